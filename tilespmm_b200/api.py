"""Python host side over the C ABI of libtilespmm_b200.so (ctypes; no torch types cross the boundary).

The class mirrors the call sequence of the upstream driver (src/main.cu:226-311): features -> threshold model
-> partition + conversion -> threshold candidates / tuning -> SpMM.  There is no CPU fallback: if the CUDA
library is missing, importing this module's `lib()` raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("TILESPMM_B200_LIB") or os.path.join(HERE, "libtilespmm_b200.so")
CLASSES = (64, 16, 8)
ARRAYS = ("orig_row", "tile_ptr", "tile_nnz", "tile_colidx", "tile_val", "panel_row")
ARRAYS64 = ("masks", "rec", "records")      # 64-row class only: export indices 6, 7, 8
_lib = None


class TileSpMMError(RuntimeError):
    pass


def lib() -> C.CDLL:
    """Loads the CUDA library; fails loudly when it has not been built (python -m tilespmm_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise TileSpMMError(f"{LIB_PATH} is missing: build it with `python -m tilespmm_b200.build` (needs nvcc)")
        L = C.CDLL(LIB_PATH)
        vp, i, ll, f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
        L.tsp_last_error.restype = C.c_char_p
        L.tsp_create.argtypes = [C.POINTER(vp), i, i]
        L.tsp_destroy.argtypes = [vp]
        L.tsp_convert_host.argtypes = [vp, i, i, ll, vp, vp, vp, f, f, i, i]
        L.tsp_convert_device.argtypes = [vp, i, i, ll, vp, vp, vp, f, f, i, i]
        L.tsp_info.argtypes = [vp, vp, vp]
        L.tsp_export.argtypes = [vp, i, i, vp, C.POINTER(ll)]
        L.tsp_top4.argtypes = [vp, i, i, vp]
        L.tsp_atom_weight.argtypes = [i, i, i]
        L.tsp_atom_weight.restype = C.c_float
        L.tsp_kernel_info.argtypes = [vp, i, i, vp]
        L.tsp_schedule.argtypes = [vp, i, i]
        L.tsp_export_schedule.argtypes = [vp, i, C.POINTER(i), vp, vp]
        L.tsp_tune.argtypes = [vp, vp, vp, i, vp, C.POINTER(f)]
        L.tsp_spmm.argtypes = [vp, vp, vp, i, vp]
        L.tsp_check_error.argtypes = [vp, vp]
        L.tsp_selftest_wait_timeout.argtypes = [vp, i]
        L.tsp_c_rows.restype = ll
        L.tsp_c_rows.argtypes = [vp]
        L.tsp_spmm_host.argtypes = [vp, vp, vp, i]
        L.tsp_spmm_host_async.argtypes = [vp, vp, vp, i, i]
        L.tsp_spmm_host_wait.argtypes = [vp, i]
        L.tsp_launch_count.restype = ll
        L.tsp_launch_count.argtypes = [vp]
        L.tsp_algorithmic_bytes.argtypes = [vp, i, i, vp]
        L.tsp_tile_bytes.argtypes = [vp, i, C.POINTER(C.c_double)]
        L.tsp_time.argtypes = [vp, i, vp, vp, i, i, C.POINTER(f)]
        L.tsp_run.argtypes = [vp, vp, vp, i, i, C.c_double, i, vp]
        L.tsp_cusparse_baseline.argtypes = [i, i, i, i, ll, vp, vp, vp, i, i, vp, vp, i, i, vp]
        L.tsp_features_from_csr.argtypes = [i, i, ll, vp, C.c_double, i, vp]
        L.tilespmm_predict_fp16.argtypes = [vp, C.POINTER(f), C.POINTER(f)]
        L.tilespmm_predict_tf32.argtypes = [vp, C.POINTER(f), C.POINTER(f)]
        L.tilespmm_predict_fp16.restype = None
        L.tilespmm_predict_tf32.restype = None
        _lib = L
    return _lib


def _p(a):
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return a.ctypes.data_as(C.c_void_p)
    if isinstance(a, int):
        return C.c_void_p(a)
    return C.c_void_p(a.data_ptr())  # a torch tensor: only its address crosses the boundary


def _check(rc: int, what: str):
    if rc != 0:
        raise TileSpMMError(f"{what} failed with status {rc}: {lib().tsp_last_error().decode()}")


def padded_width(colB: int) -> int:
    """Upstream pads the dense width to 32 or to a multiple of 64 (src/main.cu:173)."""
    return 32 if colB <= 32 else (colB + 63) // 64 * 64


def to_values(vals, precision: int) -> np.ndarray:
    """float32 -> the value type the kernels read: FP16 bit patterns (uint16) or float32 (TF32 inputs)."""
    vals = np.ascontiguousarray(vals, dtype=np.float32)
    return vals.astype(np.float16).view(np.uint16) if precision == 0 else vals


def features_from_csr(rowptr, shape, capability: float, colB: int) -> np.ndarray:
    rowptr = np.ascontiguousarray(rowptr, np.int32)
    f = np.zeros(11, dtype=np.float64)
    if not lib().tsp_features_from_csr(shape[0], shape[1], int(rowptr[-1]), _p(rowptr), capability, colB, _p(f)):
        raise TileSpMMError("inconsistent CSR row pointer")
    return f


def atom_weight(precision: int, cls: int, colB_padded: int) -> float:
    """Weight of one atomic slice in the threshold cost model (tsp_atom_weight)."""
    return float(lib().tsp_atom_weight(precision, cls, colB_padded))


def predict(precision: int, features) -> tuple[float, float]:
    f = np.ascontiguousarray(features, np.float64)
    g, d = C.c_float(0), C.c_float(0)
    (lib().tilespmm_predict_tf32 if precision else lib().tilespmm_predict_fp16)(_p(f), C.byref(g), C.byref(d))
    return g.value, d.value


class TileMatrix:
    """A sparse matrix converted to the variable 64/16/8-row tile format, resident on one GPU."""

    def __init__(self, precision: int, device: int = 0):
        self.L = lib()
        self.precision = precision
        self.device = device
        self.h = C.c_void_p()
        _check(self.L.tsp_create(C.byref(self.h), device, precision), "tsp_create")
        self.shape = None
        self.nnz = 0

    def close(self):
        if getattr(self, "h", None):
            self.L.tsp_destroy(self.h)
            self.h = None

    __del__ = close

    # -- conversion
    def convert_host(self, shape, rowptr, colidx, vals, gamma, delta, shard=(0, 1)):
        rowptr = np.ascontiguousarray(rowptr, np.int32)
        colidx = np.ascontiguousarray(colidx, np.int32)
        v = vals if (isinstance(vals, np.ndarray) and vals.dtype == np.uint16) else to_values(vals, self.precision)
        self.shape, self.nnz = tuple(shape), int(colidx.size)
        _check(self.L.tsp_convert_host(self.h, shape[0], shape[1], colidx.size, _p(rowptr), _p(colidx), _p(v),
                                       gamma, delta, shard[0], shard[1]), "tsp_convert_host")
        return self

    def convert_device(self, shape, d_rowptr, d_colidx, d_vals, nnz, gamma, delta, shard=(0, 1)):
        self.shape, self.nnz = tuple(shape), int(nnz)
        _check(self.L.tsp_convert_device(self.h, shape[0], shape[1], nnz, _p(d_rowptr), _p(d_colidx), _p(d_vals),
                                         gamma, delta, shard[0], shard[1]), "tsp_convert_device")
        return self

    # -- inspection
    def info(self):
        out = np.zeros(12, dtype=np.int32)
        rows = np.zeros(2, dtype=np.int32)
        _check(self.L.tsp_info(self.h, _p(out), _p(rows)), "tsp_info")
        self.row_range = (int(rows[0]), int(rows[1]))
        return out.reshape(3, 4)

    def array(self, cls: int, which: str) -> np.ndarray:
        w = ARRAYS.index(which) if which in ARRAYS else 6 + ARRAYS64.index(which)
        nbytes = C.c_longlong(0)
        _check(self.L.tsp_export(self.h, cls, w, None, C.byref(nbytes)), "tsp_export")
        if which == "tile_val":
            out = np.zeros(nbytes.value // (4 if self.precision else 2), dtype=np.float32 if self.precision else np.uint16)
        elif which == "masks":
            out = np.zeros(nbytes.value // (2 if self.precision else 4), dtype=np.uint16 if self.precision else np.uint32)
        elif which == "rec":
            out = np.zeros(nbytes.value // 4, dtype=np.uint32)
        elif which == "records":
            out = np.zeros(nbytes.value, dtype=np.uint8)
        else:
            out = np.zeros(nbytes.value // 4, dtype=np.int32)
        if nbytes.value:
            _check(self.L.tsp_export(self.h, cls, w, _p(out), C.byref(nbytes)), "tsp_export")
        return out

    def top4(self, cls: int, colB_padded: int) -> np.ndarray:
        out = np.zeros(4, dtype=np.int32)
        _check(self.L.tsp_top4(self.h, cls, colB_padded, _p(out)), "tsp_top4")
        return out

    def kernel_info(self, cls: int, colB_padded: int) -> np.ndarray:
        out = np.zeros(6, dtype=np.int64)
        _check(self.L.tsp_kernel_info(self.h, cls, colB_padded, _p(out)), "tsp_kernel_info")
        return out

    def schedule(self, cls: int, TH: int):
        _check(self.L.tsp_schedule(self.h, cls, TH), "tsp_schedule")
        n = C.c_int(0)
        _check(self.L.tsp_export_schedule(self.h, cls, C.byref(n), None, None), "tsp_export_schedule")
        rows = np.zeros(n.value, dtype=np.uint32)
        colstart = np.zeros(n.value + 1, dtype=np.int32)
        if n.value:
            _check(self.L.tsp_export_schedule(self.h, cls, C.byref(n), _p(rows), _p(colstart)), "tsp_export_schedule")
        return rows, colstart

    def c_rows(self) -> int:
        return int(self.L.tsp_c_rows(self.h))

    def launch_count(self) -> int:
        return int(self.L.tsp_launch_count(self.h))

    def algorithmic_bytes(self, colB_padded: int, cls: int = -1):
        out = np.zeros(3, dtype=np.float64)
        _check(self.L.tsp_algorithmic_bytes(self.h, cls, colB_padded, _p(out)), "tsp_algorithmic_bytes")
        return out

    def tile_bytes(self, cls: int = -1) -> float:
        out = C.c_double(0)
        _check(self.L.tsp_tile_bytes(self.h, cls, C.byref(out)), "tsp_tile_bytes")
        return out.value

    # -- compute
    def tune(self, d_b, d_c, colB_padded: int):
        best = np.zeros(3, dtype=np.int32)
        ms = C.c_float(0)
        _check(self.L.tsp_tune(self.h, _p(d_b), _p(d_c), colB_padded, _p(best), C.byref(ms)), "tsp_tune")
        return best, ms.value

    def spmm(self, d_b, d_c, colB_padded: int, stream: int = 0):
        _check(self.L.tsp_spmm(self.h, _p(d_b), _p(d_c), colB_padded, C.c_void_p(stream)), "tsp_spmm")

    def check_error(self, stream: int = 0):
        """Waits for `stream` (0: the device) and raises if a bounded wait ran out in a kernel of this handle."""
        _check(self.L.tsp_check_error(self.h, C.c_void_p(stream) if stream else None), "tsp_check_error")

    def spmm_host(self, h_b: np.ndarray, colB_padded: int) -> np.ndarray:
        rows = self.row_range[1] - self.row_range[0] if hasattr(self, "row_range") else self.shape[0]
        out = np.zeros((rows, colB_padded), dtype=np.float32)
        _check(self.L.tsp_spmm_host(self.h, _p(h_b), _p(out), colB_padded), "tsp_spmm_host")
        return out

    def time(self, d_b, d_c, colB_padded: int, iters: int, cls: int = -1) -> float:
        ms = C.c_float(0)
        _check(self.L.tsp_time(self.h, cls, _p(d_b), _p(d_c), colB_padded, iters, C.byref(ms)), "tsp_time")
        return ms.value

    def run(self, h_b: np.ndarray, colB_padded: int, colB_logical: int, repeat: int = 1000, cpu_pre_ms: float = 0.0,
            want_c: bool = True):
        out6 = np.zeros(6, dtype=np.float64)
        c = np.zeros((self.shape[0], colB_padded), dtype=np.float32) if want_c else None
        _check(self.L.tsp_run(self.h, _p(h_b), _p(c), colB_padded, colB_logical, cpu_pre_ms, repeat, _p(out6)), "tsp_run")
        return out6, c


def cusparse_baseline(precision, shape, rowptr, colidx, vals, h_b, colB, device=0, warmup=100, repeat=1000, want_c=True, alg=0):
    """The cuSPARSE CSR SpMM upstream runs beside its own kernels (src/main.cu:16-134); alg 1..3 select
    CUSPARSE_SPMM_CSR_ALG1..3 instead of upstream's ALG_DEFAULT."""
    rowptr = np.ascontiguousarray(rowptr, np.int32)
    colidx = np.ascontiguousarray(colidx, np.int32)
    v = vals if (isinstance(vals, np.ndarray) and vals.dtype == np.uint16) else to_values(vals, precision)
    out3 = np.zeros(3, dtype=np.float64)
    c = np.zeros((shape[0], colB), dtype=np.float32) if want_c else None
    if alg:
        _check(lib().tsp_cusparse_baseline_alg(device, precision, shape[0], shape[1], colidx.size, _p(rowptr), _p(colidx), _p(v),
                                               colB, h_b.shape[1], _p(h_b), _p(c), warmup, repeat, alg, _p(out3)), "tsp_cusparse_baseline_alg")
    else:
        _check(lib().tsp_cusparse_baseline(device, precision, shape[0], shape[1], colidx.size, _p(rowptr), _p(colidx), _p(v),
                                           colB, h_b.shape[1], _p(h_b), _p(c), warmup, repeat, _p(out3)), "tsp_cusparse_baseline")
    return out3, c


class MultiTileMatrix:
    """One matrix spread over several GPUs of this box inside one process (the tsp_multi_* layer of the C ABI): every
    device converts and multiplies a contiguous range of panels and owns the matching row slab of C; B is uploaded in
    row blocks and all-gathered over NCCL."""

    def __init__(self, precision: int, devices):
        self.L = lib()
        vp, i, ll, f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
        self.L.tsp_multi_create.argtypes = [C.POINTER(vp), i, vp, i]
        self.L.tsp_multi_destroy.argtypes = [vp]
        self.L.tsp_multi_convert_host.argtypes = [vp, i, i, ll, vp, vp, vp, f, f]
        self.L.tsp_multi_info.argtypes = [vp, vp, vp]
        self.L.tsp_multi_spmm_host.argtypes = [vp, vp, vp, i]
        self.L.tsp_multi_run.argtypes = [vp, vp, vp, i, i, C.c_double, i, vp]
        self.precision = precision
        self.devices = np.ascontiguousarray(devices, dtype=np.int32)
        self.h = C.c_void_p()
        _check(self.L.tsp_multi_create(C.byref(self.h), int(self.devices.size), _p(self.devices), precision), "tsp_multi_create")
        self.shape = None

    def close(self):
        if getattr(self, "h", None):
            self.L.tsp_multi_destroy(self.h)
            self.h = None

    __del__ = close

    def convert_host(self, shape, rowptr, colidx, vals, gamma, delta):
        rowptr = np.ascontiguousarray(rowptr, np.int32)
        colidx = np.ascontiguousarray(colidx, np.int32)
        v = vals if (isinstance(vals, np.ndarray) and vals.dtype == np.uint16) else to_values(vals, self.precision)
        self.shape = tuple(shape)
        _check(self.L.tsp_multi_convert_host(self.h, shape[0], shape[1], colidx.size, _p(rowptr), _p(colidx), _p(v), gamma, delta),
               "tsp_multi_convert_host")
        return self

    def info(self):
        out = np.zeros(12, dtype=np.int32)
        slabs = np.zeros(2 * self.devices.size, dtype=np.int32)
        _check(self.L.tsp_multi_info(self.h, _p(out), _p(slabs)), "tsp_multi_info")
        self.slabs = [tuple(int(x) for x in slabs[2 * k:2 * k + 2]) for k in range(self.devices.size)]
        return out.reshape(3, 4)

    def spmm_host(self, h_b: np.ndarray, colB_padded: int) -> np.ndarray:
        out = np.zeros((self.shape[0], colB_padded), dtype=np.float32)
        _check(self.L.tsp_multi_spmm_host(self.h, _p(h_b), _p(out), colB_padded), "tsp_multi_spmm_host")
        return out

    def run(self, h_b: np.ndarray, colB_padded: int, colB_logical: int, repeat: int = 1000):
        out6 = np.zeros(6, dtype=np.float64)
        c = np.zeros((self.shape[0], colB_padded), dtype=np.float32)
        _check(self.L.tsp_multi_run(self.h, _p(h_b), _p(c), colB_padded, colB_logical, 0.0, repeat, _p(out6)), "tsp_multi_run")
        return out6, c
