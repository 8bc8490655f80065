"""ctypes bindings of the CHECKERS: the plain-C restatement (oracle/libtile_oracle.so) and, where it was
built, the unmodified upstream sources behind oracle/_ref/libref_{fp16,tf32}.so.  Test-only."""
import ctypes as C
import hashlib
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
CLASSES = (64, 16, 8)
ARRAYS = ("orig_row", "tile_ptr", "tile_nnz", "tile_colidx", "tile_val", "panel_row")


def BN(precision, cls):
    return ((32, 16, 16), (16, 8, 8))[precision][cls]


def to_values(vals_f32, precision):
    """FP16 bit patterns (uint16) for precision 0, float32 for precision 1 (TF32 inputs are plain floats)."""
    if isinstance(vals_f32, np.ndarray) and vals_f32.dtype == np.uint16:
        return np.ascontiguousarray(vals_f32)          # already FP16 bit patterns
    vals_f32 = np.ascontiguousarray(vals_f32, dtype=np.float32)
    if precision == 0:
        return vals_f32.astype(np.float16).view(np.uint16)
    return vals_f32


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


class OrcResources(C.Structure):
    _fields_ = [("sm_count", C.c_int), ("threads_per_sm", C.c_int), ("blocks_per_sm", C.c_int),
                ("registers_per_sm", C.c_int), ("l2_bytes", C.c_int), ("shared_bytes_per_sm", C.c_longlong),
                ("threads", C.c_int), ("registers_per_thread", C.c_int), ("iteration_bytes", C.c_int),
                ("shared_bytes", C.c_longlong), ("tasks_per_block", C.c_int), ("stripes", C.c_int),
                ("atom_weight", C.c_float)]   # 0 = upstream's table


# rows of the upstream kernel table compiled into oracle/_ref (oracle/make_prefetch_stub.sh):
# index = class_group*2 + (colB != 32) with class_group 0: 8-row, 1: 16-row, 2: 64-row
UPSTREAM_KERNELS = {
    0: [(128, 46, 5120, 5120), (64, 42, 2304, 2304), (128, 46, 10240, 6144), (64, 40, 4608, 2560),
        (128, 40, 5120, 6144), (256, 40, 9216, 8192)],
    1: [(128, 52, 5120, 5120), (64, 42, 2304, 2304), (128, 48, 10240, 6144), (64, 40, 4608, 2560),
        (128, 46, 5120, 6144), (256, 54, 9216, 8192)],
}
B200_L2 = 132644864


def upstream_resources(precision, cls, colB_padded, l2_bytes=B200_L2):
    group = {0: 2, 1: 1, 2: 0}[cls]
    th, regs, smem, itb = UPSTREAM_KERNELS[precision][group * 2 + (colB_padded != 32)]
    tpb = 4 if (colB_padded == 32 and cls != 0) else 1
    stripes = 1 if colB_padded == 32 else (colB_padded + 63) // 64
    return OrcResources(148, 2048, 32, 65536, l2_bytes, 233472, th, regs, itb, smem, tpb, stripes)


class _Tiles:
    """Common accessors over a converted matrix held by either checker."""

    def info(self):
        out = np.zeros(12, dtype=np.int32)
        self._info(self.h, _ptr(out))
        return out.reshape(3, 4)  # rows, nnz, tilem, tilenum per class

    def array(self, cls, which):
        w = ARRAYS.index(which)
        nbytes = self._array(self.h, cls, w, None)
        if which == "tile_val":
            out = np.zeros(nbytes // (4 if self.precision else 2), dtype=np.float32 if self.precision else np.uint16)
        else:
            out = np.zeros(nbytes // 4, dtype=np.int32)
        if nbytes:
            self._array(self.h, cls, w, _ptr(out))
        return out

    def digest(self):
        """sha256 over every bit-exact array of the three classes, plus per-array digests."""
        per = {}
        for cls in range(3):
            for which in ARRAYS:
                per[f"{CLASSES[cls]}:{which}"] = hashlib.sha256(self.array(cls, which).tobytes()).hexdigest()[:16]
        return per


class Orc(_Tiles):
    _lib = None

    @classmethod
    def lib(cls):
        if cls._lib is None:
            L = C.CDLL(os.path.join(ORACLE_DIR, "libtile_oracle.so"))
            L.orc_convert.restype = C.c_void_p
            L.orc_convert.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_float]
            L.orc_info.argtypes = [C.c_void_p, C.c_void_p]
            L.orc_array.restype = C.c_longlong
            L.orc_array.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
            L.orc_destroy.argtypes = [C.c_void_p]
            L.orc_schedule.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
            L.orc_top4.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(OrcResources), C.c_void_p]
            L.orc_spmm_csr.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int]
            cls._lib = L
        return cls._lib

    def __init__(self, precision, shape, rowptr, colidx, vals, gamma, delta):
        L = self.lib()
        self.precision = precision
        self._info, self._array = L.orc_info, L.orc_array
        self.keep = (np.ascontiguousarray(rowptr, np.int32), np.ascontiguousarray(colidx, np.int32), to_values(vals, precision))
        self.h = L.orc_convert(precision, shape[0], shape[1], _ptr(self.keep[0]), _ptr(self.keep[1]), _ptr(self.keep[2]),
                               C.c_float(gamma), C.c_float(delta))

    def schedule(self, cls, TH):
        n = self.lib().orc_schedule(self.h, cls, TH, None, None)
        rows = np.zeros(n, dtype=np.uint32)
        colstart = np.zeros(n + 1, dtype=np.int32)
        if n:
            self.lib().orc_schedule(self.h, cls, TH, _ptr(rows), _ptr(colstart))
        return rows, colstart

    def top4(self, cls, colB_padded, res):
        out = np.zeros(4, dtype=np.int32)
        rc = self.lib().orc_top4(self.h, cls, colB_padded, C.byref(res), _ptr(out))
        assert rc == 0
        return out

    def __del__(self):
        if getattr(self, "h", None):
            self.lib().orc_destroy(self.h)
            self.h = None


def spmm_csr(precision, shape, rowptr, colidx, vals, B, ncols, trunc=True):
    """CPU CSR SpMM of the checker: returns float32 [rows, ncols]; B is [cols, ldb] (uint16 bits or float32)."""
    L = Orc.lib()
    rowptr = np.ascontiguousarray(rowptr, np.int32)
    colidx = np.ascontiguousarray(colidx, np.int32)
    v = to_values(vals, precision)
    B = np.ascontiguousarray(B)
    Cm = np.zeros((shape[0], ncols), dtype=np.float32)
    L.orc_spmm_csr(precision, int(trunc), 0, shape[0], _ptr(rowptr), _ptr(colidx), _ptr(v), _ptr(B), B.shape[1], ncols,
                   _ptr(Cm), ncols)
    return Cm


def upstream_available(precision=0):
    return os.path.exists(os.path.join(ORACLE_DIR, "_ref", f"libref_{'tf32' if precision else 'fp16'}.so"))


class Upstream(_Tiles):
    _libs = {}

    @classmethod
    def lib(cls, precision):
        if precision not in cls._libs:
            L = C.CDLL(os.path.join(ORACLE_DIR, "_ref", f"libref_{'tf32' if precision else 'fp16'}.so"))
            L.ref_convert.restype = C.c_void_p
            L.ref_convert.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_float]
            L.ref_info.argtypes = [C.c_void_p, C.c_void_p]
            L.ref_array.restype = C.c_longlong
            L.ref_array.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
            L.ref_destroy.argtypes = [C.c_void_p]
            L.ref_schedule.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
            L.ref_top4.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
            L.ref_predict.argtypes = [C.c_int, C.c_int, C.c_longlong, C.c_void_p, C.c_double, C.c_int, C.c_void_p,
                                      C.POINTER(C.c_float), C.POINTER(C.c_float)]
            L.ref_gpu_spmm.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
            L.ref_cusparse.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                       C.c_void_p, C.c_void_p, C.c_void_p]
            cls._libs[precision] = L
        return cls._libs[precision]

    def __init__(self, precision, shape, rowptr, colidx, vals, gamma, delta):
        L = self.lib(precision)
        self.precision = precision
        self.L = L
        self._info, self._array = L.ref_info, L.ref_array
        self.keep = (np.ascontiguousarray(rowptr, np.int32).copy(), np.ascontiguousarray(colidx, np.int32).copy(),
                     to_values(vals, precision).copy())
        self.h = L.ref_convert(shape[0], shape[1], int(self.keep[1].size), _ptr(self.keep[0]), _ptr(self.keep[1]),
                               _ptr(self.keep[2]), C.c_float(gamma), C.c_float(delta))

    def schedule(self, cls, TH):
        n = self.L.ref_schedule(self.h, cls, TH, None, None)
        rows = np.zeros(n, dtype=np.uint32)
        colstart = np.zeros(n + 1, dtype=np.int32)
        if n:
            self.L.ref_schedule(self.h, cls, TH, _ptr(rows), _ptr(colstart))
        return rows, colstart

    def top4(self, cls, colB_padded, l2_bytes=B200_L2):
        out = np.zeros(4, dtype=np.int32)
        self.L.ref_top4(self.h, cls, colB_padded, l2_bytes, _ptr(out))
        return out

    @classmethod
    def predict(cls, precision, shape, rowptr, capability, colB):
        L = cls.lib(precision)
        rowptr = np.ascontiguousarray(rowptr, np.int32)
        f = np.zeros(11, dtype=np.float64)
        g, d = C.c_float(0), C.c_float(0)
        rc = L.ref_predict(shape[0], shape[1], int(rowptr[-1]), _ptr(rowptr), capability, colB, _ptr(f), C.byref(g), C.byref(d))
        assert rc == 0
        return g.value, d.value, f

    def __del__(self):
        if getattr(self, "h", None):
            self.L.ref_destroy(self.h)
            self.h = None
