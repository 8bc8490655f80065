"""TEST AND MEASUREMENT INFRASTRUCTURE ONLY (not part of the product path).

Runs UPSTREAM's own SpMM -- its unmodified sources compiled for sm_100a into oracle/_ref -- on one matrix on one GPU and
prints one JSON line: upstream's model picks the thresholds (capability 10.0), upstream's host code converts, upstream's
call_tilespmm_cuda (src/csr2tile.h:826-1093) tunes and runs its 1000-pass timed loop.  bench.py starts this as a child
process, after its own timed regions, to report upstream's kernels beside this library's on the same box.

    python oracle/upstream_gpu_leg.py <dir with rp.npy ci.npy vv.npy b.npy> <precision> <rows> <cols> <colB> <colB_padded> <device>
"""
import ctypes as C
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(HERE), "tests"))

import _orc  # noqa: E402


def main():
    tmp, prec, rows, cols, colB, cb, device = sys.argv[1], *[int(x) for x in sys.argv[2:8]]
    rp, ci = np.load(os.path.join(tmp, "rp.npy")), np.load(os.path.join(tmp, "ci.npy"))
    vv, Bv = np.load(os.path.join(tmp, "vv.npy")), np.load(os.path.join(tmp, "b.npy"))
    shape = (rows, cols)
    g, d, _ = _orc.Upstream.predict(prec, shape, rp, 10.0, colB)
    t0 = time.perf_counter()
    u = _orc.Upstream(prec, shape, rp, ci, vv, g, d)
    convert_ms = (time.perf_counter() - t0) * 1e3
    out6 = np.zeros(6, dtype=np.float64)
    c = np.zeros((rows, cb), dtype=np.float32)     # upstream copies its checked result here
    rc = u.L.ref_gpu_spmm(u.h, device, cb, colB, Bv.ctypes.data_as(C.c_void_p), c.ctypes.data_as(C.c_void_p), out6.ctypes.data_as(C.c_void_p))
    if rc != 0:
        raise SystemExit(f"ref_gpu_spmm returned {rc}")
    print(json.dumps({"time_ms": float(out6[4]), "tflops": float(out6[5]), "gamma": g, "delta": d,
                      "tiles_64_16_8": [int(x) for x in u.info()[:, 3]], "best_th": [int(x) for x in out6[:3]],
                      "host_convert_ms": convert_ms, "tune_ms": float(out6[3]),
                      "protocol": "upstream call_tilespmm_cuda: its model, conversion, tuning and 1000-pass loop"}))


if __name__ == "__main__":
    main()
