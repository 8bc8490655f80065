"""Side-by-side measurement on one GPU box: this library vs the UNMODIFIED upstream kernels (oracle/_ref, built for
sm_100a) vs cuSPARSE, on the benchmark configurations, with C parity between all of them.

    python tests/compare_upstream_gpu.py [c1 c2 c3 c4] [--scale S] > compare.jsonl

Not a pytest file (it lives here because only tests may drive oracle/).  One JSON line per configuration.
Upstream is driven through its own call_tilespmm_cuda (thresholds from its own model at capability 10.0, its own
tuning, 1000 timed passes) and cusparse_spmm_all (100 warm-up + 1000 timed passes)."""
import ctypes as C
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

import _orc  # noqa: E402
from tilespmm_b200 import api, synth  # noqa: E402

PREC = {"fp16": 0, "tf32": 1}


def main():
    names = [a for a in sys.argv[1:] if a.startswith("c")] or ["c1", "c2", "c3", "c4"]
    scale = int(sys.argv[sys.argv.index("--scale") + 1]) if "--scale" in sys.argv else None
    for name in names:
        kw = {}
        if scale and name in ("c3", "c5"):
            kw["scale"] = scale
        rp, ci, v, shape, cfg = synth.make_config(name, **kw)
        prec, colB = PREC[cfg["precision"]], cfg["colB"]
        cb = api.padded_width(colB)
        B = synth.dense_b(shape[1], cb, 1, cfg["b_dist"])
        B[:, colB:] = 0
        Bv = api.to_values(B, prec).reshape(shape[1], cb)
        vv = api.to_values(v, prec)
        nnz = int(ci.size)
        rec = {"config": name, "rows": shape[0], "nnz": nnz, "precision": cfg["precision"], "colB": colB}

        want = _orc.spmm_csr(prec, shape, rp, ci, vv, Bv, cb)
        scale_c = float(np.abs(want).max())

        # ---- upstream kernels with upstream's own model
        g_up, d_up, _ = _orc.Upstream.predict(prec, shape, rp, 10.0, colB)
        t0 = time.perf_counter()
        u = _orc.Upstream(prec, shape, rp, ci, vv, g_up, d_up)
        rec["upstream_convert_s"] = time.perf_counter() - t0
        c_up = np.zeros((shape[0], cb), dtype=np.float32)
        out6 = np.zeros(6, dtype=np.float64)
        rc = u.L.ref_gpu_spmm(u.h, 0, cb, colB, Bv.ctypes.data_as(C.c_void_p), c_up.ctypes.data_as(C.c_void_p), out6.ctypes.data_as(C.c_void_p))
        assert rc == 0, rc
        rec["upstream"] = {"gamma": g_up, "delta": d_up, "tiles_64_16_8": u.info()[:, 3].tolist(), "best_th": out6[:3].tolist(),
                           "tune_ms": out6[3], "time_ms": out6[4], "tflops": out6[5],
                           "rel_err_vs_cpu": float(np.abs(c_up - want).max()) / scale_c}
        out3 = np.zeros(3, dtype=np.float64)
        c_cs = np.zeros((shape[0], colB), dtype=np.float32)
        rc = u.L.ref_cusparse(shape[0], shape[1], nnz, u.keep[0].ctypes.data_as(C.c_void_p), u.keep[1].ctypes.data_as(C.c_void_p),
                              u.keep[2].ctypes.data_as(C.c_void_p), colB, cb, Bv.ctypes.data_as(C.c_void_p),
                              c_cs.ctypes.data_as(C.c_void_p), out3.ctypes.data_as(C.c_void_p))
        assert rc == 0, rc
        rec["cusparse"] = {"time_ms": out3[1], "tflops": out3[2], "rel_err_vs_cpu": float(np.abs(c_cs - want[:, :colB]).max()) / scale_c}

        # ---- this library: its own model, and upstream's thresholds for a like-for-like tiling
        feats = api.features_from_csr(rp, shape, 10.0, colB)
        for label, (g, d) in (("ours", api.predict(prec, feats)), ("ours_upstream_thresholds", (g_up, d_up))):
            t0 = time.perf_counter()
            m = api.TileMatrix(prec).convert_host(shape, rp, ci, vv, g, d)
            conv = time.perf_counter() - t0
            info = m.info()
            out, c = m.run(Bv, cb, colB, repeat=1000)
            rec[label] = {"gamma": g, "delta": d, "tiles_64_16_8": info[:, 3].tolist(), "best_th": out[:3].tolist(), "tune_ms": out[3],
                          "time_ms": out[4], "tflops": out[5], "convert_s": conv,
                          "rel_err_vs_cpu": float(np.abs(c - want).max()) / scale_c,
                          "rel_err_vs_upstream_gpu": float(np.abs(c - c_up).max()) / scale_c}
            if label == "ours_upstream_thresholds":   # same thresholds: the tiling must be bit-identical to upstream's
                same = info.tolist() == u.info().tolist() and all(
                    np.array_equal(m.array(k, w), u.array(k, w)) for k in range(3) for w in _orc.ARRAYS)
                rec[label]["tiling_bit_exact_vs_upstream"] = bool(same)
            m.close()
        rec["speedup_vs_upstream"] = rec["ours"]["tflops"] / rec["upstream"]["tflops"]
        rec["speedup_vs_cusparse"] = rec["ours"]["tflops"] / rec["cusparse"]["tflops"]
        print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
