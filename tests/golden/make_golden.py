"""Regenerates tests/golden/tiling_golden.json and tests/golden/tiny_arrays.npz from the UNMODIFIED upstream
sources (oracle/_ref/libref_*.so, built by `make -C oracle ref` where the upstream tree is present).

Run from the repository root:  python tests/golden/make_golden.py
The JSON holds, per (case, precision, gamma, delta): the 3x4 info table (rows, nnz, panels, tiles per class),
a 64-bit digest of every bit-exact array, the schedule digests for three thresholds and the four threshold
candidates for three dense widths; plus threshold-model outputs for a list of feature vectors.
The NPZ holds complete arrays for the two smallest cases so a failure can be looked at element by element.
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import _orc  # noqa: E402
import cases  # noqa: E402


def h(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()[:16]


def main():
    golden = {"tiling": {}, "model": []}
    tiny = {}
    for name, (rp, ci, v, shape) in cases.small_cases().items():
        for prec in (0, 1):
            for (g, d) in cases.GAMMA_DELTA:
                u = _orc.Upstream(prec, shape, rp, ci, v, g, d)
                rec = {"info": u.info().tolist(), "arrays": u.digest(), "sched": {}, "top4": {}}
                for cls in range(3):
                    for TH in (8, 24, 64):
                        rows, cs = u.schedule(cls, TH)
                        rec["sched"][f"{cls}:{TH}"] = [int(rows.size), h(rows), h(cs)]
                    for cb in (32, 64, 256):
                        rec["top4"][f"{cls}:{cb}"] = u.top4(cls, cb).tolist()
                golden["tiling"][f"{name}|{prec}|{g}|{d}"] = rec
                if name in ("rand_tiny_5", "rand_dups_150") and (g, d) in ((2.0, 1.2), (0.0, 1.5), (5.0, 0.0), (5.0, 3.0)):
                    for cls in range(3):
                        for which in _orc.ARRAYS:
                            tiny[f"{name}|{prec}|{g}|{d}|{cls}|{which}"] = u.array(cls, which)
    # threshold model: upstream src/model.h through its C ABI (src/ml_predict.h:14-15)
    rng = np.random.Generator(np.random.Philox(77))
    for prec in (0, 1):
        for _ in range(400):
            rows = int(2 ** rng.uniform(8, 24))
            cols = rows if rng.random() < 0.7 else int(2 ** rng.uniform(8, 24))
            avg = float(2 ** rng.uniform(0, 8))
            nnz = int(min(rows * avg, rows * float(cols)))
            mx = int(max(avg, 1) * 2 ** rng.uniform(0, 8))
            mn = int(rng.integers(0, max(1, int(avg))))
            cap = float(rng.choice([8.0, 8.6, 8.9, 9.0, 10.0, 12.0]))
            colB = int(rng.choice([8, 32, 64, 100, 128, 256, 512]))
            f = [0.0, 0.0, float(rows), float(cols), float(nnz), 1.0 - nnz / (float(rows) * cols), nnz / rows,
                 float(mx), float(mn), cap, float(colB)]
            import ctypes as C
            g, d = C.c_float(0), C.c_float(0)
            fa = np.asarray(f, dtype=np.float64)
            _orc.Upstream.lib(prec).ref_predict_features(fa.ctypes.data_as(C.c_void_p), C.byref(g), C.byref(d))
            golden["model"].append({"precision": prec, "features": f, "gamma": g.value, "delta": d.value})
    # Matrix Market loader: upstream mmio_allinone (src/mmio_highlevel.h:307-480) on the fixtures under tests/golden/mtx
    import ctypes as C
    import glob
    L = _orc.Upstream.lib(1)
    golden["mtx"] = {}
    for path in sorted(glob.glob(os.path.join(HERE, "mtx", "*.mtx"))):
        m, n, nnz, sym = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        rp, ci, va = C.POINTER(C.c_int)(), C.POINTER(C.c_int)(), C.POINTER(C.c_float)()
        rc = L.ref_read_mtx(path.encode(), C.byref(m), C.byref(n), C.byref(nnz), C.byref(sym), C.byref(rp), C.byref(ci), C.byref(va))
        assert rc == 0, (path, rc)
        golden["mtx"][os.path.basename(path)] = {"m": m.value, "n": n.value, "nnz": nnz.value, "symmetric": sym.value,
                                                  "rowptr": [rp[i] for i in range(m.value + 1)],
                                                  "colidx": [ci[i] for i in range(nnz.value)],
                                                  "val": [float(va[i]) for i in range(nnz.value)]}
    with open(os.path.join(HERE, "tiling_golden.json"), "w") as fh:
        json.dump(golden, fh, separators=(",", ":"))
    np.savez_compressed(os.path.join(HERE, "tiny_arrays.npz"), **tiny)
    print("cases:", len(golden["tiling"]), "model rows:", len(golden["model"]))


if __name__ == "__main__":
    main()
