"""CPU test: the C-ABI library loads and exports every entry point include/tilespmm_b200.h declares
(no compute call is made -- there is no GPU here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "tilespmm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tsp_[a-z0-9_]+|tilespmm_predict_[a-z0-9]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("tsp_create", "tsp_convert_host", "tsp_convert_device", "tsp_export", "tsp_top4", "tsp_schedule",
                 "tsp_tune", "tsp_spmm", "tsp_spmm_host", "tsp_run", "tsp_cusparse_baseline",
                 "tilespmm_predict_fp16", "tilespmm_predict_tf32"):
        assert must in names


def test_library_exports_every_declared_symbol():
    path = os.path.join(ROOT, "tilespmm_b200", "libtilespmm_b200.so")
    if not os.path.exists(path):
        from tilespmm_b200 import build
        build.build()
    L = ctypes.CDLL(path)
    missing = [n for n in declared_functions() if not hasattr(L, n)]
    assert not missing, missing


def test_model_abi_returns_an_upstream_candidate():
    """The threshold model keeps upstream's C ABI (src/ml_predict.h:14-15) and answers with one of upstream's
    66 candidate pairs (src/model.h:14-38)."""
    from tilespmm_b200 import api
    gammas = [1.0, 1.4, 1.8, 2.0, 2.4, 2.8, 3.0, 3.4, 3.8, 4.0]
    deltas = [1.0, 1.2, 1.4, 1.5, 1.8, 2.0]
    cands = {(0.0, 1.5), (5.0, 0.0), (5.0, 3.0), (2.5, 1.0), (2.5, 1.2), (3.5, 1.0)} | {(g, d) for g in gammas for d in deltas}
    import numpy as np
    rng = np.random.default_rng(0)
    for _ in range(200):
        rows = int(2 ** rng.uniform(8, 24))
        avg = float(2 ** rng.uniform(0, 8))
        f = [0, 0, rows, rows, rows * avg, 1 - avg / rows, avg, avg * 2 ** rng.uniform(0, 8), 0, 10.0, float(rng.choice([32, 64, 128, 256]))]
        for prec in (0, 1):
            g, d = api.predict(prec, f)
            assert (round(g, 1), round(d, 1)) in cands


def test_features_match_upstream_definition():
    from tilespmm_b200 import api
    import numpy as np
    rp = np.array([0, 3, 3, 7, 8], dtype=np.int32)
    f = api.features_from_csr(rp, (4, 10), 10.0, 100)
    assert f.tolist() == [0.0, 0.0, 4.0, 10.0, 8.0, 1.0 - 8.0 / 40.0, 2.0, 4.0, 0.0, 10.0, 100.0]
    with pytest.raises(api.TileSpMMError):
        api.features_from_csr(np.array([1, 2], dtype=np.int32), (1, 3), 10.0, 8)
