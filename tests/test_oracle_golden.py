"""CPU tests: the plain-C restatement (oracle/tile_oracle.c) against golden vectors produced by the unmodified
upstream sources (tests/golden/make_golden.py), and against those sources live where oracle/_ref was built."""
import hashlib
import json
import os

import numpy as np
import pytest

import _orc
import cases

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "tiling_golden.json")))
TINY = np.load(os.path.join(os.path.dirname(__file__), "golden", "tiny_arrays.npz"))
CASES = cases.small_cases()


def h(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()[:16]


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("prec", [0, 1])
def test_restatement_matches_upstream_golden(name, prec):
    rp, ci, v, shape = CASES[name]
    for (g, d) in cases.GAMMA_DELTA:
        rec = GOLDEN["tiling"][f"{name}|{prec}|{g}|{d}"]
        o = _orc.Orc(prec, shape, rp, ci, v, g, d)
        assert o.info().tolist() == rec["info"], (name, prec, g, d)
        assert o.digest() == rec["arrays"], (name, prec, g, d)          # bit-exact: every tiling array
        for cls in range(3):
            for TH in (8, 24, 64):
                rows, cs = o.schedule(cls, TH)
                assert [int(rows.size), h(rows), h(cs)] == rec["sched"][f"{cls}:{TH}"]
            for cb in (32, 64, 256):
                got = o.top4(cls, cb, _orc.upstream_resources(prec, cls, cb)).tolist()
                assert got == rec["top4"][f"{cls}:{cb}"], (name, prec, g, d, cls, cb)


def test_tiny_arrays_elementwise():
    for key in TINY.files:
        name, prec, g, d, cls, which = key.split("|")
        rp, ci, v, shape = CASES[name]
        o = _orc.Orc(int(prec), shape, rp, ci, v, float(g), float(d))
        np.testing.assert_array_equal(o.array(int(cls), which), TINY[key], err_msg=key)


@pytest.mark.skipif(not (_orc.upstream_available(0) and _orc.upstream_available(1)), reason="oracle/_ref not built")
@pytest.mark.parametrize("prec", [0, 1])
def test_restatement_matches_upstream_live(prec):
    from tilespmm_b200 import synth
    for rp, ci, v, shape in (synth.stencil27(24, 5), synth.rmat_symmetric(14, 16, 6), synth.mixed_density(16384, 7),
                             cases.banded_blocks(20011, 50000, 8)):
        for (g, d) in ((2.0, 1.2), (1.4, 1.5), (3.0, 1.0), (0.0, 1.5), (5.0, 0.0), (5.0, 3.0)):
            o = _orc.Orc(prec, shape, rp, ci, v, g, d)
            u = _orc.Upstream(prec, shape, rp, ci, v, g, d)
            assert o.info().tolist() == u.info().tolist()
            assert o.digest() == u.digest()


def test_cpu_spmm_matches_numpy():
    """The CPU CSR SpMM of the checker against a float64 numpy product on exactly representable inputs."""
    rp, ci, v, shape = cases.random_csr(120, 90, 7, 31)
    rng = np.random.default_rng(3)
    B = rng.integers(-3, 4, size=(shape[1], 40)).astype(np.float32)
    v = np.round(v * 4).astype(np.float32)
    dense = np.zeros(shape, dtype=np.float64)
    for r in range(shape[0]):
        for j in range(rp[r], rp[r + 1]):
            dense[r, ci[j]] += v[j]
    want = dense @ B.astype(np.float64)
    got16 = _orc.spmm_csr(0, shape, rp, ci, v, B.astype(np.float16).view(np.uint16), 40)
    got32 = _orc.spmm_csr(1, shape, rp, ci, v, B, 40)
    np.testing.assert_array_equal(got16, want.astype(np.float32))
    np.testing.assert_array_equal(got32, want.astype(np.float32))
