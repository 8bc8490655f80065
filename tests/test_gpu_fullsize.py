"""GPU tests at the full sizes of the benchmark configurations.

Two kinds.  (1) Parity on the configurations themselves, with their own value laws: tiling bit-exact against the
checker's restatement at full size, C against the CPU CSR SpMM of the checker and against upstream's own kernels
(oracle/_ref, where it was built) within max relative error 1e-2 (FP16) / 5e-3 (TF32) at FP32 accumulation.
(2) Properties that need no CPU reference at that size: structural invariants of the tiling, exact row sums,
linearity in B, and shard concatenation."""
import ctypes as C
import functools

import numpy as np
import pytest

import _orc

pytestmark = pytest.mark.gpu

TOL = {0: 1e-2, 1: 5e-3}


@functools.lru_cache(maxsize=2)
def _config(name):
    from tilespmm_b200 import synth
    return synth.make_config(name)       # c3 is the full scale-20 R-MAT


def _configs():
    return {name: (lambda n=name: _config(n)) for name in ("c1", "c2", "c3", "c4")}


def _errors(got, want, bound):
    """(normalised, elementwise) errors of `got` against `want`: max|got - want| / max|want|, and max over the entries of
    |got - want| / (|A| |B|), the rounding-error bound of a dot product, which is a relative error per entry that stays
    meaningful where C itself cancels to nearly zero."""
    diff = np.abs(got - want)
    norm = float(diff.max()) / max(float(np.abs(want).max()), 1e-30)
    elem = float((diff / np.maximum(bound, 1e-30)).max())
    return norm, elem


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4"])
def test_baseline_config_parity_with_cpu_checker_and_upstream_gpu(name):
    """The configuration as the benchmark runs it: thresholds from the model, N(0,1) / U[-1,1] right-hand side."""
    from tilespmm_b200 import api, synth
    rp, ci, v, shape, cfg = _config(name)
    prec = 0 if cfg["precision"] == "fp16" else 1
    colB = cfg["colB"]
    cb = api.padded_width(colB)
    B = synth.dense_b(shape[1], cb, 1, cfg["b_dist"])
    B[:, colB:] = 0
    Bv = api.to_values(B, prec).reshape(shape[1], cb)
    vv = api.to_values(v, prec)
    g, d = api.predict(prec, api.features_from_csr(rp, shape, 10.0, colB))

    m = api.TileMatrix(prec).convert_host(shape, rp, ci, vv, g, d)
    info = m.info()
    o = _orc.Orc(prec, shape, rp, ci, vv, g, d)                # tiling: bit for bit at full size
    assert info.tolist() == o.info().tolist()
    for cls in range(3):
        for w in _orc.ARRAYS:
            assert np.array_equal(m.array(cls, w), o.array(cls, w)), (name, cls, w)
    del o
    got = m.spmm_host(Bv, cb)
    m.close()

    want = _orc.spmm_csr(prec, shape, rp, ci, vv, Bv, cb)
    av = np.abs(v.astype(np.float16).astype(np.float32) if prec == 0 else v)
    Ba = np.abs(Bv.view(np.float16).astype(np.float32) if prec == 0 else Bv)
    bound = _orc.spmm_csr(1, shape, rp, ci, av, Ba, cb, trunc=False)
    norm, elem = _errors(got[:, :colB], want[:, :colB], bound[:, :colB])
    assert norm <= TOL[prec] and elem <= TOL[prec], (name, norm, elem)
    assert not got[:, colB:].any()

    if not _orc.upstream_available(prec):
        pytest.skip("oracle/_ref was not built: no comparison with upstream's own kernels")
    g_up, d_up, _ = _orc.Upstream.predict(prec, shape, rp, 10.0, colB)
    u = _orc.Upstream(prec, shape, rp, ci, vv, g_up, d_up)
    c_up = np.zeros((shape[0], cb), dtype=np.float32)
    out6 = np.zeros(6, dtype=np.float64)
    rc = u.L.ref_gpu_spmm(u.h, 0, cb, colB, Bv.ctypes.data_as(C.c_void_p), c_up.ctypes.data_as(C.c_void_p), out6.ctypes.data_as(C.c_void_p))
    assert rc == 0
    norm_u, elem_u = _errors(got[:, :colB], c_up[:, :colB], bound[:, :colB])
    assert norm_u <= TOL[prec] and elem_u <= TOL[prec], (name, norm_u, elem_u)
    # and with upstream's thresholds the tiling equals upstream's own conversion, array for array
    m2 = api.TileMatrix(prec).convert_host(shape, rp, ci, vv, g_up, d_up)
    assert m2.info().tolist() == u.info().tolist()
    for cls in range(3):
        for w in _orc.ARRAYS:
            assert np.array_equal(m2.array(cls, w), u.array(cls, w)), (name, cls, w)
    m2.close()


def test_c5_sampled_rows_and_shard_concatenation():
    """Configuration 5 (symmetric R-MAT generated on the GPU, FP16, colB 128) at scale 22: 10,000 sampled rows of C
    against a CPU dot product in float64, and the tiling of 8 shards concatenated against the unsharded tiling."""
    import torch
    from tilespmm_b200 import api, synth
    scale, colB = 22, 128
    d_rp, d_ci, d_v, shape = synth.rmat_symmetric_device(scale, 16, 1005, values="u01")
    d_v = d_v.to(torch.float16)
    nnz = int(d_ci.numel())
    rp = d_rp.cpu().numpy()
    g, d = api.predict(0, api.features_from_csr(rp, shape, 10.0, colB))
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    dB = (torch.rand((shape[1], colB), generator=gen, device="cuda") * 2 - 1).to(torch.float16)

    full = api.TileMatrix(0).convert_device(shape, d_rp, d_ci, d_v, nnz, g, d)
    finfo = full.info()
    dC = torch.empty((full.c_rows(), colB), dtype=torch.float32, device="cuda")
    full.spmm(dB, dC, colB)
    torch.cuda.synchronize()

    rng = np.random.default_rng(11)
    heavy = np.argsort(np.diff(rp))[-100:]                        # the longest rows (split panels) are always sampled
    rows = np.unique(np.concatenate([rng.integers(0, shape[0], 10000), heavy]))
    rows_t = torch.from_numpy(rows).cuda()
    got = dC[rows_t].cpu().numpy().astype(np.float64)
    Bh = dB.cpu().numpy()
    worst = 0.0
    for i, r in enumerate(rows):
        a, b = int(rp[r]), int(rp[r + 1])
        cols = d_ci[a:b].cpu().numpy()
        vals = d_v[a:b].cpu().numpy().astype(np.float64)
        Bg = Bh[cols].astype(np.float64)
        want = vals @ Bg
        if a < b:
            worst = max(worst, float((np.abs(got[i] - want) / np.maximum(np.abs(vals) @ np.abs(Bg), 1e-30)).max()))
        else:
            assert not got[i].any()
    assert worst <= TOL[0], worst

    arrays = {(cls, w): full.array(cls, w) for cls in range(3) for w in _orc.ARRAYS}
    full.close()
    del dC
    at = {key: 0 for key in arrays}                                # how much of every unsharded array the shards have covered
    pinfo = np.zeros((3, 4), dtype=np.int64)
    ranges = []
    for k in range(8):
        p = api.TileMatrix(0).convert_device(shape, d_rp, d_ci, d_v, nnz, g, d, shard=(k, 8))
        pinfo += p.info()
        ranges.append(p.row_range)
        for (cls, w), whole in arrays.items():
            part = p.array(cls, w)
            if w in ("tile_ptr", "tile_nnz"):                      # prefix sums restart in every shard: compare the differences
                part, ref = np.diff(part), np.diff(whole)
            else:
                ref = whole
            assert np.array_equal(part, ref[at[(cls, w)]:at[(cls, w)] + part.size]), (k, cls, w)
            at[(cls, w)] += part.size
        p.close()
    assert pinfo.tolist() == finfo.tolist()
    assert ranges[0][0] == 0 and ranges[-1][1] == shape[0] and all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    for (cls, w), whole in arrays.items():
        assert at[(cls, w)] == (max(whole.size - 1, 0) if w in ("tile_ptr", "tile_nnz") else whole.size), (cls, w)


@pytest.mark.parametrize("name", ["c2", "c3", "c4"])
def test_fullsize_invariants_rowsums_linearity(name):
    import torch
    from tilespmm_b200 import api
    rp, ci, v, shape, cfg = _configs()[name]()
    prec = 0 if cfg["precision"] == "fp16" else 1
    colB = cfg["colB"]
    tdt = torch.float16 if prec == 0 else torch.float32
    feats = api.features_from_csr(rp, shape, 10.0, colB)
    g, d = api.predict(prec, feats)
    ones = np.ones_like(v)
    m = api.TileMatrix(prec).convert_host(shape, rp, ci, ones, g, d)          # all values 1: products are exact
    info = m.info()
    assert int(info[:, 0].sum()) == shape[0] and int(info[:, 1].sum()) == ci.size   # every row and entry in one class
    row_nnz = np.diff(rp)
    for cls in range(3):
        if info[cls, 2] == 0:
            continue
        bn = (32, 16, 16)[cls] if prec == 0 else (16, 8, 8)[cls]
        tp, tn, tc = m.array(cls, "tile_ptr"), m.array(cls, "tile_nnz"), m.array(cls, "tile_colidx")
        orow = m.array(cls, "orig_row")
        assert np.all(np.diff(tp) >= 0) and tp[-1] == info[cls, 3]
        assert tn[0] == 0 and np.all(np.diff(tn) >= 0) and tn[-1] == int(row_nnz[orow].sum()) == info[cls, 1]
        cols = tc.reshape(-1, bn)
        assert np.all(np.diff(cols, axis=1) >= 0)                              # sorted inside every tile (padding repeats the last)
        assert cols.min() >= 0 and cols.max() < shape[1]
        vals = m.array(cls, "tile_val")
        nz = np.count_nonzero(vals if prec else vals.view(np.float16))
        assert nz == info[cls, 1]                                              # no repeated entries in these generators
    # A * ones: every C entry is the row's entry count, exactly
    B = torch.ones((shape[1], colB), dtype=tdt, device="cuda")
    C = torch.full((m.c_rows(), colB), -1.0, dtype=torch.float32, device="cuda")
    m.spmm(B, C, colB)
    torch.cuda.synchronize()
    got = C[:shape[0]].cpu().numpy()
    assert np.array_equal(got[:, 0], row_nnz.astype(np.float32)) and np.array_equal(got[:, -1], row_nnz.astype(np.float32))
    assert np.array_equal(got.min(axis=1), got.max(axis=1))
    # linearity with small integers (exact in FP16/TF32 and in FP32 sums at these magnitudes)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(3)
    B1 = torch.randint(-2, 3, (shape[1], colB), generator=gen, device="cuda").to(tdt)
    B2 = torch.randint(-2, 3, (shape[1], colB), generator=gen, device="cuda").to(tdt)
    C1, C2, C12 = (torch.empty_like(C) for _ in range(3))
    m.spmm(B1, C1, colB)
    m.spmm(B2, C2, colB)
    m.spmm((B1.float() + B2.float()).to(tdt), C12, colB)
    torch.cuda.synchronize()
    assert torch.equal(C12[:shape[0]], C1[:shape[0]] + C2[:shape[0]])
    m.close()


def test_fullsize_shards_concatenate():
    import torch
    from tilespmm_b200 import api, synth
    rp, ci, v, shape, cfg = _config("c3")
    colB = 64
    feats = api.features_from_csr(rp, shape, 10.0, colB)
    g, d = api.predict(0, feats)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    B = torch.randint(-2, 3, (shape[1], colB), generator=gen, device="cuda").to(torch.float16)
    vi = np.round(v * 2).astype(np.float32)
    full = api.TileMatrix(0).convert_host(shape, rp, ci, vi, g, d)
    full.info()
    Cf = torch.empty((full.c_rows(), colB), dtype=torch.float32, device="cuda")
    full.spmm(B, Cf, colB)
    parts = []
    for k in range(8):
        p = api.TileMatrix(0).convert_host(shape, rp, ci, vi, g, d, shard=(k, 8))
        p.info()
        Cp = torch.empty((p.c_rows(), colB), dtype=torch.float32, device="cuda")
        p.spmm(B, Cp, colB)
        torch.cuda.synchronize()
        parts.append(Cp[:p.row_range[1] - p.row_range[0]].clone())
        p.close()
    torch.cuda.synchronize()
    assert torch.equal(torch.cat(parts), Cf[:shape[0]])


def test_fullsize_with_the_transposed_tcgen05_kernels():
    """Same properties with the tcgen05 kernel of the 16/8-row classes (TSP_SMALL=t, chosen once per process): R-MAT and
    the mixed-density matrix have long and split panels, which is where its two MMA issuers and out-of-order slot
    releases are exercised."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, TSP_SMALL="t")
    here = os.path.abspath(__file__)
    r = subprocess.run([sys.executable, "-m", "pytest", here, "-x", "-q", "-m", "gpu", "-k", "rowsums_linearity or shards_concatenate"],
                       env=env, capture_output=True, text=True, timeout=1800)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
