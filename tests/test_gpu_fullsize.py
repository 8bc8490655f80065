"""GPU tests at the full sizes of the benchmark configurations, through properties that need no CPU reference at that
size: structural invariants of the tiling, exact row sums, linearity in B, and shard concatenation."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _configs():
    from tilespmm_b200 import synth
    return {
        "c2": lambda: synth.make_config("c2"),                 # 27-point stencil 64^3, TF32, colB 128
        "c3": lambda: synth.make_config("c3", scale=19),       # R-MAT (scale 19 keeps the host generator to seconds)
        "c4": lambda: synth.make_config("c4"),                 # mixed density 524288^2, TF32, colB 256
    }


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
    rp, ci, v, shape, cfg = synth.make_config("c3", scale=19)
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
