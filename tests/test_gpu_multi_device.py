"""GPU tests of the in-process multi-GPU layer (tsp_multi_* in the C ABI, the CLI's --gpus): on a box with one GPU they
run over one device (no collective), on a box with several over up to four, where B is all-gathered over NCCL."""
import os
import subprocess

import numpy as np
import pytest

import _orc
import cases

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _devices():
    import torch
    return list(range(min(torch.cuda.device_count(), 4)))


@pytest.mark.parametrize("prec", [0, 1])
def test_multi_device_product_matches_cpu_checker(prec):
    import torch  # noqa: F401  (loads PyTorch's NCCL first, which the library then shares)
    from tilespmm_b200 import api, synth
    devs = _devices()
    rp, ci, v, shape = synth.rmat_symmetric(13, 16, 31)
    colB = 128
    B = synth.dense_b(shape[1], colB, 2)
    Bv = api.to_values(B, prec).reshape(shape[1], colB)
    vv = api.to_values(v, prec)
    want = _orc.spmm_csr(prec, shape, rp, ci, vv, Bv, colB)
    m = api.MultiTileMatrix(prec, devs).convert_host(shape, rp, ci, vv, 2.0, 1.2)
    info = m.info()
    assert int(info[:, 0].sum()) == shape[0] and int(info[:, 1].sum()) == ci.size
    assert m.slabs[0][0] == 0 and m.slabs[-1][1] == shape[0] and all(a[1] == b[0] for a, b in zip(m.slabs, m.slabs[1:]))
    one = api.TileMatrix(prec, 0).convert_host(shape, rp, ci, vv, 2.0, 1.2)
    assert info.tolist() == one.info().tolist()                     # the shards add up to the unsharded tiling
    tol = 1e-2 if prec == 0 else 5e-3
    for _ in range(2):                                              # twice: the device buffers are reused
        got = m.spmm_host(Bv, colB)
        assert np.abs(got - want).max() / np.abs(want).max() <= tol
    out6, c = m.run(Bv, colB, colB, repeat=20)
    assert out6[4] > 0 and out6[5] > 0
    assert np.abs(c - want).max() / np.abs(want).max() <= tol
    m.close(); one.close()


def test_cli_gpus_option(tmp_path):
    """`--gpus N` after upstream's arguments: same CSV row (19 fields), same check line."""
    from tilespmm_b200 import synth
    rp, ci, v, shape = cases.small_cases()["banded_1500"]
    mtx = tmp_path / "m.mtx"
    rows = np.repeat(np.arange(shape[0]), np.diff(rp))
    with open(mtx, "w") as fh:
        fh.write("%%MatrixMarket matrix coordinate real general\n")
        fh.write(f"{shape[0]} {shape[1]} {ci.size}\n")
        for r, c, x in zip(rows, ci, v):
            fh.write(f"{r + 1} {c + 1} {x:.6f}\n")
    n = len(_devices())
    exe = os.path.join(ROOT, "tilespmm_b200", "bin", "tilespmm_tf32")
    r = subprocess.run([exe, "-d", "0", str(mtx), "64", "--gpus", str(n)], cwd=tmp_path, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "Check... PASS!" in r.stdout
    row = open(tmp_path / "TileSpMM-TF32.csv").read().strip().split(",")
    assert len(row) == 19 and int(row[1]) == shape[0] and int(row[3]) == ci.size
    bad = subprocess.run([exe, "-d", "0", str(mtx), "64", "--gpus", "0"], cwd=tmp_path, capture_output=True, text=True, timeout=60)
    assert bad.returncode != 0
