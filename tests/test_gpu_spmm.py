"""GPU parity tests of the SpMM kernels (through the C ABI) against the CPU CSR SpMM of the checker.
Tolerance: max relative error <= 1e-2 (FP16 inputs) / 5e-3 (TF32 inputs) with FP32 accumulation, measured as
max|C - C_ref| / max|C_ref|; exact for integer-valued inputs (the upstream check, src/main.cu:315-335, allows 1e-3 absolute)."""
import numpy as np
import pytest

import _orc
import cases

pytestmark = pytest.mark.gpu

TOL = {0: 1e-2, 1: 5e-3}
CASES = cases.small_cases()


def run_case(prec, shape, rp, ci, v, g, d, colB, integer=False, seed=0, force_th=None):
    from tilespmm_b200 import api, synth
    cb = api.padded_width(colB)
    B = synth.dense_b(shape[1], cb, seed, "uniform" if prec == 0 else "normal")
    if integer:
        B = np.round(B * 3)
        v = np.round(v * 3)
    B[:, colB:] = 0
    Bv = api.to_values(B, prec).reshape(shape[1], cb)
    vv = api.to_values(v, prec)
    m = api.TileMatrix(prec).convert_host(shape, rp, ci, vv, g, d)
    m.info()
    if force_th:
        for cls in range(3):
            m.schedule(cls, force_th)
    got = m.spmm_host(Bv, cb)
    want = _orc.spmm_csr(prec, shape, rp, ci, vv, Bv, cb)
    scale = max(float(np.abs(want).max()), 1e-30)
    err = float(np.abs(got - want).max()) / scale
    m.close()
    return err, got, want


@pytest.mark.parametrize("prec", [0, 1])
@pytest.mark.parametrize("gd", [(0.0, 1.5), (5.0, 0.0), (5.0, 3.0), (2.0, 1.2)])
@pytest.mark.parametrize("colB", [32, 64, 128, 256])
def test_spmm_matches_cpu_oracle(prec, gd, colB):
    for name in ("stencil_g17", "rmat_s11", "banded_1500", "rand_ragged_203"):
        rp, ci, v, shape = CASES[name]
        err, _, _ = run_case(prec, shape, rp, ci, v, gd[0], gd[1], colB)
        assert err <= TOL[prec], (name, prec, gd, colB, err)


@pytest.mark.parametrize("prec", [0, 1])
@pytest.mark.parametrize("colB", [1, 33, 100, 192, 320])
def test_odd_widths_and_integer_inputs_are_exact(prec, colB):
    """Integer-valued inputs are exact in FP16/TF32/FP32, so every class must reproduce the CPU result bit for bit
    (upstream's own check)."""
    for name, gd in (("banded_1500", (2.0, 1.2)), ("rand_dups_150", (5.0, 0.0)), ("rand_tiny_5", (5.0, 3.0)), ("rand_wide_64x5000", (0.0, 1.5))):
        rp, ci, v, shape = CASES[name]
        if name == "rand_dups_150":
            v = np.sign(v)      # repeated entries are summed in value type: keep the sums exact
        err, got, want = run_case(prec, shape, rp, ci, v, gd[0], gd[1], colB, integer=True)
        np.testing.assert_array_equal(got, want, err_msg=f"{name} prec={prec} colB={colB}")


@pytest.mark.parametrize("prec", [0, 1])
@pytest.mark.parametrize("gd", [(0.0, 1.5), (5.0, 0.0), (5.0, 3.0)])
def test_split_panels_use_the_atomic_path(prec, gd):
    """A threshold of 8 tiles splits the long panels of a power-law matrix into slices that accumulate into C."""
    rp, ci, v, shape = CASES["rmat_s11"]
    err, got, want = run_case(prec, shape, rp, ci, v, gd[0], gd[1], 64, integer=True, force_th=8)
    np.testing.assert_allclose(got, want, rtol=0, atol=1e-3)


def test_empty_matrix_and_empty_panels_write_zeros():
    from tilespmm_b200 import api
    rp, ci, v, shape = CASES["all_empty_40"]
    for prec in (0, 1):
        m = api.TileMatrix(prec).convert_host(shape, rp, ci, v, 2.0, 1.2)
        m.info()
        B = np.ones((shape[1], 64), dtype=np.float32)
        got = m.spmm_host(api.to_values(B, prec).reshape(shape[1], 64), 64)
        assert not got.any()


def test_second_call_overwrites_instead_of_accumulating():
    """C does not have to be cleared between calls, including for split panels."""
    import torch
    from tilespmm_b200 import api, synth
    rp, ci, v, shape = CASES["rmat_s11"]
    m = api.TileMatrix(0).convert_host(shape, rp, ci, np.ones_like(v), 5.0, 3.0)
    m.info()
    m.schedule(2, 8)
    B = torch.ones((shape[1], 64), dtype=torch.float16, device="cuda")
    Cd = torch.full((m.c_rows(), 64), 7.0, dtype=torch.float32, device="cuda")
    m.spmm(B, Cd, 64)
    m.spmm(B, Cd, 64)
    torch.cuda.synchronize()
    want = np.diff(rp).astype(np.float32)
    np.testing.assert_array_equal(Cd[:shape[0], 0].cpu().numpy(), want)


def test_sharded_spmm_covers_all_rows():
    from tilespmm_b200 import api, synth
    rp, ci, v, shape = synth.rmat_symmetric(13, 16, 5)
    B = synth.dense_b(shape[1], 128, 1)
    Bv = api.to_values(B, 0).reshape(shape[1], 128)
    vv = api.to_values(v, 0)
    want = _orc.spmm_csr(0, shape, rp, ci, vv, Bv, 128)
    got = []
    for k in range(4):
        m = api.TileMatrix(0).convert_host(shape, rp, ci, vv, 2.0, 1.2, shard=(k, 4))
        m.info()
        got.append(m.spmm_host(Bv, 128))
    got = np.concatenate(got)
    assert got.shape == want.shape
    assert float(np.abs(got - want).max()) / float(np.abs(want).max()) <= 1e-2


def test_upstream_driver_mirror_and_cusparse_baseline():
    """tsp_run (the call_tilespmm_cuda mirror) against the cuSPARSE baseline with upstream's own check: integer
    inputs, |difference| <= 1e-3 (src/main.cu:315-335)."""
    from tilespmm_b200 import api, synth
    rp, ci, v, shape = synth.stencil27(16, 3)
    rng = np.random.default_rng(1325)
    for prec in (0, 1):
        vv = api.to_values(rng.integers(1, 4, size=v.size).astype(np.float32), prec)
        B = np.zeros((shape[1], 64), dtype=np.float32)
        B[:, :40] = rng.integers(1, 4, size=(shape[1], 40))
        Bv = api.to_values(B, prec).reshape(shape[1], 64)
        m = api.TileMatrix(prec).convert_host(shape, rp, ci, vv, 2.0, 1.2)
        m.info()
        out6, c = m.run(Bv, 64, 40, repeat=20)
        out3, c2 = api.cusparse_baseline(prec, shape, rp, ci, vv, Bv, 40, warmup=2, repeat=5)
        assert out6[4] > 0 and out6[5] > 0 and out3[1] > 0
        assert np.abs(c[:, :40] - c2).max() <= 1e-3


def test_async_host_path_two_slots_in_flight():
    """tsp_spmm_host_async / _wait: two calls in flight in the two staging slots give what two blocking calls give."""
    import ctypes as C
    import torch
    from tilespmm_b200 import api, synth
    rp, ci, v, shape = CASES["banded_4099"]
    m = api.TileMatrix(1).convert_host(shape, rp, ci, v, 2.0, 1.2)
    m.info()
    Bs = [torch.from_numpy(synth.dense_b(shape[1], 128, s, "normal")).pin_memory() for s in (1, 2, 3)]
    want = [m.spmm_host(b.numpy(), 128) for b in Bs]
    outs = [torch.zeros((shape[0], 128), dtype=torch.float32).pin_memory() for _ in Bs]
    L = m.L
    for i, b in enumerate(Bs):
        slot = i & 1
        if i >= 2:
            assert L.tsp_spmm_host_wait(m.h, slot) == 0
        assert L.tsp_spmm_host_async(m.h, C.c_void_p(b.data_ptr()), C.c_void_p(outs[i].data_ptr()), 128, slot) == 0, L.tsp_last_error()
    assert L.tsp_spmm_host_async(m.h, C.c_void_p(Bs[0].data_ptr()), C.c_void_p(outs[0].data_ptr()), 128, 0) == 4   # slot still in flight
    for slot in (0, 1):
        assert L.tsp_spmm_host_wait(m.h, slot) == 0
    for got, w in zip(outs, want):
        np.testing.assert_array_equal(got.numpy(), w)
    m.close()


def test_tma_gather4_variant_of_the_64_row_kernel():
    """The 64-row kernel has a second producer: TMA tile::gather4 loads instead of cp.async (TSP_SPMM64=tma, chosen once
    per process).  Run the 64-row parity cases of this file in a child process with that variant."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, TSP_SPMM64="tma")
    here = os.path.abspath(__file__)
    r = subprocess.run([sys.executable, "-m", "pytest", here, "-x", "-q", "-m", "gpu", "-k",
                        "(gd0 or exact or split) and not tma_gather4 and not async"], env=env, capture_output=True, text=True, timeout=1200)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


def test_transposed_tcgen05_variant_of_the_small_kernels():
    """The 16/8-row classes have a second kernel: persistent, tcgen05.mma on the transposed product with the accumulators
    in tensor memory (TSP_SMALL=t, chosen once per process; widths that are multiples of 64).  Run the parity cases of
    this file in a child process with that variant."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, TSP_SMALL="t")
    here = os.path.abspath(__file__)
    r = subprocess.run([sys.executable, "-m", "pytest", here, "-x", "-q", "-m", "gpu", "-k",
                        "not tma_gather4 and not transposed_tcgen05 and not async"], env=env, capture_output=True, text=True, timeout=1200)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


def test_cusparse_algorithms():
    """The stronger cuSPARSE baselines (CSR_ALG1..3) give the same product as upstream's ALG_DEFAULT."""
    import numpy as np
    from tilespmm_b200 import api, synth
    rp, ci, v, shape = synth.fixed_nnz_per_row(2048, 12, seed=11)
    vi = np.round(v * 4).astype(np.float32)
    B = np.round(synth.dense_b(shape[1], 64, 3, "uniform") * 4).astype(np.float32)
    for prec in (0, 1):
        Bv = api.to_values(B, prec).reshape(shape[1], 64)
        ref = None
        for alg in (0, 1, 2, 3):
            out3, c = api.cusparse_baseline(prec, shape, rp, ci, vi, Bv, 64, warmup=1, repeat=2, alg=alg)
            assert out3[1] > 0 and out3[2] > 0
            ref = c if ref is None else ref
            np.testing.assert_array_equal(c, ref)     # small integers: exact in every algorithm
