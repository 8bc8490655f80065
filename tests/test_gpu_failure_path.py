"""GPU test of the failure path (through the C ABI): a device-side wait that runs out must come back as TSP_ETIMEOUT,
hang nothing, leave no tensor memory allocated and leave the handle usable.  The wait is made to run out on the host's
terms: a self-test kernel polls, a bounded number of times, an mbarrier that nothing ever arrives on."""
import numpy as np
import pytest

import _orc
import cases

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_the_handle_stays_usable():
    from tilespmm_b200 import api, synth
    rp, ci, v, shape = cases.small_cases()["stencil_g17"]
    for prec in (0, 1):
        B = synth.dense_b(shape[1], 128, 4)
        Bv = api.to_values(B, prec).reshape(shape[1], 128)
        vv = api.to_values(v, prec)
        m = api.TileMatrix(prec).convert_host(shape, rp, ci, vv, 0.0, 1.5)      # all 64-row tiles: the tcgen05 kernel
        m.info()
        want = _orc.spmm_csr(prec, shape, rp, ci, vv, Bv, 128)
        tol = 1e-2 if prec == 0 else 5e-3
        before = m.spmm_host(Bv, 128)
        assert np.abs(before - want).max() / np.abs(want).max() <= tol
        for polls in (1, 1024):
            rc = m.L.tsp_selftest_wait_timeout(m.h, polls)
            assert rc == 6, rc                                                   # TSP_ETIMEOUT
            assert b"bounded wait" in m.L.tsp_last_error()
            m.check_error()                                                      # the record was cleared: no error now
        # tensor memory was freed and the context is intact: many more launches of the tensor-memory kernel succeed
        for _ in range(8):
            after = m.spmm_host(Bv, 128)
        assert np.abs(after - want).max() / np.abs(want).max() <= tol      # (slices of split panels add in any order)
        with pytest.raises(api.TileSpMMError):
            api._check(m.L.tsp_selftest_wait_timeout(m.h, 0), "tsp_selftest_wait_timeout")   # argument check
        m.close()
