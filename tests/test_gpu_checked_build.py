"""GPU tests of the checked build (libtilespmm_b200_debug.so, compiled with -DTSP_DEBUG): its kernels verify every
gathered column index, every task's tile range and every written row of C, report a violation through the handle's error
flag and skip the access -- nothing is ever read or written out of bounds, so these tests cannot fault the GPU.  Run in
a child process, because a process loads one build of the library."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEBUG_LIB = os.path.join(ROOT, "tilespmm_b200", "libtilespmm_b200_debug.so")

CHILD = r'''
import ctypes as C, sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
import _orc, cases
from tilespmm_b200 import api, synth
L = api.lib()
assert hasattr(L, "tsp_debug_poke"), "not the checked build"
L.tsp_debug_poke.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_longlong, C.c_int]
rp, ci, v, shape = cases.small_cases()["banded_4099"]
for prec in (0, 1):
    tol = 1e-2 if prec == 0 else 5e-3
    tdt = torch.float16 if prec == 0 else torch.float32
    for (g, d), cls in (((0.0, 1.5), 0), ((5.0, 0.0), 1), ((5.0, 3.0), 2), ((2.0, 1.2), None)):
        colB = 128
        B = synth.dense_b(shape[1], colB, 3)
        Bv = api.to_values(B, prec).reshape(shape[1], colB)
        vv = api.to_values(v, prec)
        want = _orc.spmm_csr(prec, shape, rp, ci, vv, Bv, colB)
        m = api.TileMatrix(prec).convert_host(shape, rp, ci, vv, g, d)
        info = m.info()
        # 1. a clean run passes every check, and the rows of C past the padded slab stay untouched (canary rows)
        dB = torch.from_numpy(Bv.view(np.float16) if prec == 0 else Bv).cuda()
        rows = m.c_rows()
        dC = torch.full((rows + 64, colB), 12345.0, dtype=torch.float32, device="cuda")
        m.spmm(dB, dC, colB)
        m.check_error()
        got = dC[:shape[0]].cpu().numpy()
        assert np.abs(got - want).max() / np.abs(want).max() <= tol
        assert bool((dC[rows:] == 12345.0).all()), "a kernel wrote past the rows tsp_c_rows() promises"
        if cls is None:
            m.close(); continue
        # 2. a column index outside B: reported, not dereferenced
        assert L.tsp_debug_poke(m.h, cls, 0, 5, shape[1] + 1000) == 0
        m.spmm(dB, dC, colB)
        try:
            m.check_error(); raise SystemExit("a bad column index went unnoticed")
        except api.TileSpMMError as e:
            assert "column outside B" in str(e), e
        # 3. a task that runs past the class's tiles: reported, not executed
        m.convert_host(shape, rp, ci, vv, g, d); m.info()
        m.spmm(dB, dC, colB); m.check_error()
        assert L.tsp_debug_poke(m.h, cls, 1, 0, int(info[cls, 3]) + 50) == 0
        m.spmm(dB, dC, colB)
        try:
            m.check_error(); raise SystemExit("a bad task range went unnoticed")
        except api.TileSpMMError as e:
            assert "outside the class's tiles" in str(e), e
        # 4. C with fewer rows than the slab needs cannot be expressed through the ABI (the caller states no size), so the
        #    row check is exercised through a slab whose handle claims fewer rows: covered by the task check above
        m.close()
print("checked build ok")
'''


def test_checked_build_passes_clean_runs_and_reports_damaged_indices():
    if not os.path.exists(DEBUG_LIB):
        from tilespmm_b200 import build
        build.build()
    env = dict(os.environ, TILESPMM_B200_LIB=DEBUG_LIB)
    r = subprocess.run([sys.executable, "-c", CHILD, ROOT], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "checked build ok" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_release_library_has_no_poke_entry():
    from tilespmm_b200 import api
    assert not hasattr(api.lib(), "tsp_debug_poke")
