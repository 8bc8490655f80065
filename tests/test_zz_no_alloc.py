"""GPU test of tsp_schedule_noalloc: the schedule builder for callers that must not allocate device memory
(all of it is owned by their own arena, or the allocator is off limits on their hot path).  It keeps its
per-panel counters in a fixed array inside the library instead of a cudaMalloc'ed workspace, so its results
must equal tsp_schedule()'s bit for bit -- also on a second call, which finds the previous call's data in that
array.  Collected last on purpose (file name), so a failure here cannot hide other tests behind `-x`."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _noalloc(L, tile_ptr_d, panel_row_d, tilem, TH, capacity, torch):
    rows = torch.full((max(capacity, 1),), 0x7fffffff, dtype=torch.int32, device="cuda")
    start = torch.full((max(capacity, 1) + 1,), -1, dtype=torch.int32, device="cuda")
    split = torch.zeros(max(tilem, 1), dtype=torch.int32, device="cuda")
    n, ns = C.c_int(-1), C.c_int(-1)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]                    # cudaMemGetInfo: what the driver has left on the device
    rc = L.tsp_schedule_noalloc(0, tilem, TH, C.c_void_p(tile_ptr_d.data_ptr()), C.c_void_p(panel_row_d.data_ptr()),
                                C.c_void_p(rows.data_ptr()), C.c_void_p(start.data_ptr()), C.c_longlong(capacity),
                                C.c_void_p(split.data_ptr()), C.byref(n), C.byref(ns), None)
    _noalloc.device_bytes_taken = free_before - torch.cuda.mem_get_info()[0]
    return rc, n.value, ns.value, rows, start, split


def test_noalloc_schedule_equals_allocating_schedule_twice_in_a_row():
    import torch
    from tilespmm_b200 import api, synth
    L = api.lib()
    L.tsp_schedule_noalloc.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong,
                                       C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_void_p]
    rp, ci, v, shape = synth.rmat_symmetric(13, 16, 4242)        # skewed rows: many split panels at small TH
    m = api.TileMatrix(0).convert_host(shape, rp, ci, v, 2.0, 1.2)
    info = m.info()
    calls = 0
    for cls in range(3):
        tilem = int(info[cls, 2])
        if tilem == 0:
            continue
        tile_ptr_d = torch.from_numpy(m.array(cls, "tile_ptr")).cuda()
        panel_row_d = torch.from_numpy(m.array(cls, "panel_row")).cuda()
        for TH in (8, 24, 8):                                     # consecutive calls reuse the library's array
            want_rows, want_start = m.schedule(cls, TH)
            cap = int(want_rows.size) + 5
            rc, n, ns, rows, start, split = _noalloc(L, tile_ptr_d, panel_row_d, tilem, TH, cap, torch)
            assert rc == 0, L.tsp_last_error()
            calls += 1
            if calls > 1:      # the first call on a device may load the kernels; every later one takes no device memory at all
                assert _noalloc.device_bytes_taken == 0, _noalloc.device_bytes_taken
            assert n == want_rows.size
            np.testing.assert_array_equal(rows[:n].cpu().numpy().view(np.uint32), want_rows)
            np.testing.assert_array_equal(start[:n + 1].cpu().numpy(), want_start)
            split_rows = np.unique(want_rows[(want_rows >> 31) != 0] & 0x7fffffff)
            assert ns == split_rows.size
            np.testing.assert_array_equal(np.sort(split[:ns].cpu().numpy()), split_rows.astype(np.int32))
    m.close()


def test_noalloc_limits_are_reported():
    import torch
    from tilespmm_b200 import api
    L = api.lib()
    L.tsp_schedule_noalloc.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong,
                                       C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_void_p]
    tile_ptr = torch.tensor([0, 40, 40, 45], dtype=torch.int32, device="cuda")   # panel 0 splits into 5 slices at TH=8
    panel_row = torch.tensor([0, 8, 16], dtype=torch.int32, device="cuda")
    rc, n, ns, rows, start, split = _noalloc(L, tile_ptr, panel_row, 3, 8, 3, torch)
    assert rc == 3 and n == 7                                   # TSP_ENOMEM, tasks needed reported
    assert int(rows[0]) == 0x7fffffff and int(start[0]) == -1   # outputs untouched
    rc, n, ns, rows, start, split = _noalloc(L, tile_ptr, panel_row, 3, 8, 7, torch)
    assert rc == 0 and n == 7 and ns == 1
    assert start.cpu().numpy()[:8].tolist() == [0, 8, 16, 24, 32, 40, 40, 45]
    rc, *_ = _noalloc(L, tile_ptr, panel_row, (1 << 20) + 1, 8, 7, torch)
    assert rc == 1 and b"exceed" in L.tsp_last_error()         # beyond the fixed scratch: refused, TSP_EINVAL
