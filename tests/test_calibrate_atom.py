"""CPU tests of the atomic-weight calibration (tilespmm_b200/calibrate_atom.py): its restatement of the cost terms
against the checker's cost model, and the fit on synthetic timings."""
from types import SimpleNamespace

import numpy as np
import pytest

from tests import _orc
from tilespmm_b200 import calibrate_atom as cal

PROPS = SimpleNamespace(max_threads_per_multi_processor=2048, regs_per_multiprocessor=65536,
                        shared_memory_per_multiprocessor=233472, multi_processor_count=148, L2_cache_size=_orc.B200_L2)


def test_fit_recovers_a_known_weight():
    rng = np.random.default_rng(3)
    tile_ptr = np.arange(0, 64 * 4096 + 1, 64, dtype=np.int32)
    info = [128, 80, 34816, 17408, 4, 1]
    cap = cal.resident_blocks(info, PROPS) * PROPS.multi_processor_count
    X = np.array([[c, e * 128 / 32.0] for c, e in (cal.cost_terms(tile_ptr, th, 128, info, cap, PROPS.L2_cache_size) for th in range(8, 65, 8))])
    for lam in (0.002, 0.01, 0.03):
        y = 0.004 * (X[:, 0] + lam * X[:, 1]) * (1 + rng.normal(0, 0.002, len(X)))
        got, raw, r2 = cal.fit_weight(X, y)
        assert abs(got - lam) < 0.1 * lam and r2 > 0.99
    # a weight outside the accepted range is clamped, never passed on
    assert cal.fit_weight(X, 0.004 * X[:, 0])[0] == cal.LO
    assert cal.fit_weight(X, 0.004 * (X[:, 0] + X[:, 1]))[0] == cal.HI


@pytest.mark.parametrize("prec,cls,cb,weight", [(1, 2, 128, 0.00960), (0, 1, 128, 0.01163), (1, 0, 32, 0.020), (0, 2, 32, 0.00360)])
def test_cost_terms_agree_with_the_checker(prec, cls, cb, weight):
    """The cheapest threshold under cost_terms + weight is the checker's first candidate (upstream's table weight)."""
    bn = {0: (32, 16, 16), 1: (16, 8, 8)}[prec][cls]
    rows = 256 * cal.BM[cls]
    rp, ci, v, shape = cal.uniform_matrix(rows, max(1, 48 * bn // cal.BM[cls]), 5 + cls)
    o = _orc.Orc(prec, shape, rp, ci, v, *cal.FORCE[cls])
    tile_ptr = o.array(cls, "tile_ptr")
    lens = np.diff(tile_ptr)
    assert lens.max() <= 5 * lens.mean()          # the skew discount of the model stays off
    res = _orc.upstream_resources(prec, cls, cb)
    info = [res.threads, res.registers_per_thread, res.shared_bytes, res.iteration_bytes, res.tasks_per_block, res.stripes]
    cap = cal.resident_blocks(info, PROPS) * PROPS.multi_processor_count
    tmax = min(128, (int(lens.max()) + 7) // 8 * 8)
    costs = {}
    for th in range(8, tmax + 1, 8):
        comp, extra = cal.cost_terms(tile_ptr, th, cb, info, cap, PROPS.L2_cache_size)
        costs[th] = np.float32(comp) + np.float32(weight / 32.0 * cb) * np.float32(extra)
    best = min(costs, key=lambda th: (costs[th], th))
    top4 = o.top4(cls, cb, res).tolist()
    # near ties may swap under float32 rounding: the checker's first choice must be within 0.1 % of the minimum here
    assert costs[top4[0]] <= costs[best] * 1.001, (top4, best, costs)


def test_library_table_is_within_the_accepted_range():
    """tsp_atom_weight is a host-side table lookup: every entry lies in the range the calibration may write."""
    from tilespmm_b200 import api
    for prec in (0, 1):
        for cls in (0, 1, 2):
            for cb in (32, 64, 128, 256):
                w = api.atom_weight(prec, cls, cb)
                assert cal.LO * 0.999 <= w <= cal.HI * 1.001, (prec, cls, cb, w)
            assert api.atom_weight(prec, cls, 64) == api.atom_weight(prec, cls, 256)   # one row for every width above 32


@pytest.mark.gpu
def test_calibration_leg_runs_on_the_gpu():
    """One small (precision, class, width) case end to end: conversion, every candidate threshold scheduled and timed, fit."""
    lam, raw, r2, n = cal.fit_case(1, 1, 128, iters=5, panels=256, tiles_per_panel=64)
    assert cal.LO <= lam <= cal.HI and n >= 3 and np.isfinite(raw) and np.isfinite(r2)
