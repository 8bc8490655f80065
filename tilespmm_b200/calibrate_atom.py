"""Calibration of the atomic-slice weight of the threshold cost model on the GPU at hand.

Upstream's get_optimal_prefetch_th (src/csr2tile.h:437-642) prices a threshold TH as

    cost(TH) = blocks/cap * TH + longest slice + l2 term + lambda_atom * (colB / 32) * (extra slices)

and hard-codes lambda_atom per {32 columns, wider} x tile class x precision, "calibrated from existing platform
data" (src/csr2tile.h:483-495) -- its own kernels on its own GPUs.  This tool is that calibration for THESE kernels:
for every (precision, class, width) it converts a seeded matrix whose panels all hold the same number of tiles (so
the skew discount of src/csr2tile.h:519 stays off), schedules every candidate TH, times the class kernel, and fits

    time(TH) = a * [blocks/cap * TH + longest slice + l2 term] + a * lambda * (colB / 32) * (extra slices)

by least squares for (a, a * lambda).  lambda is clamped to [1e-4, 0.05]: the model only orders candidates and the four
cheapest are then measured on the GPU, so a rough weight is enough, a zero or a huge one is not.

    python -m tilespmm_b200.calibrate_atom            # needs the GPU; prints the fitted table
    python -m tilespmm_b200.calibrate_atom --write    # ... and rewrites csrc/atom_table.inc (then rebuild)
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
TABLE = os.path.join(HERE, "csrc", "atom_table.inc")
FORCE = {0: (0.0, 1.5), 1: (5.0, 0.0), 2: (5.0, 3.0)}   # (gamma, delta) that puts every panel into one class
BM = {0: 64, 1: 16, 2: 8}
LO, HI = 1e-4, 0.05


def cost_terms(tile_ptr, TH, colB, info, cap, l2_bytes):
    """(computation terms, extra slices) of upstream's cost for threshold TH (src/csr2tile.h:540-612)."""
    lens = np.diff(tile_ptr)
    lens = lens[lens > 0]
    parts = (lens + TH - 1) // TH
    each = (lens + parts - 1) // parts
    tasks = int(parts.sum())
    stripes, tasks_per_block, iteration_bytes = int(info[5]), int(info[4]), int(info[3])
    blocks = (tasks * stripes + tasks_per_block - 1) // tasks_per_block
    lambda_l2 = iteration_bytes * cap / l2_bytes
    l2 = float(((1.0 - 1.0 / parts)[parts > 1]).sum()) * lambda_l2
    return blocks / cap * TH + float(each.max()) + l2, int((parts - 1).sum())


def resident_blocks(info, props):
    threads, regs, smem = int(info[0]), int(info[1]), int(info[2])
    blk = props.max_threads_per_multi_processor // threads
    blk = min(blk, props.regs_per_multiprocessor // max(1, regs * threads))
    if smem > 0:
        blk = min(blk, props.shared_memory_per_multiprocessor // smem)
    return max(1, min(blk, 32))


def uniform_matrix(rows, per_row, seed):
    """rows x rows CSR with ``per_row`` entries per row at uniformly drawn columns (repeats are rare and summed)."""
    rng = np.random.default_rng(seed)
    colidx = rng.integers(0, rows, size=rows * per_row, dtype=np.int32)
    rowptr = (np.arange(rows + 1, dtype=np.int64) * per_row).astype(np.int32)
    vals = rng.uniform(-1.0, 1.0, size=rows * per_row).astype(np.float32)
    return rowptr, colidx, vals, (rows, rows)


def fit_case(precision, cls, colB, iters=200, panels=4096, tiles_per_panel=128, seed=77, verbose=False):
    import torch
    from . import api
    bn = {0: (32, 16, 16), 1: (16, 8, 8)}[precision][cls]
    rows = panels * BM[cls]
    per_row = max(1, tiles_per_panel * bn // BM[cls])
    rp, ci, v, shape = uniform_matrix(rows, per_row, seed + 10 * cls + precision)
    cb = api.padded_width(colB)
    m = api.TileMatrix(precision).convert_host(shape, rp, ci, api.to_values(v, precision), *FORCE[cls])
    tile_ptr = m.array(cls, "tile_ptr")
    info = m.kernel_info(cls, cb)
    props = torch.cuda.get_device_properties(0)
    cap = resident_blocks(info, props) * props.multi_processor_count
    dB = torch.zeros((shape[1], cb), dtype=torch.float16 if precision == 0 else torch.float32, device="cuda")
    dB.uniform_(-1, 1)
    dC = torch.empty((m.c_rows(), cb), dtype=torch.float32, device="cuda")
    tmax = min(128, (int(np.diff(tile_ptr).max()) + 7) // 8 * 8)
    X, y, seen = [], [], set()
    for TH in range(8, tmax + 1, 8):
        comp, extra = cost_terms(tile_ptr, TH, cb, info, cap, props.L2_cache_size)
        if extra in seen:
            continue
        seen.add(extra)
        m.schedule(cls, TH)
        m.time(dB, dC, cb, 20, cls)
        t = min(m.time(dB, dC, cb, iters, cls) for _ in range(3))
        X.append([comp, extra * cb / 32.0])
        y.append(t)
        if verbose:
            print(f"    TH={TH} computation={comp:.1f} extra_slices={extra} ms={t:.5f}", flush=True)
    m.close()
    return fit_weight(X, y) + (len(y),)


def fit_weight(X, y):
    """Least-squares (a, a * lambda) of time = a * X[:, 0] + a * lambda * X[:, 1]; returns (clamped, raw, R^2)."""
    X, y = np.asarray(X, dtype=np.float64), np.asarray(y, dtype=np.float64)
    sol, *_ = np.linalg.lstsq(X, y, rcond=None)
    a, al = float(sol[0]), float(sol[1])
    lam = al / a if a > 0 else HI
    pred = X @ sol
    r2 = 1.0 - float(((y - pred) ** 2).sum()) / max(1e-30, float(((y - y.mean()) ** 2).sum()))
    return min(HI, max(LO, lam)), lam, r2


def write_table(w, gpu_name, path=TABLE):
    def row(wide):
        return "{" + ", ".join("{" + ", ".join(f"{w[(p, c, wide)]:.5f}f" for p in (0, 1)) + "}" for c in (0, 1, 2)) + "}"
    text = (
        "// Weight of one atomic slice in the threshold cost model, per {32 columns, wider} x {64-, 16-, 8-row class} x {FP16, TF32}.\n"
        "// Written by `python -m tilespmm_b200.calibrate_atom --write` from timings on the GPU named below; upstream keeps a table of\n"
        "// the same shape, calibrated for its kernels on its GPUs (src/csr2tile.h:483-495).\n"
        f"// fitted on: {gpu_name}\n"
        "static const float kAtomWeight[2][3][2] = {\n"
        f"    {row(0)},\n    {row(1)},\n}};\n")
    with open(path, "w") as f:
        f.write(text)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--write", action="store_true", help="rewrite csrc/atom_table.inc with the fitted weights")
    ap.add_argument("--out", default=TABLE, help="where --write puts the table (default: csrc/atom_table.inc)")
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--panels", type=int, default=4096)
    ap.add_argument("--tiles-per-panel", type=int, default=128)
    ap.add_argument("--verbose", action="store_true", help="print every timed threshold")
    args = ap.parse_args(argv)
    import torch
    if not torch.cuda.is_available():
        print("calibrate_atom needs a GPU", file=sys.stderr)
        return 2
    w = {}
    for precision in (0, 1):
        for cls in (0, 1, 2):
            for wide, colB in ((0, 32), (1, 128)):
                lam, raw, r2, n = fit_case(precision, cls, colB, iters=args.iters, panels=args.panels, tiles_per_panel=args.tiles_per_panel,
                                           verbose=args.verbose)
                w[(precision, cls, wide)] = lam
                print(f"precision={precision} class={BM[cls]}-row colB={colB}: lambda_atom={lam:.5f} (unclamped {raw:.5f}, R2={r2:.3f}, {n} thresholds; "
                      f"library now {api_weight(precision, cls, colB):.5f})", flush=True)
    if args.write:
        write_table(w, torch.cuda.get_device_name(0), args.out)
        print(f"wrote {args.out}; rebuild with python -m tilespmm_b200.build")
    return 0


def api_weight(precision, cls, colB):
    from . import api
    return api.atom_weight(precision, cls, colB)


if __name__ == "__main__":
    sys.exit(main())
