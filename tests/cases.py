"""Seeded test matrices shared by the golden-vector generator and the parity tests."""
import numpy as np

from tilespmm_b200 import synth

GAMMA_DELTA = [(0.0, 1.5), (5.0, 0.0), (5.0, 3.0), (1.0, 1.0), (2.0, 1.2), (3.0, 2.0), (1.4, 1.5), (3.8, 1.0),
               (2.5, 1.0), (4.0, 1.8)]


def random_csr(rows, cols, avg, seed, duplicates=False, empty_every=0):
    """Small irregular CSR: row lengths geometric-ish around ``avg``, unsorted columns, optional repeated
    (row, col) entries and empty rows."""
    rng = np.random.Generator(np.random.Philox(seed))
    lens = rng.poisson(avg, size=rows).astype(np.int64)
    lens[rng.random(rows) < 0.05] *= 6
    if empty_every:
        lens[::empty_every] = 0
    lens = np.minimum(lens, cols)
    rowptr = np.zeros(rows + 1, dtype=np.int32)
    rowptr[1:] = np.cumsum(lens)
    colidx = np.empty(int(rowptr[-1]), dtype=np.int32)
    for r in range(rows):
        n = int(lens[r])
        if n == 0:
            continue
        if duplicates:
            colidx[rowptr[r]:rowptr[r + 1]] = rng.integers(0, cols, size=n)
        else:
            colidx[rowptr[r]:rowptr[r + 1]] = rng.choice(cols, size=n, replace=False)
    vals = rng.uniform(-1.0, 1.0, size=colidx.size).astype(np.float32)
    return rowptr, colidx, vals, (rows, cols)


def banded_blocks(rows, cols, seed):
    """Clustered structure (runs of rows sharing columns) so that every class gets panels for mid thresholds."""
    rng = np.random.Generator(np.random.Philox(seed))
    rp = [0]
    ci = []
    r = 0
    while r < rows:
        run = int(rng.choice([8, 16, 24, 64, 72, 128]))
        kind = rng.integers(0, 3)
        base = rng.integers(0, max(1, cols - 200))
        shared = rng.choice(200, size=int(rng.integers(4, 60)), replace=False) + base
        for _ in range(min(run, rows - r)):
            if kind == 0:      # rows share most columns -> tall tiles pay off
                c = shared[rng.random(shared.size) < 0.8]
            elif kind == 1:    # disjoint random columns
                c = rng.choice(cols, size=int(rng.integers(0, 12)), replace=False)
            else:              # mix
                c = np.unique(np.concatenate([shared[:6], rng.choice(cols, size=3, replace=False)]))
            c = rng.permutation(c)
            ci.append(c.astype(np.int32))
            rp.append(rp[-1] + c.size)
            r += 1
    colidx = np.concatenate(ci) if ci else np.zeros(0, np.int32)
    vals = rng.standard_normal(colidx.size).astype(np.float32)
    return np.asarray(rp, dtype=np.int32), colidx, vals, (rows, cols)


def small_cases():
    """name -> (rowptr, colidx, vals, shape).  Seconds on a CPU for every checker."""
    out = {}
    out["c1_4096"] = synth.fixed_nnz_per_row(4096, 16, 1001)
    out["c1_small_517"] = synth.fixed_nnz_per_row(517, 9, 11)
    out["stencil_g12"] = synth.stencil27(12, 1002)
    out["stencil_g17"] = synth.stencil27(17, 1002)          # 4913 rows: not a multiple of 8
    out["rmat_s11"] = synth.rmat_symmetric(11, 16, 1003)
    out["rmat_s13_u01"] = synth.rmat_symmetric(13, 8, 1005, values="u01")
    out["mixed_4096"] = synth.mixed_density(4096, 1004)
    out["rand_ragged_203"] = random_csr(203, 331, 6, 21, empty_every=7)
    out["rand_dups_150"] = random_csr(150, 64, 10, 22, duplicates=True)
    out["rand_wide_64x5000"] = random_csr(64, 5000, 300, 23)
    out["rand_tiny_5"] = random_csr(5, 40, 4, 24)
    out["rand_1row"] = random_csr(1, 10, 3, 25)
    out["banded_1500"] = banded_blocks(1500, 3000, 26)
    out["banded_4099"] = banded_blocks(4099, 9000, 27)
    rp, ci, v, sh = synth.stencil27(10, 3)
    out["stencil_shuffled"] = (*synth.shuffle_within_rows(rp, ci, v, 9), sh)
    out["all_empty_40"] = (np.zeros(41, np.int32), np.zeros(0, np.int32), np.zeros(0, np.float32), (40, 17))
    return out
