"""Seeded synthetic matrices with the shapes, sizes and value distributions of the benchmark
configurations (they stand in for the public matrix collections the upstream project is measured on).

Every generator returns a CSR triple ``(rowptr int32[rows+1], colidx int32[nnz], values float32[nnz])``
plus the shape.  Values are float32; callers round them to FP16 or keep them as TF32 inputs.
Generators are deterministic for a given seed (numpy Philox streams).
"""
from __future__ import annotations

import numpy as np


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(seed))


def fixed_nnz_per_row(n: int = 4096, per_row: int = 16, seed: int = 1001):
    """Config 1: n x n, exactly ``per_row`` nonzeros per row, columns uniform without replacement,
    stored in generation order (unsorted); values U[-1, 1]."""
    rng = _rng(seed)
    cols = np.empty((n, per_row), dtype=np.int32)
    chunk = max(1, (1 << 24) // max(n, 1))
    for r0 in range(0, n, chunk):
        r1 = min(n, r0 + chunk)
        keys = rng.random((r1 - r0, n), dtype=np.float32)
        cols[r0:r1] = np.argpartition(keys, per_row - 1, axis=1)[:, :per_row].astype(np.int32)
    rowptr = (np.arange(n + 1, dtype=np.int64) * per_row).astype(np.int32)
    vals = rng.uniform(-1.0, 1.0, size=n * per_row).astype(np.float32)
    return rowptr, cols.reshape(-1), vals, (n, n)


def stencil27(g: int = 64, seed: int = 1002):
    """Config 2: 27-point stencil on a g^3 grid, x fastest, Dirichlet boundaries (outside neighbours
    dropped); diagonal 26, off-diagonals -1, each with U[-1e-3, 1e-3] jitter."""
    rng = _rng(seed)
    n = g * g * g
    idx = np.arange(n, dtype=np.int64)
    x, y, z = idx % g, (idx // g) % g, idx // (g * g)
    rows, cols, diag = [], [], []
    for dz in (-1, 0, 1):
        for dy in (-1, 0, 1):
            for dx in (-1, 0, 1):
                ok = ((x + dx >= 0) & (x + dx < g) & (y + dy >= 0) & (y + dy < g)
                      & (z + dz >= 0) & (z + dz < g))
                r = idx[ok]
                rows.append(r)
                cols.append(r + dx + dy * g + dz * g * g)
                diag.append(np.full(r.shape, dx == 0 and dy == 0 and dz == 0))
    rows, cols, diag = np.concatenate(rows), np.concatenate(cols), np.concatenate(diag)
    order = np.lexsort((cols, rows))
    rows, cols, diag = rows[order], cols[order], diag[order]
    vals = np.where(diag, 26.0, -1.0) + rng.uniform(-1e-3, 1e-3, size=rows.size)
    rowptr = np.zeros(n + 1, dtype=np.int64)
    np.add.at(rowptr, rows + 1, 1)
    return np.cumsum(rowptr).astype(np.int32), cols.astype(np.int32), vals.astype(np.float32), (n, n)


def rmat_symmetric(scale: int = 20, edge_factor: int = 16, seed: int = 1003, values: str = "one",
                   abcd=(0.57, 0.19, 0.19, 0.05)):
    """Configs 3 and 5: symmetric R-MAT, duplicates and self-loops removed; columns sorted per row.
    ``values``: "one" (all 1.0) or "u01" (uniform in (0, 1])."""
    rng = _rng(seed)
    n = 1 << scale
    m = edge_factor * n
    a, b, c, _ = abcd
    src = np.zeros(m, dtype=np.int64)
    dst = np.zeros(m, dtype=np.int64)
    for _level in range(scale):
        u = rng.random(m, dtype=np.float32)
        right = ((u >= a) & (u < a + b)) | (u >= a + b + c)   # quadrants b and d set the column bit
        down = u >= a + b                                      # quadrants c and d set the row bit
        src = (src << 1) | down
        dst = (dst << 1) | right
    keep = src != dst
    src, dst = src[keep], dst[keep]
    keys = np.concatenate([src * n + dst, dst * n + src])
    keys = np.unique(keys)
    rows, cols = keys // n, keys % n
    rowptr = np.zeros(n + 1, dtype=np.int64)
    np.add.at(rowptr, rows + 1, 1)
    if values == "one":
        vals = np.ones(keys.size, dtype=np.float32)
    else:
        vals = (1.0 - rng.random(keys.size, dtype=np.float32)).astype(np.float32)
    return np.cumsum(rowptr).astype(np.int32), cols.astype(np.int32), vals, (n, n)


def rmat_symmetric_device(scale: int, edge_factor: int, seed: int, values: str = "one", abcd=(0.57, 0.19, 0.19, 0.05),
                          device="cuda"):
    """The same R-MAT law generated on the GPU with torch (configuration 5 has ~500 M nonzeros: too slow on the host).
    Returns device tensors (rowptr int32[n+1], colidx int32[nnz], values float32[nnz]) and the shape.  Deterministic for
    a given seed on a given GPU model (torch Philox generator), so every rank of a multi-GPU run builds the same matrix."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    n = 1 << scale
    m = edge_factor * n
    a, b, c, _ = abcd
    src = torch.zeros(m, dtype=torch.int64, device=device)
    dst = torch.zeros(m, dtype=torch.int64, device=device)
    for _level in range(scale):
        u = torch.rand(m, generator=g, device=device)
        right = ((u >= a) & (u < a + b)) | (u >= a + b + c)
        down = u >= a + b
        src = (src << 1) | down
        dst = (dst << 1) | right
        del u, right, down
    keep = src != dst
    src, dst = src[keep], dst[keep]
    del keep
    keys = torch.cat([src * n + dst, dst * n + src])
    del src, dst
    keys = torch.unique(keys)
    rows = torch.div(keys, n, rounding_mode="floor")
    cols = (keys - rows * n).to(torch.int32)
    del keys
    counts = torch.bincount(rows, minlength=n)
    del rows
    rowptr = torch.zeros(n + 1, dtype=torch.int64, device=device)
    rowptr[1:] = torch.cumsum(counts, 0)
    nnz = int(rowptr[-1].item())
    if values == "one":
        vals = torch.ones(nnz, dtype=torch.float32, device=device)
    else:
        vals = 1.0 - torch.rand(nnz, generator=g, device=device)
    return rowptr.to(torch.int32), cols, vals, (n, n)


def mixed_density(n: int = 524288, seed: int = 1004, dense_fraction: float = 0.1, blocks_per_panel: int = 4,
                  density: float = 0.5, sparse_per_row: int = 4):
    """Config 4: a random ``dense_fraction`` of the 64-row panels hold ``blocks_per_panel`` 64x64 blocks of
    the given density at random block columns; every other row has ``sparse_per_row`` uniform-random
    nonzeros; values N(0, 1)."""
    rng = _rng(seed)
    panels = n // 64
    dense = np.zeros(panels, dtype=bool)
    dense[rng.choice(panels, size=max(1, int(round(panels * dense_fraction))), replace=False)] = True
    keys = []
    # sparse rows
    srows = np.repeat(np.nonzero(~np.repeat(dense, 64))[0].astype(np.int64), sparse_per_row)
    scols = rng.integers(0, n, size=srows.size, dtype=np.int64)
    keys.append(srows * n + scols)
    # dense blocks
    dp = np.nonzero(dense)[0].astype(np.int64)
    bc = rng.integers(0, n // 64, size=(dp.size, blocks_per_panel), dtype=np.int64)
    mask = rng.random((dp.size, blocks_per_panel, 64, 64), dtype=np.float32) < density
    pi, bi, ri, ci = np.nonzero(mask)
    keys.append((dp[pi] * 64 + ri) * n + bc[pi, bi] * 64 + ci)
    keys = np.unique(np.concatenate(keys))
    rows, cols = keys // n, keys % n
    rowptr = np.zeros(n + 1, dtype=np.int64)
    np.add.at(rowptr, rows + 1, 1)
    vals = rng.standard_normal(keys.size, dtype=np.float32)
    return np.cumsum(rowptr).astype(np.int32), cols.astype(np.int32), vals, (n, n)


def banded(n: int = 65536, half_bandwidth: int = 12, fill: float = 0.6, seed: int = 1006):
    """Banded matrix: every row holds a random `fill` share of the 2*half_bandwidth+1 diagonals around the main one
    (the diagonal itself always); values N(0, 1).  Neighbouring rows share almost all their columns."""
    rng = _rng(seed)
    offs = np.arange(-half_bandwidth, half_bandwidth + 1, dtype=np.int64)
    keep = rng.random((n, offs.size), dtype=np.float32) < fill
    keep[:, half_bandwidth] = True
    rows = np.repeat(np.arange(n, dtype=np.int64), offs.size).reshape(n, offs.size)
    cols = rows + offs[None, :]
    ok = keep & (cols >= 0) & (cols < n)
    r, c = rows[ok], cols[ok]
    rowptr = np.zeros(n + 1, dtype=np.int64)
    np.add.at(rowptr, r + 1, 1)
    vals = rng.standard_normal(r.size, dtype=np.float32)
    return np.cumsum(rowptr).astype(np.int32), c.astype(np.int32), vals, (n, n)


def block_diagonal(n: int = 65536, block: int = 64, density: float = 0.3, seed: int = 1007):
    """Block-diagonal matrix: dense-ish `block` x `block` blocks of the given density on the diagonal; values N(0, 1)."""
    rng = _rng(seed)
    nb = n // block
    mask = rng.random((nb, block, block), dtype=np.float32) < density
    bi, ri, ci = np.nonzero(mask)
    r, c = bi.astype(np.int64) * block + ri, bi.astype(np.int64) * block + ci
    rowptr = np.zeros(n + 1, dtype=np.int64)
    np.add.at(rowptr, r + 1, 1)
    vals = rng.standard_normal(r.size, dtype=np.float32)
    return np.cumsum(rowptr).astype(np.int32), c.astype(np.int32), vals, (n, n)


def dense_b(rows: int, cols: int, seed: int, dist: str = "uniform") -> np.ndarray:
    """Dense right-hand side, row-major float32: U[-1, 1] ("uniform") or N(0, 1) ("normal")."""
    rng = _rng(seed + 7919)
    if dist == "normal":
        return rng.standard_normal((rows, cols), dtype=np.float32)
    return (rng.random((rows, cols), dtype=np.float32) * 2.0 - 1.0).astype(np.float32)


def shuffle_within_rows(rowptr, colidx, vals, seed: int = 5):
    """Random within-row permutation of the stored entries (Matrix Market files keep file order)."""
    rng = _rng(seed)
    nnz = colidx.size
    rows = np.repeat(np.arange(rowptr.size - 1), np.diff(rowptr))
    order = np.lexsort((rng.random(nnz), rows))
    return rowptr, colidx[order], vals[order]


CONFIGS = {
    "c1": dict(gen="fixed_nnz_per_row", precision="fp16", colB=32, b_dist="uniform"),
    "c2": dict(gen="stencil27", precision="tf32", colB=128, b_dist="normal"),
    "c3": dict(gen="rmat_symmetric", precision="fp16", colB=64, b_dist="uniform"),
    "c4": dict(gen="mixed_density", precision="tf32", colB=256, b_dist="normal"),
    "c5": dict(gen="rmat_symmetric", precision="fp16", colB=128, b_dist="uniform",
               kwargs=dict(scale=24, seed=1005, values="u01")),
}


def make_config(name: str, **override):
    """CSR + meta of one named benchmark configuration (``override`` shrinks it for tests)."""
    cfg = CONFIGS[name]
    kwargs = dict(cfg.get("kwargs", {}))
    kwargs.update(override)
    rowptr, colidx, vals, shape = globals()[cfg["gen"]](**kwargs)
    return rowptr, colidx, vals, shape, cfg
