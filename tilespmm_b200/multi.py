"""Host-side plumbing of the multi-GPU path: one process per GPU, panels sharded, B broadcast once, C row-partitioned.

The shard boundaries themselves are computed inside the library (tsp_convert_* with shard_index/shard_count) from the
global panel sequence; `shard_cuts` restates that rule so that it can be checked without a GPU, and so that a host
can plan slab sizes before converting.
"""
from __future__ import annotations

import bisect

import numpy as np


def panel_cost(tiles: int, bm: int, bn: int, value_bytes: int) -> float:
    """Bytes one panel moves per SpMM at a 128-column B: tile values + column indices + gathered rows, plus its C rows,
    plus a fixed 12 KB that stands for the start-up of a task (measured: about three tile-times)."""
    return tiles * (bm * bn * value_bytes + bn * 4 + bn * 128 * value_bytes) + bm * 128 * 4.0 + 12288.0


def shard_cuts(costs, world: int):
    """Cuts a sequence of per-panel costs into `world` contiguous ranges of nearly equal total cost.
    Returns world+1 panel indices; rank r owns panels [cuts[r], cuts[r+1])."""
    prefix = np.concatenate([[0.0], np.cumsum(np.asarray(costs, dtype=np.float64))])
    n = len(prefix) - 1
    cuts = [0]
    for g in range(1, world):
        want = prefix[n] * g / world
        cuts.append(max(cuts[-1], bisect.bisect_left(prefix.tolist(), want)))
    cuts.append(n)
    return cuts


def broadcast_dense(tensor, dist, src: int = 0):
    """B is produced on one rank and replicated into every GPU's own memory (no peer reads in the kernels)."""
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        dist.broadcast(tensor, src=src)
    return tensor


def max_over_ranks(value: float, dist, device="cpu") -> float:
    """A multi-GPU time is the slowest rank's time."""
    import torch
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def slabs_cover(row_ranges, rows: int) -> bool:
    """True when the per-rank C slabs [begin, end) are contiguous, ordered and cover [0, rows)."""
    if not row_ranges or row_ranges[0][0] != 0 or row_ranges[-1][1] != rows:
        return False
    return all(a[1] == b[0] for a, b in zip(row_ranges[:-1], row_ranges[1:])) and all(a[0] <= a[1] for a in row_ranges)
