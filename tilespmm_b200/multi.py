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


def b_block_rows(rows_b: int, world: int) -> int:
    """Rows of B per rank when B is cut into `world` equal row blocks (the last block may reach past rows_b)."""
    return (rows_b + world - 1) // world


class ShardedTileMatrix:
    """One rank's share of a matrix whose panel sequence is cut across the ranks of a process group.

    Every rank converts its own contiguous range of panels (`tsp_convert_*` with shard arguments), keeps a full copy
    of B in its own memory and owns the matching row slab of C.  With host buffers (`spmm_host`) a rank uploads only its
    own 1/world row block of B from pinned memory and the ranks all-gather the blocks over the process group (NCCL over
    NVLink on GPUs) into every rank's copy, so the host-to-device traffic per step does not grow with the number of
    ranks; C slabs go back to the host per rank.  There is no reduction and no peer-memory access from the kernels.

    `engine` is the per-rank matrix: an `api.TileMatrix` (the default) or any object with the same `convert_host`,
    `convert_device`, `info`, `row_range`, `c_rows` and `spmm` -- the CPU tests pass a stand-in, because the CUDA
    library does not run without a GPU.
    """

    def __init__(self, precision: int, dist=None, device: int = 0, engine=None):
        self.precision, self.dist, self.device = precision, dist, device
        on = dist is not None and dist.is_initialized()
        self.rank = dist.get_rank() if on else 0
        self.world = dist.get_world_size() if on else 1
        if engine is None:
            from . import api
            engine = api.TileMatrix(precision, device)
        self.m = engine
        self.shape = None
        self._bufs = {}

    # -- conversion: the partition is global, only this rank's panels are converted
    def convert_host(self, shape, rowptr, colidx, vals, gamma, delta):
        self.m.convert_host(shape, rowptr, colidx, vals, gamma, delta, shard=(self.rank, self.world))
        return self._converted(shape)

    def convert_device(self, shape, d_rowptr, d_colidx, d_vals, nnz, gamma, delta):
        self.m.convert_device(shape, d_rowptr, d_colidx, d_vals, nnz, gamma, delta, shard=(self.rank, self.world))
        return self._converted(shape)

    def _converted(self, shape):
        self.shape = tuple(shape)
        self.info = self.m.info()
        self.row_range = self.m.row_range
        self._bufs = {}
        return self

    @property
    def slab_rows(self) -> int:
        return self.row_range[1] - self.row_range[0]

    def b_block(self):
        """(first, one-past-last) row of B this rank uploads in `spmm_host`."""
        per = b_block_rows(self.shape[1], self.world)
        return min(self.rank * per, self.shape[1]), min((self.rank + 1) * per, self.shape[1])

    def all_slabs(self):
        """Row ranges of every rank's C slab, in rank order (checked to tile [0, rows) without gaps)."""
        if self.world == 1:
            ranges = [tuple(self.row_range)]
        else:
            ranges = [None] * self.world
            self.dist.all_gather_object(ranges, tuple(self.row_range))
        if not slabs_cover(ranges, self.shape[0]):
            raise RuntimeError(f"the C slabs of the ranks do not tile the rows: {ranges}")
        return ranges

    # -- resident operands
    def spmm(self, d_b, d_c, colB_padded: int, stream: int = 0):
        """C slab = A[rows of this rank] * B with B (whole) and C (tsp_c_rows x colB_padded) in this rank's memory."""
        self.m.spmm(d_b, d_c, colB_padded, stream)

    # -- host operands
    def _buffers(self, slot: int, colB_padded: int, like_b, device):
        import torch
        key = (slot, colB_padded, like_b.dtype, str(device))
        if key not in self._bufs:
            per = b_block_rows(self.shape[1], self.world)
            full = torch.empty((per * self.world, colB_padded), dtype=like_b.dtype, device=device)
            c = torch.empty((self.m.c_rows(), colB_padded), dtype=torch.float32, device=device)
            self._bufs[key] = (full, c)
        return self._bufs[key]

    def spmm_host(self, h_b_block, h_c_slab, colB_padded: int, slot: int = 0, device=None):
        """One product with host operands, asynchronous on the current stream of `device`.

        h_b_block: this rank's row block of B (`b_block()` rows x colB_padded, pinned for a truly asynchronous copy);
        h_c_slab: `slab_rows` x colB_padded float32, receives this rank's rows of C.  Steps: upload of the block into
        this rank's copy of B, all-gather of the blocks (world > 1), kernels, download of the slab.  `slot` selects
        one of the device buffer sets, so that a caller can keep two steps in flight on two streams.  Returns after
        enqueueing; synchronise the stream (or the device) before reading h_c_slab."""
        import torch
        if device is None:
            device = torch.device("cuda", self.device) if h_b_block.is_pinned() or torch.cuda.is_available() else torch.device("cpu")
        full, c = self._buffers(slot, colB_padded, h_b_block, device)
        per = b_block_rows(self.shape[1], self.world)
        lo, hi = self.b_block()
        mine = full[self.rank * per:(self.rank + 1) * per]
        mine[:hi - lo].copy_(h_b_block[:hi - lo], non_blocking=True)
        if self.world > 1:
            self.dist.all_gather_into_tensor(full, mine)
        stream = torch.cuda.current_stream(device).cuda_stream if device.type == "cuda" else 0
        self.m.spmm(full, c, colB_padded, stream)
        h_c_slab.copy_(c[:self.slab_rows], non_blocking=True)
        return h_c_slab

    def close(self):
        self._bufs = {}
        if hasattr(self.m, "close"):
            self.m.close()
