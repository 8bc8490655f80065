"""CPU tests of the multi-GPU host logic with real process groups (gloo, world_size 2): shard planning, the one
broadcast of B, slab coverage and max-over-ranks timing."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tilespmm_b200 import multi


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)                      # the same matrix statistics on every rank
        tiles = rng.integers(0, 60, size=5000)
        tiles[::97] = 4000                                  # a few very long panels (power-law rows)
        costs = [multi.panel_cost(int(t), 8, 16, 2) for t in tiles]
        cuts = multi.shard_cuts(costs, world)
        mine = (cuts[rank] * 8, cuts[rank + 1] * 8)         # the C slab of this rank (8-row panels)
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        ok_cover = multi.slabs_cover(gathered, 5000 * 8)
        share = sum(costs[cuts[rank]:cuts[rank + 1]]) / sum(costs)
        b = torch.arange(12, dtype=torch.float32).reshape(3, 4) if rank == 0 else torch.zeros(3, 4)
        multi.broadcast_dense(b, dist, src=0)
        slowest = multi.max_over_ranks(1.0 + rank, dist)
        out.put((rank, ok_cover, share, b.tolist(), slowest))
    finally:
        dist.destroy_process_group()


def test_two_ranks_plan_broadcast_and_time():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_cover, share, b, slowest in res:
        assert ok_cover
        assert abs(share - 0.5) < 0.02                      # balanced by bytes, not by rows
        assert b == torch.arange(12, dtype=torch.float32).reshape(3, 4).tolist()
        assert slowest == 2.0


def test_shard_cuts_properties():
    rng = np.random.default_rng(1)
    for world in (1, 2, 3, 4, 8):
        costs = rng.random(1000) ** 4 * 100
        cuts = multi.shard_cuts(costs, world)
        assert cuts[0] == 0 and cuts[-1] == 1000 and len(cuts) == world + 1
        assert all(a <= b for a, b in zip(cuts[:-1], cuts[1:]))
        parts = [costs[a:b].sum() for a, b in zip(cuts[:-1], cuts[1:])]
        assert max(parts) - min(parts) <= 2 * costs.max() + 1e-9
    assert multi.shard_cuts([], 4) == [0, 0, 0, 0, 0]
    assert multi.shard_cuts([5.0], 2) in ([0, 0, 1], [0, 1, 1])


class _CpuEngine:
    """Stand-in for api.TileMatrix in the CPU test of ShardedTileMatrix: cuts the rows into contiguous slabs of whole
    8-row blocks balanced by entry count (the library balances by tile bytes) and multiplies its slab with the
    checker's CSR SpMM."""

    def __init__(self, precision):
        self.precision = precision

    def convert_host(self, shape, rp, ci, v, gamma, delta, shard=(0, 1)):
        self.shape, self.rp, self.ci, self.v = shape, np.asarray(rp), np.asarray(ci), np.asarray(v, np.float32)
        nb = (shape[0] + 7) // 8
        ends = np.minimum((np.arange(nb) + 1) * 8, shape[0])
        costs = np.diff(np.concatenate([[0], self.rp[ends]])).astype(np.float64) + 1.0
        cuts = multi.shard_cuts(costs, shard[1])
        self.row_range = (min(cuts[shard[0]] * 8, shape[0]), min(cuts[shard[0] + 1] * 8, shape[0]))

    def info(self):
        return np.zeros((3, 4), dtype=np.int32)

    def c_rows(self):
        return (self.row_range[1] - self.row_range[0] + 64) // 64 * 64

    def spmm(self, b, c, colB, stream=0):
        import _orc
        r0, r1 = self.row_range
        rp = (self.rp[r0:r1 + 1] - self.rp[r0]).astype(np.int32)
        ci, v = self.ci[self.rp[r0]:self.rp[r1]], self.v[self.rp[r0]:self.rp[r1]]
        out = _orc.spmm_csr(self.precision, (r1 - r0, self.shape[1]), rp, ci, v, b[:self.shape[1]].numpy(), colB, trunc=False)
        c[:r1 - r0] = torch.from_numpy(out)


def _sharded_worker(rank, world, port, out):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tilespmm_b200 import synth
        rp, ci, v, shape = synth.rmat_symmetric(10, 8, 3)           # the same matrix on every rank
        shape = (shape[0], shape[1])
        B = synth.dense_b(shape[1], 64, 2)
        sm = multi.ShardedTileMatrix(1, dist, engine=_CpuEngine(1)).convert_host(shape, rp, ci, v, 2.0, 1.2)
        slabs = sm.all_slabs()
        lo, hi = sm.b_block()
        per = multi.b_block_rows(shape[1], world)
        block = torch.zeros((per, 64), dtype=torch.float32)
        block[:hi - lo] = torch.from_numpy(B[lo:hi])                 # this rank holds (and "uploads") only its block of B
        c = torch.empty((sm.slab_rows, 64), dtype=torch.float32)
        for _ in range(2):                                           # twice: the buffers are reused
            sm.spmm_host(block, c, 64, device=torch.device("cpu"))
        out.put((rank, slabs, sm.row_range, c.numpy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_matrix_gathers_b_blocks_and_owns_a_c_slab(world):
    import _orc
    from tilespmm_b200 import synth
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_sharded_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted((q.get(timeout=180) for _ in range(world)), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    rp, ci, v, shape = synth.rmat_symmetric(10, 8, 3)
    B = synth.dense_b(shape[1], 64, 2)
    want = _orc.spmm_csr(1, shape, rp, ci, v, B, 64, trunc=False)
    got = np.concatenate([r[3] for r in res])
    assert [tuple(s) for s in res[0][1]] == [tuple(r[2]) for r in res]       # every rank saw the same slab table
    assert multi.slabs_cover([tuple(r[2]) for r in res], shape[0])
    np.testing.assert_array_equal(got, want)                                 # same arithmetic order: bit for bit
