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
