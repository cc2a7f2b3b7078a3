"""Multi-rank host logic on CPU: world_size-2 (and 3) gloo groups, no GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from d2dmoe_b200.sharding import max_over_ranks, shard, shard_bounds, sum_over_ranks


def test_shard_bounds_cover_every_item_once():
    for batch in (0, 1, 7, 32, 255, 256, 257):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                lo, hi = shard_bounds(batch, world, r)
                assert 0 <= lo <= hi <= batch
                seen += list(range(lo, hi))
            assert seen == list(range(batch))
            sizes = [shard_bounds(batch, world, r)[1] - shard_bounds(batch, world, r)[0]
                     for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x = torch.arange(37 * 5, dtype=torch.float32).reshape(37, 5)      # whole batch
        mine = shard(x, world, rank)
        # the shards of all ranks together are the batch, each row once
        total = sum_over_ranks(float(mine.sum()), dist)
        rows = sum_over_ranks(mine.shape[0], dist)
        # per-rank time, job time = the slowest rank
        t = max_over_ranks(1.0 + rank, dist)
        dist.barrier()
        q.put((rank, mine.shape[0], total, rows, t))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_gloo_ranks_partition_the_batch(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x_sum = float(torch.arange(37 * 5, dtype=torch.float32).sum())
    for rank, n, total, rows, t in res:
        assert total == x_sum and rows == 37 and t == float(world)
    assert sum(n for _, n, *_ in res) == 37
