"""Batch sharding of the layer path across the GPUs of one box.

Tokens are independent (the upstream layer flattens to [B*S, d] and every rule is
per token: architectures/moe/moefication.py:80-85,94), so the path shards by batch
with replicated weights and no collective: rank r of W takes a contiguous slice of
the batch dimension.  The only cross-rank traffic is the timing reduction
(max over ranks) of the benchmark.
"""
from __future__ import annotations


def shard_bounds(batch: int, world: int, rank: int) -> tuple[int, int]:
    """Half-open slice [lo, hi) of the batch dimension owned by `rank`: sizes differ by
    at most one, earlier ranks take the larger shards, every item belongs to one rank."""
    if world < 1 or not 0 <= rank < world or batch < 0:
        raise ValueError(f"bad shard request: batch={batch} world={world} rank={rank}")
    base, extra = divmod(batch, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard(x, world: int, rank: int):
    """This rank's slice of a [B, ...] tensor (a view)."""
    lo, hi = shard_bounds(x.shape[0], world, rank)
    return x[lo:hi]


def max_over_ranks(value: float, dist=None, device="cpu") -> float:
    """Max of a per-rank scalar (elapsed time) over all ranks; identity without a group."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, dist=None, device="cpu") -> float:
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())
