"""Whole-job numbers of N independent replicas (one process per GPU, one token stream each).

The decode path has no exchange step between replicas: each rank owns a full copy of the layer and
its own requests, so the only cross-rank traffic is the reduction of the measurements themselves.
`torch.distributed` is the plumbing (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations


def max_over_ranks(value: float, dist=None, device=None) -> float:
    """The slowest rank's value; `dist` is torch.distributed (None or uninitialised: one rank)."""
    if dist is None or not dist.is_available() or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, dist=None, device=None) -> float:
    if dist is None or not dist.is_available() or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def whole_job_rate(units_local: float, seconds_local: float, dist=None, device=None) -> dict:
    """Units processed by all ranks divided by the time of the slowest rank."""
    seconds = max_over_ranks(seconds_local, dist, device)
    units = sum_over_ranks(units_local, dist, device)
    return {"units": units, "seconds": seconds, "rate": units / seconds if seconds > 0 else 0.0}


def shard_requests(n_requests: int, rank: int, world: int) -> range:
    """Requests [lo, hi) of rank `rank` when n_requests independent token streams are dealt out
    in contiguous, near-equal blocks (the first n_requests % world ranks take one more)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank outside the world")
    base, rem = divmod(max(0, n_requests), world)
    lo = rank * base + min(rank, rem)
    return range(lo, lo + base + (1 if rank < rem else 0))
