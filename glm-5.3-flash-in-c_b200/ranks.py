"""The collectives a multi-rank run of this engine needs on the host side (one process per GPU).

The data path between expert-parallel ranks is inside the CUDA kernels (rows stored through NVLink
peer mappings, see csrc/ep_exchange.cu); what is left for the host is plumbing: agreeing that a
stage succeeded everywhere, reducing measurements, and gathering the ranks' exchange handles.
`torch.distributed` carries it (NCCL on GPUs, gloo in the CPU tests). Every rank calls every
method in the same order whatever happened on it, so a failure on one rank cannot strand the rest.
"""
from __future__ import annotations


class Ranks:
    def __init__(self, dist=None, device: str = "cpu"):
        """dist: torch.distributed (None or uninitialised = a single rank); device: where the small
        tensors of the reductions live ("cuda" under NCCL, "cpu" under gloo)."""
        self.dist = dist if (dist is not None and dist.is_available() and dist.is_initialized()) else None
        self.device = device
        self.world = self.dist.get_world_size() if self.dist else 1
        self.rank = self.dist.get_rank() if self.dist else 0

    def _sync(self):
        if self.device.startswith("cuda"):
            import torch
            torch.cuda.synchronize()

    def barrier(self):
        self._sync()
        if self.dist:
            self.dist.barrier()
        self._sync()

    def reduce(self, value: float, op: str) -> float:
        """max / min / sum of one float over the ranks."""
        if not self.dist:
            return float(value)
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64, device=self.device)
        ops = {"max": self.dist.ReduceOp.MAX, "min": self.dist.ReduceOp.MIN, "sum": self.dist.ReduceOp.SUM}
        self.dist.all_reduce(t, op=ops[op])
        return float(t.item())

    def all_ok(self, flag: bool) -> bool:
        """True only if every rank passed True."""
        return self.reduce(1.0 if flag else 0.0, "min") > 0.5

    def gather(self, obj) -> list:
        """Every rank's object, in rank order, on every rank."""
        if not self.dist:
            return [obj]
        out = [None] * self.world
        self.dist.all_gather_object(out, obj)
        return out

    def connect(self, engine):
        """Exchange the expert-parallel handles of all ranks and map them (nothing to do for one rank)."""
        if self.world > 1:
            engine.ep_connect(self.gather(engine.ep_export()))


def expert_range(n_experts: int, rank: int, world: int) -> range:
    """Routed experts [lo, hi) that expert-parallel rank `rank` of `world` owns in every MoE layer."""
    if world < 1 or not 0 <= rank < world or n_experts % world:
        raise ValueError("the ranks must divide the experts evenly")
    per = n_experts // world
    return range(rank * per, (rank + 1) * per)


def strong_scaling_rate(units: float, seconds_local: float, ranks: Ranks) -> dict:
    """All ranks work on the same units together: units / the slowest rank's time."""
    seconds = ranks.reduce(seconds_local, "max")
    return {"units": float(units), "seconds": seconds, "rate": units / seconds if seconds > 0 else 0.0}
