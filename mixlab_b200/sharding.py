"""Host-side helpers for running the primitives on several GPUs of one node.

The primitives have no exchange step: units are independent per (batch, head), so a job is
sharded by batch, one process per GPU, and the only collectives are the ones the
measurement needs (a barrier and a max over ranks of the device time).  Works with any
torch.distributed backend (nccl on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """[lo, hi) of `total` units owned by `rank`; remainders go to the lowest ranks."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, rem = divmod(total, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def rank_seed(base_seed: int, rank: int, index: int = 0) -> int:
    """Distinct, reproducible input seed per (rank, sequence)."""
    return 1000 * (rank + 1) + base_seed * 100003 + index


def max_over_ranks(value: float, device=None) -> float:
    """MAX all-reduce of a scalar (the step time of the slowest rank)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def whole_job_rate(units_per_rank: int, world: int, seconds: float) -> float:
    """Aggregate units/s of a weak-scaled job: every rank processed `units_per_rank` in `seconds`
    (the max over ranks)."""
    return world * units_per_rank / seconds
