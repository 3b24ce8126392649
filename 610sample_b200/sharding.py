"""Partition of the (batch, head) slices over the GPUs of one box.

Every (batch, head) slice of an attention call is independent, so multi-GPU runs
give each rank a contiguous range of slices and need no collective on the kernel
path.  The reference has no distributed code; this is the only multi-GPU logic
the hot path needs.
"""
from __future__ import annotations

from typing import Tuple


def shard_range(n_slices: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of the slices owned by `rank`; sizes differ by at most one and
    earlier ranks take the larger shares."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    if n_slices < 0:
        raise ValueError("n_slices must be >= 0")
    base, extra = divmod(n_slices, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def max_over_ranks(value: float, device=None) -> float:
    """Max of a per-rank scalar (elapsed time) over the default process group;
    the value itself when torch.distributed is not initialised."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
