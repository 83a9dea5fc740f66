"""Replica bookkeeping for multi-GPU runs of the xnor path.

The path has no exchange step: every GPU holds a full copy of the packed weights and works on its own slice of
the image batch ("replicas only").  What is shared is host-side arithmetic only: how a global batch is cut into
per-rank slices, and how per-rank timings combine into one throughput figure (the slowest rank sets the time).
torch.distributed is used for the barrier and the max -- NCCL on GPUs, gloo in the CPU tests.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


def shard_batch(global_batch: int, world: int) -> List[Tuple[int, int]]:
    """[(first image, count)] per rank: contiguous slices, sizes differ by at most one, earlier ranks get the extras."""
    if global_batch < 0 or world <= 0:
        raise ValueError("global_batch must be >= 0 and world > 0")
    base, extra = divmod(global_batch, world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((start, n))
        start += n
    return out


def max_over_ranks(value: float, device: torch.device | str = "cpu") -> float:
    """The slowest rank's value (identity when no process group is initialised)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device: torch.device | str = "cpu") -> float:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def aggregate_images_per_s(images_this_rank: int, ms_this_rank: float, device: torch.device | str = "cpu") -> float:
    """Whole-job images/s: all ranks' images divided by the slowest rank's time."""
    total = sum_over_ranks(float(images_this_rank), device)
    ms = max_over_ranks(ms_this_rank, device)
    return total / (ms * 1e-3)
