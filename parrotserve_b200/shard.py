"""Collective-free partitioning of the attention path over the GPUs of one box.

The path has no exchange step: attention is independent per head and per prefix group, the KV
fill likewise (the reference itself scales by independent engine replicas, one per GPU,
``scripts/launch/launch_4_vicuna_7b.sh:8-17``). A rank therefore owns either a contiguous range
of heads of every cache block, or whole prefix groups with their rows. ``torch.distributed`` is
used by the harness only: a barrier around timed regions and a MAX-reduce of per-rank times.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def head_range(num_heads: int, world: int, rank: int) -> range:
    """Heads owned by `rank` when `num_heads` are split as evenly as possible, in order."""
    if not 0 <= rank < world:
        raise ValueError("rank outside the world")
    base, extra = divmod(num_heads, world)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


def group_assignment(group_bytes: Sequence[float], world: int) -> List[List[int]]:
    """Greedy longest-first assignment of prefix groups (with the KV bytes each one and its rows
    must stream) to ranks; returns the group indices of every rank."""
    order = sorted(range(len(group_bytes)), key=lambda g: -group_bytes[g])
    load = [0.0] * world
    owned: List[List[int]] = [[] for _ in range(world)]
    for g in order:
        r = min(range(world), key=lambda i: load[i])
        owned[r].append(g)
        load[r] += group_bytes[g]
    for o in owned:
        o.sort()
    return owned


def max_over_ranks(values_ms: Sequence[float], device: torch.device) -> List[float]:
    """Element-wise maximum of per-rank timings (the job takes as long as its slowest rank)."""
    t = torch.tensor(list(values_ms), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def whole_job_rate(units_per_rank: int, world: int, ms_per_step: float) -> float:
    """Units (decode tokens) all ranks complete per second when each rank does `units_per_rank`
    per step and a step takes `ms_per_step` on the slowest rank."""
    return units_per_rank * world / (ms_per_step * 1e-3)
