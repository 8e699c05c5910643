"""Collective-free partitioning of the attention path over the GPUs of one box, and the
harness-side helpers that go with it.

The path has no exchange step: attention is independent per head and per prefix group, the KV
fill likewise (the reference itself scales by independent engine replicas, one per GPU,
``scripts/launch/launch_4_vicuna_7b.sh:8-17``). A rank therefore owns a contiguous range of the
heads of every cache block (or whole prefix groups with their rows). ``torch.distributed`` is
used by the harness only: a barrier around timed regions, a MAX-reduce of per-rank times, and an
all-gather of the ranks' outputs along the head dimension for verification.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist


def head_range(num_heads: int, world: int, rank: int) -> range:
    """Heads owned by `rank` when `num_heads` are split as evenly as possible, in order."""
    if not 0 <= rank < world:
        raise ValueError("rank outside the world")
    base, extra = divmod(num_heads, world)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


def max_over_ranks(values_ms: Sequence[float], device: torch.device) -> List[float]:
    """Element-wise maximum of per-rank timings (the job takes as long as its slowest rank)."""
    t = torch.tensor(list(values_ms), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def gather_heads(out_local: torch.Tensor) -> torch.Tensor:
    """All ranks' ``[rows, heads_local, D]`` outputs joined along the head dimension, in rank order
    (equal head counts per rank). The one collective of the harness; nothing on the path needs it."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return out_local
    parts = [torch.empty_like(out_local) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, out_local.contiguous())
    return torch.cat(parts, dim=1)


def sample_rows_every_group(wl, n: int, seed: int = 0) -> List[int]:
    """A seeded sample of rows that contains the first row of every non-empty prefix group and the
    rows with the shortest and the longest private context."""
    rng = np.random.default_rng(seed)
    must = set()
    offs = wl.group_row_offsets
    for g in range(wl.num_groups):
        if offs[g + 1] > offs[g]:
            must.add(int(offs[g]))
    must.add(int(np.argmin(wl.suffix_lens)))
    must.add(int(np.argmax(wl.suffix_lens)))
    rest = [r for r in rng.permutation(wl.num_rows).tolist() if r not in must]
    return sorted(must | set(rest[: max(0, n - len(must))]))


def compact_sample(wl, tensors: Dict[str, torch.Tensor], rows: Sequence[int], local_head: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, dict]:
    """Cuts the sub-problem of the sampled `rows` and ONE head out of a materialised workload, on
    the device: only the cache blocks those rows attend (their groups' prefixes and their own
    suffixes), renumbered densely, with the metadata rewritten to match. What comes back is small
    enough to gather from every rank and to hand to the CPU oracle, whatever the size of the caches.
    Returns (query [n, 1, D], key blocks [m, 1, D/x, B, x], value blocks [m, 1, D, B], metadata)."""
    if wl.seg_kv_lens is not None:
        raise ValueError("workloads with causal segments are not sampled here")
    b = wl.block_size
    offs = wl.group_row_offsets
    groups = [int(np.searchsorted(offs, r, side="right") - 1) for r in rows]
    used: List[int] = []
    g_tabs = {}
    for g in sorted(set(groups)):
        nb = (int(wl.group_prefix_lens[g]) + b - 1) // b
        g_tabs[g] = wl.group_tables[g][:nb].tolist()
        used += g_tabs[g]
    s_tabs = []
    for r in rows:
        nb = (int(wl.suffix_lens[r]) + b - 1) // b
        s_tabs.append(wl.suffix_tables[r][:nb].tolist())
        used += s_tabs[-1]
    uniq = sorted(set(used))
    remap = {old: new for new, old in enumerate(uniq)}
    dev = tensors["query"].device
    sel = torch.tensor(uniq, dtype=torch.long, device=dev)
    hsel = slice(local_head, local_head + 1)
    kc = tensors["key_cache"][:, hsel].index_select(0, sel).contiguous()
    vc = tensors["value_cache"][:, hsel].index_select(0, sel).contiguous()
    q = tensors["query"][:, hsel].index_select(0, torch.tensor(list(rows), dtype=torch.long, device=dev)).contiguous()
    counts = [0] * (wl.num_groups + 1)
    for g in groups:
        counts[g + 1] += 1
    meta = {
        "group_row_offsets": np.cumsum(counts).tolist(),
        "group_prefix_lens": [int(x) for x in wl.group_prefix_lens],
        "group_tables": [[remap[x] for x in g_tabs.get(g, [])] for g in range(wl.num_groups)],
        "suffix_lens": [int(wl.suffix_lens[r]) for r in rows],
        "suffix_tables": [[remap[x] for x in tab] for tab in s_tabs],
    }
    return q, kc, vc, meta
