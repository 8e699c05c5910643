"""Attention function for ParrotServe's builtin engine on the B200 kernels.

Same three-method contract as the reference's ``AttnFunc`` classes
(``parrot/engine/builtin/attn_func.py:31-55``): ``__init__(layer_idx, scaling, num_heads,
head_dim)``, static ``init_iteration_state(iteration_state, builtin_config, jobs, num_heads,
head_size)`` and ``forward(q, k, v, iteration_state)``; token order is all Fill tokens, then one
token per Generate job (``iter_state.py:16-27``). It replaces
``xFormersFill_SharedPromptsGenerate`` (``attn_func.py:408-696``):

* the shared context is the lowest common ancestor of all jobs' contexts (``attn_func.py:411-459``);
* KV fill uses a FLAT ragged slot mapping (one slot per new token; the reference pads it to 2-D,
  which its kernel then indexes flat, ``attn_func.py:567,589-593``);
* every query token is one row of a single grouped attention call: a Generate token attends
  shared prefix ++ its private context; the new tokens of a Fill job form one causal segment, in
  which the i-th token attends shared prefix ++ the job's private context up to and including
  itself (bottom-right causal, the mask the reference builds at ``attn_func.py:541-546``), on the
  tensor cores. No gather into contiguous buffers, no xformers.

The metadata builder is pure Python/numpy so it is testable without a GPU; ``install()``
registers the class under a new name without editing Parrot.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import numpy as np
import torch
from torch import nn

ATTN_FUNC_NAME = "b200_shared_prompts_generate"


# ---------------------------------------------------------------------------------------------
# metadata (host side, no torch device work)
# ---------------------------------------------------------------------------------------------
def _lca(a, b):
    """Lowest common ancestor of two context-tree nodes (``parent_context`` / ``depth``), or None."""
    while a is not None and b is not None and a is not b:
        if a.depth > b.depth:
            a = a.parent_context
        elif a.depth < b.depth:
            b = b.parent_context
        else:
            a, b = a.parent_context, b.parent_context
    return a if a is b else None


def shared_context_node(jobs: Sequence):
    """The context every query row of the iteration may attend in full, or None.

    It is the common ancestor of the jobs' contexts (a lone job's own context), as in the reference
    (``attn_func.py:441-459``), with one restriction the reference does not need because it never
    applies the shared length to Fill rows (``attn_func.py:541-546, 631-675``): a Fill job's own
    context already holds the tokens the job is adding (the runner allocates them before the
    metadata is built, ``builtin_runner.py:97-99``), and those must stay under the causal mask of
    the job's segment. So while the candidate is the context of a Fill job, its parent takes its
    place (a forked parent is padded to a block multiple, ``block_context.py:30-38``)."""
    if not len(jobs):
        return None
    node = jobs[0].context
    for job in jobs[1:]:
        node = _lca(node, job.context)
        if node is None:
            return None
    fill_contexts = {id(job.context) for job in jobs if _is_fill(job)}
    while node is not None and id(node) in fill_contexts:
        node = node.parent_context
    return node


def shared_context_len(jobs: Sequence) -> int:
    """Length of the context shared by every job (0 when there is none): see shared_context_node."""
    node = shared_context_node(jobs)
    return 0 if node is None else node.get_context_len()


def _deepest_shared_nodes(jobs: Sequence) -> list:
    """For every job the deepest proper ancestor of its context that at least one other job also
    has on its path, or None (a job's own context still receives tokens, so it is never shared)."""
    count = {}
    for job in jobs:
        node = job.context
        while node is not None:
            count[id(node)] = count.get(id(node), 0) + 1
            node = node.parent_context
    out = []
    for job in jobs:
        node = job.context.parent_context
        while node is not None and count[id(node)] < 2:
            node = node.parent_context
        out.append(node)
    return out


def _strided_blocks(ctx, start: int, stop: Optional[int], step: int) -> List[int]:
    """Block ids of the tokens at positions start, start + step, ... (< stop) of a context's whole
    token sequence, ancestors first: ``ctx.get_context_block_ids()[start:stop:step]`` without building
    the per-token list of the whole context, which costs one list element per TOKEN of every job in
    every iteration (parrot/engine/context/block_context.py:107-114). Walks the ancestor chain and
    slices each context's own ``token_kv_block_ids``: O(depth + blocks returned)."""
    if not hasattr(ctx, "token_kv_block_ids"):
        return ctx.get_context_block_ids()[start:stop:step]
    chain = []
    while ctx is not None:
        chain.append(ctx)
        ctx = ctx.parent_context
    out: List[int] = []
    off = 0
    for node in reversed(chain):
        ids = node.token_kv_block_ids
        end = off + len(ids) if stop is None else min(off + len(ids), stop)
        lo = max(start, off)
        if lo < end:
            first = start + -(-(lo - start) // step) * step  # first position >= lo on the stride
            if first < end:
                out.extend(ids[first - off:end - off:step])
        off += len(ids)
        if stop is not None and off >= stop:
            break
    return out


def _last_slots(ctx, n: int) -> List[int]:
    """Slot ids of the last n tokens of a context (the tokens a job adds live in its own context)."""
    own = getattr(ctx, "token_kv_slot_ids", None)
    if own is not None and len(own) >= n:
        return own[len(own) - n:]
    return ctx.get_context_slot_ids()[-n:]


def _is_fill(job) -> bool:
    return hasattr(job, "token_ids") and job.token_ids is not None and not hasattr(job, "sampling_config")


class IterationMetadata:
    """Tables of one iteration. Field names shared with the reference's IterationState
    (``flash_context_len``, ``flash_block_table``, ``paged_context_lens``, ``paged_block_tables``,
    ``slot_mapping``) keep the reference's meaning for the Generate jobs; ``row_*`` cover every
    query token (Fill tokens first)."""

    def __init__(self, jobs: Sequence, block_size: int, two_level: bool = False):
        b = block_size
        self.block_size = b
        self.two_level = bool(two_level)
        self.flash_context_len = shared_context_len(jobs) if len(jobs) else 0
        n_shared_blocks = (self.flash_context_len + b - 1) // b
        pad_len = n_shared_blocks * b
        ctx0 = _strided_blocks(jobs[0].context, 0, pad_len, b) if len(jobs) else []
        self.flash_block_table = np.asarray(ctx0, dtype=np.int32)

        # Second sharing level (two_level): below the context shared by ALL jobs, the deepest context
        # that at least two jobs still share (an application prompt under a system prompt). A job's
        # private part then starts after that context; maximal runs of consecutive rows under the
        # same context form one inner prefix group (rows cannot be reordered here).
        inner_nodes = _deepest_shared_nodes(jobs) if (self.two_level and len(jobs) > 1) else [None] * len(jobs)
        run_keys: List[Optional[int]] = []    # per row: id of its inner context or None
        run_nodes = {}

        self.num_fill_tokens: List[int] = []
        self.num_generation_jobs = 0
        slot_mapping: List[int] = []
        row_lens: List[int] = []
        row_tables: List[List[int]] = []
        paged_lens, paged_tables = [], []
        seg_offsets, seg_kv, seg_tabs = [0], [], []
        seen_generate = False
        for job, node in zip(jobs, inner_nodes):
            # the runner sorts Fill jobs before Generate jobs (parrot/engine/builtin/builtin_runner.py:75-76);
            # the causal segments below are the leading rows because of it
            if _is_fill(job) and seen_generate:
                raise ValueError("Fill jobs must precede Generate jobs in an iteration")
            seen_generate = seen_generate or not _is_fill(job)
            ctx_len = job.context.get_context_len()
            shared_len, start = self.flash_context_len, pad_len
            if node is not None and node.get_context_len() > pad_len:
                shared_len = node.get_context_len()          # a forked context: already a block multiple
                start = (shared_len + b - 1) // b * b
                run_nodes[id(node)] = node
            key = id(node) if start > pad_len else None
            n_rows = len(job.token_ids) if _is_fill(job) else 1
            run_keys += [key] * n_rows
            private = _strided_blocks(job.context, start, None, b)
            if _is_fill(job):
                n = len(job.token_ids)
                self.num_fill_tokens.append(n)
                slot_mapping.extend(_last_slots(job.context, n))
                # one causal segment: token i sees the request's first kv - n + i + 1 private tokens
                # (the shared context never reaches into a Fill job's own context, see
                # shared_context_node, so all n new tokens lie in the private part)
                if n > 0:
                    seg_offsets.append(seg_offsets[-1] + n)
                    seg_kv.append(ctx_len - shared_len)
                    seg_tabs.append(private)
                for i in range(n):
                    row_lens.append(0)
                    row_tables.append([])
            else:
                self.num_generation_jobs += 1
                slot_mapping.extend(_last_slots(job.context, 1))
                row_lens.append(ctx_len - shared_len)
                row_tables.append(private)
                paged_lens.append(ctx_len - shared_len)
                paged_tables.append(private)
        self.slot_mapping = np.asarray(slot_mapping, dtype=np.int64)
        self.row_suffix_lens = np.asarray(row_lens, dtype=np.int32)
        self.row_suffix_tables = _pad(row_tables)
        # Fill jobs come first in the batch, so their rows are [0, num_total_fill_tokens)
        self.seg_row_offsets = np.asarray(seg_offsets, dtype=np.int32)
        self.seg_kv_lens = np.asarray(seg_kv, dtype=np.int32)
        self.seg_tables = _pad(seg_tabs)
        self.paged_context_lens = np.asarray(paged_lens, dtype=np.int32)
        self.paged_block_tables = _pad(paged_tables)
        # inner groups: runs of consecutive rows under the same inner context (prefix = the tokens of that
        # context beyond the one shared by all; rows outside any get a zero-length prefix)
        offs, lens, tabs = [0], [], []
        for r, key in enumerate(run_keys + [object()]):
            if r == len(run_keys) or (r > 0 and key != run_keys[r - 1]):
                if r > 0:
                    prev = run_keys[r - 1]
                    offs.append(r)
                    if prev is None:
                        lens.append(0)
                        tabs.append([])
                    else:
                        node = run_nodes[prev]
                        lens.append(node.get_context_len() - pad_len)
                        tabs.append(_strided_blocks(node, pad_len, None, b))
        self.inner_row_offsets = np.asarray(offs, dtype=np.int32)
        self.inner_prefix_lens = np.asarray(lens, dtype=np.int32)
        self.inner_tables = _pad(tabs)

    @property
    def num_total_fill_tokens(self) -> int:
        return int(sum(self.num_fill_tokens))

    @property
    def num_rows(self) -> int:
        return int(self.row_suffix_lens.shape[0])


def _pad(rows: List[List[int]]) -> np.ndarray:
    width = max([len(r) for r in rows] + [0])
    out = np.zeros((len(rows), width), dtype=np.int32)
    for i, r in enumerate(rows):
        out[i, : len(r)] = r
    return out


_staging = {}  # device index -> [page-locked buffer, event of the last upload from it]


def _upload_packed(arrays: dict, dev: torch.device) -> dict:
    """All index arrays of an iteration in ONE host-to-device transfer from a reused page-locked
    buffer (a dozen separate small pageable uploads cost more than the attention of a layer);
    returns device tensors (views of one allocation) under the same names."""
    if dev.type != "cuda":
        return {n: torch.from_numpy(np.ascontiguousarray(a)).to(dev) for n, a in arrays.items()}
    offs, total = {}, 0
    for n, a in arrays.items():
        offs[n] = total
        total += (a.nbytes + 15) // 16 * 16
    st = _staging.setdefault(dev.index, [None, None])
    if st[0] is None or st[0].numel() < total:
        st[0], st[1] = torch.empty(max(total, 1 << 16), dtype=torch.uint8).pin_memory(), None
    if st[1] is not None:
        st[1].synchronize()   # the previous iteration's upload has long finished; this makes it certain
    host = st[0].numpy()
    for n, a in arrays.items():
        flat = np.ascontiguousarray(a).reshape(-1).view(np.uint8)
        host[offs[n]:offs[n] + flat.size] = flat
    d = torch.empty(max(total, 16), dtype=torch.uint8, device=dev)
    d[:total].copy_(st[0][:total], non_blocking=True)
    st[1] = torch.cuda.Event()
    st[1].record(torch.cuda.current_stream(dev))
    out = {}
    for n, a in arrays.items():
        out[n] = d[offs[n]:offs[n] + a.nbytes].view(torch.from_numpy(np.empty(0, dtype=a.dtype)).dtype).view(a.shape)
    return out


# ---------------------------------------------------------------------------------------------
# the attention function
# ---------------------------------------------------------------------------------------------
class B200SharedPromptsGenerate(nn.Module):
    """Drop-in for ``xFormersFill_SharedPromptsGenerate``."""

    # (layer_idx) -> (k_cache, v_cache); install() points this at parrot.engine.builtin.mem
    kv_cache_getter: Optional[Callable[[int], tuple]] = None
    # True: also share, per run of consecutive jobs, the deepest context those jobs have in common
    # below the one shared by all (two-level context trees); the reference shares one level only
    two_level: bool = False
    # True: when the metadata of an iteration is built, read the device status word the kernels of
    # the PREVIOUS iteration left (the runner has synchronised in between, builtin_runner.py:168, so
    # this costs one 4-byte copy) and raise if they recorded a fault. The outputs of such an
    # iteration were already overwritten with NaN by the merge kernel.
    check_status: bool = True
    _last_call = None

    def __init__(self, layer_idx: int, scaling: float, num_heads: int, head_dim: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.scaling = scaling
        self.num_heads = num_heads
        self.head_dim = head_dim

    @staticmethod
    def init_iteration_state(iteration_state, builtin_config, jobs, num_heads: int, head_size: int):
        from . import ops

        cls = B200SharedPromptsGenerate
        prev, cls._last_call = cls._last_call, None
        if prev is not None and cls.check_status:
            word = prev.status()
            if word != 0:
                names = {1: "a bounded wait expired", 2: "an index outside the cache or the batch", 3: "a work list overflowed"}
                raise RuntimeError(f"the attention kernels of the previous iteration recorded a fault: "
                                   f"{names.get(word, 'status ' + str(word))}; its outputs were set to NaN")
        meta = IterationMetadata(jobs, builtin_config.block_size, two_level=B200SharedPromptsGenerate.two_level)
        dev = torch.device(builtin_config.device)
        for job in jobs:
            if _is_fill(job):
                iteration_state.num_fill_tokens.append(len(job.token_ids))
            else:
                iteration_state.generation_sampling_config.append(job.sampling_config)
        rows = meta.num_rows
        dv = _upload_packed({
            "flash_block_table": meta.flash_block_table, "paged_context_lens": meta.paged_context_lens,
            "paged_block_tables": meta.paged_block_tables, "slot_mapping": meta.slot_mapping,
            "all_rows": np.asarray([0, rows], dtype=np.int32), "flash_len": np.asarray([meta.flash_context_len], dtype=np.int32),
            "row_suffix_lens": meta.row_suffix_lens, "row_suffix_tables": meta.row_suffix_tables,
            "inner_row_offsets": meta.inner_row_offsets, "inner_prefix_lens": meta.inner_prefix_lens,
            "inner_tables": meta.inner_tables, "seg_row_offsets": meta.seg_row_offsets,
            "seg_kv_lens": meta.seg_kv_lens, "seg_tables": meta.seg_tables}, dev)
        iteration_state.flash_context_len = meta.flash_context_len
        iteration_state.flash_block_table = dv["flash_block_table"]
        iteration_state.paged_context_lens = dv["paged_context_lens"]
        iteration_state.paged_block_tables = dv["paged_block_tables"]
        iteration_state.slot_mapping = dv["slot_mapping"]
        iteration_state.b200_meta = meta
        if rows == 0:
            iteration_state.b200_call = None
            return
        shared = dict(row_offsets=dv["all_rows"], prefix_lens=dv["flash_len"],
                      tables=dv["flash_block_table"].reshape(1, -1) if meta.flash_block_table.size else None)
        if meta.two_level and int(meta.inner_prefix_lens.sum()) > 0:
            # the context shared by all jobs becomes the outer level, the contexts shared by runs of jobs the groups
            levels = dict(
                outer_row_offsets=shared["row_offsets"], outer_prefix_lens=shared["prefix_lens"],
                outer_tables=shared["tables"] if shared["tables"] is not None else torch.zeros((1, 1), dtype=torch.int32, device=dev),
                group_row_offsets=dv["inner_row_offsets"], group_prefix_lens=dv["inner_prefix_lens"],
                group_tables=dv["inner_tables"] if meta.inner_tables.size else None)
        else:
            levels = dict(group_row_offsets=shared["row_offsets"], group_prefix_lens=shared["prefix_lens"],
                          group_tables=shared["tables"])
        has_seg = len(meta.seg_kv_lens) > 0
        # The attention call performs the KV fill itself (one launch less per layer, for a decode batch
        # no fill launch at all) when every Generate row's new token lies in its private part; a lone
        # Generate job is the exception (its whole context, new token included, is the shared prefix).
        n_fill_rows = meta.num_total_fill_tokens
        iteration_state.b200_fused_fill = bool((meta.row_suffix_lens[n_fill_rows:] > 0).all())
        iteration_state.b200_call = ops.AttentionCall(
            num_rows=rows, num_heads=num_heads, head_size=head_size, block_size=builtin_config.block_size,
            dtype=builtin_config.dtype, device=dev, suffix_lens=dv["row_suffix_lens"],
            suffix_tables=dv["row_suffix_tables"], **levels,
            seg_row_offsets=dv["seg_row_offsets"] if has_seg else None,
            seg_kv_lens=dv["seg_kv_lens"] if has_seg else None,
            seg_tables=dv["seg_tables"] if has_seg else None,
            slot_mapping=dv["slot_mapping"] if iteration_state.b200_fused_fill else None,
        )
        iteration_state.b200_planned = False
        cls._last_call = iteration_state.b200_call

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, iteration_state):
        from . import ops

        getter = type(self).kv_cache_getter
        if getter is None:
            raise RuntimeError("B200SharedPromptsGenerate.kv_cache_getter is not set (call install())")
        k_cache, v_cache = getter(self.layer_idx)
        output = torch.empty_like(q)
        call = iteration_state.b200_call
        fused = call is not None and iteration_state.b200_fused_fill
        if not fused:
            ops.vllm_reshape_and_cache(k, v, k_cache, v_cache, iteration_state.slot_mapping)
        if call is not None:
            if not iteration_state.b200_planned:  # once per iteration; every layer reuses the lists
                call.plan(q, output, k_cache, v_cache)
                iteration_state.b200_planned = True
            call.params.scale = float(self.scaling)
            if fused:  # KV fill and attention as one call
                call.run(q, output, k_cache, v_cache, key_new=k.view(q.shape[0], -1, self.head_dim),
                         value_new=v.view(q.shape[0], -1, self.head_dim))
            else:
                call.run(q, output, k_cache, v_cache)
        return output.view(-1, self.num_heads * self.head_dim)


def install() -> str:
    """Registers ``B200SharedPromptsGenerate`` with an importable Parrot without editing it:
    name list, name -> class lookup on ``BuiltinConfig`` (``attn_func.py:704-737``) and
    name -> VLLM cache layout (``mem_layout.py:18-22``). Returns the registered name."""
    from parrot.engine.builtin import attn_func as ref_attn
    from parrot.engine.builtin import mem as ref_mem
    from parrot.engine.builtin.mem_layout import ATTN_FUNC_LAYOUT_MAP, MemLayout
    from parrot.engine.config import BuiltinConfig

    if ATTN_FUNC_NAME not in ref_attn.ATTN_FUNCS:
        ref_attn.ATTN_FUNCS.append(ATTN_FUNC_NAME)
        ATTN_FUNC_LAYOUT_MAP[ATTN_FUNC_NAME] = MemLayout.VLLM
        previous = BuiltinConfig._get_attn_func

        def _get_attn_func(self, name: str):
            if name == ATTN_FUNC_NAME:
                return B200SharedPromptsGenerate
            return previous(self, name)

        BuiltinConfig._get_attn_func = _get_attn_func
    B200SharedPromptsGenerate.kv_cache_getter = staticmethod(
        lambda layer: (ref_mem.get_k_cache(layer), ref_mem.get_v_cache(layer)))
    return ATTN_FUNC_NAME
