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


def shared_context_len(jobs: Sequence) -> int:
    """Length of the context shared by every job: the whole context of a lone job, else the
    context length of the jobs' common ancestor (0 when there is none)."""
    if len(jobs) == 1:
        return jobs[0].context.get_context_len()
    node = jobs[0].context
    for job in jobs[1:]:
        node = _lca(node, job.context)
        if node is None:
            return 0
    return node.get_context_len()


def _is_fill(job) -> bool:
    return hasattr(job, "token_ids") and job.token_ids is not None and not hasattr(job, "sampling_config")


class IterationMetadata:
    """Tables of one iteration. Field names shared with the reference's IterationState
    (``flash_context_len``, ``flash_block_table``, ``paged_context_lens``, ``paged_block_tables``,
    ``slot_mapping``) keep the reference's meaning for the Generate jobs; ``row_*`` cover every
    query token (Fill tokens first)."""

    def __init__(self, jobs: Sequence, block_size: int):
        b = block_size
        self.block_size = b
        self.flash_context_len = shared_context_len(jobs) if len(jobs) else 0
        n_shared_blocks = (self.flash_context_len + b - 1) // b
        pad_len = n_shared_blocks * b
        ctx0 = jobs[0].context.get_context_block_ids() if len(jobs) else []
        self.flash_block_table = np.asarray(ctx0[:pad_len:b], dtype=np.int32)

        self.num_fill_tokens: List[int] = []
        self.num_generation_jobs = 0
        slot_mapping: List[int] = []
        row_lens: List[int] = []
        row_tables: List[List[int]] = []
        paged_lens, paged_tables = [], []
        seg_offsets, seg_kv, seg_tabs = [0], [], []
        for job in jobs:
            blocks = job.context.get_context_block_ids()
            slots = job.context.get_context_slot_ids()
            ctx_len = job.context.get_context_len()
            private = blocks[pad_len::b]
            if _is_fill(job):
                n = len(job.token_ids)
                self.num_fill_tokens.append(n)
                slot_mapping.extend(slots[-n:])
                # one causal segment: token i sees the request's first kv - n + i + 1 private tokens
                seg_offsets.append(seg_offsets[-1] + n)
                seg_kv.append(max(ctx_len - self.flash_context_len, n))
                seg_tabs.append(private)
                for i in range(n):
                    row_lens.append(0)
                    row_tables.append([])
            else:
                self.num_generation_jobs += 1
                slot_mapping.extend(slots[-1:])
                row_lens.append(ctx_len - self.flash_context_len)
                row_tables.append(private)
                paged_lens.append(ctx_len - self.flash_context_len)
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


# ---------------------------------------------------------------------------------------------
# the attention function
# ---------------------------------------------------------------------------------------------
class B200SharedPromptsGenerate(nn.Module):
    """Drop-in for ``xFormersFill_SharedPromptsGenerate``."""

    # (layer_idx) -> (k_cache, v_cache); install() points this at parrot.engine.builtin.mem
    kv_cache_getter: Optional[Callable[[int], tuple]] = None

    def __init__(self, layer_idx: int, scaling: float, num_heads: int, head_dim: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.scaling = scaling
        self.num_heads = num_heads
        self.head_dim = head_dim

    @staticmethod
    def init_iteration_state(iteration_state, builtin_config, jobs, num_heads: int, head_size: int):
        from . import ops

        meta = IterationMetadata(jobs, builtin_config.block_size)
        dev = torch.device(builtin_config.device)
        for job in jobs:
            if _is_fill(job):
                iteration_state.num_fill_tokens.append(len(job.token_ids))
            else:
                iteration_state.generation_sampling_config.append(job.sampling_config)
        i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        iteration_state.flash_context_len = meta.flash_context_len
        iteration_state.flash_block_table = i32(meta.flash_block_table)
        iteration_state.paged_context_lens = i32(meta.paged_context_lens)
        iteration_state.paged_block_tables = i32(meta.paged_block_tables)
        iteration_state.slot_mapping = i32(meta.slot_mapping)
        iteration_state.b200_meta = meta
        if meta.num_rows == 0:
            iteration_state.b200_call = None
            return
        rows = meta.num_rows
        iteration_state.b200_call = ops.AttentionCall(
            num_rows=rows, num_heads=num_heads, head_size=head_size, block_size=builtin_config.block_size,
            dtype=builtin_config.dtype, device=dev, suffix_lens=i32(meta.row_suffix_lens),
            suffix_tables=i32(meta.row_suffix_tables),
            group_row_offsets=torch.tensor([0, rows], dtype=torch.int32, device=dev),
            group_prefix_lens=torch.tensor([meta.flash_context_len], dtype=torch.int32, device=dev),
            group_tables=i32(meta.flash_block_table).reshape(1, -1) if meta.flash_block_table.size else None,
            seg_row_offsets=i32(meta.seg_row_offsets) if len(meta.seg_kv_lens) else None,
            seg_kv_lens=i32(meta.seg_kv_lens) if len(meta.seg_kv_lens) else None,
            seg_tables=i32(meta.seg_tables) if len(meta.seg_kv_lens) else None,
        )
        iteration_state.b200_planned = False

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, iteration_state):
        from . import ops

        getter = type(self).kv_cache_getter
        if getter is None:
            raise RuntimeError("B200SharedPromptsGenerate.kv_cache_getter is not set (call install())")
        k_cache, v_cache = getter(self.layer_idx)
        ops.vllm_reshape_and_cache(k, v, k_cache, v_cache, iteration_state.slot_mapping)
        output = torch.empty_like(q)
        call = iteration_state.b200_call
        if call is not None:
            if not iteration_state.b200_planned:  # once per iteration; every layer reuses the lists
                call.plan(q, output, k_cache, v_cache)
                iteration_state.b200_planned = True
            call.params.scale = float(self.scaling)
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
