"""Stand-in for the reference's native module ``parrot.attention_ops`` (csrc/attention.cpp:49-62):
the same three entry points with the same positional arguments, writing into ``out`` in place.
Each forwards to the C-ABI function of the same name prefixed ``pb_``.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from ._lib import check, lib
from .ops import Workspace, _dtype_code, _kv_geometry, _require_cuda, _stream


def _prepare(out, query, key_cache, value_cache, head_mapping, block_tables, context_lens, block_size, alibi_slopes):
    if alibi_slopes is not None:
        raise RuntimeError("alibi_slopes is not supported (the reference always passes None)")
    _require_cuda(out, query, key_cache, value_cache, block_tables, context_lens)
    nb, hkv, d, b, kbs, khs = _kv_geometry(key_cache, value_cache)
    if b != block_size:
        raise RuntimeError(f"Unsupported block size: {block_size}")
    num_seqs, num_heads, head_size = query.shape
    if head_size != d:
        raise RuntimeError(f"Unsupported head size: {head_size}")
    if not out.is_contiguous():
        raise RuntimeError("out must be contiguous")
    if block_tables.dtype != torch.int32 or context_lens.dtype != torch.int32:
        raise RuntimeError("block_tables and context_lens must be int32")
    if head_mapping is not None and head_mapping.dtype != torch.int32:
        raise RuntimeError("head_mapping must be int32")
    block_tables = block_tables.contiguous()
    max_blocks = block_tables.shape[1] if block_tables.dim() == 2 else 0
    nbytes = lib().pb_single_query_workspace_bytes(num_seqs, num_heads, head_size, block_size, max_blocks)
    if nbytes == 0:
        raise _lib.PbError(_lib.PB_ERR_UNSUPPORTED, "pb_single_query_workspace_bytes")
    ws = Workspace.get(query.device, nbytes)
    tail = (block_size, max_blocks * block_size, num_seqs, num_heads, hkv, head_size, max_blocks, query.stride(0),
            kbs, khs, nb, _dtype_code(query), ws.data_ptr(), ws.numel(), _stream(query))
    return block_tables, tail


def single_query_cached_kv_attention(out, query, key_cache, value_cache, head_mapping, scale, block_tables,
                                     block_lens, block_nums, context_lens, block_size, max_context_len,
                                     alibi_slopes: Optional[torch.Tensor] = None) -> None:
    """csrc/attention.cpp:4-17. The reference kernel never reads ``block_lens`` and walks
    ``block_nums[seq]`` table entries, masking tokens at or beyond ``context_lens[seq]``
    (csrc/attention/attention_kernels.cu:159-162,203); here ceil(context_len / block_size) blocks
    are walked, the same attention for every consistent ``block_nums``, so both tensors are dropped."""
    bt, tail = _prepare(out, query, key_cache, value_cache, head_mapping, block_tables, context_lens, block_size, alibi_slopes)
    rc = lib().pb_single_query_cached_kv_attention(
        out.data_ptr(), query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
        None if head_mapping is None else head_mapping.data_ptr(), float(scale), bt.data_ptr(),
        context_lens.data_ptr(), *tail)
    check(rc, "pb_single_query_cached_kv_attention")


def single_query_cached_kv_prev_attention(out, query, key_cache, value_cache, head_mapping, scale, block_tables,
                                          context_lens, qk_maxs, exp_sums, block_size, max_context_len,
                                          alibi_slopes: Optional[torch.Tensor] = None) -> None:
    """csrc/attention.cpp:19-32: also writes the base-2 row maxima and exponent sums."""
    bt, tail = _prepare(out, query, key_cache, value_cache, head_mapping, block_tables, context_lens, block_size, alibi_slopes)
    rc = lib().pb_single_query_cached_kv_prev_attention(
        out.data_ptr(), query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
        None if head_mapping is None else head_mapping.data_ptr(), float(scale), bt.data_ptr(),
        context_lens.data_ptr(), qk_maxs.data_ptr(), exp_sums.data_ptr(), *tail)
    check(rc, "pb_single_query_cached_kv_prev_attention")


def single_query_cached_kv_post_attention(out, query, key_cache, value_cache, head_mapping, scale, block_tables,
                                          context_lens, prev_qk_maxs, prev_exp_sums, block_size, max_context_len,
                                          alibi_slopes: Optional[torch.Tensor] = None) -> None:
    """csrc/attention.cpp:34-47: merges in place with the partial result already in ``out``."""
    bt, tail = _prepare(out, query, key_cache, value_cache, head_mapping, block_tables, context_lens, block_size, alibi_slopes)
    rc = lib().pb_single_query_cached_kv_post_attention(
        out.data_ptr(), query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
        None if head_mapping is None else head_mapping.data_ptr(), float(scale), bt.data_ptr(),
        context_lens.data_ptr(), prev_qk_maxs.data_ptr(), prev_exp_sums.data_ptr(), *tail)
    check(rc, "pb_single_query_cached_kv_post_attention")
