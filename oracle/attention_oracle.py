"""CPU oracle for the shared-prefix paged attention path. TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference`` legs
of ``bench.py`` may import this module; the product (``parrotserve_b200``) never does.

Pinning: ``reference_port_paged_attention`` is checked against outputs of the reference's own
``paged_flash_attention_reference`` (run in the build container, fixtures under
``tests/golden/``); the gold functions are checked against the port on the same fixtures.

Restated from the reference (file:line relative to the ParrotServe tree):
  * torch reference attention        parrot/engine/builtin/kernels/shared_flash_decoding.py:382-404
  * per-token gather form            3rdparty/vllm/tests/kernels/test_attention.py:14-66
  * bottom-right causal with context 3rdparty/vllm/tests/kernels/test_attention.py:104-156
  * fill / gather references         3rdparty/vllm/tests/kernels/test_cache.py:70-114, 118-165
  * cache layout                     parrot/engine/builtin/mem.py:69-82, 3rdparty/vllm/csrc/cache_kernels.cu:155-178
  * merge algebra                    csrc/attention/attention_post_kernels.cu:321-340,
                                     parrot/engine/builtin/kernels/shared_flash_decoding.py:168-199
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch


# --------------------------------------------------------------------------------------------
# Port of the reference's torch reference attention (what the CPU baseline times).
# --------------------------------------------------------------------------------------------
def reference_port_paged_attention(
    query: torch.Tensor,  # [num_seqs, num_heads, head_size]
    key_cache: torch.Tensor,  # [num_blocks, num_kv_heads, head_size/x, block_size, x]
    value_cache: torch.Tensor,  # [num_blocks, num_kv_heads, head_size, block_size]
    head_mapping: torch.Tensor,  # [num_heads]
    context_lens: torch.Tensor,  # [num_seqs]
    block_tables: torch.Tensor,  # [num_seqs, max_num_blocks_per_seq]
) -> torch.Tensor:
    """Same algorithm, same operation order as shared_flash_decoding.py:382-404: per sequence,
    gather every block of the (padded) table row, scale q, logits by einsum, -inf beyond the
    context length, softmax, weighted sum by einsum. Works in the dtype of its inputs."""
    num_heads, head_size = query.shape[1], query.shape[2]
    scale = head_size ** -0.5
    hm = head_mapping.long()
    rows = []
    for s in range(query.shape[0]):
        table = block_tables[s].long()
        n = int(context_lens[s])
        v = value_cache[table]  # [nb, Hkv, D, B]
        k = key_cache[table].transpose(-1, -2).reshape(v.shape)  # [nb, Hkv, D/x, x, B] -> [nb, Hkv, D, B]
        v = v[:, hm].transpose(1, 3).reshape(-1, head_size, num_heads)  # [nb*B, D, H]
        k = k[:, hm].transpose(1, 3).reshape(-1, head_size, num_heads)
        logits = torch.einsum("hd,ndh->hn", query[s] * scale, k)
        logits[:, n:] = float("-inf")
        probs = torch.softmax(logits, dim=-1)
        rows.append(torch.einsum("hn,ndh->hd", probs, v).unsqueeze(0))
    return torch.cat(rows)


# --------------------------------------------------------------------------------------------
# Gold oracle: per-token gather, float64 accumulation, natural-exp softmax, no epsilon.
# --------------------------------------------------------------------------------------------
def gather_tokens(cache_k: torch.Tensor, cache_v: torch.Tensor, table: Sequence[int], n_tokens: int, heads):
    """K, V rows [n_tokens, len(heads), D] of the first n_tokens tokens addressed by `table`
    (token j lives in block table[j // B] at offset j % B)."""
    b = cache_v.shape[3]
    nb = (n_tokens + b - 1) // b
    if nb == 0:
        d = cache_v.shape[2]
        z = torch.zeros((0, len(heads), d), dtype=torch.float64)
        return z, z.clone()
    idx = torch.as_tensor(list(table[:nb]), dtype=torch.long)
    hs = torch.as_tensor(list(heads), dtype=torch.long)
    kb = cache_k[idx][:, hs]  # [nb, h, D/x, B, x]
    vb = cache_v[idx][:, hs]  # [nb, h, D, B]
    nbk, h, dx, bb, x = kb.shape
    k = kb.permute(0, 3, 1, 2, 4).reshape(nbk * bb, h, dx * x)[:n_tokens]
    v = vb.permute(0, 3, 1, 2).reshape(nbk * bb, h, vb.shape[2])[:n_tokens]
    return k.double(), v.double()


def gold_row_attention(q_row: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """q_row [h, D], k/v [n, h, D] float64 -> [h, D] float64 (zeros when n == 0)."""
    if k.shape[0] == 0:
        return torch.zeros_like(q_row, dtype=torch.float64)
    logits = torch.einsum("hd,nhd->hn", q_row.double() * scale, k)
    probs = torch.softmax(logits, dim=-1)
    return torch.einsum("hn,nhd->hd", probs, v)


def gold_grouped_attention(
    query: torch.Tensor,  # [rows, H, D]
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    group_row_offsets: Optional[Sequence[int]],  # [G+1] or None
    group_prefix_lens: Optional[Sequence[int]],
    group_tables: Optional[Sequence[Sequence[int]]],
    suffix_lens: Sequence[int],
    suffix_tables: Sequence[Sequence[int]],
    rows: Optional[Sequence[int]] = None,
    heads: Optional[Sequence[int]] = None,
    head_mapping: Optional[Sequence[int]] = None,
    scale: Optional[float] = None,
    seg_row_offsets: Optional[Sequence[int]] = None,
    seg_kv_lens: Optional[Sequence[int]] = None,
    seg_tables: Optional[Sequence[Sequence[int]]] = None,
    outer_row_offsets: Optional[Sequence[int]] = None,
    outer_prefix_lens: Optional[Sequence[int]] = None,
    outer_tables: Optional[Sequence[Sequence[int]]] = None,
) -> torch.Tensor:
    """Attention of each selected row over prefix(group(row)) ++ suffix(row): the identity the
    shared-prefix kernels are pinned by (shared result == ordinary paged attention over the
    concatenated block table). Returns float64 [len(rows), len(heads), D]."""
    n_rows, n_heads, d = query.shape
    scale = d ** -0.5 if scale is None else scale
    rows = list(range(n_rows)) if rows is None else list(rows)
    heads = list(range(n_heads)) if heads is None else list(heads)
    kv_heads = heads if head_mapping is None else [int(head_mapping[h]) for h in heads]
    row_group = [-1] * n_rows
    if group_row_offsets is not None:
        for g in range(len(group_row_offsets) - 1):
            for r in range(int(group_row_offsets[g]), int(group_row_offsets[g + 1])):
                row_group[r] = g
    # causal segments: row i of a segment of n rows sees the first kv - n + i + 1 tokens of its table
    # (bottom-right aligned mask, 3rdparty/vllm/tests/kernels/test_attention.py:104-156)
    row_seg = {}
    if seg_row_offsets is not None:
        for s in range(len(seg_row_offsets) - 1):
            r0, r1 = int(seg_row_offsets[s]), int(seg_row_offsets[s + 1])
            for r in range(r0, r1):
                row_seg[r] = (s, int(seg_kv_lens[s]) - (r1 - r0) + (r - r0) + 1)
    # outer prefix groups: a context shared above the groups (two-level context trees,
    # tests/engine/builtin/test_shared_prefix.py:57-115); its tokens come first
    row_outer = [-1] * n_rows
    if outer_row_offsets is not None:
        for o in range(len(outer_row_offsets) - 1):
            for r in range(int(outer_row_offsets[o]), int(outer_row_offsets[o + 1])):
                row_outer[r] = o
    prefix_cache, outer_cache = {}, {}
    out = torch.zeros((len(rows), len(heads), d), dtype=torch.float64)
    for i, r in enumerate(rows):
        g = row_group[r]
        ks, vs = [], []
        o = row_outer[r]
        if o >= 0 and int(outer_prefix_lens[o]) > 0:
            if o not in outer_cache:
                outer_cache[o] = gather_tokens(key_cache, value_cache, outer_tables[o], int(outer_prefix_lens[o]), kv_heads)
            ks.append(outer_cache[o][0])
            vs.append(outer_cache[o][1])
        if g >= 0 and int(group_prefix_lens[g]) > 0:
            if g not in prefix_cache:
                prefix_cache[g] = gather_tokens(key_cache, value_cache, group_tables[g], int(group_prefix_lens[g]), kv_heads)
            ks.append(prefix_cache[g][0])
            vs.append(prefix_cache[g][1])
        if r in row_seg:
            sidx, vis = row_seg[r]
            k, v = gather_tokens(key_cache, value_cache, seg_tables[sidx], vis, kv_heads)
            ks.append(k)
            vs.append(v)
        n = int(suffix_lens[r]) if suffix_lens is not None else 0
        if n > 0:
            k, v = gather_tokens(key_cache, value_cache, suffix_tables[r], n, kv_heads)
            ks.append(k)
            vs.append(v)
        if ks:
            out[i] = gold_row_attention(query[r][heads], torch.cat(ks), torch.cat(vs), scale)
    return out


def gold_stats(q_row: torch.Tensor, k: torch.Tensor, scale: float):
    """Base-2 statistics of one row: (max, sum 2^(logit - max)) per head, the convention of
    csrc/attention/attention_post_kernels.cu:147,223 (logits multiplied by log2 e)."""
    logits = torch.einsum("hd,nhd->hn", q_row.double() * scale, k) * 1.4426950408889634
    m = logits.max(dim=-1).values
    l = torch.exp2(logits - m[:, None]).sum(dim=-1)
    return m, l


def merge_partials(outs: Sequence[torch.Tensor], ms: Sequence[torch.Tensor], ls: Sequence[torch.Tensor]):
    """LSE merge of normalised partial outputs [.., D] with base-2 (max, sum) statistics [..]:
    w_i = l_i 2^(m_i - M) / sum_j l_j 2^(m_j - M)   (attention_post_kernels.cu:321-340)."""
    m_all = torch.stack(list(ms))
    M = m_all.max(dim=0).values
    w = torch.stack([l * torch.exp2(m - M) for m, l in zip(ms, ls)])
    L = w.sum(dim=0)
    out = sum(o * (wi / L)[..., None] for o, wi in zip(outs, w))
    return out, M, L


def gold_causal_with_context(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """Bottom-right aligned causal attention: query i of q_len sees keys j <= i + ctx_len - q_len
    (3rdparty/vllm/tests/kernels/test_attention.py:104-156). q [q_len,h,D], k/v [ctx_len,h,D]."""
    q_len, ctx_len = q.shape[0], k.shape[0]
    logits = torch.einsum("qhd,khd->hqk", q.double() * scale, k.double())
    mask = torch.triu(torch.ones(q_len, ctx_len, dtype=torch.bool), diagonal=ctx_len - q_len + 1)
    logits = logits.masked_fill(mask, float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(logits, dim=-1), v.double())


# --------------------------------------------------------------------------------------------
# Byte-exact references for the cache fill / gather / moves (numpy).
# --------------------------------------------------------------------------------------------
def _np(t):
    if isinstance(t, torch.Tensor):
        if t.dtype == torch.bfloat16:
            return t.contiguous().view(torch.int16).numpy()
        return t.contiguous().numpy()
    return np.asarray(t)


def fill_reference(key, value, key_cache, value_cache, slot_mapping):
    """In-place indexed assignment of test_cache.py:103-111 on numpy views (bit patterns).
    key/value [T,H,D]; key_cache [NB,H,D/x,B,x]; value_cache [NB,H,D,B]; negative slots skipped."""
    key, value = _np(key), _np(value)
    t, h, d = key.shape
    x = key_cache.shape[4]
    b = key_cache.shape[3]
    rk = key.reshape(t, h, d // x, x)
    for i, s in enumerate(np.asarray(slot_mapping).reshape(-1).tolist()):
        if s < 0:
            continue
        key_cache[s // b, :, :, s % b, :] = rk[i]
        value_cache[s // b, :, :, s % b] = value[i]


def gather_reference(key_cache, value_cache, slot_mapping):
    """Inverse of fill_reference (test_cache.py:118-165): returns key, value [T,H,D]."""
    nb, h, dx, b, x = key_cache.shape
    slots = np.asarray(slot_mapping).reshape(-1)
    blk, off = slots // b, slots % b
    k = key_cache[blk, :, :, off, :].reshape(len(slots), h, dx * x)
    v = value_cache[blk, :, :, off]
    return k, v


def move_rows_reference(src, dest, src_idx, dest_idx):
    """dest[dest_idx[i]] = src[src_idx[i]] (tokens_moving.py:25-64)."""
    dest[np.asarray(dest_idx)] = src[np.asarray(src_idx)]


def rotary_neox_reference(positions, query, key, cos_sin_cache, head_size: int):
    """NeoX rotary embedding, float64: the arithmetic of rotary_embedding_neox_kernel
    (3rdparty/vllm/csrc/pos_encoding_kernels.cu:7-60) on numpy arrays.

    positions [T] int; query [T, Hq*head_size], key [T, Hk*head_size] (any float dtype, read as
    float64); cos_sin_cache [max_position, rot_dim] = cos(rot_dim/2) | sin(rot_dim/2) per row.
    For each head: x = elements [0, rot_dim/2), y = [rot_dim/2, rot_dim);
    out_x = x*cos - y*sin, out_y = y*cos + x*sin; elements >= rot_dim pass through.
    Returns (query, key) as float64 arrays of the input shapes; the caller rounds to the storage type."""
    pos = np.asarray(positions).reshape(-1)
    cs = np.asarray(cos_sin_cache, dtype=np.float64)
    rot = cs.shape[1]
    e = rot // 2
    cos, sin = cs[pos, :e], cs[pos, e:]  # [T, e]

    def rot_one(a):
        a = np.asarray(a, dtype=np.float64)
        t = a.shape[0]
        v = a.reshape(t, -1, head_size).copy()
        x, y = v[:, :, :e].copy(), v[:, :, e:rot].copy()
        v[:, :, :e] = x * cos[:, None, :] - y * sin[:, None, :]
        v[:, :, e:rot] = y * cos[:, None, :] + x * sin[:, None, :]
        return v.reshape(a.shape)

    return rot_one(query), rot_one(key)
