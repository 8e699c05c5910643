"""Seeded synthetic workloads with the shapes of the five benchmark configurations.

The reference measures this path on no public dataset; these generators stand alone. Metadata
(lengths, group assignment, block permutation) comes from a CPU generator seeded ``1000 + cfg``
so it is identical on every machine; payload (Q/K/V ~ N(0,1)) is generated per head with seed
``2000 + cfg`` so a head-sharded rank holds exactly the slices a single GPU would hold.

Layout facts used (parrot/engine/builtin/mem.py:69-82): K ``[NB, H, D/x, B, x]``,
V ``[NB, H, D, B]``, ``x = 16 / element_size``; every row's private context starts in a fresh
block, prefix lengths are block multiples (a forked parent is padded, block_context.py:30-38),
block-table rows are 0-padded like the reference's (attn_func.py:564-567).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

HEAD_SIZE = 128
BLOCK_SIZE = 16


@dataclasses.dataclass
class Workload:
    name: str
    cfg: int
    dtype: torch.dtype
    num_heads: int
    head_size: int
    block_size: int
    num_blocks: int
    group_row_offsets: np.ndarray  # [G+1] int32
    group_prefix_lens: np.ndarray  # [G] int32
    group_tables: np.ndarray  # [G, max_prefix_blocks] int32
    suffix_lens: np.ndarray  # [rows] int32
    suffix_tables: np.ndarray  # [rows, max_blocks] int32
    # KV fill of the iteration's new tokens (flat ragged slot mapping) and, for prefill rows,
    # which new-token range belongs to which request
    fill_slots: np.ndarray  # [T_new] int64
    num_prefill_tokens: int = 0
    prefill_lens: Sequence[int] = ()
    # causal segments (prefill requests): rows [seg_row_offsets[s], seg_row_offsets[s+1]) are the
    # request's new tokens; token i sees the first seg_kv_lens[s] - n + i + 1 tokens of seg_tables[s]
    seg_row_offsets: Optional[np.ndarray] = None
    seg_kv_lens: Optional[np.ndarray] = None
    seg_tables: Optional[np.ndarray] = None

    @property
    def num_rows(self) -> int:
        return int(self.suffix_lens.shape[0])

    @property
    def num_groups(self) -> int:
        return int(self.group_prefix_lens.shape[0])

    @property
    def elem_bytes(self) -> int:
        return torch.empty((), dtype=self.dtype).element_size()

    def algorithmic_bytes(self, num_heads: Optional[int] = None, include_fill: bool = True) -> Dict[str, float]:
        """Bytes one layer call must move: each group's prefix KV once, every row's private KV,
        Q read + O write, and the fill (read new K,V + write them into the cache)."""
        h = self.num_heads if num_heads is None else num_heads
        per_tok = 2 * self.head_size * self.elem_bytes * h
        used = np.diff(self.group_row_offsets) > 0
        prefix = float(self.group_prefix_lens[used].sum()) * per_tok
        suffix = float(self.suffix_lens.sum()) * per_tok
        if self.seg_kv_lens is not None:  # a request's private KV is read once for all its new tokens
            suffix += float(self.seg_kv_lens.sum()) * per_tok
        qo = 2.0 * self.num_rows * h * self.head_size * self.elem_bytes
        fill = 2.0 * len(self.fill_slots) * per_tok if include_fill else 0.0
        return {"prefix": prefix, "suffix": suffix, "qo": qo, "fill": fill, "total": prefix + suffix + qo + fill}

    # ---- payload ----
    def materialize(self, device, heads: Optional[Sequence[int]] = None, seed: Optional[int] = None):
        """Allocates caches and queries for the given head subset on `device` and fills them with
        N(0,1). Returns a dict of tensors (device) including int32 metadata."""
        heads = list(range(self.num_heads)) if heads is None else list(heads)
        seed = 2000 + self.cfg if seed is None else seed
        dev = torch.device(device)
        e = self.elem_bytes
        x = 16 // e
        hl, d, b, nb = len(heads), self.head_size, self.block_size, self.num_blocks
        kc = torch.empty((nb, hl, d // x, b, x), dtype=self.dtype, device=dev)
        vc = torch.empty((nb, hl, d, b), dtype=self.dtype, device=dev)
        q = torch.empty((self.num_rows, hl, d), dtype=self.dtype, device=dev)
        t_new = len(self.fill_slots)
        k_new = torch.empty((t_new, hl, d), dtype=self.dtype, device=dev)
        v_new = torch.empty((t_new, hl, d), dtype=self.dtype, device=dev)
        gen = torch.Generator(device=dev)
        for i, h in enumerate(heads):
            gen.manual_seed(seed * 4096 + h)
            kc[:, i].copy_(torch.randn((nb, d // x, b, x), generator=gen, device=dev, dtype=torch.float32))
            vc[:, i].copy_(torch.randn((nb, d, b), generator=gen, device=dev, dtype=torch.float32))
            q[:, i].copy_(torch.randn((self.num_rows, d), generator=gen, device=dev, dtype=torch.float32))
            if t_new:
                k_new[:, i].copy_(torch.randn((t_new, d), generator=gen, device=dev, dtype=torch.float32))
                v_new[:, i].copy_(torch.randn((t_new, d), generator=gen, device=dev, dtype=torch.float32))
        i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
        return {
            "query": q, "key_cache": kc, "value_cache": vc, "k_new": k_new, "v_new": v_new,
            "group_row_offsets": i32(self.group_row_offsets), "group_prefix_lens": i32(self.group_prefix_lens),
            "group_tables": i32(self.group_tables), "suffix_lens": i32(self.suffix_lens),
            "suffix_tables": i32(self.suffix_tables),
            "fill_slots": torch.from_numpy(np.ascontiguousarray(self.fill_slots, dtype=np.int64)).to(dev),
            "head_mapping": torch.arange(hl, dtype=torch.int32, device=dev),
            "seg_row_offsets": None if self.seg_kv_lens is None else i32(self.seg_row_offsets),
            "seg_kv_lens": None if self.seg_kv_lens is None else i32(self.seg_kv_lens),
            "seg_tables": None if self.seg_kv_lens is None else i32(self.seg_tables),
        }


def _blocks(n_tokens: int, b: int) -> int:
    return (n_tokens + b - 1) // b


def _deal(perm: np.ndarray, cursor: List[int], n: int) -> np.ndarray:
    out = perm[cursor[0]: cursor[0] + n]
    if len(out) != n:
        raise RuntimeError("block pool exhausted")
    cursor[0] += n
    return out


def _pad_rows(rows: List[np.ndarray]) -> np.ndarray:
    width = max([len(r) for r in rows] + [0])
    out = np.zeros((len(rows), width), dtype=np.int32)
    for i, r in enumerate(rows):
        out[i, : len(r)] = r
    return out


def _assemble(name, cfg, dtype, heads, prefix_lens, row_groups, suffix_lens, *, identity=False, num_blocks=None,
              slack=1.1, rng=None, new_token_rows=None, prefill=None) -> Workload:
    """prefix_lens [G]; row_groups [rows] sorted ascending; suffix_lens [rows]."""
    b = BLOCK_SIZE
    g = len(prefix_lens)
    need = sum(_blocks(p, b) for p in prefix_lens) + sum(_blocks(int(s), b) for s in suffix_lens)
    nb = num_blocks if num_blocks is not None else int(need * slack) + 8
    if identity:
        perm = np.arange(nb, dtype=np.int64)
    else:
        perm = rng.permutation(nb)
    cur = [0]
    gtabs = [_deal(perm, cur, _blocks(p, b)) for p in prefix_lens]
    stabs = [_deal(perm, cur, _blocks(int(s), b)) for s in suffix_lens]
    offs = np.zeros(g + 1, dtype=np.int32)
    for r in row_groups:
        offs[r + 1] += 1
    offs = np.cumsum(offs).astype(np.int32)
    suffix_tables = _pad_rows(stabs)
    # new tokens of the iteration: the last token of every decode row (default), or as given
    fill = []
    if new_token_rows is None:
        new_token_rows = [(r, int(suffix_lens[r]) - 1, 1) for r in range(len(suffix_lens)) if suffix_lens[r] > 0]
    for r, first_tok, n in new_token_rows:
        for t in range(first_tok, first_tok + n):
            fill.append(int(stabs[r][t // b]) * b + t % b)
    return Workload(
        name=name, cfg=cfg, dtype=dtype, num_heads=heads, head_size=HEAD_SIZE, block_size=b, num_blocks=nb,
        group_row_offsets=offs, group_prefix_lens=np.asarray(prefix_lens, dtype=np.int32),
        group_tables=_pad_rows(gtabs), suffix_lens=np.asarray(suffix_lens, dtype=np.int32),
        suffix_tables=suffix_tables, fill_slots=np.asarray(fill, dtype=np.int64),
        num_prefill_tokens=0 if prefill is None else int(sum(prefill)), prefill_lens=tuple(prefill or ()),
    )


def make_workload(cfg: int, shrink: int = 1, num_heads: Optional[int] = None) -> Workload:
    """Builds configuration `cfg` (1..5). `shrink` divides every length (prefixes stay block
    multiples) for quick tests; 1 = the full benchmark shape."""
    rng = np.random.default_rng(1000 + cfg)
    b = BLOCK_SIZE
    sh = max(1, shrink)

    def plen(tokens):
        return max(b, (tokens // sh) // b * b)

    def slen(lo, hi, n):
        hi = max(lo, hi // sh)
        return rng.integers(lo, hi + 1, size=n)

    if cfg == 1:  # CPU plumbing: fp32, contiguous KV
        suf = slen(1, 64, 4)
        return _assemble("cfg1_fp32_1x512_4seq", 1, torch.float32, num_heads or 32, [plen(512)], [0] * 4, suf,
                         identity=True, slack=1.0, rng=rng)
    if cfg == 2:  # LLaMA-7B decode step
        lo = max(1, 32 // sh)
        suf = rng.integers(lo, max(lo, 512 // sh) + 1, size=64)
        return _assemble("cfg2_llama7b_4096prefix_64seq", 2, torch.float16, num_heads or 32, [plen(4096)], [0] * 64,
                         suf, rng=rng)
    if cfg == 3:  # ragged multi-group, 13B heads
        g = 8
        w = np.arange(1, g + 1, dtype=np.float64) ** -1.2
        groups = np.sort(rng.choice(g, size=256, p=w / w.sum()))
        suf = slen(1, 2048, 256)
        return _assemble("cfg3_llama13b_8groups_256seq", 3, torch.float16, num_heads or 40,
                         [plen(1024 * (i + 1)) for i in range(g)], groups.tolist(), suf, rng=rng)
    if cfg == 4:  # continuous-batching iteration: 16 prefills + 240 decodes over one 2048 prefix
        q_lens = slen(max(1, 256 // sh), 1024, 16)
        dec = slen(1, 1024, 240)
        # every prefill token is a row; row i of a request sees that request's first i+1 new tokens
        return _assemble_cfg4(q_lens, dec, plen(2048), max(2 * 1024, 200000 // sh) // b, rng, num_heads or 32)
    if cfg == 5:  # box-scale head-sharded decode, bf16
        g = 32
        per = max(1, 64 // (sh if sh > 1 else 1))
        groups = np.repeat(np.arange(g), per)
        suf = slen(1, 1024, len(groups))
        return _assemble("cfg5_box_32groups_2048seq_bf16", 5, torch.bfloat16, num_heads or 64,
                         [plen(16384)] * g, groups.tolist(), suf, rng=rng)
    raise ValueError(f"unknown config {cfg}")


def _assemble_cfg4(q_lens, dec_lens, prefix_len, num_blocks, rng, heads) -> Workload:
    b = BLOCK_SIZE
    perm = rng.permutation(num_blocks)
    cur = [0]
    gtab = _deal(perm, cur, _blocks(prefix_len, b))
    suffix_lens, stabs, fill = [], [], []
    seg_offs, seg_tabs = [0], []
    for ql in q_lens:
        blocks = _deal(perm, cur, _blocks(int(ql), b))
        seg_offs.append(seg_offs[-1] + int(ql))
        seg_tabs.append(blocks)
        for i in range(int(ql)):
            suffix_lens.append(0)  # the request's own tokens are its causal segment, not a suffix
            stabs.append(blocks[:0])
            fill.append(int(blocks[i // b]) * b + i % b)
    for dl in dec_lens:
        blocks = _deal(perm, cur, _blocks(int(dl), b))
        suffix_lens.append(int(dl))
        stabs.append(blocks)
        t = int(dl) - 1
        fill.append(int(blocks[t // b]) * b + t % b)
    rows = len(suffix_lens)
    return Workload(
        name="cfg4_contbatch_16prefill_240decode", cfg=4, dtype=torch.float16, num_heads=heads, head_size=HEAD_SIZE,
        block_size=b, num_blocks=num_blocks, group_row_offsets=np.asarray([0, rows], dtype=np.int32),
        group_prefix_lens=np.asarray([prefix_len], dtype=np.int32), group_tables=_pad_rows([gtab]),
        suffix_lens=np.asarray(suffix_lens, dtype=np.int32), suffix_tables=_pad_rows(stabs),
        fill_slots=np.asarray(fill, dtype=np.int64), num_prefill_tokens=int(sum(int(x) for x in q_lens)),
        prefill_lens=tuple(int(x) for x in q_lens),
        seg_row_offsets=np.asarray(seg_offs, dtype=np.int32), seg_kv_lens=np.asarray([int(x) for x in q_lens], dtype=np.int32),
        seg_tables=_pad_rows(seg_tabs),
    )
