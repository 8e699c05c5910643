"""CPU tests of the host side: C-ABI exports, workload generators, iteration metadata against
the reference's own output, and the multi-rank helpers under gloo (world size 2)."""
import json
import os
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def test_library_exports_every_declared_symbol():
    import ctypes

    from parrotserve_b200 import _lib

    header = (ROOT / "include" / "parrot_b200_attn.h").read_text()
    declared = set(re.findall(r"\b(pb_[a-z0-9_]+)\s*\(", header))
    declared -= {"pb_dtype", "pb_status", "pb_stats_mode", "pb_attn_params"}
    assert len(declared) >= 15
    handle = _lib.lib()  # loads without a GPU; no compute call is made here
    for name in declared:
        assert hasattr(handle, name), f"{name} is declared but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert handle.pb_abi_version() == 3
    # the ctypes mirror of pb_attn_params has the size the compiler gives the C struct
    body = re.search(r"typedef struct pb_attn_params \{(.*?)\} pb_attn_params;", header, re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = re.findall(r"(\w+)\s*;", body)
    assert names == [f[0] for f in _lib.PbAttnParams._fields_], "ctypes mirror and header disagree"
    body = re.search(r"typedef struct pb_host_step \{(.*?)\} pb_host_step;", header, re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    assert re.findall(r"(\w+)\s*;", body) == [f[0] for f in _lib.PbHostStep._fields_]
    p = _lib.PbAttnParams()
    p.num_rows, p.num_heads, p.num_kv_heads, p.head_size, p.block_size = 64, 32, 32, 128, 16
    p.dtype, p.suffix_table_stride, p.num_groups, p.group_table_stride = _lib.PB_F16, 32, 1, 256
    assert handle.pb_attn_workspace_bytes(ctypes.byref(p)) > 0
    p.head_size = 72
    assert handle.pb_attn_workspace_bytes(ctypes.byref(p)) == 0  # unsupported shape is reported, not guessed


def test_torch_shim_exports_the_reference_modules_surface():
    """The compiled torch extension has the function names of parrot.attention_ops
    (csrc/attention.cpp:49-62) and vllm.cache_ops (3rdparty/vllm/csrc/cache.cpp:30-46); CPU tensors are
    refused with a RuntimeError, as TORCH_CHECK does in the reference."""
    from parrotserve_b200 import torch_ops

    attention_ops, cache_ops = torch_ops.load()
    for name in ("single_query_cached_kv_attention", "single_query_cached_kv_prev_attention", "single_query_cached_kv_post_attention"):
        assert callable(getattr(attention_ops, name))
    for name in ("swap_blocks", "copy_blocks", "reshape_and_cache", "gather_cached_kv"):
        assert callable(getattr(cache_ops, name))
    k = torch.zeros((2, 2, 16), dtype=torch.float16)
    kc = torch.zeros((4, 2, 2, 16, 8), dtype=torch.float16)
    vc = torch.zeros((4, 2, 16, 16), dtype=torch.float16)
    with pytest.raises(RuntimeError):
        cache_ops.reshape_and_cache(k, k, kc, vc, torch.tensor([1, 2], dtype=torch.int32))
    with pytest.raises(RuntimeError):
        cache_ops.swap_blocks(kc, kc.clone(), {0: 1})  # CPU -> CPU: "Invalid device combination"
    with pytest.raises(TypeError):
        attention_ops.single_query_cached_kv_attention(k)  # the 13-argument signature


def test_ops_fail_loudly_without_a_gpu_or_on_cpu_tensors():
    import parrotserve_b200 as pb

    q = torch.zeros((1, 2, 128), dtype=torch.float16)
    kc = torch.zeros((4, 2, 16, 16, 8), dtype=torch.float16)
    vc = torch.zeros((4, 2, 128, 16), dtype=torch.float16)
    with pytest.raises(RuntimeError):
        pb.vllm_paged_attention(q, kc, vc, None, torch.tensor([3], dtype=torch.int32), torch.tensor([[0]], dtype=torch.int32))
    with pytest.raises(RuntimeError):
        pb.vllm_reshape_and_cache(q, q, kc, vc, torch.tensor([3]))


@pytest.mark.parametrize("cfg", [1, 2, 3, 4, 5])
def test_workload_generators_are_consistent(cfg):
    from parrotserve_b200.workloads import make_workload

    wl = make_workload(cfg, shrink=1 if cfg in (1, 2) else 8)
    again = make_workload(cfg, shrink=1 if cfg in (1, 2) else 8)
    assert np.array_equal(wl.suffix_tables, again.suffix_tables) and np.array_equal(wl.group_tables, again.group_tables)
    b = wl.block_size
    used = []
    for g in range(wl.num_groups):
        assert wl.group_prefix_lens[g] % b == 0
        used += wl.group_tables[g][: wl.group_prefix_lens[g] // b].tolist()
    per_job_tables = {}
    for r in range(wl.num_rows):
        nb = (int(wl.suffix_lens[r]) + b - 1) // b
        per_job_tables[tuple(wl.suffix_tables[r][:nb].tolist())] = None
        assert (wl.suffix_tables[r][nb:] == 0).all()  # rows are 0-padded like the reference's
    if cfg != 4:  # config 4: the rows of one prefill request share that request's blocks
        for tbl in per_job_tables:
            used += list(tbl)
        assert len(used) == len(set(used)), "a physical block is dealt twice"
    assert max(used) < wl.num_blocks
    assert wl.group_row_offsets[0] == 0 and wl.group_row_offsets[-1] == wl.num_rows
    assert (np.diff(wl.group_row_offsets) >= 0).all()
    assert len(wl.fill_slots) == len(set(wl.fill_slots.tolist()))
    if cfg == 2:
        assert wl.num_rows == 64 and wl.group_prefix_lens.tolist() == [4096]
        assert wl.suffix_lens.min() >= 32 and wl.suffix_lens.max() <= 512
        ab = wl.algorithmic_bytes()
        assert abs(ab["prefix"] - 4096 * 32 * 512) < 1 and ab["total"] > 3.0e8


def _tree_from_golden(case):
    from tests.fake_parrot import Context, Fill, Generate, Pool

    pool = Pool()
    b = case["block_size"]
    root = None
    if case["root_len"]:
        root = Context(0, None, pool, b)
        root.allocate(case["root_len"])
    jobs, cid = [], 1
    for cached, n_new in case.get("fills", []):
        ctx = Context(cid, root, pool, b)
        ctx.allocate(cached)
        ctx.allocate(n_new)
        jobs.append(Fill(ctx, list(range(n_new))))
        cid += 1
    for extra in case["children"]:
        ctx = Context(cid, root, pool, b)
        ctx.allocate(extra)
        ctx.allocate(1)  # the slot of the token generated in this iteration
        jobs.append(Generate(ctx))
        cid += 1
    return jobs


def _check_metadata_against_reference_case(meta, jobs, case):
    """`meta`: an IterationMetadata-shaped object; `case`: what the reference's builder produced."""
    b = case["block_size"]
    fills = case.get("fills", [])
    n_fill = len(fills)
    # the Generate side keeps the reference's meaning whenever the shared length is the reference's
    lone_fill = n_fill == 1 and len(jobs) == 1
    if not lone_fill:
        assert meta.flash_context_len == case["flash_context_len"]
        assert meta.flash_block_table.tolist() == case["flash_block_table"]
        assert meta.paged_context_lens.tolist() == case["paged_context_lens"]
        width = len(case["paged_block_tables"][0]) if case["paged_block_tables"] else 0
        assert [r[:width] for r in meta.paged_block_tables.tolist()] == case["paged_block_tables"]
    # slot mapping: the reference pads it to [jobs, max_new]; ours is the same slots, flat and ragged
    new_counts = [f[1] for f in fills] + [1] * len(case["children"])
    assert meta.slot_mapping.tolist() == [s for row, n in zip(case["slot_mapping"], new_counts) for s in row[:n]]
    assert meta.num_rows == sum(new_counts) and meta.num_fill_tokens == case.get("num_fill_tokens", [])
    if not n_fill:
        assert meta.num_total_fill_tokens == 0
        return
    # Fill side: the reference hands xformers (q_len, kv_len = whole context) per job with a bottom-right
    # causal mask and gathers every context slot; ours splits the same tokens into shared prefix
    # (attended in full) + causal segment, and addresses them through block tables
    assert np.diff(meta.seg_row_offsets).tolist() == case["fill_q_lens"]
    assert (meta.seg_kv_lens + meta.flash_context_len).tolist() == case["fill_kv_lens"]
    off = 0
    for s_idx, kv in enumerate(case["fill_kv_lens"]):
        want = case["fill_slots"][off:off + kv]
        off += kv
        shared = [int(meta.flash_block_table[t // b]) * b + t % b for t in range(meta.flash_context_len)]
        own = [int(meta.seg_tables[s_idx][t // b]) * b + t % b for t in range(int(meta.seg_kv_lens[s_idx]))]
        # a forked parent is padded to a block multiple and the padding counts as context (the
        # reference gathers those slots too)
        assert shared + own == want, case["name"]
    assert off == len(case["fill_slots"])


def test_iteration_metadata_matches_the_reference_builder():
    """Fixtures: output of the reference's init_iteration_state over its own BlockContext trees,
    Generate-only batches, mixed Fill + Generate batches and iterations of one Fill job."""
    from parrotserve_b200.attn_func import IterationMetadata

    cases = json.loads((ROOT / "tests/golden/iteration_state_ref.json").read_text())
    assert {c["name"] for c in cases} >= {"fork3_root64", "fork2_root20_padded", "single_job", "fill2_gen3_root40",
                                         "lone_fill_no_parent", "lone_fill_with_parent_and_cache"}
    for case in cases:
        jobs = _tree_from_golden(case)
        # the stand-in contexts reproduce the reference's slot allocation
        assert [j.context.get_context_slot_ids() for j in jobs] == case["context_slot_ids"], case["name"]
        meta = IterationMetadata(jobs, case["block_size"])
        _check_metadata_against_reference_case(meta, jobs, case)
        if case["name"] == "lone_fill_no_parent":
            # the reference calls the lone job's whole context "shared" but never applies that to Fill
            # rows; here the shared prefix is applied to every row, so it must stop before the job's tokens
            assert case["flash_context_len"] == 20 and meta.flash_context_len == 0
        if case["name"] == "lone_fill_with_parent_and_cache":
            assert case["flash_context_len"] == 81 and meta.flash_context_len == 48


def test_iteration_metadata_mixed_fill_and_generate():
    from parrotserve_b200.attn_func import IterationMetadata
    from tests.fake_parrot import Context, Fill, Generate, Pool

    pool, b = Pool(), 16
    root = Context(0, None, pool, b)
    root.allocate(40)  # padded to 48 when forked
    f_ctx = Context(1, root, pool, b)
    f_ctx.allocate(5)   # earlier private tokens
    f_ctx.allocate(20)  # this iteration's fill
    g_ctx = Context(2, root, pool, b)
    g_ctx.allocate(7)
    g_ctx.allocate(1)
    meta = IterationMetadata([Fill(f_ctx, list(range(20))), Generate(g_ctx)], b)
    assert meta.flash_context_len == 48 and meta.flash_block_table.tolist() == [0, 1, 2]
    assert meta.num_fill_tokens == [20] and meta.num_generation_jobs == 1 and meta.num_rows == 21
    # the Fill job is one causal segment over its 5 cached + 20 new private tokens: its i-th new
    # token sees the first 25 - 20 + i + 1 of them; fill rows carry no suffix of their own
    assert meta.row_suffix_lens.tolist() == [0] * 20 + [8]
    assert meta.seg_row_offsets.tolist() == [0, 20] and meta.seg_kv_lens.tolist() == [25]
    assert meta.seg_tables[0].tolist() == f_ctx.blocks[::b]
    assert meta.slot_mapping.tolist() == f_ctx.get_context_slot_ids()[-20:] + g_ctx.get_context_slot_ids()[-1:]
    assert meta.row_suffix_tables[20].tolist()[:1] == g_ctx.blocks[::b]
    assert meta.paged_context_lens.tolist() == [8]


def test_iteration_metadata_two_level_context_tree():
    """Two-level option: the context shared by all jobs stays the outer level; runs of consecutive jobs
    under a common deeper context become inner groups whose rows' private parts start after it."""
    from parrotserve_b200.attn_func import IterationMetadata
    from tests.fake_parrot import Context, Fill, Generate, Pool

    b = 16
    pool = Pool()
    root = Context(0, None, pool, b)
    root.allocate(64)
    app1, app2 = Context(1, root, pool, b), Context(2, root, pool, b)
    app1.allocate(30)   # padded to 32 when first forked
    app2.allocate(16)

    def generate(cid, parent, cached):
        ctx = Context(cid, parent, pool, b)
        ctx.allocate(cached)
        ctx.allocate(1)
        return Generate(ctx)

    f_ctx = Context(10, app1, pool, b)
    f_ctx.allocate(5)
    f_ctx.allocate(20)
    jobs = [Fill(f_ctx, list(range(20))), generate(11, app1, 3), generate(12, app1, 17),
            generate(13, app2, 0), generate(14, app2, 40), generate(15, root, 9)]
    meta = IterationMetadata(jobs, b, two_level=True)
    assert meta.flash_context_len == 64 and meta.flash_block_table.tolist() == [0, 1, 2, 3]
    assert meta.inner_row_offsets.tolist() == [0, 22, 24, 25]
    assert meta.inner_prefix_lens.tolist() == [32, 16, 0]
    assert meta.inner_tables.tolist() == [app1.get_context_block_ids()[64::b] , [app2.get_context_block_ids()[64], 0], [0, 0]]
    assert meta.row_suffix_lens.tolist()[20:] == [4, 18, 1, 41, 10]
    assert meta.seg_kv_lens.tolist() == [25]
    assert meta.seg_tables.tolist() == [f_ctx.get_context_block_ids()[96::b]]
    # every row's three levels add up to its context
    one = IterationMetadata(jobs, b)
    inner_of_row = np.repeat(meta.inner_prefix_lens, np.diff(meta.inner_row_offsets))
    assert (meta.row_suffix_lens[20:] + inner_of_row[20:] == one.row_suffix_lens[20:]).all()
    assert meta.seg_kv_lens[0] + 32 == one.seg_kv_lens[0]
    # the reference-named fields do not change with the option off, and one job alone has no inner level
    assert one.row_suffix_lens.tolist()[20:] == [36, 50, 17, 57, 10]
    solo = IterationMetadata(jobs[1:2], b, two_level=True)
    assert solo.inner_prefix_lens.tolist() == [0]
    with pytest.raises(ValueError):
        IterationMetadata(jobs[1:2] + jobs[0:1], b)


def test_two_level_metadata_describes_the_same_attention():
    """The two-level metadata, fed to the grouped oracle, gives every query token the attention
    over its job's whole context up to itself (small sizes, CPU only)."""
    from oracle import attention_oracle as orc
    from parrotserve_b200.attn_func import IterationMetadata
    from tests.fake_parrot import Context, Fill, Generate, Pool

    h, d, b, nb, x = 2, 32, 16, 64, 8
    g = torch.Generator().manual_seed(5)
    kc = torch.randn((nb, h, d // x, b, x), generator=g)
    vc = torch.randn((nb, h, d, b), generator=g)
    pool = Pool()
    root = Context(0, None, pool, b)
    root.allocate(40)
    app1, app2 = Context(1, root, pool, b), Context(2, root, pool, b)
    app1.allocate(50)
    app2.allocate(16)
    jobs, counts = [], []
    for cid, (parent, cached, n_new) in enumerate([(app1, 7, 21), (app2, 0, 9), (app1, 0, 1), (app1, 19, 1),
                                                   (app2, 3, 1), (app2, 16, 1), (root, 5, 1)], start=10):
        ctx = Context(cid, parent, pool, b)
        ctx.allocate(cached)
        ctx.allocate(n_new)
        jobs.append(Fill(ctx, list(range(n_new))) if n_new > 1 else Generate(ctx))
        counts.append(n_new)
    t = sum(counts)
    q = torch.randn((t, h, d), generator=g)
    m = IterationMetadata(jobs, b, two_level=True)
    assert m.inner_prefix_lens.tolist() == [64, 16, 64, 16, 0]
    out = orc.gold_grouped_attention(
        q, kc, vc, m.inner_row_offsets, m.inner_prefix_lens, m.inner_tables, m.row_suffix_lens, m.row_suffix_tables,
        seg_row_offsets=m.seg_row_offsets, seg_kv_lens=m.seg_kv_lens, seg_tables=m.seg_tables,
        outer_row_offsets=[0, t], outer_prefix_lens=[m.flash_context_len], outer_tables=[m.flash_block_table.tolist()])
    row = 0
    for job, n in zip(jobs, counts):
        slots = job.context.get_context_slot_ids()
        for i in range(n):
            vis = slots[:len(slots) - n + i + 1]
            blk, off = torch.tensor([s // b for s in vis]), torch.tensor([s % b for s in vis])
            kk = kc[blk, :, :, off, :].reshape(len(vis), h, -1).double()
            vv = vc[blk, :, :, off].double()
            ref = orc.gold_row_attention(q[row].double(), kk, vv, d ** -0.5)
            assert (out[row] - ref).abs().max().item() < 1e-9, row
            row += 1


def _one_level_oracle_rows(meta, jobs, counts, q, kc, vc, b, d):
    """Grouped oracle over one-level metadata and, beside it, the per-row reference: every query token
    attends its job's whole context up to and including itself."""
    from oracle import attention_oracle as orc

    t = sum(counts)
    h = q.shape[1]
    has_seg = len(meta.seg_kv_lens) > 0
    out = orc.gold_grouped_attention(
        q, kc, vc, [0, t], [meta.flash_context_len], [meta.flash_block_table.tolist()], meta.row_suffix_lens,
        meta.row_suffix_tables, seg_row_offsets=meta.seg_row_offsets if has_seg else None,
        seg_kv_lens=meta.seg_kv_lens if has_seg else None, seg_tables=meta.seg_tables if has_seg else None)
    row = 0
    for job, n in zip(jobs, counts):
        slots = job.context.get_context_slot_ids()
        for i in range(n):
            vis = slots[:len(slots) - n + i + 1]
            blk, off = torch.tensor([s // b for s in vis]), torch.tensor([s % b for s in vis])
            kk = kc[blk, :, :, off, :].reshape(len(vis), h, -1).double()
            vv = vc[blk, :, :, off].double()
            ref = orc.gold_row_attention(q[row].double(), kk, vv, d ** -0.5)
            assert (out[row] - ref).abs().max().item() < 1e-9, row
            row += 1
    assert row == t


def test_single_job_iterations_and_fill_contexts_never_shared():
    """An iteration of ONE job (the first prefill of any request is one), and a batch whose common
    ancestor is a Fill job's own context: the shared prefix never reaches into the context a Fill job
    is adding tokens to, so those tokens stay under the job's causal mask."""
    from parrotserve_b200.attn_func import IterationMetadata, shared_context_len
    from tests.fake_parrot import Context, Fill, Generate, Pool

    h, d, b, nb, x = 2, 32, 16, 64, 8
    g = torch.Generator().manual_seed(9)
    kc = torch.randn((nb, h, d // x, b, x), generator=g)
    vc = torch.randn((nb, h, d, b), generator=g)

    def fresh(parent_len):
        pool = Pool()
        parent = None
        if parent_len:
            parent = Context(0, None, pool, b)
            parent.allocate(parent_len)
        return pool, parent

    # [Fill] alone: no parent / a parent / a parent and earlier tokens of its own
    for parent_len, cached, n_new in ((0, 0, 20), (0, 0, 1), (40, 0, 20), (40, 13, 20), (0, 33, 7)):
        pool, parent = fresh(parent_len)
        ctx = Context(1, parent, pool, b)
        ctx.allocate(cached)
        ctx.allocate(n_new)
        jobs = [Fill(ctx, list(range(n_new)))]
        meta = IterationMetadata(jobs, b)
        want_shared = 0 if parent is None else parent.get_context_len()
        assert meta.flash_context_len == want_shared == shared_context_len(jobs)
        assert meta.seg_row_offsets.tolist() == [0, n_new] and meta.seg_kv_lens.tolist() == [cached + n_new]
        assert meta.seg_tables.shape == (1, (cached + n_new + b - 1) // b)
        assert meta.row_suffix_lens.tolist() == [0] * n_new and meta.num_rows == n_new
        assert meta.slot_mapping.tolist() == ctx.get_context_slot_ids()[-n_new:]
        q = torch.randn((n_new, h, d), generator=g)
        _one_level_oracle_rows(meta, jobs, [n_new], q, kc, vc, b, d)

    # [Generate] alone: the whole context is the shared prefix (the reference's rule), true length masked
    for parent_len, cached in ((0, 19), (48, 0), (40, 30)):
        pool, parent = fresh(parent_len)
        ctx = Context(1, parent, pool, b)
        ctx.allocate(cached)
        ctx.allocate(1)
        jobs = [Generate(ctx)]
        meta = IterationMetadata(jobs, b)
        assert meta.flash_context_len == ctx.get_context_len()
        assert meta.row_suffix_lens.tolist() == [0] and meta.row_suffix_tables.shape[1] == 0
        assert len(meta.seg_kv_lens) == 0
        _one_level_oracle_rows(meta, jobs, [1], torch.randn((1, h, d), generator=g), kc, vc, b, d)

    # a Fill job on context C together with Generate jobs on children of C: the common ancestor is C
    # itself, which still receives the Fill job's tokens
    pool, parent = fresh(32)
    c = Context(1, parent, pool, b)
    c.allocate(16)                      # earlier tokens of C
    kids = [Context(2 + i, c, pool, b) for i in range(2)]   # forked before the new fill (pads C)
    c.allocate(16)                      # this iteration's Fill tokens
    for i, kid in enumerate(kids):
        kid.allocate(5 * i)
        kid.allocate(1)
    jobs = [Fill(c, list(range(16)))] + [Generate(k) for k in kids]
    meta = IterationMetadata(jobs, b)
    assert meta.flash_context_len == parent.get_context_len() == 32   # not C's 64
    assert meta.seg_kv_lens.tolist() == [32] and meta.paged_context_lens.tolist() == [33, 38]
    _one_level_oracle_rows(meta, jobs, [16, 1, 1], torch.randn((18, h, d), generator=g), kc, vc, b, d)

    # a Fill job without tokens adds no segment and no rows
    pool, parent = fresh(16)
    e_ctx, g_ctx = Context(1, parent, pool, b), Context(2, parent, pool, b)
    g_ctx.allocate(1)
    meta = IterationMetadata([Fill(e_ctx, []), Generate(g_ctx)], b)
    assert meta.num_rows == 1 and len(meta.seg_kv_lens) == 0 and meta.seg_row_offsets.tolist() == [0]


def test_strided_block_lookup_matches_slicing_the_whole_context():
    """The O(blocks) table lookup against the per-token list of the whole context, over random
    context chains, starts, stops and a context type without the per-token attributes."""
    from parrotserve_b200.attn_func import _last_slots, _strided_blocks
    from tests.fake_parrot import Context, Pool

    rng = np.random.default_rng(8)
    for case in range(40):
        b = int(rng.choice([4, 16]))
        pool = Pool()
        ctx = None
        for depth in range(int(rng.integers(1, 5))):
            ctx = Context(depth, ctx, pool, b)
            ctx.allocate(int(rng.integers(0, 70)))
        ctx.allocate(1)
        whole = ctx.get_context_block_ids()
        for _ in range(10):
            start = int(rng.integers(0, len(whole) + 3))
            stop = None if rng.random() < 0.5 else int(rng.integers(0, len(whole) + 3))
            assert _strided_blocks(ctx, start, stop, b) == whole[start:stop:b], (case, start, stop)
        n = int(rng.integers(1, len(ctx.token_kv_slot_ids) + 1))
        assert _last_slots(ctx, n) == ctx.get_context_slot_ids()[-n:]

    class Opaque:   # only the methods of the context interface
        parent_context = None

        def get_context_block_ids(self):
            return list(range(50))

        def get_context_slot_ids(self):
            return list(range(100, 150))

    assert _strided_blocks(Opaque(), 16, None, 16) == [16, 32, 48]
    assert _last_slots(Opaque(), 2) == [148, 149]


def test_install_registers_the_attention_function(monkeypatch):
    """install() against stand-ins shaped like the registry it patches (a name list and a lookup
    method hung on BuiltinConfig, parrot/engine/builtin/attn_func.py:704-737; the name -> layout map,
    mem_layout.py:18-22; the per-layer cache getters, mem.py:179-188)."""
    import enum
    import types

    from parrotserve_b200 import attn_func as af

    class MemLayout(enum.Enum):
        NORMAL = 1
        VLLM = 3

    class BuiltinConfig:
        def _get_attn_func(self, name):
            if name == "xformers_with_buffer":
                return "reference class"
            raise ValueError(name)

    mods = {
        "parrot": types.ModuleType("parrot"),
        "parrot.engine": types.ModuleType("parrot.engine"),
        "parrot.engine.builtin": types.ModuleType("parrot.engine.builtin"),
        "parrot.engine.builtin.attn_func": types.ModuleType("parrot.engine.builtin.attn_func"),
        "parrot.engine.builtin.mem": types.ModuleType("parrot.engine.builtin.mem"),
        "parrot.engine.builtin.mem_layout": types.ModuleType("parrot.engine.builtin.mem_layout"),
        "parrot.engine.config": types.ModuleType("parrot.engine.config"),
    }
    for name, m in mods.items():
        if name.count(".") < 3:
            m.__path__ = []
        parent, _, leaf = name.rpartition(".")
        if parent:
            setattr(mods[parent], leaf, m)
        monkeypatch.setitem(sys.modules, name, m)
    mods["parrot.engine.builtin.attn_func"].ATTN_FUNCS = ["xformers_with_buffer"]
    mods["parrot.engine.builtin.mem_layout"].MemLayout = MemLayout
    mods["parrot.engine.builtin.mem_layout"].ATTN_FUNC_LAYOUT_MAP = {"xformers_with_buffer": MemLayout.NORMAL}
    mods["parrot.engine.builtin.mem"].get_k_cache = lambda layer: ("k", layer)
    mods["parrot.engine.builtin.mem"].get_v_cache = lambda layer: ("v", layer)
    mods["parrot.engine.config"].BuiltinConfig = BuiltinConfig
    monkeypatch.setattr(af.B200SharedPromptsGenerate, "kv_cache_getter", None)

    name = af.install()
    assert name == af.ATTN_FUNC_NAME and af.install() == name        # a second call changes nothing
    assert mods["parrot.engine.builtin.attn_func"].ATTN_FUNCS.count(name) == 1
    assert mods["parrot.engine.builtin.mem_layout"].ATTN_FUNC_LAYOUT_MAP[name] is MemLayout.VLLM
    cfg = BuiltinConfig()
    assert cfg._get_attn_func(name) is af.B200SharedPromptsGenerate
    assert cfg._get_attn_func("xformers_with_buffer") == "reference class"  # the reference's names still resolve
    with pytest.raises(ValueError):
        cfg._get_attn_func("nonsense")
    assert af.B200SharedPromptsGenerate.kv_cache_getter(3) == (("k", 3), ("v", 3))


def test_sampler_install_swaps_the_forward_of_the_reference_class(monkeypatch):
    import types

    from parrotserve_b200 import sampler as sm

    class RefSampler(torch.nn.Module):   # shaped like parrot/engine/builtin/models/sampler.py:13-17
        def __init__(self, config, embd_weight):
            super().__init__()
            self.embd_weight, self.vocab_size = embd_weight, config.vocab_size

        def forward(self, hidden_states, sampling_config):
            raise AssertionError("the reference forward must not run after install()")

    names = ["parrot", "parrot.engine", "parrot.engine.builtin", "parrot.engine.builtin.models",
             "parrot.engine.builtin.models.sampler"]
    mods = {n: types.ModuleType(n) for n in names}
    for n, m in mods.items():
        m.__path__ = []
        parent, _, leaf = n.rpartition(".")
        if parent:
            setattr(mods[parent], leaf, m)
        monkeypatch.setitem(sys.modules, n, m)
    mods[names[-1]].Sampler = RefSampler
    sm.install()
    s = RefSampler(types.SimpleNamespace(vocab_size=11), torch.zeros((11, 4)))
    out = s(torch.zeros((0, 4)), [])          # the empty batch needs no GPU
    assert out.dtype == torch.int64 and out.shape == (0,)
    with pytest.raises(AssertionError):
        s(torch.zeros((2, 4)), [object()])    # one sampling config per row, as in the reference


def test_head_and_group_partitions():
    from parrotserve_b200 import shard

    for heads, world in ((32, 8), (40, 8), (64, 8), (5, 2), (3, 4)):
        got = [h for r in range(world) for h in shard.head_range(heads, world, r)]
        assert got == list(range(heads))
        sizes = [len(shard.head_range(heads, world, r)) for r in range(world)]
        assert max(sizes) - min(sizes) <= 1


def test_compact_sample_describes_the_same_attention():
    """The sub-problem the multi-GPU verification cuts out on the device (sampled rows, one head, only
    the blocks those rows attend, renumbered) gives the oracle the same rows as the whole problem."""
    from oracle import attention_oracle as orc
    from parrotserve_b200 import shard
    from parrotserve_b200.workloads import make_workload

    for cfg, shrink in ((2, 16), (3, 32), (5, 128)):
        wl = make_workload(cfg, shrink=shrink, num_heads=3)
        t = wl.materialize("cpu")
        rows = shard.sample_rows_every_group(wl, 9, seed=cfg)
        offs = wl.group_row_offsets
        assert all(int(offs[g]) in rows for g in range(wl.num_groups) if offs[g + 1] > offs[g])
        q1, kc1, vc1, meta = shard.compact_sample(wl, t, rows, local_head=1)
        assert q1.shape[:2] == (len(rows), 1) and kc1.shape[0] == vc1.shape[0] < wl.num_blocks
        small = orc.gold_grouped_attention(q1.float(), kc1.float(), vc1.float(), meta["group_row_offsets"], meta["group_prefix_lens"],
                                           meta["group_tables"], meta["suffix_lens"], meta["suffix_tables"])
        whole = orc.gold_grouped_attention(t["query"].float(), t["key_cache"].float(), t["value_cache"].float(),
                                           wl.group_row_offsets.tolist(), wl.group_prefix_lens.tolist(), wl.group_tables.tolist(),
                                           wl.suffix_lens.tolist(), wl.suffix_tables.tolist(), rows=rows, heads=[1])
        assert torch.equal(small, whole)


_GLOO_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO_ROOT"])
from parrotserve_b200 import shard
from parrotserve_b200.workloads import make_workload
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
wl = make_workload(2, shrink=8)
heads = shard.head_range(wl.num_heads, world, rank)
t = wl.materialize("cpu", heads=heads)
assert t["key_cache"].shape[1] == len(heads)
# a rank's shard holds exactly the slices a single process would hold for those heads
full = wl.materialize("cpu", heads=range(wl.num_heads)) if rank == 0 else None
if rank == 0:
    assert torch.equal(full["key_cache"][:, heads.start:heads.stop], t["key_cache"])
    assert torch.equal(full["query"][:, heads.start:heads.stop], t["query"])
ms = shard.max_over_ranks([10.0 + rank, 5.0 - rank], torch.device("cpu"))
assert ms == [10.0 + world - 1, 5.0], ms
# the harness's one collective: outputs joined along the head dimension, in rank order
mine = torch.full((3, len(heads), 2), float(rank))
joined = shard.gather_heads(mine)
assert joined.shape == (3, wl.num_heads, 2) and all(float(joined[0, h, 0]) == h // len(heads) for h in range(wl.num_heads))
count = torch.tensor([len(heads)]); dist.all_reduce(count)
assert int(count) == wl.num_heads
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_two_rank_head_sharding_under_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER)
    env = dict(os.environ, REPO_ROOT=str(ROOT), MASTER_ADDR="127.0.0.1", MASTER_PORT="29653", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
