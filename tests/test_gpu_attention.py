"""GPU parity: the CUDA attention path (through the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

import parrotserve_b200 as pb
from parrotserve_b200.workloads import make_workload
from tests.helpers import assert_close_to_oracle, oracle_for_workload, sample_rows
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_grouped(wl, t, **tuning):
    call = pb.AttentionCall(
        num_rows=wl.num_rows, num_heads=t["query"].shape[1], head_size=wl.head_size, block_size=wl.block_size,
        dtype=wl.dtype, device=t["query"].device, suffix_lens=t["suffix_lens"], suffix_tables=t["suffix_tables"],
        group_row_offsets=t["group_row_offsets"], group_prefix_lens=t["group_prefix_lens"],
        group_tables=t["group_tables"], seg_row_offsets=t.get("seg_row_offsets"), seg_kv_lens=t.get("seg_kv_lens"),
        seg_tables=t.get("seg_tables"), **tuning,
    )
    out = torch.empty_like(t["query"])
    call.run(t["query"], out, t["key_cache"], t["value_cache"])
    assert call.status() == 0
    return out


@pytest.mark.parametrize("cfg,shrink", [(1, 1), (2, 8), (2, 1), (3, 16), (4, 8), (5, 64)])
@pytest.mark.parametrize("dense_min_rows,row_tile", [(0, 128), (0, 256), (1 << 30, 0)])
def test_configs_match_oracle(cfg, shrink, dense_min_rows, row_tile):
    heads = {1: 4, 2: 32 if shrink == 1 else 4, 3: 5, 4: 3, 5: 2}[cfg]
    wl = make_workload(cfg, shrink=shrink, num_heads=heads)
    t = wl.materialize(DEV)
    out = run_grouped(wl, t, dense_min_rows=dense_min_rows, dense_row_tile=row_tile)
    rows = sample_rows(wl, 24, seed=cfg)
    if wl.seg_kv_lens is not None:  # first, last and tile-boundary tokens of prefill requests
        offs = wl.seg_row_offsets.tolist()
        for a, b in zip(offs[:3], offs[1:4]):
            rows += [a, b - 1] + [r for r in (a + 127, a + 128, a + 129) if r < b]
        rows = sorted(set(rows))
    hs = list(range(min(heads, 4)))
    if cfg in (1, 2) and shrink == 1:  # the configurations the full oracle is cheap for: every row, every head
        rows, hs = list(range(wl.num_rows)), list(range(heads))
    ref = oracle_for_workload(wl, t, rows=rows, heads=hs)
    route = f"dense, row tile {row_tile}" if dense_min_rows == 0 else "single-query"
    assert_close_to_oracle(out[rows][:, hs], ref, wl.dtype, f"cfg{cfg}/shrink{shrink}/{route} prefix route")


@pytest.mark.parametrize("cfg,heads,row_tile", [(3, None, 0), (4, None, 128), (4, None, 256), (5, 8, 0)])
def test_full_size_configs_on_a_sample(cfg, heads, row_tile):
    """Configs 3, 4 and the per-GPU shard of config 5 (8 of its 64 heads) at FULL size; the oracle
    is evaluated on a seeded sample of (row, head) pairs that contains every group's first row, the
    shortest and longest private context and, for prefill requests, first / last / tile-boundary rows."""
    wl = make_workload(cfg, num_heads=heads)
    t = wl.materialize(DEV)
    out = run_grouped(wl, t, dense_row_tile=row_tile)
    rows = sample_rows(wl, 40, seed=100 + cfg)
    if wl.seg_kv_lens is not None:
        offs = wl.seg_row_offsets.tolist()
        for a, b in zip(offs[:-1], offs[1:]):
            rows += [a, b - 1] + [r for r in (a + 127, a + 128, a + 255, a + 256) if r < b]
        rows = sorted(set(rows))
    h = t["query"].shape[1]
    hs = sorted({0, 1, h // 2, h - 1})
    ref = oracle_for_workload(wl, t, rows=rows, heads=hs)
    assert_close_to_oracle(out[rows][:, hs], ref, wl.dtype, f"cfg{cfg} full size")


def _mini(dtype, num_heads, prefix_len, suffix_lens, nb=64, seed=0, groups=None, d=128, b=16):
    """Hand-built problem on DEV: one prefix group (or `groups` = [(prefix_len, n_rows), ...])."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = 16 // torch.empty((), dtype=dtype).element_size()
    kc = torch.randn((nb, num_heads, d // x, b, x), generator=g, device=DEV).to(dtype)
    vc = torch.randn((nb, num_heads, d, b), generator=g, device=DEV).to(dtype)
    groups = groups if groups is not None else [(prefix_len, len(suffix_lens))]
    rng = np.random.default_rng(seed)
    perm = rng.permutation(nb).tolist()
    gt, offs = [], [0]
    for pl, n in groups:
        k = (pl + b - 1) // b
        gt.append([perm.pop() for _ in range(k)])
        offs.append(offs[-1] + n)
    st = []
    for s in suffix_lens:
        k = (s + b - 1) // b
        st.append([perm.pop() for _ in range(k)])
    width = max([len(r) for r in st] + [1])
    gwidth = max([len(r) for r in gt] + [1])
    pad = lambda rows, w: [r + [0] * (w - len(r)) for r in rows]
    q = torch.randn((len(suffix_lens), num_heads, d), generator=g, device=DEV).to(dtype)
    meta = dict(offs=offs, plens=[pl for pl, _ in groups], gt=pad(gt, gwidth), sl=list(suffix_lens), st=pad(st, width))
    return q, kc, vc, meta


def _run_mini(q, kc, vc, meta, **tuning):
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    return pb.flash_paged_attention_grouped(q, kc, vc, None, i32(meta["plens"]), i32(meta["gt"]), i32(meta["offs"]),
                                            i32(meta["sl"]), i32(meta["st"]), **tuning)


def _oracle_mini(q, kc, vc, meta):
    return orc.gold_grouped_attention(q.float().cpu(), kc.float().cpu(), vc.float().cpu(), meta["offs"], meta["plens"],
                                      meta["gt"], meta["sl"], meta["st"])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("dense_min_rows,row_tile", [(0, 128), (0, 256), (1 << 30, 0)])
def test_ragged_edges(dtype, dense_min_rows, row_tile):
    # suffix lengths around the block size, a zero-length suffix, a prefix that is not a block multiple
    sl = [0, 1, 15, 16, 17, 31, 32, 33, 100, 7, 64, 65]
    q, kc, vc, meta = _mini(dtype, 3, 40, sl, nb=96, seed=1)
    out = _run_mini(q, kc, vc, meta, dense_min_rows=dense_min_rows, dense_row_tile=row_tile)
    assert_close_to_oracle(out, _oracle_mini(q, kc, vc, meta), dtype, "ragged edges")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("dense_min_rows", [0, 1 << 30])
def test_groups_empty_single_and_no_prefix(dtype, dense_min_rows):
    # group 0: empty (no rows); group 1: one row; group 2: zero-length prefix; group 3: many rows
    groups = [(64, 0), (48, 1), (0, 3), (200, 9)]
    sl = [5, 1, 16, 40, 3, 0, 17, 33, 2, 90, 16, 8, 1]
    q, kc, vc, meta = _mini(dtype, 2, 0, sl, nb=128, seed=2, groups=groups)
    out = _run_mini(q, kc, vc, meta, dense_min_rows=dense_min_rows)
    assert_close_to_oracle(out, _oracle_mini(q, kc, vc, meta), dtype, "group edge cases")


def test_row_with_nothing_to_attend_is_zero():
    q, kc, vc, meta = _mini(torch.float16, 2, 0, [0, 4], nb=16, seed=3)
    out = _run_mini(q, kc, vc, meta)
    assert torch.count_nonzero(out[0]) == 0
    assert_close_to_oracle(out, _oracle_mini(q, kc, vc, meta), torch.float16, "empty row")


def test_reference_signature_single_group_and_padded_tables():
    # flash_paged_attention(query, key_cache, value_cache, head_mapping, flash_context_len,
    #                       flash_block_table, paged_context_lens, paged_block_tables)
    sl = [6, 18, 34]
    q, kc, vc, meta = _mini(torch.float16, 4, 64, sl, nb=32, seed=4)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    hm = torch.arange(4, dtype=torch.int32, device=DEV)
    out = pb.flash_paged_attention(q, kc, vc, hm, 64, i32(meta["gt"][0]), i32(sl), i32(meta["st"]))
    out2 = pb.paged_flash_attention(q, kc, vc, hm, 64, i32(meta["gt"][0]), i32(sl), i32(meta["st"]))
    ref = _oracle_mini(q, kc, vc, meta)
    assert_close_to_oracle(out, ref, torch.float16, "flash_paged_attention")
    assert torch.equal(out, out2)
    # single job: the whole context is shared, the private table is [1, 0] wide
    out1 = pb.flash_paged_attention(q[:1], kc, vc, hm, 64, i32(meta["gt"][0]), i32([0]),
                                    torch.zeros((1, 0), dtype=torch.int32, device=DEV))
    m1 = dict(meta, offs=[0, 1], sl=[0], st=[[0]])
    assert_close_to_oracle(out1, _oracle_mini(q[:1], kc, vc, m1), torch.float16, "single job")


def test_unshared_paged_attention_and_strided_query():
    sl = [1, 16, 100, 37]
    q, kc, vc, meta = _mini(torch.float16, 4, 0, sl, nb=32, seed=5, groups=[])
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    hm = torch.arange(4, dtype=torch.int32, device=DEV)
    # q as a strided view of a fused qkv projection output (models/llama.py:111-112)
    qkv = torch.randn((len(sl), 3 * 4 * 128), device=DEV).half()
    qv = qkv.chunk(3, dim=-1)[0].view(-1, 4, 128)
    out = pb.vllm_paged_attention(qv, kc, vc, hm, i32(sl), i32(meta["st"]))
    ref = orc.gold_grouped_attention(qv.float().cpu(), kc.float().cpu(), vc.float().cpu(), None, None, None, sl, meta["st"])
    assert_close_to_oracle(out, ref, torch.float16, "vllm_paged_attention")


def test_head_mapping_gqa():
    # 4 query heads onto 2 kv heads
    sl = [20, 3]
    q, kc, vc, meta = _mini(torch.float16, 2, 32, sl, nb=16, seed=6)
    g = torch.Generator(device=DEV).manual_seed(7)
    q4 = torch.randn((2, 4, 128), generator=g, device=DEV).half()
    hm = torch.tensor([0, 0, 1, 1], dtype=torch.int32, device=DEV)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    out = pb.flash_paged_attention(q4, kc, vc, hm, 32, i32(meta["gt"][0]), i32(sl), i32(meta["st"]))
    ref = orc.gold_grouped_attention(q4.float().cpu(), kc.float().cpu(), vc.float().cpu(), meta["offs"], meta["plens"],
                                     meta["gt"], sl, meta["st"], head_mapping=[0, 0, 1, 1])
    assert_close_to_oracle(out, ref, torch.float16, "gqa")


def test_prev_post_native_entry_points():
    """prev writes normalised out + base-2 stats; post merges a second context into it in place:
    prev(A) then post(B) == attention over A ++ B (csrc/attention.cpp:19-47)."""
    from parrotserve_b200 import attention_ops as aops

    sl_a, sl_b = [30, 16, 5], [9, 40, 1]
    q, kc, vc, ma = _mini(torch.float16, 3, 0, sl_a, nb=48, seed=8, groups=[])
    rng = np.random.default_rng(9)
    used = {b for r in ma["st"] for b in r}
    free = [b for b in rng.permutation(48).tolist() if b not in used]
    stb = [[free.pop() for _ in range((s + 15) // 16)] for s in sl_b]
    w = max(len(r) for r in stb)
    stb = [r + [0] * (w - len(r)) for r in stb]
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    hm = torch.arange(3, dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    qk_max = torch.zeros((3, 3), dtype=torch.float32, device=DEV)
    exp_sum = torch.zeros((3, 3), dtype=torch.float32, device=DEV)
    scale = 128 ** -0.5
    aops.single_query_cached_kv_prev_attention(out, q, kc, vc, hm, scale, i32(ma["st"]), i32(sl_a), qk_max, exp_sum,
                                               16, len(ma["st"][0]) * 16, None)
    ref_a = orc.gold_grouped_attention(q.float().cpu(), kc.float().cpu(), vc.float().cpu(), None, None, None, sl_a, ma["st"])
    assert_close_to_oracle(out, ref_a, torch.float16, "prev out")
    for r in range(3):
        k, _ = orc.gather_tokens(kc.float().cpu(), vc.float().cpu(), ma["st"][r], sl_a[r], [0, 1, 2])
        m, l = orc.gold_stats(q[r].float().cpu(), k, scale)
        assert torch.allclose(qk_max[r].double().cpu(), m, atol=1e-3)
        assert torch.allclose(exp_sum[r].double().cpu(), l, rtol=2e-3)
    aops.single_query_cached_kv_post_attention(out, q, kc, vc, hm, scale, i32(stb), i32(sl_b), qk_max, exp_sum,
                                               16, w * 16, None)
    both_tabs = [ma["st"][r][: (sl_a[r] + 15) // 16] + stb[r] for r in range(3)]
    # A's last block may be ragged, so build the oracle from explicit token gathers
    kcf, vcf, qf = kc.float().cpu(), vc.float().cpu(), q.float().cpu()
    for r in range(3):
        ka, va = orc.gather_tokens(kcf, vcf, ma["st"][r], sl_a[r], [0, 1, 2])
        kb, vb = orc.gather_tokens(kcf, vcf, stb[r], sl_b[r], [0, 1, 2])
        ref = orc.gold_row_attention(qf[r], torch.cat([ka, kb]), torch.cat([va, vb]), scale)
        # out passed through an fp16 round trip between the two calls
        assert (out[r].double().cpu() - ref).abs().max().item() < 4e-3
    # plain 13-argument form; block_lens / block_nums are ignored
    out_p = torch.empty_like(q)
    aops.single_query_cached_kv_attention(out_p, q, kc, vc, hm, scale, i32(ma["st"]), None, None, i32(sl_a), 16,
                                          len(ma["st"][0]) * 16, None)
    assert_close_to_oracle(out_p, ref_a, torch.float16, "plain")
    # post with zeroed statistics (no earlier partial) must not produce NaN
    out_z = torch.full_like(q, float("nan"))
    z = torch.zeros((3, 3), dtype=torch.float32, device=DEV)
    aops.single_query_cached_kv_post_attention(out_z, q, kc, vc, hm, scale, i32(ma["st"]), i32(sl_a), z, z.clone(),
                                               16, len(ma["st"][0]) * 16, None)
    assert_close_to_oracle(out_z, ref_a, torch.float16, "post without prev")


def test_rejects_bad_arguments():
    q, kc, vc, meta = _mini(torch.float16, 2, 16, [4], nb=8, seed=10)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError):  # head size 72 is outside the compiled set (64, 80, 96, 112, 128, 256)
        pb.vllm_paged_attention(torch.zeros((1, 2, 72), dtype=torch.float16, device=DEV),
                                torch.zeros((8, 2, 9, 16, 8), dtype=torch.float16, device=DEV),
                                torch.zeros((8, 2, 72, 16), dtype=torch.float16, device=DEV), None, i32([4]), i32([[0]]))
    with pytest.raises(RuntimeError):  # dtype mismatch
        pb.vllm_paged_attention(q.float(), kc, vc, None, i32([4]), i32([[0]]))
    with pytest.raises(RuntimeError):  # CPU tensors: there is no CPU path
        pb.vllm_paged_attention(q.cpu(), kc.cpu(), vc.cpu(), None, torch.tensor([4], dtype=torch.int32),
                                torch.tensor([[0]], dtype=torch.int32))
    with pytest.raises(RuntimeError):  # rows per tensor-core work item: 0 (default), 128 or 256
        pb.AttentionCall(num_rows=1, num_heads=2, head_size=128, block_size=16, dtype=torch.float16, device=q.device,
                         suffix_lens=i32([4]), suffix_tables=i32([[0]]), dense_row_tile=64).run(q, torch.empty_like(q), kc, vc)
    # an out-of-range block id is reported through the status word, not by a fault
    call = pb.AttentionCall(num_rows=1, num_heads=2, head_size=128, block_size=16, dtype=torch.float16,
                            device=q.device, suffix_lens=i32([4]), suffix_tables=i32([[9999]]))
    out = torch.empty_like(q)
    call.run(q, out, kc, vc)
    assert call.status() == 2
    assert torch.isnan(out).all()  # a call that recorded a fault hands out NaN, never plausible numbers


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("d,row_tile", [(128, 128), (128, 256), (80, 0)])
def test_causal_segments_with_cached_context(dtype, d, row_tile):
    """Prefill requests with earlier private tokens: segment i sees kv - n + i + 1 of its tokens
    after the shared prefix. fp32 and head sizes other than 128 have no tensor-core path and take
    the single-query route."""
    b, h, nb = 16, 2, 160
    g = torch.Generator(device=DEV).manual_seed(21)
    x = 16 // torch.empty((), dtype=dtype).element_size()
    kc = torch.randn((nb, h, d // x, b, x), generator=g, device=DEV).to(dtype)
    vc = torch.randn((nb, h, d, b), generator=g, device=DEV).to(dtype)
    rng = np.random.default_rng(22)
    perm = rng.permutation(nb).tolist()
    take = lambda n: [perm.pop() for _ in range(n)]
    plen = 70
    ptab = take((plen + b - 1) // b)
    segs = [(0, 150), (37, 20), (16, 1), (300, 130)]  # (cached private tokens, new tokens)
    seg_offs, seg_kv, seg_tabs = [0], [], []
    for cached, n in segs:
        seg_offs.append(seg_offs[-1] + n)
        seg_kv.append(cached + n)
        seg_tabs.append(take((cached + n + b - 1) // b))
    dec = [5, 64, 0]
    rows = seg_offs[-1] + len(dec)
    stabs = [[] for _ in range(seg_offs[-1])] + [take((n + b - 1) // b) for n in dec]
    slens = [0] * seg_offs[-1] + dec
    pad = lambda rr: [r + [0] * (max(len(q) for q in rr) - len(r)) for r in rr]
    q = torch.randn((rows, h, d), generator=g, device=DEV).to(dtype)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    call = pb.AttentionCall(
        num_rows=rows, num_heads=h, head_size=d, block_size=b, dtype=dtype, device=q.device, suffix_lens=i32(slens),
        suffix_tables=i32(pad(stabs)), group_row_offsets=i32([0, rows]), group_prefix_lens=i32([plen]),
        group_tables=i32([ptab]), seg_row_offsets=i32(seg_offs), seg_kv_lens=i32(seg_kv), seg_tables=i32(pad(seg_tabs)),
        dense_row_tile=row_tile)
    out = torch.empty_like(q)
    call.run(q, out, kc, vc)
    assert call.status() == 0
    ref = orc.gold_grouped_attention(q.float().cpu(), kc.float().cpu(), vc.float().cpu(), [0, rows], [plen], [ptab], slens,
                                     pad(stabs), seg_row_offsets=seg_offs, seg_kv_lens=seg_kv, seg_tables=pad(seg_tabs))
    assert_close_to_oracle(out, ref, dtype, "causal segments")


@pytest.mark.parametrize("row_tile", [128, 256])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_causal_segments_joined_straddling_and_outside_groups(dtype, row_tile):
    """The planner's cases around prefill requests and prefix groups: requests inside a dense group
    (planned together with the prefix, with plain group rows before them), back to back with cached
    context, a request that straddles two groups, a request inside a group too small for the
    tensor-core kernel, a request whose rows belong to no group, and decode rows after all of them."""
    b, d, h, nb = 16, 128, 2, 500
    g = torch.Generator(device=DEV).manual_seed(31)
    x = 16 // torch.empty((), dtype=dtype).element_size()
    kc = torch.randn((nb, h, d // x, b, x), generator=g, device=DEV).to(dtype)
    vc = torch.randn((nb, h, d, b), generator=g, device=DEV).to(dtype)
    rng = np.random.default_rng(32)
    perm = rng.permutation(nb).tolist()
    blocks = lambda n: [perm.pop() for _ in range((n + b - 1) // b)]
    rows = 400
    group_offs, plens = [0, 320, 360, 363], [200, 72, 48]  # rows 363.. are in no group
    ptabs = [blocks(p) for p in plens]
    # consecutive segments from row 10 on: (new tokens, cached private tokens)
    segs = [(140, 0), (20, 33), (130, 5), (60, 9), (3, 7), (10, 0)]  # 4th straddles groups 0/1, 5th in the 3-row group
    seg_offs, seg_kv, seg_tabs = [10], [], []
    for n, cached in segs:
        seg_offs.append(seg_offs[-1] + n)
        seg_kv.append(cached + n)
        seg_tabs.append(blocks(cached + n))
    assert seg_offs[-1] == 373
    slens = [0] * rows
    for r in list(range(0, 10)) + list(range(373, rows)):  # decode rows before and after the prefill rows
        slens[r] = int(rng.integers(0, 70))
    stabs = [blocks(n) for n in slens]
    pad = lambda rr: [r + [0] * (max(len(q) for q in rr) - len(r)) for r in rr]
    q = torch.randn((rows, h, d), generator=g, device=DEV).to(dtype)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    call = pb.AttentionCall(
        num_rows=rows, num_heads=h, head_size=d, block_size=b, dtype=dtype, device=q.device, suffix_lens=i32(slens),
        suffix_tables=i32(pad(stabs)), group_row_offsets=i32(group_offs), group_prefix_lens=i32(plens),
        group_tables=i32(pad(ptabs)), seg_row_offsets=i32(seg_offs), seg_kv_lens=i32(seg_kv), seg_tables=i32(pad(seg_tabs)),
        dense_row_tile=row_tile)
    out = torch.empty_like(q)
    call.run(q, out, kc, vc)
    assert call.status() == 0
    ref = orc.gold_grouped_attention(q.float().cpu(), kc.float().cpu(), vc.float().cpu(), group_offs, plens, pad(ptabs), slens,
                                     pad(stabs), seg_row_offsets=seg_offs, seg_kv_lens=seg_kv, seg_tables=pad(seg_tabs))
    assert_close_to_oracle(out, ref, dtype, "segments joined / straddling / outside groups")
    # with statistics requested no row may be finished by the dense kernel alone: every row goes
    # through the merge, which is where (max, sum) are produced
    from parrotserve_b200 import _lib
    qk_max = torch.zeros((rows, h), dtype=torch.float32, device=DEV)
    exp_sum = torch.zeros((rows, h), dtype=torch.float32, device=DEV)
    out_s = torch.empty_like(q)
    call.run(q, out_s, kc, vc, qk_max=qk_max, exp_sum=exp_sum, stats_mode=_lib.PB_STATS_SAVE)
    assert call.status() == 0
    assert_close_to_oracle(out_s, ref, dtype, "same problem with statistics saved")
    assert bool((exp_sum[10:373] > 0).all()) and bool(torch.isfinite(qk_max[10:373]).all())  # every prefill row sees a token
    # the same problem with the tensor-core route closed for the groups (dense_min_rows above every group):
    # prefixes through the single-query kernel, segments on their own
    call2 = pb.AttentionCall(
        num_rows=rows, num_heads=h, head_size=d, block_size=b, dtype=dtype, device=q.device, suffix_lens=i32(slens),
        suffix_tables=i32(pad(stabs)), group_row_offsets=i32(group_offs), group_prefix_lens=i32(plens),
        group_tables=i32(pad(ptabs)), seg_row_offsets=i32(seg_offs), seg_kv_lens=i32(seg_kv), seg_tables=i32(pad(seg_tabs)),
        dense_min_rows=100000, dense_row_tile=row_tile)
    out2 = torch.empty_like(q)
    call2.run(q, out2, kc, vc)
    assert call2.status() == 0
    assert_close_to_oracle(out2, ref, dtype, "segments with single-query prefixes")


def test_two_planned_calls_keep_their_own_work_lists():
    """Two planned calls on one device, run alternately: each owns its workspace, so the plan of one
    never disturbs the work lists of the other."""
    dtype = torch.float16
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    problems, calls, outs = [], [], []
    for seed, (plen, sl) in enumerate([(200, [5, 70, 16, 33, 1, 90, 8, 64]), (48, [100, 3, 17])]):
        q, kc, vc, meta = _mini(dtype, 2, plen, sl, nb=96, seed=40 + seed)
        call = pb.AttentionCall(
            num_rows=len(sl), num_heads=2, head_size=128, block_size=16, dtype=dtype, device=q.device,
            suffix_lens=i32(meta["sl"]), suffix_tables=i32(meta["st"]), group_row_offsets=i32(meta["offs"]),
            group_prefix_lens=i32(meta["plens"]), group_tables=i32(meta["gt"]))
        out = torch.empty_like(q)
        call.plan(q, out, kc, vc)
        problems.append((q, kc, vc, meta))
        calls.append(call)
        outs.append(out)
    assert calls[0].workspace.data_ptr() != calls[1].workspace.data_ptr()
    for k in (0, 1, 0, 1):
        q, kc, vc, meta = problems[k]
        outs[k].zero_()
        calls[k].run(q, outs[k], kc, vc)
        assert calls[k].status() == 0
        assert_close_to_oracle(outs[k], _oracle_mini(q, kc, vc, meta), dtype, f"planned call {k}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("d", [64, 80, 96, 112, 256])
def test_other_head_sizes(dtype, d):
    """The other head sizes of the reference's paged-attention kernels (64, 80, 96, 112, 256;
    csrc/attention/attention_kernels.cu:457-478): prefixes and suffixes both go through the single-query
    kernel, grouped and plain."""
    groups = [(100, 6), (48, 1), (0, 2)]
    sl = [5, 70, 16, 33, 1, 90, 8, 64, 17]
    q, kc, vc, meta = _mini(dtype, 3, 0, sl, nb=96, seed=50, groups=groups, d=d)
    out = _run_mini(q, kc, vc, meta)
    assert_close_to_oracle(out, _oracle_mini(q, kc, vc, meta), dtype, f"head size {d}, grouped")
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    plain = pb.vllm_paged_attention(q, kc, vc, None, i32(meta["sl"]), i32(meta["st"]))
    ref = orc.gold_grouped_attention(q.float().cpu(), kc.float().cpu(), vc.float().cpu(), None, None, None, meta["sl"], meta["st"])
    assert_close_to_oracle(plain, ref, dtype, f"head size {d}, plain")


@pytest.mark.parametrize("seed", list(range(24)))
def test_random_problems_match_oracle(seed, outer=None):
    """Seeded random problems over everything the planner distinguishes: up to four prefix groups
    (some empty, some below the tensor-core gate, prefix lengths off the block and tile sizes),
    prefill requests of random lengths with random cached context laid first in the batch (so they
    fall inside, across and outside groups as the dice decide), decode rows with random suffixes,
    fp16 / bf16, 1-3 heads; from seed 12 on also up to three outer prefix groups (a second,
    independent partition of the rows)."""
    rng = np.random.default_rng(1000 + seed)
    dtype = [torch.float16, torch.bfloat16][seed % 2]
    b, d, h = 16, 128, int(rng.integers(1, 4))
    n_seg = int(rng.integers(0, 4))
    segs = [(int(rng.integers(1, 200)), int(rng.integers(0, 40))) for _ in range(n_seg)]  # (new tokens, cached)
    n_dec = int(rng.integers(1, 40))
    seg_rows = sum(n for n, _ in segs)
    rows = seg_rows + n_dec
    n_groups = int(rng.integers(0, 5))
    cuts = sorted(rng.integers(0, rows + 1, size=max(n_groups - 1, 0)).tolist())
    covered = int(rng.integers(rows // 2, rows + 1)) if n_groups else 0  # rows beyond it are in no group
    group_offs = [0] + [min(c, covered) for c in cuts] + [covered] if n_groups else [0]
    plens = [int(rng.choice([0, 7, 16, 100, 128, 200, 300])) for _ in range(n_groups)]
    nb = 64 + sum((p + b - 1) // b for p in plens) + sum((n + c + b - 1) // b for n, c in segs) + n_dec * 6
    with_outer = seed >= 12 if outer is None else outer
    nb += 3 * 17 if with_outer else 0   # room for three outer prefixes
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = 16 // torch.empty((), dtype=dtype).element_size()
    kc = torch.randn((nb, h, d // x, b, x), generator=g, device=DEV).to(dtype)
    vc = torch.randn((nb, h, d, b), generator=g, device=DEV).to(dtype)
    perm = rng.permutation(nb).tolist()
    blocks = lambda n: [perm.pop() for _ in range((n + b - 1) // b)]
    ptabs = [blocks(p) for p in plens]
    seg_offs, seg_kv, seg_tabs = [0], [], []
    for n, cached in segs:
        seg_offs.append(seg_offs[-1] + n)
        seg_kv.append(n + cached)
        seg_tabs.append(blocks(n + cached))
    slens = [0] * seg_rows + [int(rng.integers(0, 90)) for _ in range(n_dec)]
    stabs = [blocks(n) for n in slens]
    n_outer = int(rng.integers(1, 4)) if with_outer else 0
    outer_offs, olens, otabs = None, None, None
    if n_outer:
        ocuts = sorted(rng.integers(0, rows + 1, size=n_outer - 1).tolist())
        ocovered = int(rng.integers(rows // 2, rows + 1))
        outer_offs = [0] + [min(c, ocovered) for c in ocuts] + [ocovered]
        olens = [int(rng.choice([0, 5, 16, 90, 128, 260])) for _ in range(n_outer)]
        otabs = [blocks(n) for n in olens]
    pad = lambda rr: [r + [0] * (max([len(q) for q in rr] + [1]) - len(r)) for r in rr]
    q = torch.randn((rows, h, d), generator=g, device=DEV).to(dtype)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    kw = {}
    if n_groups:
        kw.update(group_row_offsets=i32(group_offs), group_prefix_lens=i32(plens), group_tables=i32(pad(ptabs)))
    if n_seg:
        kw.update(seg_row_offsets=i32(seg_offs), seg_kv_lens=i32(seg_kv), seg_tables=i32(pad(seg_tabs)))
    if n_outer:
        kw.update(outer_row_offsets=i32(outer_offs), outer_prefix_lens=i32(olens), outer_tables=i32(pad(otabs)))
    outs = {}
    for row_tile in (128, 256):  # both forms of the tensor-core kernel on every problem
        call = pb.AttentionCall(num_rows=rows, num_heads=h, head_size=d, block_size=b, dtype=dtype, device=q.device,
                                suffix_lens=i32(slens), suffix_tables=i32(pad(stabs)), dense_row_tile=row_tile, **kw)
        outs[row_tile] = torch.empty_like(q)
        call.run(q, outs[row_tile], kc, vc)
        assert call.status() == 0
    ref = orc.gold_grouped_attention(
        q.float().cpu(), kc.float().cpu(), vc.float().cpu(), group_offs if n_groups else None, plens if n_groups else None,
        pad(ptabs) if n_groups else None, slens, pad(stabs), seg_row_offsets=seg_offs if n_seg else None,
        seg_kv_lens=seg_kv if n_seg else None, seg_tables=pad(seg_tabs) if n_seg else None,
        outer_row_offsets=outer_offs, outer_prefix_lens=olens, outer_tables=pad(otabs) if n_outer else None)
    for row_tile, out in outs.items():
        assert_close_to_oracle(out, ref, dtype, f"random problem {seed}, row tile {row_tile}: groups {group_offs} {plens}, "
                                                f"segments {segs}, decodes {n_dec}, outer {outer_offs} {olens}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("dense_min_rows", [0, 1 << 30])
def test_two_level_prefix_sharing(dtype, dense_min_rows):
    """A two-level context tree: one system prompt shared by every request (outer group), three
    application prompts shared by subsets (groups), private contexts, and a prefill request inside
    one application; plus a second outer group too small for the tensor-core kernel and rows under no
    outer prefix. Every row attends outer ++ group ++ own-context tokens exactly once each."""
    b, d, h, nb = 16, 128, 2, 420
    g = torch.Generator(device=DEV).manual_seed(61)
    x = 16 // torch.empty((), dtype=dtype).element_size()
    kc = torch.randn((nb, h, d // x, b, x), generator=g, device=DEV).to(dtype)
    vc = torch.randn((nb, h, d, b), generator=g, device=DEV).to(dtype)
    rng = np.random.default_rng(62)
    perm = rng.permutation(nb).tolist()
    blocks = lambda n: [perm.pop() for _ in range((n + b - 1) // b)]
    rows = 230
    outer_offs, outer_lens = [0, 200, 203], [300, 40]      # rows 203.. have no outer prefix
    group_offs, plens = [0, 150, 190, 215], [130, 64, 20]  # group 2 straddles the end of the outer groups
    seg_offs, seg_kv = [0, 140], [140 + 25]                # one prefill request of 140 tokens (25 cached) in group 0
    otabs, ptabs, seg_tabs = [blocks(n) for n in outer_lens], [blocks(n) for n in plens], [blocks(seg_kv[0])]
    slens = [0] * 140 + [int(rng.integers(0, 80)) for _ in range(rows - 140)]
    stabs = [blocks(n) for n in slens]
    pad = lambda rr: [r + [0] * (max([len(q) for q in rr] + [1]) - len(r)) for r in rr]
    q = torch.randn((rows, h, d), generator=g, device=DEV).to(dtype)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    call = pb.AttentionCall(
        num_rows=rows, num_heads=h, head_size=d, block_size=b, dtype=dtype, device=q.device, suffix_lens=i32(slens),
        suffix_tables=i32(pad(stabs)), group_row_offsets=i32(group_offs), group_prefix_lens=i32(plens),
        group_tables=i32(pad(ptabs)), seg_row_offsets=i32(seg_offs), seg_kv_lens=i32(seg_kv), seg_tables=i32(pad(seg_tabs)),
        outer_row_offsets=i32(outer_offs), outer_prefix_lens=i32(outer_lens), outer_tables=i32(pad(otabs)),
        dense_min_rows=dense_min_rows)
    out = torch.empty_like(q)
    call.run(q, out, kc, vc)
    assert call.status() == 0
    ref = orc.gold_grouped_attention(
        q.float().cpu(), kc.float().cpu(), vc.float().cpu(), group_offs, plens, pad(ptabs), slens, pad(stabs),
        seg_row_offsets=seg_offs, seg_kv_lens=seg_kv, seg_tables=pad(seg_tabs),
        outer_row_offsets=outer_offs, outer_prefix_lens=outer_lens, outer_tables=pad(otabs))
    assert_close_to_oracle(out, ref, dtype, "two-level prefix sharing")


def _bits(x):
    return x.detach().cpu().contiguous().view(torch.int16 if x.element_size() == 2 else torch.int32).numpy()


@pytest.mark.parametrize("cfg,shrink,heads,dtype", [(2, 8, 4, None), (2, 1, 8, None), (3, 16, 5, None), (5, 64, 2, None),
                                                    (1, 1, 4, None), (4, 8, 3, None), (2, 8, 4, torch.bfloat16)])
def test_attention_call_performs_the_kv_fill(cfg, shrink, heads, dtype):
    """The attention call given the step's new tokens (key_new / value_new + slot_mapping) must leave
    the caches exactly as the fill followed by the attention leaves them, and give the attention over
    the FILLED caches: for decode batches the suffix kernel does the fill on the fly (no fill launch),
    for batches with prefill requests (config 4) the call runs the fill kernel first."""
    wl = make_workload(cfg, shrink=shrink, num_heads=heads)
    if dtype is not None:
        wl.dtype = dtype
    t = wl.materialize(DEV)
    assert len(wl.fill_slots) == wl.num_rows  # every row brings one new token, in row order
    # poison the new tokens' cache slots: a kernel that read them from the cache would show
    b = wl.block_size
    slots = t["fill_slots"]
    t["key_cache"][slots // b, :, :, slots % b, :] = 77.0
    t["value_cache"][slots // b, :, :, slots % b] = -55.0
    kr, vr = _bits(t["key_cache"]).copy(), _bits(t["value_cache"]).copy()
    orc.fill_reference(_bits(t["k_new"]), _bits(t["v_new"]), kr, vr, wl.fill_slots)
    call = pb.AttentionCall(
        num_rows=wl.num_rows, num_heads=heads, head_size=wl.head_size, block_size=b, dtype=wl.dtype, device=t["query"].device,
        suffix_lens=t["suffix_lens"], suffix_tables=t["suffix_tables"], group_row_offsets=t["group_row_offsets"],
        group_prefix_lens=t["group_prefix_lens"], group_tables=t["group_tables"], seg_row_offsets=t.get("seg_row_offsets"),
        seg_kv_lens=t.get("seg_kv_lens"), seg_tables=t.get("seg_tables"), slot_mapping=t["fill_slots"])
    out = torch.empty_like(t["query"])
    call.plan(t["query"], out, t["key_cache"], t["value_cache"])
    call.run(t["query"], out, t["key_cache"], t["value_cache"], key_new=t["k_new"], value_new=t["v_new"])
    assert call.status() == 0
    assert np.array_equal(_bits(t["key_cache"]), kr) and np.array_equal(_bits(t["value_cache"]), vr), "cache contents differ from the fill's"
    rows = sample_rows(wl, 16, seed=cfg)
    if wl.seg_kv_lens is not None:
        offs = wl.seg_row_offsets.tolist()
        rows = sorted(set(rows + [offs[0], offs[1] - 1]))
    hs = list(range(min(heads, 4)))
    ref = oracle_for_workload(wl, t, rows=rows, heads=hs)  # over the caches as they are now: filled
    assert_close_to_oracle(out[rows][:, hs], ref, wl.dtype, f"cfg{cfg}/shrink{shrink} with the fill inside the call")
    # a second layer call on the same plan (the caches already hold the tokens) gives the same result
    out2 = torch.empty_like(out)
    call.run(t["query"], out2, t["key_cache"], t["value_cache"], key_new=t["k_new"], value_new=t["v_new"])
    assert torch.equal(out, out2)


def test_new_token_that_is_not_the_end_of_its_row_is_reported():
    """Decode batch, fill inside the call: a slot that is not the last position of its row's suffix
    cannot ride along with the row's last block; the planner records it and the output is NaN."""
    wl = make_workload(2, shrink=8, num_heads=2)
    t = wl.materialize(DEV)
    slots = t["fill_slots"].clone()
    slots[3] = slots[3] - 1 if int(slots[3]) % wl.block_size else slots[3] + 1
    call = pb.AttentionCall(
        num_rows=wl.num_rows, num_heads=2, head_size=wl.head_size, block_size=wl.block_size, dtype=wl.dtype, device=t["query"].device,
        suffix_lens=t["suffix_lens"], suffix_tables=t["suffix_tables"], group_row_offsets=t["group_row_offsets"],
        group_prefix_lens=t["group_prefix_lens"], group_tables=t["group_tables"], slot_mapping=slots)
    out = torch.zeros_like(t["query"])
    call.run(t["query"], out, t["key_cache"], t["value_cache"], key_new=t["k_new"], value_new=t["v_new"])
    assert call.status() == 2 and torch.isnan(out).all()
    with pytest.raises(RuntimeError):  # new tokens without slots
        pb.AttentionCall(num_rows=wl.num_rows, num_heads=2, head_size=wl.head_size, block_size=wl.block_size, dtype=wl.dtype,
                         device=t["query"].device, suffix_lens=t["suffix_lens"], suffix_tables=t["suffix_tables"]).run(
            t["query"], out, t["key_cache"], t["value_cache"], key_new=t["k_new"], value_new=t["v_new"])
    # a C caller that builds the lists WITHOUT the slots and then asks the attention call for the fill:
    # no item carries a token, so nothing would be written; recorded as a fault instead of passing silently
    late = pb.AttentionCall(
        num_rows=wl.num_rows, num_heads=2, head_size=wl.head_size, block_size=wl.block_size, dtype=wl.dtype, device=t["query"].device,
        suffix_lens=t["suffix_lens"], suffix_tables=t["suffix_tables"], group_row_offsets=t["group_row_offsets"],
        group_prefix_lens=t["group_prefix_lens"], group_tables=t["group_tables"])
    late.plan(t["query"], out, t["key_cache"], t["value_cache"])
    late.params.slot_mapping, late.params.slot_is_i64 = t["fill_slots"].data_ptr(), 1
    late._has_slots = True
    late.run(t["query"], out, t["key_cache"], t["value_cache"], key_new=t["k_new"], value_new=t["v_new"])
    assert late.status() == 2 and torch.isnan(out).all()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("b,d", [(8, 128), (32, 128), (8, 80), (32, 80), (8, 112), (32, 64), (8, 256), (32, 256), (8, 96)])
def test_other_block_sizes(dtype, b, d):
    """Block sizes 8 and 32 (the reference dispatches 8 / 16 / 32, csrc/attention/attention_kernels.cu:504-524)
    over its head sizes: grouped shared-prefix attention, plain paged attention, prev + post, and the KV
    fill inside the call."""
    groups = [(100, 6), (3 * b, 1), (0, 2)]
    sl = [5, 70, b, 2 * b + 1, 1, 90, b - 1, 4 * b, b + 1]
    q, kc, vc, meta = _mini(dtype, 3, 0, sl, nb=128 if b == 8 else 48, seed=60 + b, groups=groups, d=d, b=b)
    out = _run_mini(q, kc, vc, meta)
    assert_close_to_oracle(out, _oracle_mini(q, kc, vc, meta), dtype, f"block size {b}, head size {d}, grouped")
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    plain = pb.vllm_paged_attention(q, kc, vc, None, i32(meta["sl"]), i32(meta["st"]))
    ref = orc.gold_grouped_attention(q.float().cpu(), kc.float().cpu(), vc.float().cpu(), None, None, None, meta["sl"], meta["st"])
    assert_close_to_oracle(plain, ref, dtype, f"block size {b}, head size {d}, plain")
    # the native entry points: prev over the suffixes, then post over the (same) tables merges two copies
    # of the same context, which leaves the attention unchanged
    n, h = q.shape[0], q.shape[1]
    o2 = torch.zeros_like(q)
    m = torch.zeros((n, h), dtype=torch.float32, device=DEV)
    l = torch.zeros((n, h), dtype=torch.float32, device=DEV)
    hm = torch.arange(h, dtype=torch.int32, device=DEV)
    pb.attention_ops.single_query_cached_kv_prev_attention(o2, q, kc, vc, hm, d ** -0.5, i32(meta["st"]), i32(meta["sl"]), m, l, b,
                                                           len(meta["st"][0]) * b, None)
    pb.attention_ops.single_query_cached_kv_post_attention(o2, q, kc, vc, hm, d ** -0.5, i32(meta["st"]), i32(meta["sl"]), m, l, b,
                                                           len(meta["st"][0]) * b, None)
    assert_close_to_oracle(o2, ref, dtype, f"block size {b}, head size {d}, prev + post")
    # KV fill inside the call: the last token of every non-empty row comes from key_new / value_new
    rows = [r for r, s_ in enumerate(meta["sl"]) if s_ > 0]
    slots = torch.full((n,), -1, dtype=torch.int64, device=DEV)
    for r in rows:
        t_ = meta["sl"][r] - 1
        slots[r] = meta["st"][r][t_ // b] * b + t_ % b
    g = torch.Generator(device=DEV).manual_seed(5)
    k_new = torch.randn((n, 3, d), generator=g, device=DEV).to(dtype)
    v_new = torch.randn((n, 3, d), generator=g, device=DEV).to(dtype)
    kr, vr = _bits(kc).copy(), _bits(vc).copy()
    orc.fill_reference(_bits(k_new), _bits(v_new), kr, vr, slots.cpu().numpy())
    call = pb.AttentionCall(num_rows=n, num_heads=3, head_size=d, block_size=b, dtype=dtype, device=q.device,
                            suffix_lens=i32(meta["sl"]), suffix_tables=i32(meta["st"]), group_row_offsets=i32(meta["offs"]),
                            group_prefix_lens=i32(meta["plens"]), group_tables=i32(meta["gt"]), slot_mapping=slots)
    out_f = torch.empty_like(q)
    call.run(q, out_f, kc, vc, key_new=k_new, value_new=v_new)
    assert call.status() == 0
    assert np.array_equal(_bits(kc), kr) and np.array_equal(_bits(vc), vr)
    assert_close_to_oracle(out_f, _oracle_mini(q, kc, vc, meta), dtype, f"block size {b}, head size {d}, fill inside the call")


def test_head_shards_equal_the_unsharded_result():
    """Head sharding (the multi-GPU partition): every rank holds the slices of its heads, generated per
    (seed, global head); the shards' outputs joined along the head dimension equal the unsharded run
    (to accumulation order: the chunking of the work lists depends on the head count) and the oracle."""
    from parrotserve_b200.shard import head_range

    wl = make_workload(2, shrink=4, num_heads=8)
    full = wl.materialize(DEV)
    out_full = run_grouped(wl, full)
    parts = []
    for rank in range(4):
        heads = head_range(8, 4, rank)
        shard_wl = make_workload(2, shrink=4, num_heads=len(heads))
        t = shard_wl.materialize(DEV, heads=heads)
        assert torch.equal(t["key_cache"], full["key_cache"][:, heads.start:heads.stop])
        assert torch.equal(t["query"], full["query"][:, heads.start:heads.stop])
        parts.append(run_grouped(shard_wl, t))
    joined = torch.cat(parts, dim=1)
    assert (joined.float() - out_full.float()).abs().max().item() <= 1e-3
    rows = sample_rows(wl, 12, seed=3)
    ref = oracle_for_workload(wl, full, rows=rows)
    assert_close_to_oracle(joined[rows], ref, wl.dtype, "head shards joined")
