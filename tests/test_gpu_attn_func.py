"""GPU parity of the drop-in attention function: a mixed Fill + Generate iteration through
`B200SharedPromptsGenerate.forward` (KV fill + grouped attention) against the CPU oracle."""
import types

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from parrotserve_b200.attn_func import B200SharedPromptsGenerate
from tests.fake_parrot import Context, Fill, Generate, IterationState, Pool
from tests.helpers import assert_close_to_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _token_rows(ctx, cache_k, cache_v, n_tokens, heads):
    slots = ctx.get_context_slot_ids()[:n_tokens]
    b = cache_v.shape[3]
    blk = torch.tensor([s // b for s in slots])
    off = torch.tensor([s % b for s in slots])
    k = cache_k[blk, :, :, off, :].reshape(len(slots), cache_k.shape[1], -1)[:, heads]
    v = cache_v[blk, :, :, off][:, heads]
    return k.double(), v.double()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("root_len", [64, 40, 0])
def test_mixed_fill_generate_iteration(dtype, root_len):
    h, d, b, nb = 4, 128, 16, 128
    g = torch.Generator(device=DEV).manual_seed(11)
    x = 8
    kc = torch.randn((nb, h, d // x, b, x), generator=g, device=DEV).to(dtype)
    vc = torch.randn((nb, h, d, b), generator=g, device=DEV).to(dtype)
    pool = Pool()
    root = None
    if root_len:
        root = Context(0, None, pool, b)
        root.allocate(root_len)
    jobs, new_counts = [], []
    for cid, (cached, n_new) in enumerate([(0, 37), (9, 20)], start=1):  # two Fill jobs
        ctx = Context(cid, root, pool, b)
        ctx.allocate(cached)
        ctx.allocate(n_new)
        jobs.append(Fill(ctx, list(range(n_new))))
        new_counts.append(n_new)
    for cid, cached in enumerate([0, 15, 16, 70], start=10):  # four Generate jobs
        ctx = Context(cid, root, pool, b)
        ctx.allocate(cached)
        ctx.allocate(1)
        jobs.append(Generate(ctx))
        new_counts.append(1)
    t_new = sum(new_counts)
    qkv = torch.randn((t_new, 3 * h * d), generator=g, device=DEV).to(dtype)
    q, k, v = (c.view(-1, h, d) for c in qkv.chunk(3, dim=-1))  # strided views, as the model produces them

    cfg = types.SimpleNamespace(block_size=b, device=DEV, dtype=dtype)
    state = IterationState()
    B200SharedPromptsGenerate.init_iteration_state(state, cfg, jobs, h, d)
    assert state.num_fill_tokens == [37, 20] and len(state.generation_sampling_config) == 4
    B200SharedPromptsGenerate.kv_cache_getter = staticmethod(lambda layer: (kc, vc))
    layer = B200SharedPromptsGenerate(0, d ** -0.5, h, d)
    out = layer(q, k, v, state).view(t_new, h, d)
    # a second layer call reuses the plan
    out2 = layer(q, k, v, state).view(t_new, h, d)
    assert torch.equal(out, out2)
    assert state.b200_call.status() == 0

    # oracle: after the fill, every query token attends its job's context up to and including itself
    kcf, vcf, qf = kc.float().cpu(), vc.float().cpu(), q.float().cpu()
    heads = list(range(h))
    ref = torch.zeros((t_new, h, d), dtype=torch.float64)
    row = 0
    for job, n in zip(jobs, new_counts):
        ctx_len = job.context.get_context_len()
        for i in range(n):
            visible = ctx_len - n + i + 1
            kk, vv = _token_rows(job.context, kcf, vcf, visible, heads)
            ref[row] = orc.gold_row_attention(qf[row], kk, vv, d ** -0.5)
            row += 1
    assert_close_to_oracle(out, ref, dtype, f"attn func root={root_len}")
    # the bottom-right causal oracle gives the same rows for a whole Fill job
    job, n = jobs[0], new_counts[0]
    kk, vv = _token_rows(job.context, kcf, vcf, job.context.get_context_len(), heads)
    causal = orc.gold_causal_with_context(qf[:n], kk, vv, d ** -0.5)
    assert (causal - ref[:n]).abs().max().item() < 1e-9


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_two_level_context_tree_iteration(dtype):
    """A two-level context tree (a root shared by all, two application prompts below it) through the
    attention function with `two_level` on: same rows as attending each job's whole context."""
    h, d, b, nb = 4, 128, 16, 160
    g = torch.Generator(device=DEV).manual_seed(23)
    x = 8
    kc = torch.randn((nb, h, d // x, b, x), generator=g, device=DEV).to(dtype)
    vc = torch.randn((nb, h, d, b), generator=g, device=DEV).to(dtype)
    pool = Pool()
    root = Context(0, None, pool, b)
    root.allocate(96)
    app1, app2 = Context(1, root, pool, b), Context(2, root, pool, b)
    app1.allocate(150)
    app2.allocate(33)
    jobs, new_counts = [], []

    def add(cid, parent, cached, n_new):
        ctx = Context(cid, parent, pool, b)
        ctx.allocate(cached)
        ctx.allocate(n_new)
        jobs.append(Fill(ctx, list(range(n_new))) if n_new > 1 else Generate(ctx))
        new_counts.append(n_new)

    add(10, app1, 7, 45)
    for cid, cached in enumerate([0, 3, 31, 64], start=11):
        add(cid, app1, cached, 1)
    add(20, app2, 0, 19)
    for cid, cached in enumerate([0, 18], start=21):
        add(cid, app2, cached, 1)
    add(30, root, 12, 1)
    # the runner's order: Fill jobs first, otherwise as submitted (builtin_runner.py:75-76)
    order = sorted(range(len(jobs)), key=lambda i: isinstance(jobs[i], Generate))
    jobs, new_counts = [jobs[i] for i in order], [new_counts[i] for i in order]
    t_new = sum(new_counts)
    qkv = torch.randn((t_new, 3 * h * d), generator=g, device=DEV).to(dtype)
    q, k, v = (c.view(-1, h, d) for c in qkv.chunk(3, dim=-1))

    cfg = types.SimpleNamespace(block_size=b, device=DEV, dtype=dtype)
    B200SharedPromptsGenerate.kv_cache_getter = staticmethod(lambda layer: (kc, vc))
    layer = B200SharedPromptsGenerate(0, d ** -0.5, h, d)
    outs = []
    try:
        for two_level in (True, False):
            B200SharedPromptsGenerate.two_level = two_level
            state = IterationState()
            B200SharedPromptsGenerate.init_iteration_state(state, cfg, jobs, h, d)
            outs.append(layer(q, k, v, state).view(t_new, h, d).clone())
            assert state.b200_call.status() == 0
    finally:
        B200SharedPromptsGenerate.two_level = False

    kcf, vcf, qf = kc.float().cpu(), vc.float().cpu(), q.float().cpu()
    heads = list(range(h))
    ref = torch.zeros((t_new, h, d), dtype=torch.float64)
    row = 0
    for job, n in zip(jobs, new_counts):
        ctx_len = job.context.get_context_len()
        for i in range(n):
            kk, vv = _token_rows(job.context, kcf, vcf, ctx_len - n + i + 1, heads)
            ref[row] = orc.gold_row_attention(qf[row], kk, vv, d ** -0.5)
            row += 1
    assert_close_to_oracle(outs[0], ref, dtype, "attn func, two levels")
    assert_close_to_oracle(outs[1], ref, dtype, "attn func, one level")


def _forward_and_check(jobs, new_counts, dtype, seed, what):
    """One iteration through init_iteration_state + forward; every query token must equal the
    attention over its job's context up to and including itself (after the fill)."""
    h, d, b, nb = 4, 128, 16, 96
    x = 16 // torch.empty((), dtype=dtype).element_size()
    g = torch.Generator(device=DEV).manual_seed(seed)
    kc = torch.randn((nb, h, d // x, b, x), generator=g, device=DEV).to(dtype)
    vc = torch.randn((nb, h, d, b), generator=g, device=DEV).to(dtype)
    t_new = sum(new_counts)
    qkv = torch.randn((t_new, 3 * h * d), generator=g, device=DEV).to(dtype)
    q, k, v = (c.view(-1, h, d) for c in qkv.chunk(3, dim=-1))
    cfg = types.SimpleNamespace(block_size=b, device=DEV, dtype=dtype)
    state = IterationState()
    B200SharedPromptsGenerate.init_iteration_state(state, cfg, jobs, h, d)
    B200SharedPromptsGenerate.kv_cache_getter = staticmethod(lambda layer: (kc, vc))
    layer = B200SharedPromptsGenerate(0, d ** -0.5, h, d)
    out = layer(q, k, v, state).view(t_new, h, d)
    assert state.b200_call.status() == 0
    kcf, vcf, qf = kc.float().cpu(), vc.float().cpu(), q.float().cpu()
    ref = torch.zeros((t_new, h, d), dtype=torch.float64)
    abs_ref = torch.zeros_like(ref)  # the same attention over |V|: bound of the weights' rounding (bf16)
    row = 0
    for job, n in zip(jobs, new_counts):
        ctx_len = job.context.get_context_len()
        for i in range(n):
            kk, vv = _token_rows(job.context, kcf, vcf, ctx_len - n + i + 1, list(range(h)))
            ref[row] = orc.gold_row_attention(qf[row], kk, vv, d ** -0.5)
            abs_ref[row] = orc.gold_row_attention(qf[row], kk, vv.abs(), d ** -0.5)
            row += 1
    assert_close_to_oracle(out, ref, dtype, what, abs_ref=abs_ref)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("parent_len,cached,n_new", [(0, 0, 20), (0, 0, 1), (40, 0, 150), (40, 13, 20), (0, 33, 7)])
def test_single_fill_job_iteration(dtype, parent_len, cached, n_new):
    """The first prefill of a request is an iteration of one Fill job: its tokens form a causal
    segment over the job's own context; only a parent context is a (non-causal) shared prefix."""
    b = 16
    pool = Pool()
    parent = None
    if parent_len:
        parent = Context(0, None, pool, b)
        parent.allocate(parent_len)
    ctx = Context(1, parent, pool, b)
    ctx.allocate(cached)
    ctx.allocate(n_new)
    _forward_and_check([Fill(ctx, list(range(n_new)))], [n_new], dtype, 31, f"lone fill {parent_len}/{cached}/{n_new}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("parent_len,cached", [(0, 19), (48, 0), (40, 30)])
def test_single_generate_job_iteration(dtype, parent_len, cached):
    b = 16
    pool = Pool()
    parent = None
    if parent_len:
        parent = Context(0, None, pool, b)
        parent.allocate(parent_len)
    ctx = Context(1, parent, pool, b)
    ctx.allocate(cached)
    ctx.allocate(1)
    _forward_and_check([Generate(ctx)], [1], dtype, 32, f"lone generate {parent_len}/{cached}")


def test_fill_job_whose_context_is_the_common_ancestor():
    """Generate jobs on children of the context a Fill job is extending: the shared prefix stops at
    that context's parent, the Fill tokens stay causal, the children see all of them."""
    b = 16
    pool = Pool()
    parent = Context(0, None, pool, b)
    parent.allocate(32)
    c = Context(1, parent, pool, b)
    c.allocate(16)
    kids = [Context(2 + i, c, pool, b) for i in range(3)]
    c.allocate(16)
    for i, kid in enumerate(kids):
        kid.allocate(9 * i)
        kid.allocate(1)
    _forward_and_check([Fill(c, list(range(16)))] + [Generate(k) for k in kids], [16, 1, 1, 1], torch.float16, 33,
                       "fill context is the common ancestor")
