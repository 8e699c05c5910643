"""Generates the golden fixtures in this directory by running the REFERENCE's own code on CPU.

Run in the build container only (needs the read-only reference checkout):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py <path to the ParrotServe checkout>

Outputs (committed):
  paged_attention_ref.npz    inputs + outputs of the reference's torch reference attention
                             ``paged_flash_attention_reference``
                             (parrot/engine/builtin/kernels/shared_flash_decoding.py:382-404)
  iteration_state_ref.json   block tables / lengths / slot mappings built by the reference's
                             ``xFormersFill_SharedPromptsGenerate.init_iteration_state``
                             (parrot/engine/builtin/attn_func.py:461-599) from its own
                             ``BlockContext`` trees (parrot/engine/context/block_context.py)

  rotary_neox_ref.npz        inputs + outputs of ``RefRotaryEmbeddingNeox``, the torch reference
                             implementation the vendored vLLM tests check the rotary kernel against
                             (3rdparty/vllm/tests/kernels/test_pos_encoding.py:9-79), fp32 on CPU

  sampler_probs_ref.npz      hidden states, embedding, temperatures, top-p values and the probability
                             rows the reference's ``Sampler.forward`` hands to ``torch.multinomial``
                             (parrot/engine/builtin/models/sampler.py:19-66), fp32 on CPU; the call to
                             ``torch.multinomial`` is wrapped to record its argument, nothing else

  causal_context_ref.npz     inputs + outputs of ``ref_masked_attention`` with the additive
                             bottom-right-aligned causal mask of the vendored vLLM test's
                             with-context reference (3rdparty/vllm/tests/kernels/test_attention.py:14-27,
                             mask as built at :128-129), fp32 on CPU: the arithmetic the reference
                             delegates to xformers for Fill jobs that have cached context

The reference modules import native extensions that do not exist here (``vllm.cache_ops``,
``parrot.attention_ops``, ``xformers``); empty stub modules stand in for those names. No
arithmetic of the reference is patched.
"""
from __future__ import annotations

import importlib.util
import json
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _stub(name: str, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    sys.modules[name] = m
    return m


def install_stubs():
    import triton  # noqa: F401  (real triton is present; the kernels are never launched)

    vllm = _stub("vllm")
    vllm.__path__ = []
    for sub in ("cache_ops", "attention_ops", "layernorm_ops", "pos_encoding_ops"):
        setattr(vllm, sub, _stub(f"vllm.{sub}"))
    xf = _stub("xformers")
    xf.__path__ = []
    ops = _stub("xformers.ops")
    ops.__path__ = []
    fmha = _stub("xformers.ops.fmha")
    fmha.__path__ = []

    class _Mask:
        def __init__(self, q, kv):
            self.q_seqlen, self.kv_seqlen = list(q), list(kv)

        @classmethod
        def from_seqlens(cls, q_seqlen, kv_seqlen=None):
            return cls(q_seqlen, kv_seqlen if kv_seqlen is not None else q_seqlen)

    ab = _stub("xformers.ops.fmha.attn_bias", BlockDiagonalCausalFromBottomRightMask=_Mask,
               BlockDiagonalCausalMask=_Mask)
    fmha.attn_bias = ab
    fmha.cutlass = _stub("xformers.ops.fmha.cutlass")
    ops.fmha = fmha
    xf.ops = ops


def load_reference_attention(ref_root: Path):
    sys.path.insert(0, str(ref_root))
    parrot = sys.modules.get("parrot")
    import parrot  # noqa: F811  (pure-python package init)

    parrot.attention_ops = _stub("parrot.attention_ops")
    path = ref_root / "parrot/engine/builtin/kernels/shared_flash_decoding.py"
    spec = importlib.util.spec_from_file_location("_ref_shared_flash_decoding", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.paged_flash_attention_reference


def attention_cases():
    """(name, num_seqs, num_heads, head_size, block_size, num_blocks, context lens, seed)."""
    return [
        ("tiny", 3, 2, 16, 8, 12, [1, 8, 19], 11),
        ("ragged", 5, 2, 64, 16, 24, [1, 15, 16, 17, 100], 12),
        ("cfg1_like", 3, 2, 128, 16, 40, [512 + 3, 512 + 64, 33], 13),
    ]


def make_attention_fixture(ref_fn):
    out = {}
    for name, s, h, d, b, nb, lens, seed in attention_cases():
        g = torch.Generator().manual_seed(seed)
        x = 4  # fp32
        # values are rounded to fp16 so the fixture can store them in half the space, exactly
        q = torch.randn((s, h, d), generator=g).half().float()
        kc = torch.randn((nb, h, d // x, b, x), generator=g).half().float()
        vc = torch.randn((nb, h, d, b), generator=g).half().float()
        maxb = max((n + b - 1) // b for n in lens)
        tables = torch.zeros((s, maxb), dtype=torch.int32)
        for i, n in enumerate(lens):
            k = (n + b - 1) // b
            tables[i, :k] = torch.randperm(nb, generator=g)[:k].to(torch.int32)
        hm = torch.arange(h, dtype=torch.int32)
        cl = torch.tensor(lens, dtype=torch.int32)
        # the reference indexes with the table row directly: int64 needed on CPU
        o = ref_fn(q, kc, vc, hm.long(), cl, tables.long())
        for key, val in (("q", q), ("kc", kc), ("vc", vc), ("tables", tables), ("lens", cl), ("out", o)):
            out[f"{name}.{key}"] = val.half().numpy() if key in ("q", "kc", "vc") else val.numpy()
    np.savez_compressed(HERE / "paged_attention_ref.npz", **out)
    print("wrote paged_attention_ref.npz", {k: v.shape for k, v in out.items() if k.endswith(".out")})


def make_iteration_state_fixture():
    from transformers import PretrainedConfig

    from parrot.engine.config import BuiltinConfig
    from parrot.engine.context.block_context import BlockContext
    from parrot.engine.primitive_job import Fill, Generate
    from parrot.sampling_config import SamplingConfig
    from parrot.utils import RecyclePool
    import parrot.engine.builtin.attn_func  # noqa: F401  (registers the attn-func lookup on BuiltinConfig)
    from parrot.engine.builtin.iter_state import IterationState

    cases = []

    def run_case(name, root_len, children, block_size=16, with_fill=None):
        pool = RecyclePool()
        cfg = BuiltinConfig(num_kv_cache_blocks=4096, attn_func="xformers_fill_shared_prompts_generate",
                            block_size=block_size, device="cpu")
        hf = PretrainedConfig(num_attention_heads=4, hidden_size=64)
        root = BlockContext(0, None, pool, block_size)
        root.allocate(root_len)
        jobs, cid = [], 1
        for extra in children:
            ctx = BlockContext(cid, root, pool, block_size)
            ctx.allocate(extra)
            job = Generate(session_id=0, task_id=cid, context_id=cid, parent_context_id=0,
                           sampling_config=SamplingConfig())
            job.context = ctx
            ctx.allocate(1)  # the slot of the token generated in this iteration (builtin_runner.py:97-101)
            jobs.append(job)
            cid += 1
        st = IterationState(jobs, hf, cfg)
        cases.append({
            "name": name, "block_size": block_size, "root_len": root_len, "children": list(children),
            "flash_context_len": int(st.flash_context_len),
            "flash_block_table": st.flash_block_table.tolist(),
            "paged_context_lens": st.paged_context_lens.tolist(),
            "paged_block_tables": st.paged_block_tables.tolist(),
            "slot_mapping": st.slot_mapping.tolist(),
            "context_block_ids": [sorted(set(j.context.get_context_block_ids())) for j in jobs],
            "context_slot_ids": [j.context.get_context_slot_ids() for j in jobs],
            "context_lens": [j.context.get_context_len() for j in jobs],
        })

    def run_fill_case(name, root_len, fills, children, block_size=16):
        """A tree with Fill jobs (cached tokens, new tokens) before the Generate jobs, as the runner
        orders them (builtin_runner.py:75-76)."""
        pool = RecyclePool()
        cfg = BuiltinConfig(num_kv_cache_blocks=4096, attn_func="xformers_fill_shared_prompts_generate",
                            block_size=block_size, device="cpu")
        hf = PretrainedConfig(num_attention_heads=4, hidden_size=64)
        root = None
        if root_len:
            root = BlockContext(0, None, pool, block_size)
            root.allocate(root_len)
        jobs, cid = [], 1
        for cached, n_new in fills:
            ctx = BlockContext(cid, root, pool, block_size)
            ctx.allocate(cached)
            job = Fill(session_id=0, task_id=cid, context_id=cid, parent_context_id=0 if root else -1,
                       token_ids=list(range(n_new)))
            job.context = ctx
            ctx.allocate(n_new)  # the runner allocates the new tokens before the metadata is built
            jobs.append(job)
            cid += 1
        for extra in children:
            ctx = BlockContext(cid, root, pool, block_size)
            ctx.allocate(extra)
            job = Generate(session_id=0, task_id=cid, context_id=cid, parent_context_id=0 if root else -1,
                           sampling_config=SamplingConfig())
            job.context = ctx
            ctx.allocate(1)
            jobs.append(job)
            cid += 1
        st = IterationState(jobs, hf, cfg)
        bias = st.q_kv_attn_bias  # the stub mask records the sequence lengths the reference passes
        cases.append({
            "name": name, "block_size": block_size, "root_len": root_len, "fills": [list(f) for f in fills],
            "children": list(children),
            "flash_context_len": int(st.flash_context_len),
            "flash_block_table": st.flash_block_table.tolist(),
            "paged_context_lens": st.paged_context_lens.tolist(),
            "paged_block_tables": st.paged_block_tables.tolist(),
            "slot_mapping": st.slot_mapping.tolist(),
            "num_fill_tokens": list(st.num_fill_tokens),
            "fill_q_lens": list(bias.q_seqlen), "fill_kv_lens": list(bias.kv_seqlen),
            "fill_slots": st.fill_slots.tolist(),
            "context_slot_ids": [j.context.get_context_slot_ids() for j in jobs],
            "context_lens": [j.context.get_context_len() for j in jobs],
        })

    run_case("fork3_root64", 64, [5, 17, 33])
    run_case("fork2_root20_padded", 20, [0, 3])
    run_case("single_job", 40, [7])
    run_fill_case("fill2_gen3_root40", 40, [(0, 37), (9, 20)], [0, 15, 70])
    run_fill_case("lone_fill_no_parent", 0, [(0, 20)], [])
    run_fill_case("lone_fill_with_parent_and_cache", 40, [(13, 20)], [])
    (HERE / "iteration_state_ref.json").write_text(json.dumps(cases, indent=1))
    print("wrote iteration_state_ref.json", [c["name"] for c in cases])


def make_rotary_fixture(ref_root: Path):
    """Runs the vendored vLLM test's own torch reference of the NeoX rotary embedding on CPU."""
    path = ref_root / "3rdparty/vllm/tests/kernels/test_pos_encoding.py"
    spec = importlib.util.spec_from_file_location("_ref_test_pos_encoding", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)  # imports the stubbed vllm.pos_encoding_ops; no kernel is called
    out = {}
    for name, (t, h, d, rot, max_pos) in {"full_128": (9, 3, 128, 128, 64), "partial_64of128": (7, 2, 128, 64, 32),
                                          "head64": (5, 4, 64, 64, 40)}.items():
        g = torch.Generator().manual_seed(4000 + t)
        positions = torch.randint(0, max_pos, (t,), generator=g)
        q = torch.randn((t, h, d), generator=g)
        k = torch.randn((t, h, d), generator=g)
        # the cos/sin table exactly as the test builds it for the kernel (test_pos_encoding.py:99-105)
        inv_freq = 1.0 / (10000 ** (torch.arange(0, rot, 2) / rot))
        freqs = torch.einsum("i,j -> ij", torch.arange(max_pos).float(), inv_freq.float())
        cos_sin = torch.cat((freqs.cos(), freqs.sin()), dim=-1)
        ref = mod.RefRotaryEmbeddingNeox(dim=rot, max_position_embeddings=max_pos)
        with torch.inference_mode():
            rq, rk = ref(positions, q, k)
        for key, val in (("positions", positions), ("q", q), ("k", k), ("cos_sin", cos_sin), ("q.out", rq), ("k.out", rk)):
            out[f"{name}.{key}"] = val.numpy()
    np.savez_compressed(HERE / "rotary_neox_ref.npz", **out)
    print("wrote rotary_neox_ref.npz", sorted({k.split(".")[0] for k in out}))


def make_causal_fixture(ref_root: Path):
    """Runs the vendored vLLM test's own ``ref_masked_attention`` on CPU with the additive mask its
    with-context reference builds (``triu(ones(q_len, ctx_len), diagonal=ctx_len - q_len + 1) * -1e5``,
    test_attention.py:128-129; that helper itself pins the mask to 'cuda', so the two lines are
    evaluated here on the CPU)."""
    path = ref_root / "3rdparty/vllm/tests/kernels/test_attention.py"
    spec = importlib.util.spec_from_file_location("_ref_test_attention", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)  # imports the stubbed xformers / vllm.attention_ops; no kernel is called
    out = {}
    for name, (q_len, ctx_len, h, d) in {"square_5": (5, 5, 2, 16), "ctx20_q7": (7, 20, 2, 64),
                                         "ctx33_q1": (1, 33, 3, 32), "ctx200_q64": (64, 200, 2, 128)}.items():
        g = torch.Generator().manual_seed(5000 + q_len)
        q = torch.randn((q_len, h, d), generator=g).half().float()
        k = torch.randn((ctx_len, h, d), generator=g).half().float()
        v = torch.randn((ctx_len, h, d), generator=g).half().float()
        attn_mask = torch.triu(torch.ones(q_len, ctx_len), diagonal=ctx_len - q_len + 1) * -1e5
        attn_mask = attn_mask.to(dtype=torch.float32)
        with torch.inference_mode():
            o = mod.ref_masked_attention(q, k, v, 1.0 / (d ** 0.5), attn_mask=attn_mask)
        for key, val in (("q", q.half()), ("k", k.half()), ("v", v.half()), ("out", o)):
            out[f"{name}.{key}"] = val.numpy()
    np.savez_compressed(HERE / "causal_context_ref.npz", **out)
    print("wrote causal_context_ref.npz", {k: v.shape for k, v in out.items() if k.endswith(".out")})


def make_sampler_fixture(ref_root: Path):
    """Runs the reference's Sampler on CPU and records the probabilities it samples from."""
    from transformers import PretrainedConfig

    from parrot.sampling_config import SamplingConfig

    path = ref_root / "parrot/engine/builtin/models/sampler.py"
    spec = importlib.util.spec_from_file_location("_ref_sampler", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    recorded = []
    real_multinomial = torch.multinomial

    def recording_multinomial(probs, *args, **kwargs):
        recorded.append(probs.detach().clone())
        return real_multinomial(probs, *args, **kwargs)

    out = {}
    cases = {
        # name: (vocab, hidden, temperatures, top_ps, seed, logit scale)
        "mixed": (512, 16, [1.0, 0.7, 1.3, 1.0, 0.5, 2.0], [1.0, 0.9, 0.5, 0.3, 0.95, 0.8], 71, 1.0),
        "peaked": (300, 8, [1.0, 1.0, 0.25], [0.6, 0.05, 0.9], 72, 3.0),
        "plain": (257, 8, [1.0, 1.0], [1.0, 1.0], 73, 1.0),
    }
    torch.multinomial = recording_multinomial
    try:
        for name, (vocab, hidden, temps, top_ps, seed, scale) in cases.items():
            g = torch.Generator().manual_seed(seed)
            embd = torch.randn((vocab, hidden), generator=g) * scale
            hs = torch.randn((len(temps), hidden), generator=g)
            sampler = mod.Sampler(PretrainedConfig(vocab_size=vocab), embd)
            recorded.clear()
            with torch.inference_mode():
                ids = sampler(hs, [SamplingConfig(temperature=t, top_p=p) for t, p in zip(temps, top_ps)])
            assert len(recorded) == 1 and ids.shape == (len(temps),)
            for key, val in (("embd", embd), ("hidden", hs), ("temperature", torch.tensor(temps)),
                             ("top_p", torch.tensor(top_ps)), ("probs", recorded[0])):
                out[f"{name}.{key}"] = val.numpy()
    finally:
        torch.multinomial = real_multinomial
    np.savez_compressed(HERE / "sampler_probs_ref.npz", **out)
    print("wrote sampler_probs_ref.npz", {k: v.shape for k, v in out.items() if k.endswith(".probs")})


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to the ParrotServe checkout>")
    ref_root = Path(sys.argv[1])
    install_stubs()
    if len(sys.argv) > 2 and sys.argv[2] == "sampler":   # only this fixture
        sys.path.insert(0, str(ref_root))
        make_sampler_fixture(ref_root)
        return
    ref_fn = load_reference_attention(ref_root)
    make_attention_fixture(ref_fn)
    make_iteration_state_fixture()
    make_rotary_fixture(ref_root)
    make_causal_fixture(ref_root)
    make_sampler_fixture(ref_root)


if __name__ == "__main__":
    main()
