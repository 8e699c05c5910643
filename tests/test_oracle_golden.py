"""CPU tests: the oracle against fixtures produced by the reference's own code."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc

GOLD = Path(__file__).resolve().parent / "golden"
CASES = ["tiny", "ragged", "cfg1_like"]


def _load(name):
    z = np.load(GOLD / "paged_attention_ref.npz")
    g = lambda k: torch.from_numpy(z[f"{name}.{k}"])
    return g("q").float(), g("kc").float(), g("vc").float(), g("tables"), g("lens"), g("out")


@pytest.mark.parametrize("name", CASES)
def test_port_matches_reference_output(name):
    # same algorithm in the same operation order: agreement to float32 rounding
    q, kc, vc, tables, lens, ref = _load(name)
    hm = torch.arange(q.shape[1])
    out = orc.reference_port_paged_attention(q, kc, vc, hm, lens, tables)
    assert torch.allclose(out, ref, atol=2e-6, rtol=1e-5), (out - ref).abs().max()


@pytest.mark.parametrize("name", CASES)
def test_gold_matches_reference_output(name):
    q, kc, vc, tables, lens, ref = _load(name)
    out = orc.gold_grouped_attention(q, kc, vc, None, None, None, lens.tolist(), tables.tolist())
    assert (out - ref.double()).abs().max().item() < 5e-6


@pytest.mark.parametrize("name", ["ragged", "cfg1_like"])
def test_shared_prefix_identity(name):
    """Splitting a context into (shared prefix, private suffix) does not change the result:
    the identity that pins the shared-prefix kernels."""
    q, kc, vc, tables, lens, ref = _load(name)
    b = vc.shape[3]
    # use row 1's first block as everybody's "prefix": rebuild rows as prefix ++ own tokens
    ptab = tables[1, :1].tolist()
    plen = b
    rows = [i for i in range(q.shape[0]) if lens[i] > 0]
    full_tabs = [ptab + tables[i].tolist() for i in rows]
    full = orc.gold_grouped_attention(q[rows], kc, vc, None, None, None, [plen + int(lens[i]) for i in rows], full_tabs)
    split = orc.gold_grouped_attention(q[rows], kc, vc, [0, len(rows)], [plen], [ptab],
                                       [int(lens[i]) for i in rows], [tables[i].tolist() for i in rows])
    assert (full - split).abs().max().item() < 1e-12


def test_merge_partials_is_exact_split_softmax():
    g = torch.Generator().manual_seed(5)
    h, d, n = 3, 16, 50
    q = torch.randn((h, d), generator=g, dtype=torch.float64)
    k = torch.randn((n, h, d), generator=g, dtype=torch.float64)
    v = torch.randn((n, h, d), generator=g, dtype=torch.float64)
    scale = d ** -0.5
    whole = orc.gold_row_attention(q, k, v, scale)
    cuts = [0, 7, 7, 31, 50]  # includes an empty-free uneven split
    outs, ms, ls = [], [], []
    for a, b in zip(cuts[:-1], cuts[1:]):
        if a == b:
            continue
        outs.append(orc.gold_row_attention(q, k[a:b], v[a:b], scale))
        m, l = orc.gold_stats(q, k[a:b], scale)
        ms.append(m)
        ls.append(l)
    merged, M, L = orc.merge_partials(outs, ms, ls)
    assert (merged - whole).abs().max().item() < 1e-12
    m_all, l_all = orc.gold_stats(q, k, scale)
    assert torch.allclose(M, m_all) and torch.allclose(L, l_all)
    # associativity: merging in another order gives the same result
    merged2, _, _ = orc.merge_partials(outs[::-1], ms[::-1], ls[::-1])
    assert (merged2 - whole).abs().max().item() < 1e-12


def test_causal_with_context_matches_rowwise():
    g = torch.Generator().manual_seed(6)
    h, d, ctx, ql = 2, 8, 11, 4
    q = torch.randn((ql, h, d), generator=g)
    k = torch.randn((ctx, h, d), generator=g)
    v = torch.randn((ctx, h, d), generator=g)
    out = orc.gold_causal_with_context(q, k, v, d ** -0.5)
    for i in range(ql):
        n = ctx - ql + i + 1
        row = orc.gold_row_attention(q[i], k[:n].double(), v[:n].double(), d ** -0.5)
        assert (out[i] - row).abs().max().item() < 1e-12


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_fill_gather_reference_roundtrip(dtype):
    # the shapes of the reference's own cache test (3rdparty/vllm/tests/kernels/test_cache.py:179-186)
    rng = np.random.default_rng(0)
    t, h, d, b, nb = 3, 2, 16, 8, 2
    x = 16 // np.dtype(dtype).itemsize
    key = rng.standard_normal((t, h, d)).astype(dtype)
    value = rng.standard_normal((t, h, d)).astype(dtype)
    kc = rng.standard_normal((nb, h, d // x, b, x)).astype(dtype)
    vc = rng.standard_normal((nb, h, d, b)).astype(dtype)
    kc0, vc0 = kc.copy(), vc.copy()
    slots = rng.choice(nb * b, size=t, replace=False)
    orc.fill_reference(key, value, kc, vc, slots)
    # element-level address formula of the layout (cache_kernels.cu:170-178)
    for i, s in enumerate(slots):
        for hh in range(h):
            for dd in range(d):
                assert kc.reshape(-1)[((s // b * h + hh) * (d // x) + dd // x) * b * x + (s % b) * x + dd % x] == key[i, hh, dd]
                assert vc.reshape(-1)[((s // b * h + hh) * d + dd) * b + s % b] == value[i, hh, dd]
    k2, v2 = orc.gather_reference(kc, vc, slots)
    assert np.array_equal(k2, key) and np.array_equal(v2, value)
    # untouched slots keep their bytes
    mask = np.ones(nb * b, dtype=bool)
    mask[slots] = False
    others = np.nonzero(mask)[0]
    ka, va = orc.gather_reference(kc, vc, others)
    kb, vb = orc.gather_reference(kc0, vc0, others)
    assert np.array_equal(ka, kb) and np.array_equal(va, vb)


@pytest.mark.parametrize("name", ["full_128", "partial_64of128", "head64"])
def test_rotary_oracle_matches_reference_torch_implementation(name):
    """The rotary oracle against outputs of RefRotaryEmbeddingNeox, the torch reference the vendored
    vLLM test checks the kernel with (3rdparty/vllm/tests/kernels/test_pos_encoding.py:27-79)."""
    fx = np.load(GOLD / "rotary_neox_ref.npz")
    q, k = fx[f"{name}.q"], fx[f"{name}.k"]
    t, h, d = q.shape
    oq, ok = orc.rotary_neox_reference(fx[f"{name}.positions"], q.reshape(t, -1), k.reshape(t, -1),
                                       fx[f"{name}.cos_sin"], d)
    assert np.abs(oq.reshape(t, h, d) - fx[f"{name}.q.out"]).max() < 2e-6  # the reference computes in fp32
    assert np.abs(ok.reshape(t, h, d) - fx[f"{name}.k.out"]).max() < 2e-6
    rot = fx[f"{name}.cos_sin"].shape[1]
    assert np.array_equal(oq.reshape(t, h, d)[..., rot:], q[..., rot:].astype(np.float64))  # pass-through part


def test_sampler_oracle_matches_reference_probabilities():
    """The probability rows the reference's Sampler hands to torch.multinomial
    (parrot/engine/builtin/models/sampler.py:31-63, fp32 on CPU), including the nucleus sets."""
    from oracle import sampler_oracle as so

    z = np.load(GOLD / "sampler_probs_ref.npz")
    for name in sorted({k.split(".")[0] for k in z.files}):
        logits = z[f"{name}.hidden"].astype(np.float64) @ z[f"{name}.embd"].astype(np.float64).T
        probs = so.nucleus_probs_reference(logits, z[f"{name}.temperature"], z[f"{name}.top_p"])
        ref = z[f"{name}.probs"]
        assert np.abs(probs - ref).max() < 2e-6, name
        assert ((probs > 0) == (ref > 0)).all(), name
        assert np.allclose(probs.sum(axis=1), 1.0)


def test_sampler_oracle_draw_and_ties():
    from oracle import sampler_oracle as so

    # ties at the nucleus edge go by index, as a stable descending sort orders them
    logits = np.log(np.array([[0.1, 0.3, 0.3, 0.3]]))
    p = so.nucleus_probs_reference(logits, np.array([1.0]), np.array([0.5]))
    assert np.allclose(p, [[0.0, 0.5, 0.5, 0.0]])       # mass before the 3rd tied token is 0.6 > 0.5
    assert so.sample_inverse_cdf(p, np.array([0.49]))[0] == 1 and so.sample_inverse_cdf(p, np.array([0.5]))[0] == 2
    # empirical frequencies of the inverse-CDF draw follow the probabilities
    rng = np.random.default_rng(3)
    probs = np.array([[0.5, 0.0, 0.25, 0.25]])
    ids = np.array([so.sample_inverse_cdf(probs, np.array([u]))[0] for u in rng.random(4000)])
    freq = np.bincount(ids, minlength=4) / 4000
    assert np.abs(freq - probs[0]).max() < 0.03 and freq[1] == 0
