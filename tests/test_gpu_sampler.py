"""GPU parity of the device sampler (`pb_sample_top_p` through `ops.sample_top_p` and the
reference-shaped `Sampler` module) against the CPU oracle of the reference's sampler
(parrot/engine/builtin/models/sampler.py:19-66).

The kernel computes probabilities in float32 (2^-40 fixed point), the oracle in float64, so a draw
is compared through the oracle's CDF: the kernel's token must own the uniform number up to TOL, plus
the probability of the one token at the nucleus edge when top_p falls within EDGE of it."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import sampler_oracle as so
from parrotserve_b200 import ops
from parrotserve_b200.sampler import Sampler

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLD = Path(__file__).resolve().parent / "golden"
TOL = 2e-5
EDGE = 1e-5


def _check_draws(logits: torch.Tensor, temperature, top_p, uniforms: torch.Tensor, ids: torch.Tensor, what: str):
    lg = logits.float().cpu().numpy().astype(np.float64)
    t = np.asarray(temperature, dtype=np.float64)
    p = np.asarray(top_p, dtype=np.float64)
    probs = so.nucleus_probs_reference(lg, t, p)
    margin = so.nucleus_margin(lg, t, p)
    u = uniforms.cpu().numpy().astype(np.float64)
    got = ids.cpu().numpy()
    want = so.sample_inverse_cdf(probs, u)
    assert ids.dtype == torch.int64 and got.shape == want.shape
    exact = 0
    for r in range(lg.shape[0]):
        k = int(got[r])
        assert 0 <= k < lg.shape[1], (what, r, k)
        variants = [probs[r]]
        if p[r] < 1.0 and margin[r, 0] < EDGE:   # the token at the nucleus edge may fall either way
            e = int(margin[r, 2])
            alt = probs[r].copy()
            if alt[e] > 0:
                alt[e] = 0.0
            else:   # its un-normalised weight relative to the kept mass
                x = lg[r] / t[r]
                alt[e] = np.exp(x[e] - x.max()) / np.exp(x[probs[r] > 0] - x.max()).sum()
            if alt.sum() > 0:
                variants.append(alt / alt.sum())
        ok = False
        for pr in variants:
            cdf = np.cumsum(pr)
            ok = ok or (pr[k] > 0 and cdf[k] - pr[k] - TOL <= u[r] <= cdf[k] + TOL)
        cdf = np.cumsum(probs[r])
        assert ok, f"{what}: row {r} u={u[r]} drew token {k}, which owns [{cdf[k] - probs[r, k]}, {cdf[k]}] (p={probs[r, k]})"
        exact += int(k == want[r])
    return exact / lg.shape[0]


def test_golden_rows_many_uniforms():
    """Rows of the reference fixture, 64 uniform numbers each."""
    z = np.load(GOLD / "sampler_probs_ref.npz")
    g = torch.Generator(device=DEV).manual_seed(5)
    for name in sorted({k.split(".")[0] for k in z.files}):
        logits = torch.tensor(z[f"{name}.hidden"].astype(np.float64) @ z[f"{name}.embd"].astype(np.float64).T,
                              dtype=torch.float32, device=DEV).repeat_interleave(64, dim=0)
        temp = np.repeat(z[f"{name}.temperature"], 64)
        top_p = np.repeat(z[f"{name}.top_p"], 64)
        u = torch.rand(logits.shape[0], generator=g, device=DEV)
        ids = ops.sample_top_p(logits, temp.tolist(), top_p.tolist(), u)
        frac = _check_draws(logits, temp, top_p, u, ids, name)
        assert frac > 0.98, (name, frac)
        assert torch.equal(ids, ops.sample_top_p(logits, temp.tolist(), top_p.tolist(), u))  # repeats bit for bit


def test_ties_at_the_nucleus_edge_go_by_index():
    logits = torch.tensor(np.log([[0.1, 0.3, 0.3, 0.3]]), dtype=torch.float32, device=DEV).repeat(4, 1)
    u = torch.tensor([0.0, 0.49, 0.51, 0.999], device=DEV)
    ids = ops.sample_top_p(logits, None, [0.5] * 4, u)
    assert ids.tolist() == [1, 1, 2, 2]
    # a flat row: top_p keeps the first floor(top_p * V) + 1 tokens by index, each equally likely
    v = 5000
    flat = torch.zeros((6, v), dtype=torch.float16, device=DEV)
    u = torch.tensor([0.0, 0.1003, 0.5001, 0.7302, 0.9999, 0.33331], device=DEV)
    ids = ops.sample_top_p(flat, None, [0.25] * 6, u)
    assert ids.tolist() == [int(float(x) * 1251) for x in u.tolist()]
    # without top-p every token of the flat row can be drawn
    ids = ops.sample_top_p(flat, None, None, u)
    assert ids.tolist() == [int(float(x) * v) for x in u.tolist()]


def test_tie_classes_at_the_edge_small_and_large():
    """A handful of ties at the nucleus edge (settled by one warp) and several dozen (settled by an
    index-ordered scan of the row): the first ties by index are kept, as many as the mass allows."""
    v = 1000
    p = np.full(v, 0.1 / 994)
    p[7] = 0.4
    ties = [3, 100, 500, 501, 900]
    p[ties] = 0.1
    logits = torch.tensor(np.log(p)[None, :], dtype=torch.float32, device=DEV).repeat(4, 1)
    u = torch.tensor([0.1, 0.5, 0.8, 0.95], device=DEV)
    ids = ops.sample_top_p(logits, None, [0.65] * 4, u)
    assert ids.tolist() == [3, 7, 100, 500]
    _check_draws(logits, [1.0] * 4, [0.65] * 4, u, ids, "five ties")

    v = 2000
    p = np.full(v, 0.2 / 1949)
    p[0] = 0.3
    p[10:60] = 0.01
    logits = torch.tensor(np.log(p)[None, :], dtype=torch.float32, device=DEV).repeat(3, 1)
    u = torch.tensor([0.2, 0.7, 0.99], device=DEV)
    ids = ops.sample_top_p(logits, None, [0.505] * 3, u)
    assert ids.tolist() == [0, 15, 30]
    _check_draws(logits, [1.0] * 3, [0.505] * 3, u, ids, "fifty ties")
    # top_p = 0 keeps the leader only
    assert ops.sample_top_p(logits, None, [0.0] * 3, u).tolist() == [0, 0, 0]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("vocab", [32000, 50272, 32003])
def test_model_sized_vocabularies(dtype, vocab):
    rows = 48
    g = torch.Generator(device=DEV).manual_seed(vocab)
    logits = (torch.randn((rows, vocab), generator=g, device=DEV) * 2.5).to(dtype)
    logits[3, 17] = float("-inf")
    logits[5, :100] = 9.0     # a block of tied leaders
    temp = [1.0, 0.7, 1.5, 0.3] * (rows // 4)
    top_p = [1.0, 0.9, 0.5, 0.95, 0.1, 0.999] * (rows // 6)
    u = torch.rand(rows, generator=g, device=DEV)
    ids = ops.sample_top_p(logits, temp, top_p, u)
    frac = _check_draws(logits, temp, top_p, u, ids, f"{dtype} V={vocab}")
    assert frac > 0.9, frac
    # a padded row stride (a slice of a wider matrix)
    wide = torch.zeros((rows, vocab + 24), dtype=dtype, device=DEV)
    wide[:, :vocab] = logits
    assert torch.equal(ops.sample_top_p(wide[:, :vocab], temp, top_p, u), ids)


@pytest.mark.parametrize("seed", list(range(16)))
def test_small_and_odd_vocabularies(seed):
    """Vocabulary sizes around the kernel's vector width and tile size, rows that are not 16-byte
    aligned, flat rows, half of the row masked with -inf, extreme temperatures and top_p 0 / 1."""
    rng = np.random.default_rng(seed)
    vocab = [1, 2, 3, 7, 8, 9, 31, 100, 1000, 4097, 8191, 8192, 8193, 20001, 32000, 65537][seed]
    rows = int(rng.integers(2, 12))
    dtype = [torch.float16, torch.bfloat16, torch.float32][seed % 3]
    scale = [0.0, 0.5, 2.5, 8.0][seed % 4]
    g = torch.Generator(device=DEV).manual_seed(seed)
    logits = (torch.randn((rows, vocab), generator=g, device=DEV) * scale).to(dtype)
    if vocab > 3 and seed % 2:
        logits[:, : vocab // 2] = float("-inf")
    temp = [float(rng.choice([1.0, 0.5, 1.7, 0.05])) for _ in range(rows)]
    top_p = [float(rng.choice([1.0, 0.9, 0.5, 0.1, 0.0, 0.999])) for _ in range(rows)]
    u = torch.rand(rows, generator=g, device=DEV)
    ids = ops.sample_top_p(logits, temp, top_p, u)
    _check_draws(logits, temp, top_p, u, ids, f"vocab {vocab} {dtype} scale {scale}")
    assert torch.equal(ids, ops.sample_top_p(logits, temp, top_p, u))
    if vocab > 3 and seed % 2:
        assert (ids >= vocab // 2).all()   # masked tokens are never drawn


def test_frequencies_follow_the_nucleus_distribution():
    v, n = 1000, 20000
    g = torch.Generator(device=DEV).manual_seed(9)
    row = torch.randn((1, v), generator=g, device=DEV) * 2.0
    logits = row.expand(n, v).contiguous()
    u = torch.rand(n, generator=g, device=DEV)
    ids = ops.sample_top_p(logits, [0.8] * n, [0.9] * n, u)
    probs = so.nucleus_probs_reference(row.cpu().numpy(), np.array([0.8]), np.array([0.9]))[0]
    freq = np.bincount(ids.cpu().numpy(), minlength=v) / n
    assert freq[probs == 0].sum() == 0                       # nothing outside the nucleus
    assert 0.5 * np.abs(freq - probs).sum() < 0.06           # total variation; sampling noise ~0.03 here
    top = np.argsort(-probs)[:5]
    assert np.abs(freq[top] - probs[top]).max() < 0.01


def test_sampler_module_has_the_reference_interface():
    class Cfg:
        vocab_size = 4096

    class SC:
        def __init__(self, temperature, top_p):
            self.temperature, self.top_p = temperature, top_p

    g = torch.Generator(device=DEV).manual_seed(1)
    embd = torch.randn((4096, 64), generator=g, device=DEV).half()
    hs = torch.randn((5, 64), generator=g, device=DEV).half()
    sampler = Sampler(Cfg(), embd)
    sampler.generator = torch.Generator(device=DEV).manual_seed(77)
    cfgs = [SC(1.0, 1.0), SC(0.5, 0.9), SC(1.0, 0.2), SC(2.0, 1.0), SC(0.9, 0.6)]
    ids = sampler(hs, cfgs)
    u = torch.rand(5, generator=torch.Generator(device=DEV).manual_seed(77), device=DEV)
    logits = torch.matmul(hs, embd.t())
    assert ids.dtype == torch.int64 and ids.shape == (5,)
    assert torch.equal(ids, ops.sample_top_p(logits, [c.temperature for c in cfgs], [c.top_p for c in cfgs], u))
    _check_draws(logits, [c.temperature for c in cfgs], [c.top_p for c in cfgs], u, ids, "module")
    assert sampler(hs[:0], []).shape == (0,)
    with pytest.raises(ValueError):
        ops.sample_top_p(logits, [0.0] * 5, None, u)


def test_c_entry_rejects_bad_arguments():
    from parrotserve_b200 import _lib

    lib = _lib.lib()
    logits = torch.zeros((2, 8), dtype=torch.float16, device=DEV)
    u = torch.zeros(2, device=DEV)
    ids = torch.zeros(2, dtype=torch.int64, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    call = lambda *a: lib.pb_sample_top_p(*a, stream)
    ok = (logits.data_ptr(), _lib.PB_F16, 2, 8, 8, None, None, u.data_ptr(), ids.data_ptr())
    assert call(*ok) == _lib.PB_OK
    assert call(logits.data_ptr(), _lib.PB_F16, -1, 8, 8, None, None, u.data_ptr(), ids.data_ptr()) == _lib.PB_ERR_INVALID_ARG
    assert call(logits.data_ptr(), _lib.PB_F16, 2, 0, 8, None, None, u.data_ptr(), ids.data_ptr()) == _lib.PB_ERR_INVALID_ARG
    assert call(logits.data_ptr(), _lib.PB_F16, 2, 8, 7, None, None, u.data_ptr(), ids.data_ptr()) == _lib.PB_ERR_INVALID_ARG
    assert call(None, _lib.PB_F16, 2, 8, 8, None, None, u.data_ptr(), ids.data_ptr()) == _lib.PB_ERR_INVALID_ARG
    assert call(logits.data_ptr(), _lib.PB_F16, 2, 8, 8, None, None, None, ids.data_ptr()) == _lib.PB_ERR_INVALID_ARG
    assert call(logits.data_ptr(), 9, 2, 8, 8, None, None, u.data_ptr(), ids.data_ptr()) == _lib.PB_ERR_UNSUPPORTED
    assert call(None, _lib.PB_F16, 0, 8, 8, None, None, None, None) == _lib.PB_OK   # an empty batch touches nothing
    with pytest.raises(RuntimeError):
        ops.sample_top_p(logits.t(), None, None, u)          # vocabulary must be the unit-stride dimension
    with pytest.raises(RuntimeError):
        ops.sample_top_p(logits, None, None, torch.zeros(3, device=DEV))
    with pytest.raises(RuntimeError):
        ops.sample_top_p(logits.cpu(), None, None, u)         # no CPU fallback
