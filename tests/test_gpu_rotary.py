"""GPU parity of the NeoX rotary embedding fused with the KV fill (`pb_rotary_reshape_and_cache`):
against the float64 oracle, against the outputs of the reference's own torch implementation
(golden fixture), and bit-exact cache contents against rotary-then-fill composed on the host."""
from pathlib import Path

import numpy as np
import pytest
import torch

import parrotserve_b200 as pb
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLD = Path(__file__).resolve().parent / "golden"


def bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    return t.view(torch.int16 if t.element_size() == 2 else torch.int32).numpy()


def cos_sin_table(max_pos, rot, dtype):
    inv_freq = 1.0 / (10000 ** (torch.arange(0, rot, 2) / rot))
    freqs = torch.einsum("i,j -> ij", torch.arange(max_pos).float(), inv_freq.float())
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).to(dtype=dtype, device=DEV)


def rounded(x64: np.ndarray, dtype) -> torch.Tensor:
    """float64 oracle values rounded once to the storage type."""
    return torch.from_numpy(x64).to(dtype)


def assert_rotated(got: torch.Tensor, want64: np.ndarray, dtype, what):
    want = rounded(want64, dtype)
    g, w = got.detach().cpu().float(), want.float()
    if dtype == torch.float32:
        assert (g - w).abs().max().item() <= 1e-6 * max(1.0, w.abs().max().item()), what
        return
    # one rounding of an fp32 value that is itself within half an fp32 ulp of the exact one: at
    # most one storage ulp from the correctly rounded result, and almost always equal to it
    ulp = torch.maximum(w.abs(), torch.tensor(2.0 ** -14)) * (2.0 ** (-10 if dtype == torch.float16 else -7))
    assert ((g - w).abs() <= ulp).all(), what
    assert (g == w).float().mean().item() > 0.999, what


@pytest.mark.parametrize("name", ["full_128", "partial_64of128", "head64"])
def test_rotation_matches_reference_torch_outputs(name):
    fx = np.load(GOLD / "rotary_neox_ref.npz")
    q = torch.from_numpy(fx[f"{name}.q"]).to(DEV)
    k = torch.from_numpy(fx[f"{name}.k"]).to(DEV)
    t, h, d = q.shape
    pb.vllm_rotary_emb(torch.from_numpy(fx[f"{name}.positions"]).to(DEV), q.view(t, -1), k.view(t, -1),
                       torch.from_numpy(fx[f"{name}.cos_sin"]).to(DEV), d)
    assert np.abs(q.cpu().numpy() - fx[f"{name}.q.out"]).max() < 2e-6
    assert np.abs(k.cpu().numpy() - fx[f"{name}.k.out"]).max() < 2e-6


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("t,hq,hk,d,rot", [(5, 4, 4, 128, 128), (33, 8, 2, 128, 64), (64, 3, 3, 64, 64), (17, 2, 2, 256, 128)])
def test_rotation_only_in_place(dtype, t, hq, hk, d, rot):
    g = torch.Generator(device=DEV).manual_seed(t)
    max_pos = 97
    # q, k as strided views of one fused projection output, as the model produces them
    qkv = torch.randn((t, (hq + 2 * hk) * d), generator=g, device=DEV).to(dtype)
    q, k = qkv[:, : hq * d], qkv[:, hq * d: (hq + hk) * d]
    v_before = qkv[:, (hq + hk) * d:].clone()
    positions = torch.randint(0, max_pos, (t,), generator=g, device=DEV)
    cs = cos_sin_table(max_pos, rot, dtype)
    wq, wk = orc.rotary_neox_reference(positions.cpu().numpy(), q.cpu().double().numpy(), k.cpu().double().numpy(),
                                       cs.cpu().double().numpy(), d)
    pb.vllm_rotary_emb(positions, q, k, cs, d)
    assert_rotated(q, wq, dtype, "query")
    assert_rotated(k, wk, dtype, "key")
    assert torch.equal(qkv[:, (hq + hk) * d:], v_before)  # the neighbouring columns are untouched


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("write_back", [False, True])
def test_fused_rotary_fill_matches_rotary_then_fill(dtype, write_back):
    h, d, b, nb, rot, max_pos = 3, 128, 16, 40, 128, 300
    g = torch.Generator(device=DEV).manual_seed(7)
    x = 16 // torch.empty((), dtype=dtype).element_size()
    kc = torch.randn((nb, h, d // x, b, x), generator=g, device=DEV).to(dtype)
    vc = torch.randn((nb, h, d, b), generator=g, device=DEV).to(dtype)
    # prefill-like runs (full blocks, mid-block start and end), lone decode tokens, one skipped token
    runs = [(5 * b, 3 * b), (9 * b + 7, 20), (14 * b, 5), (20 * b + 15, 1), (21 * b, 1), (2 * b + 3, 12)]
    slots = []
    for s0, n in runs:
        slots += list(range(s0, s0 + n))
    slots[40] = -1
    slots = np.asarray(slots, dtype=np.int64)
    t = len(slots)
    qkv = torch.randn((t, 3 * h * d), generator=g, device=DEV).to(dtype)
    q, k, v = qkv.chunk(3, dim=-1)
    k0 = k.clone()
    positions = torch.randint(0, max_pos, (t,), generator=g, device=DEV)
    cs = cos_sin_table(max_pos, rot, dtype)
    wq, wk = orc.rotary_neox_reference(positions.cpu().numpy(), q.cpu().double().numpy(), k.cpu().double().numpy(),
                                       cs.cpu().double().numpy(), d)
    kr, vr = bits(kc).copy(), bits(vc).copy()
    pb.rotary_reshape_and_cache(positions, q, k, v, kc, vc, torch.tensor(slots, device=DEV), cs, d, write_key_back=write_back)
    assert_rotated(q, wq, dtype, "query")
    # what landed in the K cache is the rotated key, rounded once; read it back through the gather
    keep = slots >= 0
    k_back, v_back = torch.zeros((t, h, d), dtype=dtype, device=DEV), torch.zeros((t, h, d), dtype=dtype, device=DEV)
    pb.gather_cached_kv(k_back, v_back, kc, vc, torch.tensor(slots, device=DEV))
    assert_rotated(k_back.view(t, -1)[keep], wk[keep], dtype, "cached key")
    assert np.array_equal(bits(v_back.view(t, -1))[keep], bits(v)[keep])  # values are pure byte movement
    # nothing but the addressed slots changed: the fill of the device's own rotated keys reproduces the cache
    orc.fill_reference(bits(k_back), bits(v_back), kr, vr, slots)
    assert np.array_equal(bits(kc), kr) and np.array_equal(bits(vc), vr)
    if write_back:
        assert np.array_equal(bits(k)[keep], bits(k_back.view(t, -1))[keep])  # same bits as the cache got
    else:
        assert torch.equal(k, k0)


def test_rotary_rejects_unsupported_shapes():
    q = torch.zeros((2, 128), dtype=torch.float16, device=DEV)
    cs = torch.zeros((8, 24), dtype=torch.float16, device=DEV)  # halves of 12 elements: not whole 16-byte chunks
    with pytest.raises(RuntimeError):
        pb.vllm_rotary_emb(torch.zeros(2, dtype=torch.int64, device=DEV), q, q.clone(), cs, 128)
    with pytest.raises(RuntimeError):  # dtype mismatch between table and tensors
        pb.vllm_rotary_emb(torch.zeros(2, dtype=torch.int64, device=DEV), q, q.clone(), cs.float(), 128)
