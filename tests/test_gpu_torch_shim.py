"""GPU parity THROUGH the compiled torch-extension shim, imported under the reference's module
names (``attention_ops``, ``cache_ops``): plain / prev / post attention with the reference's
positional argument lists (csrc/attention.cpp:4-47) and fill / gather / copy / swap of cache blocks
(3rdparty/vllm/csrc/cache.cpp:6-28), against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from parrotserve_b200 import torch_ops
from tests.helpers import assert_close_to_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bits(x):
    return x.detach().cpu().contiguous().view(torch.int16 if x.element_size() == 2 else torch.int32).numpy()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("b", [16, 8, 32])
def test_attention_ops_through_the_shim(dtype, b):
    attention_ops, _ = torch_ops.load()
    h, d, nb = 4, 128, 160
    x = 16 // torch.empty((), dtype=dtype).element_size()
    g = torch.Generator(device=DEV).manual_seed(40 + b)
    kc = torch.randn((nb, h, d // x, b, x), generator=g, device=DEV).to(dtype)
    vc = torch.randn((nb, h, d, b), generator=g, device=DEV).to(dtype)
    lens_a, lens_b = [37, 1, 4 * b, 4 * b + 1, 200], [5, 64, 3, b, 90]
    rng = np.random.default_rng(b)
    perm = rng.permutation(nb).tolist()

    def tables(lens):
        rows = [[perm.pop() for _ in range((n + b - 1) // b)] for n in lens]
        w = max(len(r) for r in rows)
        return torch.tensor([r + [0] * (w - len(r)) for r in rows], dtype=torch.int32, device=DEV)

    ta, tb = tables(lens_a), tables(lens_b)
    la, lb = (torch.tensor(v, dtype=torch.int32, device=DEV) for v in (lens_a, lens_b))
    n = len(lens_a)
    # q as a strided view of a fused qkv projection, as the models hand it over
    qkv = torch.randn((n, 3 * h * d), generator=g, device=DEV).to(dtype)
    q = qkv[:, : h * d].view(n, h, d)
    hm = torch.arange(h, dtype=torch.int32, device=DEV)
    scale = d ** -0.5
    qf, kf, vf = q.float().cpu(), kc.float().cpu(), vc.float().cpu()

    out = torch.zeros((n, h, d), dtype=dtype, device=DEV)
    unused = torch.zeros((n, ta.shape[1]), dtype=torch.int32, device=DEV)
    nums = ((la + b - 1) // b).to(torch.int32)
    attention_ops.single_query_cached_kv_attention(out, q, kc, vc, hm, scale, ta, unused, nums, la, b, ta.shape[1] * b, None)
    ref_a = orc.gold_grouped_attention(qf, kf, vf, None, None, None, lens_a, ta.tolist())
    assert_close_to_oracle(out, ref_a, dtype, f"shim plain, block {b}")

    # prev over context A, post over context B == attention over A ++ B
    o2 = torch.zeros_like(out)
    m = torch.zeros((n, h), dtype=torch.float32, device=DEV)
    l = torch.zeros((n, h), dtype=torch.float32, device=DEV)
    attention_ops.single_query_cached_kv_prev_attention(o2, q, kc, vc, hm, scale, ta, la, m, l, b, ta.shape[1] * b, None)
    assert_close_to_oracle(o2, ref_a, dtype, f"shim prev, block {b}")
    attention_ops.single_query_cached_kv_post_attention(o2, q, kc, vc, hm, scale, tb, lb, m, l, b, tb.shape[1] * b, None)
    both = []
    for i in range(n):
        ka, va = orc.gather_tokens(kf, vf, ta[i].tolist(), lens_a[i], range(h))
        kb, vb = orc.gather_tokens(kf, vf, tb[i].tolist(), lens_b[i], range(h))
        both.append(orc.gold_row_attention(qf[i], torch.cat([ka, kb]), torch.cat([va, vb]), scale))
    assert_close_to_oracle(o2, torch.stack(both), dtype, f"shim prev + post, block {b}")
    with pytest.raises(RuntimeError):  # the reference's TORCH_CHECK on the block size
        attention_ops.single_query_cached_kv_attention(out, q, kc, vc, hm, scale, ta, unused, nums, la, b * 2, ta.shape[1] * b, None)
    with pytest.raises(RuntimeError):
        attention_ops.single_query_cached_kv_attention(out, q, kc, vc, hm, scale, ta, unused, nums, la, b, ta.shape[1] * b,
                                                       torch.zeros(h, device=DEV))


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_cache_ops_through_the_shim(dtype):
    _, cache_ops = torch_ops.load()
    t, h, d, b, nb = 37, 3, 128, 16, 24
    x = 16 // torch.empty((), dtype=dtype).element_size()
    g = torch.Generator(device=DEV).manual_seed(3)
    kc = torch.randn((nb, h, d // x, b, x), generator=g, device=DEV).to(dtype)
    vc = torch.randn((nb, h, d, b), generator=g, device=DEV).to(dtype)
    qkv = torch.randn((t, 3 * h * d), generator=g, device=DEV).to(dtype)
    _, k, v = (c.view(t, h, d) for c in qkv.chunk(3, dim=-1))
    slots = torch.tensor(np.random.default_rng(1).permutation(nb * b)[:t].astype(np.int32), device=DEV)
    kr, vr = _bits(kc).copy(), _bits(vc).copy()
    orc.fill_reference(_bits(k), _bits(v), kr, vr, slots.cpu().numpy())
    cache_ops.reshape_and_cache(k, v, kc, vc, slots)
    assert np.array_equal(_bits(kc), kr) and np.array_equal(_bits(vc), vr)
    k2, v2 = torch.zeros((t, h, d), dtype=dtype, device=DEV), torch.zeros((t, h, d), dtype=dtype, device=DEV)
    cache_ops.gather_cached_kv(k2, v2, kc, vc, slots)
    assert torch.equal(k2, k) and torch.equal(v2, v)
    # copy_blocks over two layers, swap_blocks device -> host -> device
    kc2, vc2 = kc.clone(), vc.clone()
    before = [c.clone() for c in (kc, vc, kc2, vc2)]
    cache_ops.copy_blocks([kc, kc2], [vc, vc2], {0: [5, 6], 3: [7]})
    for c, old in zip((kc, vc, kc2, vc2), before):
        want = old.clone()
        want[5], want[6], want[7] = old[0], old[0], old[3]
        assert torch.equal(c, want)
    host = torch.zeros((nb,) + tuple(kc.shape[1:]), dtype=dtype).pin_memory()
    cache_ops.swap_blocks(kc, host, {1: 2, 2: 9})
    torch.cuda.synchronize()
    assert torch.equal(host[2], kc[1].cpu()) and torch.equal(host[9], kc[2].cpu())
    back = torch.zeros_like(kc)
    cache_ops.swap_blocks(host, back, {2: 4})
    torch.cuda.synchronize()
    assert torch.equal(back[4], kc[1])
