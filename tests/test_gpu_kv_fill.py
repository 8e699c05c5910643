"""GPU parity of the cache fill / gather / moves: bit-exact against the numpy references."""
import numpy as np
import pytest
import torch

import parrotserve_b200 as pb
from parrotserve_b200.workloads import make_workload
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    return t.view(torch.int16 if t.element_size() == 2 else torch.int32).numpy()


def _caches(dtype, nb, h, d, b, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = 16 // torch.empty((), dtype=dtype).element_size()
    kc = torch.randn((nb, h, d // x, b, x), generator=g, device=DEV).to(dtype)
    vc = torch.randn((nb, h, d, b), generator=g, device=DEV).to(dtype)
    return kc, vc, g


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("t,h,d,b,nb", [(3, 2, 16, 8, 2), (37, 3, 128, 16, 64), (300, 5, 64, 32, 40), (129, 2, 256, 16, 32)])
def test_fill_scattered_slots_bit_exact(dtype, t, h, d, b, nb):
    kc, vc, g = _caches(dtype, nb, h, d, b, 0)
    # strided views of a fused qkv tensor, as the reference's own test builds them
    qkv = torch.randn((t, 3, h, d), generator=g, device=DEV).to(dtype)
    _, key, value = qkv.unbind(dim=1)
    rng = np.random.default_rng(1)
    slots = rng.choice(nb * b, size=t, replace=False)
    kr, vr = bits(kc).copy(), bits(vc).copy()
    orc.fill_reference(bits(key), bits(value), kr, vr, slots)
    pb.vllm_reshape_and_cache(key, value, kc, vc, torch.tensor(slots, dtype=torch.int32, device=DEV))
    assert np.array_equal(bits(kc), kr) and np.array_equal(bits(vc), vr)
    # and back
    k2, v2 = torch.zeros_like(key.contiguous()), torch.zeros_like(value.contiguous())
    pb.gather_cached_kv(k2, v2, kc, vc, torch.tensor(slots, dtype=torch.int64, device=DEV))
    assert np.array_equal(bits(k2), bits(key)) and np.array_equal(bits(v2), bits(value))


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_fill_runs_partial_blocks_and_skips(dtype):
    # prefill-like runs: full blocks, a run starting mid-block, a run ending mid-block, lone tokens, skipped tokens
    h, d, b, nb = 3, 128, 16, 32
    kc, vc, g = _caches(dtype, nb, h, d, b, 2)
    runs = [(5 * b, 3 * b), (9 * b + 7, 20), (14 * b, 5), (20 * b + 15, 1), (21 * b, 1), (2 * b + 3, 12)]
    slots = []
    for s0, n in runs:
        slots += list(range(s0, s0 + n))
    slots[40] = -1  # a padded token
    slots = np.asarray(slots, dtype=np.int64)
    t = len(slots)
    key = torch.randn((t, h, d), generator=g, device=DEV).to(dtype)
    value = torch.randn((t, h, d), generator=g, device=DEV).to(dtype)
    kr, vr = bits(kc).copy(), bits(vc).copy()
    orc.fill_reference(bits(key), bits(value), kr, vr, slots)
    pb.vllm_reshape_and_cache(key, value, kc, vc, torch.tensor(slots, device=DEV))
    assert np.array_equal(bits(kc), kr) and np.array_equal(bits(vc), vr)
    keep = slots >= 0
    k2, v2 = torch.zeros_like(key), torch.zeros_like(value)
    pb.gather_cached_kv(k2, v2, kc, vc, torch.tensor(slots, device=DEV))
    assert np.array_equal(bits(k2)[keep], bits(key)[keep]) and np.array_equal(bits(v2)[keep], bits(value)[keep])
    assert not bits(k2)[~keep].any()


@pytest.mark.parametrize("dtype,b", [(torch.float16, 16), (torch.float32, 16), (torch.bfloat16, 32), (torch.float16, 8)])
def test_fill_prefill_sized_batch_bit_exact(dtype, b):
    """A prefill-sized batch (more than 2048 tokens, where the launch uses fewer head groups per token): runs of whole
    blocks, runs that start or end inside a block, lone tokens and padded (-1) tokens, in random order."""
    h, d, nb = 3, 128, 400
    kc, vc, g = _caches(dtype, nb, h, d, b, 5)
    rng = np.random.default_rng(77)
    order = rng.permutation(nb).tolist()
    slots = []
    while len(slots) < 2600 and order:
        blk = order.pop()
        kind = int(rng.integers(0, 6))
        if kind <= 2:  # a request's run over several whole blocks (physically scattered), odd length so windows shift
            n_blocks = int(rng.integers(1, 5))
            blks = [blk] + [order.pop() for _ in range(min(n_blocks - 1, len(order)))]
            for bb in blks:
                slots += list(range(bb * b, bb * b + b))
            tail = order.pop() if order else None
            if tail is not None:
                slots += list(range(tail * b, tail * b + int(rng.integers(1, b))))
        elif kind == 3:  # starts inside a block
            off = int(rng.integers(1, b))
            slots += list(range(blk * b + off, blk * b + b))
        elif kind == 4:  # a lone token
            slots.append(blk * b + int(rng.integers(0, b)))
        else:  # padded tokens
            slots += [-1] * int(rng.integers(1, 4))
    slots = np.asarray(slots, dtype=np.int64)
    t = len(slots)
    assert t >= 2048
    key = torch.randn((t, h, d), generator=g, device=DEV).to(dtype)
    value = torch.randn((t, h, d), generator=g, device=DEV).to(dtype)
    kr, vr = bits(kc).copy(), bits(vc).copy()
    orc.fill_reference(bits(key), bits(value), kr, vr, slots)
    pb.vllm_reshape_and_cache(key, value, kc, vc, torch.tensor(slots, device=DEV))
    assert np.array_equal(bits(kc), kr) and np.array_equal(bits(vc), vr)
    keep = slots >= 0
    k2, v2 = torch.zeros_like(key), torch.zeros_like(value)
    pb.gather_cached_kv(k2, v2, kc, vc, torch.tensor(slots, device=DEV))
    assert np.array_equal(bits(k2)[keep], bits(key)[keep]) and np.array_equal(bits(v2)[keep], bits(value)[keep])
    assert not bits(k2)[~keep].any()


def test_fill_config4_shape_and_decode_reference_layout():
    wl = make_workload(4, shrink=8, num_heads=4)
    t = wl.materialize(DEV)
    kc, vc = t["key_cache"], t["value_cache"]
    kr, vr = bits(kc).copy(), bits(vc).copy()
    orc.fill_reference(bits(t["k_new"]), bits(t["v_new"]), kr, vr, wl.fill_slots)
    pb.vllm_reshape_and_cache(t["k_new"], t["v_new"], kc, vc, t["fill_slots"])
    assert np.array_equal(bits(kc), kr) and np.array_equal(bits(vc), vr)
    # the reference AttnFunc's 2-D [num_jobs, 1] mapping of a pure-decode batch is accepted as is
    wl2 = make_workload(2, shrink=8, num_heads=2)
    t2 = wl2.materialize(DEV)
    kr, vr = bits(t2["key_cache"]).copy(), bits(t2["value_cache"]).copy()
    orc.fill_reference(bits(t2["k_new"]), bits(t2["v_new"]), kr, vr, wl2.fill_slots)
    pb.vllm_reshape_and_cache(t2["k_new"], t2["v_new"], t2["key_cache"], t2["value_cache"],
                              t2["fill_slots"].to(torch.int32).view(-1, 1))
    assert np.array_equal(bits(t2["key_cache"]), kr) and np.array_equal(bits(t2["value_cache"]), vr)
    with pytest.raises(RuntimeError):  # a zero-padded ragged 2-D mapping is ambiguous
        pb.vllm_reshape_and_cache(t2["k_new"], t2["v_new"], t2["key_cache"], t2["value_cache"],
                                  torch.zeros((len(wl2.fill_slots), 2), dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_move_tokens_from_blocked_caches(dtype):
    h, d, b, nb = 5, 128, 16, 24
    kc, vc, g = _caches(dtype, nb, h, d, b, 3)
    rng = np.random.default_rng(4)
    n = 200
    src = rng.integers(0, nb * b, size=n)
    dst = rng.permutation(256)[:n]
    kd = torch.zeros((256, h, d), dtype=dtype, device=DEV)
    vd = torch.zeros((256, h, d), dtype=dtype, device=DEV)
    pb.move_tokens_from_blocked_k_cache(kc, kd, torch.tensor(src, device=DEV), torch.tensor(dst, device=DEV))
    pb.move_tokens_from_blocked_v_cache(vc, vd, torch.tensor(src, device=DEV), torch.tensor(dst, device=DEV))
    kref, vref = orc.gather_reference(bits(kc), bits(vc), src)
    ke, ve = np.zeros_like(bits(kd)), np.zeros_like(bits(vd))
    ke[dst], ve[dst] = kref, vref
    assert np.array_equal(bits(kd), ke) and np.array_equal(bits(vd), ve)
    with pytest.raises(AssertionError):
        pb.move_tokens_from_blocked_k_cache(kc, kd, torch.tensor(src, device=DEV), torch.tensor(dst[:-1], device=DEV))


@pytest.mark.parametrize("dtype,h,d", [(torch.float16, 96, 128), (torch.float32, 3, 20), (torch.bfloat16, 1, 7)])
def test_discontinuous_move_tokens(dtype, h, d):
    g = torch.Generator(device=DEV).manual_seed(5)
    src = torch.randn((300, h, d), generator=g, device=DEV).to(dtype)
    dst = torch.randn((280, h, d), generator=g, device=DEV).to(dtype)
    rng = np.random.default_rng(6)
    si, di = rng.permutation(300)[:150], rng.permutation(280)[:150]
    expect = bits(dst).copy()
    orc.move_rows_reference(bits(src), expect, si, di)
    pb.discontinuous_move_tokens(src, dst, torch.tensor(si, device=DEV), torch.tensor(di, device=DEV))
    assert np.array_equal(bits(dst), expect)


def test_fill_then_attend_roundtrip_at_full_config2():
    """Size-independent property at the benchmark shape: after the fill, gathering the filled
    slots returns the new rows bit for bit, and every other cache byte is untouched."""
    wl = make_workload(2)
    t = wl.materialize(DEV)
    kc, vc = t["key_cache"], t["value_cache"]
    k0, v0 = kc.clone(), vc.clone()
    pb.vllm_reshape_and_cache(t["k_new"], t["v_new"], kc, vc, t["fill_slots"])
    k2, v2 = torch.empty_like(t["k_new"]), torch.empty_like(t["v_new"])
    pb.gather_cached_kv(k2, v2, kc, vc, t["fill_slots"])
    assert torch.equal(k2, t["k_new"]) and torch.equal(v2, t["v_new"])
    blk = torch.unique(t["fill_slots"] // 16)
    mask = torch.ones(kc.shape[0], dtype=torch.bool, device=DEV)
    mask[blk] = False
    assert torch.equal(kc[mask], k0[mask]) and torch.equal(vc[mask], v0[mask])


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_copy_blocks_and_swap_blocks_bit_exact(dtype):
    """Whole-block copies inside the caches of several layers and swaps GPU <-> host, against numpy
    indexing; the shapes and mappings follow the reference's own cache test
    (3rdparty/vllm/tests/kernels/test_cache.py:9-67)."""
    from parrotserve_b200 import cache_ops

    layers, nb, h, d, b = 3, 40, 4, 64, 16
    x = 16 // torch.empty((), dtype=dtype).element_size()
    g = torch.Generator(device=DEV).manual_seed(5)
    kcs = [torch.randn((nb, h, d // x, b, x), generator=g, device=DEV).to(dtype) for _ in range(layers)]
    vcs = [torch.randn((nb, h, d, b), generator=g, device=DEV).to(dtype) for _ in range(layers)]
    rng = np.random.default_rng(6)
    srcs = rng.choice(nb // 2, size=6, replace=False).tolist()
    free = (nb // 2 + rng.permutation(nb // 2)).tolist()
    mapping = {s: [free.pop(), free.pop()] if i % 2 else [free.pop()] for i, s in enumerate(srcs)}
    want_k, want_v = [bits(k).copy() for k in kcs], [bits(v).copy() for v in vcs]
    for s, dsts in mapping.items():
        for dd in dsts:
            for wk, wv in zip(want_k, want_v):
                wk[dd], wv[dd] = wk[s], wv[s]
    cache_ops.copy_blocks(kcs, vcs, mapping)
    for k, v, wk, wv in zip(kcs, vcs, want_k, want_v):
        assert np.array_equal(bits(k), wk) and np.array_equal(bits(v), wv)
    # swap out to a pinned host cache and back in at other places (a run of consecutive pairs and lone ones)
    host = torch.zeros((24,) + tuple(kcs[0].shape[1:]), dtype=dtype).pin_memory()
    out_map = {3: 10, 4: 11, 5: 12, 20: 0, 31: 23}
    cache_ops.swap_blocks(kcs[0], host, out_map)
    torch.cuda.synchronize()
    for s, dd in out_map.items():
        assert np.array_equal(bits(host[dd]), want_k[0][s])
    in_map = {10: 39, 11: 1, 0: 2}
    cache_ops.swap_blocks(host, kcs[1], in_map)
    torch.cuda.synchronize()
    for s, dd in in_map.items():
        assert np.array_equal(bits(kcs[1][dd]), bits(host[s]))
    with pytest.raises(RuntimeError):  # a block outside the destination cache is refused before anything is copied
        cache_ops.swap_blocks(kcs[0], host, {0: 24})
