"""The allocation-free entry point, for hosts that may not call cudaMalloc (a plugin invoked
inside another runtime's capture, a worker whose device memory pool is owned by its engine).

It must give the same attention as the workspace form, and as the CPU oracle, on two calls in a
row: the second call finds the first call's leftovers in the library's fixed scratch array and
must not be affected by them. Such a caller never sees the array's address, so the status word
the kernels leave in it is read through an entry point of its own. Collected last so that a
failure here cannot hide the result of any other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from parrotserve_b200 import _lib
from parrotserve_b200.ops import Workspace

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ATOL = 2e-3  # the tolerance of the attention parity tests


def _problem(seed, num_seqs, num_heads, lens, nb=96):
    g = torch.Generator(device=DEV).manual_seed(seed)
    d, b, x = 128, 16, 8
    q = torch.randn((num_seqs, num_heads, d), generator=g, device=DEV).half()
    kc = torch.randn((nb, num_heads, d // x, b, x), generator=g, device=DEV).half()
    vc = torch.randn((nb, num_heads, d, b), generator=g, device=DEV).half()
    rng = np.random.default_rng(seed)
    width = max((n + b - 1) // b for n in lens)
    tables = np.zeros((num_seqs, width), dtype=np.int32)
    for i, n in enumerate(lens):
        k = (n + b - 1) // b
        tables[i, :k] = rng.permutation(nb)[:k]
    return q, kc, vc, torch.tensor(tables, device=DEV), torch.tensor(lens, dtype=torch.int32, device=DEV)


def _call(static, q, kc, vc, tables, lens):
    lib = _lib.lib()
    s, h, d = q.shape
    out = torch.full_like(q, float("nan"))
    stream = torch.cuda.current_stream().cuda_stream
    head = (out.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), None, d ** -0.5, tables.data_ptr(), lens.data_ptr())
    sizes = (16, tables.shape[1] * 16, s, h, h, d, tables.shape[1], q.stride(0), kc.stride(0), kc.stride(1), kc.shape[0], _lib.PB_F16)
    if static:
        rc = lib.pb_single_query_cached_kv_attention_static(*head, *sizes, stream)
    else:
        need = lib.pb_single_query_workspace_bytes(s, h, d, 16, tables.shape[1])
        ws = Workspace.get(q.device, need, tag="no_alloc_test")
        rc = lib.pb_single_query_cached_kv_attention(*head, *sizes, ws.data_ptr(), ws.numel(), stream)
    torch.cuda.synchronize()
    return rc, out


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    # two different problems back to back through the same fixed scratch
    for seed, lens in ((1, [100, 1, 16, 17, 333, 64]), (2, [5, 250, 31])):
        q, kc, vc, tables, cl = _problem(seed, len(lens), 4, lens)
        rc_w, out_w = _call(False, q, kc, vc, tables, cl)
        rc_s, out_s = _call(True, q, kc, vc, tables, cl)
        assert rc_w == _lib.PB_OK and rc_s == _lib.PB_OK
        assert torch.isfinite(out_s).all()
        assert (out_s.float() - out_w.float()).abs().max().item() <= ATOL
        # the status word of the built-in array: clean after a good call
        word = C.c_int32(-1)
        assert _lib.lib().pb_static_scratch_status(torch.cuda.current_stream().cuda_stream, C.byref(word)) == _lib.PB_OK
        assert word.value == 0
        # and against the CPU oracle (plain paged attention = no prefix group)
        n = len(lens)
        ref = orc.gold_grouped_attention(q.float().cpu(), kc.float().cpu(), vc.float().cpu(), None, None, None,
                                         cl.tolist(), tables.tolist())
        assert (out_s.double().cpu() - ref).abs().max().item() <= ATOL, seed


def test_static_scratch_entry_rejects_oversize_problems():
    lib = _lib.lib()
    cap = lib.pb_static_scratch_bytes()
    assert cap == 32 << 20
    s, h, maxb = 4096, 32, 256  # needs far more than the fixed array
    assert lib.pb_single_query_workspace_bytes(s, h, 128, 16, maxb) > cap
    q, kc, vc, tables, cl = _problem(3, 2, 2, [4, 9], nb=8)
    stream = torch.cuda.current_stream().cuda_stream
    out = torch.empty_like(q)
    rc = lib.pb_single_query_cached_kv_attention_static(
        out.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), None, 128 ** -0.5, tables.data_ptr(), cl.data_ptr(),
        16, maxb * 16, s, h, h, 128, maxb, q.stride(0), kc.stride(0), kc.stride(1), kc.shape[0], _lib.PB_F16, stream)
    assert rc == _lib.PB_ERR_WORKSPACE
