"""Shared helpers of the parity tests: run the CPU oracle on a materialised workload."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

from oracle import attention_oracle as orc

# Tolerance of the attention parity tests (max-abs against the float64-accumulated oracle).
# fp16 and fp32 outputs: 2e-3. bf16 carries 8 significand bits, which enters twice: the stored
# result is rounded to them (up to 2^-9 relative, on every route), and on the tensor-core route the
# softmax weights are rounded to them as the A operand of P.V (the instruction takes both operands
# in one 16-bit format, and V is bf16; an fp16 P beside bf16 V is rejected by the hardware as an
# illegal instruction). The first term is bounded by 2^-8 |ref|, the second by 2^-8 times the same
# attention taken over |V| (`abs_ref`: the weights' rounding errors do not cancel the way the values
# do); a test that has no `abs_ref` at hand uses |ref| for it. What the kernels actually reach is
# logged per test (PB_PARITY_LOG).
ATOL = 2e-3


def tolerance(dtype: torch.dtype, ref: torch.Tensor, abs_ref=None) -> torch.Tensor:
    tol = torch.full_like(ref, ATOL, dtype=torch.float64)
    if dtype == torch.bfloat16:
        spread = ref.abs().double() if abs_ref is None else abs_ref.abs().double()
        tol = tol + (ref.abs().double() + spread) * 2.0 ** -8
    return tol


def assert_close_to_oracle(out: torch.Tensor, ref: torch.Tensor, dtype: torch.dtype, what: str = "", abs_ref=None):
    out = out.detach().double().cpu()
    ref = ref.double()
    assert out.shape == ref.shape, (out.shape, ref.shape)
    assert torch.isfinite(out).all(), f"{what}: non-finite output"
    err = (out - ref).abs()
    tol = tolerance(dtype, ref, abs_ref)
    worst = (err - tol).max().item()
    log = os.environ.get("PB_PARITY_LOG")
    if log:  # measured error of every parity comparison, one JSON line each
        with open(log, "a") as f:
            f.write(json.dumps({"what": what, "dtype": str(dtype).replace("torch.", ""), "max_abs_err": err.max().item(),
                                "max_abs_ref": ref.abs().max().item(), "elements": int(ref.numel())}) + "\n")
    assert worst <= 0, f"{what}: max-abs error {err.max().item():.3e} exceeds tolerance (worst excess {worst:.3e})"


def oracle_for_workload(wl, tensors, rows=None, heads=None):
    """float64 oracle output [len(rows), len(heads), D] for a materialised workload dict."""
    if heads is not None:
        # only the sampled heads leave the device (the full-size caches are several GB)
        hsel = torch.as_tensor(list(heads), device=tensors["query"].device)
        q = tensors["query"].index_select(1, hsel).float().cpu()
        kc = tensors["key_cache"].index_select(1, hsel).float().cpu()
        vc = tensors["value_cache"].index_select(1, hsel).float().cpu()
        heads = list(range(len(heads)))
    else:
        q = tensors["query"].float().cpu()
        kc = tensors["key_cache"].float().cpu()
        vc = tensors["value_cache"].float().cpu()
    return orc.gold_grouped_attention(
        q, kc, vc, wl.group_row_offsets.tolist(), wl.group_prefix_lens.tolist(), wl.group_tables.tolist(),
        wl.suffix_lens.tolist(), wl.suffix_tables.tolist(), rows=rows, heads=heads,
        seg_row_offsets=None if wl.seg_kv_lens is None else wl.seg_row_offsets.tolist(),
        seg_kv_lens=None if wl.seg_kv_lens is None else wl.seg_kv_lens.tolist(),
        seg_tables=None if wl.seg_kv_lens is None else wl.seg_tables.tolist(),
    )


def sample_rows(wl, n: int, seed: int = 0):
    """A seeded sample of rows that always contains each group's first row and the rows with the
    shortest and longest private context."""
    rng = np.random.default_rng(seed)
    must = set()
    offs = wl.group_row_offsets
    for g in range(wl.num_groups):
        if offs[g + 1] > offs[g]:
            must.add(int(offs[g]))
    must.add(int(np.argmin(wl.suffix_lens)))
    must.add(int(np.argmax(wl.suffix_lens)))
    rest = [r for r in rng.permutation(wl.num_rows).tolist() if r not in must]
    rows = sorted(must | set(rest[: max(0, n - len(must))]))
    return rows
