"""Runs one shared-prefix attention shape a few times and prints its device time: the command to
put under a profiler when a single shape (rather than a whole benchmark configuration) is of interest.

    python -m parrotserve_b200.probe --rows 1024 --prefix 2048 --suffix 1 --heads 32 --iters 5

One prefix group of ``--prefix`` tokens shared by ``--rows`` single-token queries, each with a
private suffix of ``--suffix`` tokens; fp16, head size 128, block size 16, seeded random block tables.

    python -m parrotserve_b200.probe --sampler --rows 64 --vocab 32000 --top-p 0.9

times the token sampler instead: ``--rows`` rows of ``--vocab`` seeded random fp16 logits, temperature 0.8.
"""
from __future__ import annotations

import argparse

import numpy as np
import torch

from . import AttentionCall
from .workloads import _assemble


def sampler_probe(args) -> None:
    from .ops import sample_top_p

    g = torch.Generator(device="cuda:0").manual_seed(0)
    logits = (torch.randn((args.rows, args.vocab), generator=g, device="cuda:0") * 2.5).half()
    temp = torch.full((args.rows,), 0.8, device="cuda:0")
    top_p = torch.full((args.rows,), args.top_p, device="cuda:0") if args.top_p < 1.0 else None
    u = torch.rand(args.rows, generator=g, device="cuda:0")
    for _ in range(2):
        ids = sample_top_p(logits, temp, top_p, u)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        ids = sample_top_p(logits, temp, top_p, u)
    e1.record()
    torch.cuda.synchronize()
    print(f"sampler rows {args.rows} vocab {args.vocab} top_p {args.top_p}: "
          f"{e0.elapsed_time(e1) / args.iters * 1e3:.1f} us per call (launch overhead included), first ids {ids[:4].tolist()}")


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", type=int, default=64)
    ap.add_argument("--prefix", type=int, default=4096)
    ap.add_argument("--suffix", type=int, default=1)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--dense-ctas", type=int, default=0, help="0 = let the planner split the SMs")
    ap.add_argument("--sampler", action="store_true", help="time the token sampler instead of attention")
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--top-p", type=float, default=0.9)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the path has no CPU implementation")
    if args.sampler:
        return sampler_probe(args)
    rng = np.random.default_rng(0)
    wl = _assemble("probe", 2, torch.float16, args.heads, [args.prefix], [0] * args.rows,
                   np.full(args.rows, args.suffix, dtype=np.int64), rng=rng)
    t = wl.materialize("cuda:0")
    out = torch.empty_like(t["query"])
    call = AttentionCall(
        num_rows=wl.num_rows, num_heads=args.heads, head_size=128, block_size=16, dtype=wl.dtype, device=out.device,
        suffix_lens=t["suffix_lens"], suffix_tables=t["suffix_tables"], group_row_offsets=t["group_row_offsets"],
        group_prefix_lens=t["group_prefix_lens"], group_tables=t["group_tables"], dense_ctas=args.dense_ctas)
    call.plan(t["query"], out, t["key_cache"], t["value_cache"])
    for _ in range(2):
        call.run(t["query"], out, t["key_cache"], t["value_cache"])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        call.run(t["query"], out, t["key_cache"], t["value_cache"])
    e1.record()
    torch.cuda.synchronize()
    print(f"rows {args.rows} prefix {args.prefix} suffix {args.suffix} heads {args.heads}: "
          f"{e0.elapsed_time(e1) / args.iters * 1e3:.1f} us per call, device status {call.status()}")


if __name__ == "__main__":
    main()
