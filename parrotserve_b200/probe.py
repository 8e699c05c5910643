"""Runs one shared-prefix attention shape a few times and prints its device time: the command to
put under a profiler when a single shape (rather than a whole benchmark configuration) is of interest.

    python -m parrotserve_b200.probe --rows 1024 --prefix 2048 --suffix 1 --heads 32 --iters 5

One prefix group of ``--prefix`` tokens shared by ``--rows`` single-token queries, each with a
private suffix of ``--suffix`` tokens; fp16, head size 128, block size 16, seeded random block tables.
"""
from __future__ import annotations

import argparse

import numpy as np
import torch

from . import AttentionCall
from .workloads import _assemble


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", type=int, default=64)
    ap.add_argument("--prefix", type=int, default=4096)
    ap.add_argument("--suffix", type=int, default=1)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--dense-ctas", type=int, default=0, help="0 = let the planner split the SMs")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the path has no CPU implementation")
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
