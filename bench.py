#!/usr/bin/env python
"""Benchmark of the shared-prefix decode attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-gpu]
                    [--config 2|3|4|5] [--split heads|groups] [--heads H]

One step = one attention-layer call of the continuous-batching iteration over one batch of
synthetic input: KV fill of the iteration's new tokens, shared-prefix stage, per-sequence suffix
stage, merge. Workload (N = 1): the LLaMA-7B decode shape, fp16, 32 heads x 128, one 4096-token
shared prefix, 64 sequences with private suffixes U{32..512}, paged KV with block 16 and seeded
random block tables.

With N GPUs (launched by torchrun, one rank per GPU) the SAME batch is split by attention heads:
rank r owns a contiguous range of the heads of every cache block, attention and fill are
independent per head, so nothing is exchanged on the path (strong scaling; `value` = the batch's
tokens / max-over-ranks step time). Outside the timed region the ranks' outputs are gathered over
NCCL and checked on rank 0 against the CPU oracle on a seeded sample of (row, head) pairs that
covers every rank. `--split groups` is the other collective-free partition (every rank its own
prefix group and rows: weak scaling); at N > 1 its number is reported in the sub-key `groups_split`.

Timing: W warm-up steps, then R regions of EXACTLY K steps each (CUDA events, barrier and device
synchronisation on both sides, max over ranks per region); `value` and `ms_per_step` are the MEDIAN
region, min and max are listed beside it. The steps rotate over distinct cache copies (or touch
more than L2 per step), so no step finds its KV in L2.

Prints ONE JSON line (rank 0): metric "decode_attn_tokens_per_s", `value` with inputs resident in
HBM, `e2e` through the host-buffer entry point with the copies inside the timed region,
`roofline` of the dominant (suffix) kernel against the measured HBM peak, `cpu_baseline` = the
oracle's port of the reference's torch attention timed on the host cores, `reference_gpu` = the
reference's own GPU kernels on this GPU when their build is present (baseline/_ref).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import re
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "decode_attn_tokens_per_s"
UNIT = "tokens/s"
REGIONS = 25  # timed regions of K steps each; the median is reported


def _peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def _captured_traffic(workload: str, heads: int):
    """DRAM bytes of one suffix-kernel launch from the committed ncu summary of that kernel, or None
    when the summary was taken on another workload (the summary states both in one line)."""
    f = ROOT / "profiles" / "sq_attn_kernel_cfg2_ncu_full.md"
    if not f.exists():
        return None
    m = re.search(r"traffic_bytes_per_launch\s*=\s*(\d+)\s*\(workload\s+(\S+),\s*(\d+)\s+heads\)", f.read_text())
    if not m or m.group(2) != workload or int(m.group(3)) != heads:
        return None
    return float(m.group(1))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


class CpuReference:
    """The port of the reference's torch reference attention
    (parrot/engine/builtin/kernels/shared_flash_decoding.py:382-404) on the host cores: fp32,
    over the CONCATENATED block table (prefix ++ suffix), which is what that function computes."""

    def __init__(self, wl, n_seqs: int):
        import numpy as np
        import torch

        from oracle import attention_oracle as orc

        self.orc, self.wl, self.n = orc, wl, n_seqs
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        t = wl.materialize("cpu")
        self.q = t["query"][:n_seqs].float()
        self.kc, self.vc = t["key_cache"].float(), t["value_cache"].float()
        plen = int(wl.group_prefix_lens[0])
        ptab = wl.group_tables[0][: (plen + wl.block_size - 1) // wl.block_size]
        rows, lens = [], []
        for r in range(n_seqs):
            nb = (int(wl.suffix_lens[r]) + wl.block_size - 1) // wl.block_size
            rows.append(np.concatenate([ptab, wl.suffix_tables[r][:nb]]))
            lens.append(plen + int(wl.suffix_lens[r]))
        width = max(len(r) for r in rows)
        self.tables = torch.zeros((n_seqs, width), dtype=torch.long)
        for i, r in enumerate(rows):
            self.tables[i, : len(r)] = torch.from_numpy(r.astype(np.int64))
        self.hm = torch.arange(self.q.shape[1])
        self.cl = torch.tensor(lens, dtype=torch.int32)
        self.sample = (f"{n_seqs} of {wl.num_rows} sequences x {self.q.shape[1]} heads of {wl.name}, fp32, "
                       f"prefix+suffix gathered per sequence, {self.cores} host threads")

    def run(self, n=None) -> float:
        """One pass over the sample; returns decode tokens/s."""
        n = self.n if n is None else n
        t0 = time.perf_counter()
        self.orc.reference_port_paged_attention(self.q[:n], self.kc, self.vc, self.hm, self.cl[:n], self.tables[:n])
        return n / (time.perf_counter() - t0)


def _config(full, world: int, split_heads: bool):
    """The workload description both arms print (identical for the same command line)."""
    h = full.num_heads // world if split_heads else full.num_heads
    return {
        "workload": full.name, "heads": full.num_heads, "heads_per_gpu": h, "head_size": full.head_size,
        "block_size": full.block_size, "prefix_tokens": int(full.group_prefix_lens.sum()), "sequences": full.num_rows,
        "suffix_tokens": int(full.suffix_lens.sum()), "new_tokens_filled_per_step": len(full.fill_slots),
        "partition": (f"one batch, its {full.num_heads} heads split over the ranks ({h} per GPU), no collective on the path"
                      if split_heads else ("one GPU" if world == 1 else "one prefix group (its own batch) per GPU, no collective on the path")),
    }


def run_reference(args):
    """`--impl reference`: the reference's own CPU implementation of the path (its torch
    reference attention, restated in oracle/), all host threads, on a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from parrotserve_b200.workloads import make_workload

    wl = make_workload(args.config, num_heads=args.heads or None)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    ref = CpuReference(wl, min(wl.num_rows, 16))
    for _ in range(args.warmup):
        ref.run(2)
    t0 = time.perf_counter()
    rates = [ref.run() for _ in range(args.steps)]
    dt = (time.perf_counter() - t0) / max(1, args.steps)
    value = sum(rates) / len(rates)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 and args.split == "heads" else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": _config(wl, world, world > 1 and args.split == "heads"),
        "note": "reference torch attention (CPU port) on the host cores of rank 0, bounded sample per step",
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": ref.cores, "kind": "port", "sample": "each step: " + ref.sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_reference_gpu(args):
    """`--impl reference-gpu`: the reference's own GPU kernels (built unmodified into baseline/_ref/
    by baseline/build_ref.py) on this GPU and this workload, beside ours. One JSON line."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch

    import parrotserve_b200 as pb
    from baseline import ref_gpu
    from parrotserve_b200.workloads import make_workload

    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference-gpu", "unavailable": "no CUDA device"}))
        return
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    wl = make_workload(2)
    sets = [wl.materialize(dev, seed=2002 + 17 * c) for c in range(4)]
    for t in sets:
        pb.vllm_reshape_and_cache(t["k_new"], t["v_new"], t["key_cache"], t["value_cache"], t["fill_slots"])
    # this library's results on copy 0 (parity-tested against the CPU oracle), to compare the
    # reference kernels' results with: whole attention, shared prefix alone, private suffixes alone
    t = sets[0]
    plen = int(wl.group_prefix_lens[0])
    ours = {
        "full": pb.flash_paged_attention(t["query"], t["key_cache"], t["value_cache"], None, plen, t["group_tables"][0],
                                         t["suffix_lens"], t["suffix_tables"]),
        "prefix": pb.flash_paged_attention(t["query"], t["key_cache"], t["value_cache"], None, plen, t["group_tables"][0],
                                           torch.zeros_like(t["suffix_lens"]), t["suffix_tables"]),
        "suffix": pb.vllm_paged_attention(t["query"], t["key_cache"], t["value_cache"], None, t["suffix_lens"], t["suffix_tables"]),
    }
    torch.cuda.synchronize(dev)
    rep = ref_gpu.run(wl, sets, args.steps, args.warmup, ours=ours)
    print(json.dumps({"impl": "reference-gpu", "metric": METRIC, "unit": UNIT, **rep}))


def run_probe(args):
    """`--probe rows,prefix,suffix[,heads[,dense_ctas]]`: one shared-prefix attention shape a few
    times (one prefix group shared by `rows` single-token queries, each with a private suffix), or
    `--probe-sampler rows,vocab,top_p`: the token sampler. The command to put under a profiler when
    one shape rather than a benchmark configuration is of interest; prints the device time per call."""
    import numpy as np
    import torch

    import parrotserve_b200 as pb
    from parrotserve_b200.workloads import _assemble

    dev = torch.device("cuda", 0)
    iters = max(1, args.steps if args.steps < 50 else 5)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.probe_sampler:
        rows, vocab, top_p = args.probe_sampler.split(",")
        rows, vocab, top_p = int(rows), int(vocab), float(top_p)
        g = torch.Generator(device=dev).manual_seed(0)
        logits = (torch.randn((rows, vocab), generator=g, device=dev) * 2.5).half()
        temp = torch.full((rows,), 0.8, device=dev)
        tp = torch.full((rows,), top_p, device=dev) if top_p < 1.0 else None
        u = torch.rand(rows, generator=g, device=dev)
        fn = lambda: pb.sample_top_p(logits, temp, tp, u)
        what = f"sampler rows {rows} vocab {vocab} top_p {top_p}"
    else:
        v = [int(x) for x in args.probe.split(",")]
        rows, prefix, suffix = v[0], v[1], v[2]
        heads = v[3] if len(v) > 3 else 32
        dense_ctas = v[4] if len(v) > 4 else 0
        rng = np.random.default_rng(0)
        wl = _assemble("probe", 2, torch.float16, heads, [prefix], [0] * rows, np.full(rows, suffix, dtype=np.int64), rng=rng)
        t = wl.materialize(dev)
        out = torch.empty_like(t["query"])
        call = pb.AttentionCall(
            num_rows=wl.num_rows, num_heads=heads, head_size=128, block_size=16, dtype=wl.dtype, device=dev,
            suffix_lens=t["suffix_lens"], suffix_tables=t["suffix_tables"], group_row_offsets=t["group_row_offsets"],
            group_prefix_lens=t["group_prefix_lens"], group_tables=t["group_tables"], dense_ctas=dense_ctas,
            dense_row_tile=args.dense_row_tile)
        call.plan(t["query"], out, t["key_cache"], t["value_cache"])
        fn = lambda: call.run(t["query"], out, t["key_cache"], t["value_cache"])
        what = f"attention rows {rows} prefix {prefix} suffix {suffix} heads {heads}"
    for _ in range(2):
        fn()
    torch.cuda.synchronize(dev)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize(dev)
    print(json.dumps({"probe": what, "us_per_call": e0.elapsed_time(e1) / iters * 1e3, "calls": iters}))


def _stats(ms_regions, steps):
    per = sorted(m / steps for m in ms_regions)
    return {"median": statistics.median(per), "min": per[0], "max": per[-1], "regions": len(per)}


def _verify(wl, full_heads, t, out, world, rank, dist):
    """Outside the timed region: gathers every rank's output over NCCL (along the head dimension) and
    checks, on rank 0, a seeded sample of (row, head) pairs that covers every rank and every prefix
    group against the CPU oracle. The K/V the oracle needs is cut out on the device: only the blocks
    the sampled rows attend, the first head of every rank."""
    import torch

    from oracle import attention_oracle as orc
    from parrotserve_b200.shard import compact_sample, gather_heads, sample_rows_every_group

    if wl.seg_kv_lens is not None:
        return {"note": "not verified here (causal segments): see tests/test_gpu_attention.py"}
    rows = sample_rows_every_group(wl, 12, seed=7)
    q1, kc1, vc1, meta = compact_sample(wl, t, rows, local_head=0)
    if world > 1:
        pieces = []
        for x in (q1, kc1, vc1):
            buf = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(buf, x)
            pieces.append(buf)
        out_full = gather_heads(out)  # [rows, all heads, D]
    else:
        pieces = [[q1], [kc1], [vc1]]
        out_full = out
    if rank != 0:
        return None
    per_rank = full_heads // world
    worst = 0.0
    for r in range(world):
        q, kc, vc = (pieces[i][r].float().cpu() for i in range(3))
        ref = orc.gold_grouped_attention(q, kc, vc, meta["group_row_offsets"], meta["group_prefix_lens"], meta["group_tables"],
                                         meta["suffix_lens"], meta["suffix_tables"])
        got = out_full[rows][:, r * per_rank].double().cpu()
        worst = max(worst, float((got - ref[:, 0]).abs().max().item()))
    return {"pairs": len(rows) * world, "rows": len(rows), "heads": [r * per_rank for r in range(world)],
            "max_abs_vs_oracle": worst, "within_2e-3": bool(worst <= 2e-3),
            "how": "outputs all-gathered over NCCL along the head dimension; oracle on the first head of every rank x a seeded "
                   "row sample that contains every prefix group"}


def run_ours(args):
    import torch
    import torch.distributed as dist

    import parrotserve_b200 as pb
    from parrotserve_b200 import _lib
    from parrotserve_b200.shard import head_range, max_over_ranks
    from parrotserve_b200.workloads import make_workload

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the path has no CPU implementation")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    full = make_workload(args.config, num_heads=args.heads or None)
    full_heads = full.num_heads
    split_heads = args.split == "heads" and world > 1
    if split_heads:
        if full_heads % world:
            raise SystemExit(f"{full_heads} heads do not split evenly over {world} ranks")
        my_heads = list(head_range(full_heads, world, rank))
    else:
        my_heads = list(range(full_heads))
    wl = make_workload(args.config, num_heads=len(my_heads))
    h = len(my_heads)
    # rotate over distinct cache copies so no step finds its KV in L2; the larger configurations
    # (several GB touched per step) need no rotation and would not fit four times
    copies = 4 if args.config <= 2 else 1
    # payload is generated per (seed, global head): a head's content does not depend on N. With the
    # groups split every rank is another batch, so the seed carries the rank.
    seed0 = 2000 + args.config + (0 if split_heads or world == 1 else 1000 * rank)
    sets = [wl.materialize(dev, heads=my_heads, seed=seed0 + 17 * c) for c in range(copies)]
    t0 = sets[0]
    out = torch.empty_like(t0["query"])
    tuning = dict(suffix_chunk_blocks=args.chunk, dense_ctas=args.dense_ctas, dense_row_tile=args.dense_row_tile)
    call = pb.AttentionCall(
        num_rows=wl.num_rows, num_heads=h, head_size=wl.head_size, block_size=wl.block_size, dtype=wl.dtype, device=dev,
        suffix_lens=t0["suffix_lens"], suffix_tables=t0["suffix_tables"], group_row_offsets=t0["group_row_offsets"],
        group_prefix_lens=t0["group_prefix_lens"], group_tables=t0["group_tables"], seg_row_offsets=t0.get("seg_row_offsets"),
        seg_kv_lens=t0.get("seg_kv_lens"), seg_tables=t0.get("seg_tables"),
        slot_mapping=None if args.separate_fill else t0["fill_slots"], **tuning)
    call.plan(t0["query"], out, t0["key_cache"], t0["value_cache"])  # once per iteration, reused by every layer
    stream = torch.cuda.current_stream(dev)
    has_dense = wl.dtype in (torch.float16, torch.bfloat16)
    # every query row brings one new token (decode rows their next token, prefill rows themselves): the
    # attention call performs the KV fill; for a decode batch that is no launch of its own
    fill_launch = 1 if (args.separate_fill or wl.seg_kv_lens is not None) else 0
    launches_per_step = fill_launch + (1 if has_dense else 0) + 2  # (fill,) dense prefix, suffix, merge

    def step(i, ev=None):
        t = sets[i % copies]
        if ev is not None:  # the library records these around the suffix kernel of the next call
            _lib.lib().pb_attn_set_timing_events(ev[0].cuda_event, ev[1].cuda_event)
        if args.separate_fill:
            pb.vllm_reshape_and_cache(t["k_new"], t["v_new"], t["key_cache"], t["value_cache"], t["fill_slots"])
            call.run(t["query"], out, t["key_cache"], t["value_cache"])
        else:
            call.run(t["query"], out, t["key_cache"], t["value_cache"], key_new=t["k_new"], value_new=t["v_new"])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for i in range(args.warmup):
        step(i)
    barrier()
    if call.status() != 0:
        raise SystemExit(f"device status {call.status()}")
    verified = None
    if not args.no_verify:
        step(0)  # `out` = the result on cache copy 0, the copy the verification reads
        barrier()
        verified = _verify(wl, full_heads, t0, out, world if split_heads else 1, rank if split_heads else 0, dist)

    # ---- timed regions: exactly K steps each, device-timed ----
    K = args.steps
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # The K steps are replayed from CUDA graphs of a few dozen steps each (about the layer calls of one forward pass), so the number does not depend on
    # how fast this host issues launches (a serving engine captures its decode iteration the same
    # way); the same K steps issued from Python are timed beside it and the faster way is reported.
    graph, graph_steps = None, 0
    if not args.eager:
        for cand in ((args.graph_steps,) if args.graph_steps > 0 else ()) + (40, 8, 4, 5, 10, 2, 1):
            if K % cand == 0 and cand % copies == 0:
                graph_steps = cand
                break
        if graph_steps:
            try:
                graph = torch.cuda.CUDAGraph()
                side = torch.cuda.Stream(device=dev)
                side.wait_stream(stream)
                with torch.cuda.graph(graph, stream=side):
                    for i in range(graph_steps):
                        step(args.warmup + i)
                torch.cuda.synchronize(dev)
            except RuntimeError:
                graph = None

    def timed(fn):
        barrier()
        e0.record(stream)
        fn()
        e1.record(stream)
        barrier()
        return e0.elapsed_time(e1)

    def eager_steps():
        for i in range(K):
            step(args.warmup + i)

    def graph_replay():
        for _ in range(K // graph_steps):
            graph.replay()

    regions = max(1, args.regions)
    ms_eager = [timed(eager_steps) for _ in range(max(3, regions // 5))]
    ms_graph = [timed(graph_replay) for _ in range(regions)] if graph is not None else []
    # Extra pass with the suffix kernel bracketed by CUDA events (recorded by the library on the
    # launching stream). Bracketing serialises it against the prefix kernel it normally overlaps
    # with, so this pass gives the kernel's own duration, not the step time.
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    for a, b in kev:
        a.record(stream), b.record(stream)
    barrier()
    for i in range(K):
        step(args.warmup + i, kev[i])
    barrier()
    suffix_ms = statistics.median(a.elapsed_time(b) for a, b in kev)
    # One layer call on its own: nothing before it on the device, nothing after it until it has
    # finished (what a model sees between two GEMMs, where no neighbouring attention call hides the
    # ramp and the tail), issued from Python.
    lat = []
    for i in range(min(K, 50)):
        torch.cuda.synchronize(dev)
        e0.record(stream)
        step(args.warmup + i)
        e1.record(stream)
        torch.cuda.synchronize(dev)
        lat.append(e0.elapsed_time(e1))
    single_call_ms = statistics.median(lat)
    clocks = sampler.stop() if rank == 0 else None

    # ---- e2e: the host-buffer entry point, copies inside the timed region ----
    e2e = None
    if not args.skip_e2e:
        e2e = _run_e2e(args, pb, wl, sets, copies, h, dev, stream, barrier, world, split_heads, max_over_ranks)

    # ---- the other partition (weak scaling by prefix groups), device-timed only ----
    groups_split = None
    if split_heads and not args.skip_groups:
        del sets, call
        torch.cuda.empty_cache()
        groups_split = _run_groups_split(args, pb, dev, stream, barrier, world, rank, max_over_ranks)

    # max over ranks, region by region
    ms_eager = max_over_ranks(ms_eager, dev)
    ms_graph = max_over_ranks(ms_graph, dev) if ms_graph else []
    suffix_ms, single_call_ms = max_over_ranks([suffix_ms, single_call_ms], dev)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    st_eager = _stats(ms_eager, K)
    st_graph = _stats(ms_graph, K) if ms_graph else None
    use_graph = st_graph is not None and st_graph["median"] <= st_eager["median"]
    st = st_graph if use_graph else st_eager
    launch_mode = (f"K steps replayed from CUDA graphs of {graph_steps} steps" if use_graph else "K steps issued from Python")
    tokens = wl.num_rows * (1 if split_heads or world == 1 else world)
    ms_per_step = st["median"]
    value = tokens / (ms_per_step * 1e-3)
    ab = wl.algorithmic_bytes()
    peak, which = _peaks()
    # dominant kernel: the suffix (single-query) kernel; algorithmic bytes of one launch = private
    # KV of every row + their Q rows (the partials it writes are scratch, not counted)
    suffix_bytes = ab["suffix"] + ab["qo"] / 2
    achieved = suffix_bytes / (suffix_ms * 1e-3) / 1e9
    traffic = _captured_traffic(wl.name, h) if world == 1 else None
    cpu = None
    if not args.no_cpu_baseline and world == 1:
        ref = CpuReference(full, min(full.num_rows, 16))
        ref.run(2)
        rate = max(ref.run(), ref.run())
        cpu = {"value": rate, "unit": UNIT, "cores": ref.cores, "kind": "port", "sample": ref.sample}
    ref_gpu = None
    if world == 1 and args.config == 2 and not args.no_reference_gpu and (ROOT / "baseline" / "_ref" / "attention_ops.so").exists():
        ref_gpu = _reference_gpu_subprocess(local)
        if ref_gpu and ref_gpu.get("flash_paged_attention", {}).get("tokens_per_s"):
            ref_gpu["ours_over_reference_flash_paged_attention"] = value / ref_gpu["flash_paged_attention"]["tokens_per_s"]
    dtype = "f32" if wl.elem_bytes == 4 else ("bf16" if wl.dtype == torch.bfloat16 else "f16")
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong" if split_heads else "weak", "vs_baseline": None,
        "dtype": dtype, "data": "synthetic",
        "config": _config(full, world, split_heads),
        "timing": {
            "l2": f"{ab['total'] / 1e6:.0f} MB touched per step per GPU, rotating over {copies} distinct cache copies",
            "plan": "work lists built once per iteration (outside the layer call), as AttnFunc.init_iteration_state does",
            "launch": launch_mode,
            "regions": f"{st['regions']} regions of {K} steps; value = median region, max over ranks per region",
            "ms_per_step_min_max": [st["min"], st["max"]],
            "ms_per_step_by_launch": {"python": st_eager, "cuda_graph": st_graph},
            "single_call_latency_ms": single_call_ms,
            "single_call_note": "one layer call alone on an idle device (median of up to 50, CUDA events, issued from Python): "
                                "the ramp and tail that back-to-back steps hide behind each other are exposed",
        },
        "algorithmic_bytes_per_step": ab["total"],
        "achieved_gbs_whole_step": ab["total"] / (ms_per_step * 1e-3) / 1e9,
        "frac_of_hbm_peak_whole_step": ab["total"] / (ms_per_step * 1e-3) / 1e9 / peak,
        "frac_of_nominal_8tbs_whole_step": ab["total"] / (ms_per_step * 1e-3) / 8e12,
        "roofline": {"kernel": "sq_attn_kernel (suffix stage)", "bound": "hbm", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "frac_of_nominal_8tbs": achieved / 8000.0, "peak_source": which,
                     "traffic": traffic,
                     "traffic_note": ("dram read+write of one launch, read from the committed ncu summary profiles/sq_attn_kernel_cfg2_ncu_full.md"
                                      if traffic else "no ncu capture of this workload is committed"),
                     "algorithmic_bytes": suffix_bytes, "avg_launch_ms": suffix_ms},
        "cpu_baseline": cpu,
        "e2e": e2e,
        "gpu_launches": launches_per_step * K,
        "gpu_launches_note": (f"{launches_per_step} kernels per step (" + ("KV fill, " if fill_launch else "") +
                              f"dense prefix, suffix" + ("" if fill_launch else " incl. the KV fill of the new tokens") +
                              f", merge) x {K} steps of one timed region"),
        "verified": verified,
        "groups_split": groups_split,
        "reference_gpu": ref_gpu,
        "clocks": clocks,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def _host_step_args(wl, t0, h, dev):
    return dict(
        num_rows=wl.num_rows, num_heads=h, head_size=wl.head_size, block_size=wl.block_size, dtype=wl.dtype, device=dev,
        max_suffix_blocks=t0["suffix_tables"].shape[1], num_new_tokens=t0["k_new"].shape[0],
        group_row_offsets=t0["group_row_offsets"], group_prefix_lens=t0["group_prefix_lens"], group_tables=t0["group_tables"],
        seg_row_offsets=t0.get("seg_row_offsets"), seg_kv_lens=t0.get("seg_kv_lens"), seg_tables=t0.get("seg_tables"))


def _run_e2e(args, pb, wl, sets, copies, h, dev, stream, barrier, world, split_heads, max_over_ranks):
    """The same step through pb_attention_step_host: pinned host q / new k,v / slots / suffix lengths
    and tables in, result out to pinned host memory, the work lists rebuilt every step. Three ways
    of driving it: one step at a time (the call returns when the result is on the host: what a
    caller gets from `HostStep.step_graph`), and two or three steps in flight (`HostStepPipeline`)."""
    import torch

    K = args.steps
    t0 = sets[0]
    host = {k: t0[k].cpu().pin_memory() for k in ("query", "k_new", "v_new", "fill_slots", "suffix_lens", "suffix_tables")}
    hs_args = _host_step_args(wl, t0, h, dev)

    def load(slot):
        slot.h_query.copy_(host["query"]), slot.h_key_new.copy_(host["k_new"]), slot.h_value_new.copy_(host["v_new"])
        slot.h_slots.copy_(host["fill_slots"]), slot.h_suffix_lens.copy_(host["suffix_lens"])
        slot.h_suffix_tables.copy_(host["suffix_tables"])

    hstep = pb.HostStep(**hs_args)
    load(hstep)
    regions = max(3, args.regions // 3)

    def e2e_step(i):  # one CUDA-graph launch per step (captured per cache copy), then a stream synchronize
        t = sets[i % copies]
        hstep.step_graph(t["key_cache"], t["value_cache"], replan=True)

    for i in range(max(3 * copies, args.warmup)):  # every cache copy: eager call, capture, replay
        e2e_step(i)
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    serial = []
    for _ in range(regions):
        barrier()
        f0.record(stream)
        for i in range(K):
            e2e_step(i)
        f1.record(stream)
        barrier()
        serial.append(f0.elapsed_time(f1))
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = hstep.h_out.numel() * hstep.h_out.element_size()
    del hstep

    def pipelined(depth):
        pipe = pb.HostStepPipeline(depth=depth, **hs_args)
        for slot in pipe.slots:
            load(slot)

        def pipe_step(i):
            t = sets[i % copies]
            return 0 if pipe.submit(t["key_cache"], t["value_cache"], replan=True) is None else 1

        for i in range(max(3 * math.lcm(depth, copies), args.warmup)):  # every (slot, cache) pair: eager, capture, replay
            pipe_step(i)
        pipe.drain()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        res = []
        for _ in range(regions):
            barrier()
            g0.record(stream)
            for s_ in pipe.streams:
                s_.wait_stream(stream)
            delivered = 0
            for i in range(K):
                delivered += pipe_step(i)
            delivered += len(pipe.drain())
            for s_ in pipe.streams:
                stream.wait_stream(s_)
            g1.record(stream)
            barrier()
            assert delivered == K
            res.append(g0.elapsed_time(g1))
        return res

    depths = [args.e2e_depth] if args.e2e_depth > 0 else [2, 3]
    piped = {d_: pipelined(d_) for d_ in depths} if copies >= 2 else {}
    serial = max_over_ranks(serial, dev)
    piped = {d_: max_over_ranks(v, dev) for d_, v in piped.items()}
    tokens = wl.num_rows * (1 if split_heads or world == 1 else world)
    modes = {"one_step_at_a_time": _stats(serial, K), **{f"{d_}_steps_in_flight": _stats(v, K) for d_, v in piped.items()}}
    best = min(modes, key=lambda k: modes[k]["median"])
    ms = modes[best]["median"]
    return {"value": tokens / (ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "ms_per_step": ms, "mode": best,
            "mode_note": "value = the fastest of the modes below (median region each); a caller of HostStep.step_graph gets "
                         "one_step_at_a_time, a caller of HostStepPipeline(depth) the n_steps_in_flight figures",
            "ms_per_step_by_mode": modes}


def _run_groups_split(args, pb, dev, stream, barrier, world, rank, max_over_ranks):
    """The other collective-free partition: every rank its own prefix group with its rows (its own
    batch of the benchmark shape): weak scaling, device-timed, issued from Python."""
    import torch

    from parrotserve_b200.workloads import make_workload

    wl = make_workload(args.config, num_heads=args.heads or None)
    copies = 4 if args.config <= 2 else 1
    sets = [wl.materialize(dev, seed=2000 + args.config + 1000 * rank + 17 * c) for c in range(copies)]
    t0 = sets[0]
    out = torch.empty_like(t0["query"])
    call = pb.AttentionCall(
        num_rows=wl.num_rows, num_heads=wl.num_heads, head_size=wl.head_size, block_size=wl.block_size, dtype=wl.dtype, device=dev,
        suffix_lens=t0["suffix_lens"], suffix_tables=t0["suffix_tables"], group_row_offsets=t0["group_row_offsets"],
        group_prefix_lens=t0["group_prefix_lens"], group_tables=t0["group_tables"], seg_row_offsets=t0.get("seg_row_offsets"),
        seg_kv_lens=t0.get("seg_kv_lens"), seg_tables=t0.get("seg_tables"), slot_mapping=t0["fill_slots"])
    call.plan(t0["query"], out, t0["key_cache"], t0["value_cache"])

    def step(i):
        t = sets[i % copies]
        call.run(t["query"], out, t["key_cache"], t["value_cache"], key_new=t["k_new"], value_new=t["v_new"])

    K = args.steps
    for i in range(args.warmup):
        step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    res = []
    for _ in range(max(3, args.regions // 5)):
        barrier()
        e0.record(stream)
        for i in range(K):
            step(args.warmup + i)
        e1.record(stream)
        barrier()
        res.append(e0.elapsed_time(e1))
    res = max_over_ranks(res, dev)
    st = _stats(res, K)
    return {"scaling": "weak", "partition": "one prefix group (its own batch) per GPU", "ms_per_step": st["median"],
            "value": wl.num_rows * world / (st["median"] * 1e-3), "unit": UNIT, "launch": "issued from Python", "stats": st}


def _reference_gpu_subprocess(local: int):
    """Runs `bench.py --impl reference-gpu` in a child process (the reference's kernels never share a
    process with ours) and returns its report, or a one-line reason."""
    env = dict(os.environ, LOCAL_RANK=str(local), RANK="0", WORLD_SIZE="1")
    try:
        r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference-gpu", "--steps", "50", "--warmup", "10"],
                           capture_output=True, text=True, timeout=600, env=env)
    except (OSError, subprocess.TimeoutExpired) as exc:
        return {"unavailable": f"{type(exc).__name__}"}
    for ln in reversed(r.stdout.strip().splitlines()):
        if ln.startswith("{"):
            try:
                rep = json.loads(ln)
                rep.pop("impl", None)
                return rep
            except ValueError:
                pass
    return {"unavailable": f"child exited {r.returncode}: " + (r.stderr.strip().splitlines()[-1][:200] if r.stderr.strip() else "no output")}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--config", type=int, default=2, help="benchmark configuration 2..5 (2 is the headline one)")
    ap.add_argument("--split", choices=["heads", "groups"], default="heads",
                    help="N > 1: one batch with its heads split over the ranks (strong scaling, default) or every rank "
                         "its own prefix group (weak scaling)")
    ap.add_argument("--heads", type=int, default=0, help="override the head count of the whole batch")
    ap.add_argument("--regions", type=int, default=REGIONS, help="timed regions of K steps each (the median is reported)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-gpu", action="store_true")
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true", help="device-timed part only (kernel experiments)")
    ap.add_argument("--skip-groups", action="store_true", help="N > 1: do not also time the groups split")
    ap.add_argument("--chunk", type=int, default=0, help="suffix chunk in blocks (0: library default)")
    ap.add_argument("--dense-ctas", type=int, default=0, help="SMs of the dense prefix kernel (0: the planner's split)")
    ap.add_argument("--eager", action="store_true", help="time the Python call path only, no CUDA graph")
    ap.add_argument("--separate-fill", action="store_true",
                    help="KV fill as a call of its own before the attention call (the reference's sequence of two calls) "
                         "instead of letting the attention call perform it")
    ap.add_argument("--e2e-depth", type=int, default=0, help="host steps in flight in the pipelined e2e measurement (0: try 2 and 3)")
    ap.add_argument("--graph-steps", type=int, default=0, help="steps per captured CUDA graph (must divide --steps; 0 = 40, about one forward pass of layers, else 8, 4, ...)")
    ap.add_argument("--dense-row-tile", type=int, default=0, choices=[0, 128, 256],
                    help="query rows per work item of the tensor-core kernel (0 = the library's choice)")
    ap.add_argument("--probe", default="", help="rows,prefix,suffix[,heads[,dense_ctas]]: time one attention shape and exit")
    ap.add_argument("--probe-sampler", default="", help="rows,vocab,top_p: time the token sampler and exit")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.probe or args.probe_sampler:
        run_probe(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference-gpu":
        run_reference_gpu(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
