"""GPU parity of the host-buffer entry point (`pb_attention_step_host` through `HostStep`):
inputs and result in page-locked host memory, one library call per layer. It must give exactly
what the device-tensor operators give on the same data (same kernels), and match the oracle."""
import pytest
import torch

import parrotserve_b200 as pb
from parrotserve_b200.workloads import make_workload
from tests.helpers import assert_close_to_oracle, oracle_for_workload, sample_rows

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_host_step_matches_device_operators_and_oracle():
    wl = make_workload(2, shrink=8)
    t = wl.materialize(DEV, seed=5)
    kc_ref, vc_ref = t["key_cache"].clone(), t["value_cache"].clone()
    # device-tensor path: fill, then attention
    pb.vllm_reshape_and_cache(t["k_new"], t["v_new"], kc_ref, vc_ref, t["fill_slots"])
    plen = int(wl.group_prefix_lens[0])
    want = pb.flash_paged_attention(t["query"], kc_ref, vc_ref, None, plen, t["group_tables"][0],
                                    t["suffix_lens"], t["suffix_tables"])

    host = {k: t[k].cpu().pin_memory() for k in ("query", "k_new", "v_new", "fill_slots", "suffix_lens", "suffix_tables")}
    out_host = torch.empty(tuple(t["query"].shape), dtype=t["query"].dtype).pin_memory()
    step = pb.HostStep(
        num_rows=wl.num_rows, num_heads=wl.num_heads, head_size=wl.head_size, block_size=wl.block_size, dtype=wl.dtype,
        device=torch.device(DEV), max_suffix_blocks=t["suffix_tables"].shape[1], num_new_tokens=t["k_new"].shape[0],
        group_row_offsets=t["group_row_offsets"], group_prefix_lens=t["group_prefix_lens"], group_tables=t["group_tables"])
    kc, vc = t["key_cache"], t["value_cache"]
    step.run(host["query"], host["k_new"], host["v_new"], host["fill_slots"].to(torch.int64), host["suffix_lens"],
             host["suffix_tables"], out_host, kc, vc)
    assert step.call.status() == 0
    assert torch.equal(kc, kc_ref) and torch.equal(vc, vc_ref)  # the fill is bit-exact
    assert torch.equal(out_host, want.cpu())
    rows = sample_rows(wl, 6)
    tensors = dict(t, key_cache=kc, value_cache=vc)
    ref = oracle_for_workload(wl, tensors, rows=rows, heads=[0, wl.num_heads - 1])
    assert_close_to_oracle(out_host[rows][:, [0, wl.num_heads - 1]], ref, wl.dtype, "host step")

    # second layer of the same iteration: lengths unchanged, no re-plan, no re-upload of the tables
    out2 = torch.empty_like(out_host).pin_memory()
    step.run(host["query"], host["k_new"], host["v_new"], host["fill_slots"].to(torch.int64), None, None, out2, kc, vc,
             replan=False)
    assert torch.equal(out2, out_host)

    # inputs produced straight into the step's own page-locked views: one merged upload
    step.h_query.copy_(host["query"]), step.h_key_new.copy_(host["k_new"]), step.h_value_new.copy_(host["v_new"])
    step.h_slots.copy_(host["fill_slots"]), step.h_suffix_lens.copy_(host["suffix_lens"])
    step.h_suffix_tables.copy_(host["suffix_tables"])
    step.h_out.zero_()
    step.run(step.h_query, step.h_key_new, step.h_value_new, step.h_slots, step.h_suffix_lens, step.h_suffix_tables,
             step.h_out, kc, vc)
    assert step.call.status() == 0
    assert torch.equal(step.h_out, out_host)
    # the hot-loop form of the same call
    step.h_out.zero_()
    got = step.step(kc, vc)
    assert got is step.h_out and torch.equal(step.h_out, out_host)
    step.h_out.zero_()
    step.step(kc, vc, replan=False)
    assert torch.equal(step.h_out, out_host)
    # the result written straight into the mapped host buffer by the last kernel (an option of the C entry)
    step.io.direct_out = 1
    step.h_out.zero_()
    step.step(kc, vc)
    assert torch.equal(step.h_out, out_host)
    step.io.direct_out = 0
    # the same step replayed from a captured CUDA graph (first call eager, second captures, third replays)
    for _ in range(3):
        step.h_out.zero_()
        got = step.step_graph(kc, vc)
        assert got is step.h_out and torch.equal(step.h_out, out_host)
    assert step.call.status() == 0


def test_pipelined_host_steps_give_the_serial_results():
    """Two host steps in flight on their own streams and staging buffers: every step's result equals
    what the device operators give for that step's inputs, in submission order."""
    wl = make_workload(2, shrink=8)
    dev = torch.device(DEV)
    steps = []
    for seed in range(5):   # five steps, each on its own data and cache
        t = wl.materialize(DEV, seed=20 + seed)
        kc_ref, vc_ref = t["key_cache"].clone(), t["value_cache"].clone()
        pb.vllm_reshape_and_cache(t["k_new"], t["v_new"], kc_ref, vc_ref, t["fill_slots"])
        want = pb.flash_paged_attention(t["query"], kc_ref, vc_ref, None, int(wl.group_prefix_lens[0]),
                                        t["group_tables"][0], t["suffix_lens"], t["suffix_tables"])
        steps.append((t, want.cpu()))
    t0 = steps[0][0]
    pipe = pb.HostStepPipeline(
        depth=2, num_rows=wl.num_rows, num_heads=wl.num_heads, head_size=wl.head_size, block_size=wl.block_size,
        dtype=wl.dtype, device=dev, max_suffix_blocks=t0["suffix_tables"].shape[1], num_new_tokens=t0["k_new"].shape[0],
        group_row_offsets=t0["group_row_offsets"], group_prefix_lens=t0["group_prefix_lens"], group_tables=t0["group_tables"])
    results = []
    for rnd in range(3):   # first use of a cache by a slot runs eagerly, the second captures, later ones replay
        results.clear()
        for t, _ in steps:
            slot = pipe.next_slot()
            slot.h_query.copy_(t["query"].cpu()), slot.h_key_new.copy_(t["k_new"].cpu()), slot.h_value_new.copy_(t["v_new"].cpu())
            slot.h_slots.copy_(t["fill_slots"].cpu()), slot.h_suffix_lens.copy_(t["suffix_lens"].cpu())
            slot.h_suffix_tables.copy_(t["suffix_tables"].cpu())
            done = pipe.submit(t["key_cache"], t["value_cache"])
            if done is not None:
                results.append(done.h_out.clone())
        results += [s.h_out.clone() for s in pipe.drain()]
        assert len(results) == len(steps)
        for (_, want), got in zip(steps, results):
            assert torch.equal(got, want), rnd
    assert all(s.call.status() == 0 for s in pipe.slots)


def test_host_step_rejects_device_or_misshaped_inputs():
    wl = make_workload(2, shrink=16)
    t = wl.materialize(DEV, seed=6)
    step = pb.HostStep(
        num_rows=wl.num_rows, num_heads=wl.num_heads, head_size=wl.head_size, block_size=wl.block_size, dtype=wl.dtype,
        device=torch.device(DEV), max_suffix_blocks=t["suffix_tables"].shape[1], num_new_tokens=t["k_new"].shape[0],
        group_row_offsets=t["group_row_offsets"], group_prefix_lens=t["group_prefix_lens"], group_tables=t["group_tables"])
    out_host = torch.empty(tuple(t["query"].shape), dtype=t["query"].dtype)
    with pytest.raises(RuntimeError):  # a device tensor where a host tensor is expected
        step.run(t["query"], None, None, None, None, None, out_host, t["key_cache"], t["value_cache"])
    with pytest.raises(RuntimeError):  # wrong number of rows
        step.run(t["query"].cpu()[:-1], None, None, None, None, None, out_host, t["key_cache"], t["value_cache"])
