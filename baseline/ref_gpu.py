"""Times the reference's OWN GPU kernels (built unmodified into ``baseline/_ref/`` by
``baseline/build_ref.py``) on the benchmark's configuration-2 workload, on the same GPU as ours.

What is timed, each on the same tensors (fp16, rotating over distinct cache copies so that no
call finds its KV in L2), CUDA events around K calls after W warm-up calls:

* ``flash_paged_attention``  — the function the reference's attention class calls
  (parrot/engine/builtin/kernels/shared_flash_decoding.py:285-329): Triton prefix kernel (+ Triton
  reduce) then the CUDA ``post`` kernel. If Triton rejects the kernel source (it was written for
  Triton 2.1), the compiler's message is recorded and the call is reported as "did not compile";
  its arithmetic is never patched.
* ``single_query_cached_kv_post_attention`` alone (csrc/attention/attention_post_kernels.cu:365-527)
  over the private suffixes — the counterpart of our suffix kernel + merge.
* ``single_query_cached_kv_attention`` unshared (csrc/attention/attention_kernels.cu:539-570) over
  prefix ++ suffix per sequence — what prefix sharing removes.
* ``reshape_and_cache`` (3rdparty/vllm/csrc/cache_kernels.cu:142-224) for the step's new tokens.

Outputs are compared with ours where the call ran (max-abs difference), so a number is never
reported for a kernel that computed something else.
"""
from __future__ import annotations

import importlib.machinery
import importlib.util
import sys
import types
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"


def _load_ext(name: str):
    path = REF / (name + ".so")
    if not path.exists():
        return None
    loader = importlib.machinery.ExtensionFileLoader(name, str(path))
    spec = importlib.util.spec_from_loader(name, loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


def load_reference():
    """(attention_ops, cache_ops, shared_flash_decoding module or None, note)."""
    import torch  # noqa: F401  (the extensions link against torch's libraries)

    attention_ops, cache_ops = _load_ext("attention_ops"), _load_ext("cache_ops")
    sfd, note = None, ""
    py = REF / "shared_flash_decoding.py"
    if attention_ops is not None and cache_ops is not None and py.exists():
        # the file does `from vllm import cache_ops` and `from parrot import attention_ops`
        saved = {k: sys.modules.get(k) for k in ("vllm", "parrot")}
        vllm, parrot = types.ModuleType("vllm"), types.ModuleType("parrot")
        vllm.cache_ops, parrot.attention_ops = cache_ops, attention_ops
        sys.modules["vllm"], sys.modules["parrot"] = vllm, parrot
        try:
            spec = importlib.util.spec_from_file_location("_ref_shared_flash_decoding", py)
            sfd = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(sfd)
        except Exception as exc:  # import-time failure of the Triton decorators
            sfd, note = None, f"{type(exc).__name__}: {str(exc).strip().splitlines()[-1][:200]}"
        finally:
            for k, v in saved.items():
                if v is None:
                    sys.modules.pop(k, None)
                else:
                    sys.modules[k] = v
    return attention_ops, cache_ops, sfd, note


def _time(fn, steps: int, warmup: int, torch, dev) -> float:
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1) / steps


def run(wl, sets, steps: int, warmup: int, ours: dict = None) -> dict:
    """`sets`: materialised copies of the workload (dicts of device tensors); `ours`: this library's
    outputs on copy 0 for the whole attention ("full"), the shared prefix alone ("prefix") and the
    private suffixes alone ("suffix"), to compare the reference's results with. Returns a report."""
    import torch

    ours = ours or {}

    attention_ops, cache_ops, sfd, note = load_reference()
    if attention_ops is None or cache_ops is None:
        return {"unavailable": "baseline/_ref holds no built reference extensions (run baseline/build_ref.py where the checkout is)"}
    dev = sets[0]["query"].device
    copies = len(sets)
    b, rows, h = wl.block_size, wl.num_rows, wl.num_heads
    plen = int(wl.group_prefix_lens[0])
    npb = (plen + b - 1) // b
    hm = torch.arange(h, dtype=torch.int32, device=dev)
    flash_table = sets[0]["group_tables"][0][:npb].contiguous()
    lens, tables = sets[0]["suffix_lens"], sets[0]["suffix_tables"]
    scale = wl.head_size ** -0.5
    max_ctx = tables.shape[1] * b
    rep = {"workload": wl.name, "tokens_per_call": rows, "steps": steps, "warmup": warmup}

    def rate(ms):
        return {"ms_per_call": ms, "tokens_per_s": rows / (ms * 1e-3)}

    def diff(out, key="full"):
        ref = ours.get(key)
        return None if ref is None else float((out.float() - ref.float()).abs().max().item())

    # --- flash_paged_attention: Triton prefix stage + CUDA post kernel ---
    if sfd is None:
        rep["flash_paged_attention"] = {"status": "did not import", "message": note}
    else:
        try:
            t = sets[0]
            out = sfd.flash_paged_attention(t["query"], t["key_cache"], t["value_cache"], hm, plen, flash_table, lens, tables)
            torch.cuda.synchronize(dev)
            ms = _time(lambda i: sfd.flash_paged_attention(sets[i % copies]["query"], sets[i % copies]["key_cache"],
                                                           sets[i % copies]["value_cache"], hm, plen, flash_table, lens, tables),
                       steps, warmup, torch, dev)
            rep["flash_paged_attention"] = {"status": "ran", **rate(ms), "max_abs_vs_ours": diff(out)}
            # its Triton stage alone (the shared prefix), to see which stage a difference comes from
            pm = torch.zeros((rows, h), dtype=torch.float32, device=dev)
            ps = torch.zeros((rows, h), dtype=torch.float32, device=dev)
            pout = torch.empty_like(t["query"])
            sfd.triton_flash_attention(t["query"], t["key_cache"], t["value_cache"], hm, plen, pm, ps, flash_table, pout,
                                       load_mid_results=False, save_mid_results=True)
            torch.cuda.synchronize(dev)
            rep["flash_paged_attention"]["triton_prefix_stage_max_abs_vs_ours"] = diff(pout, "prefix")
        except Exception as exc:
            msg = str(exc).strip().splitlines()
            rep["flash_paged_attention"] = {"status": "did not compile or run", "error": type(exc).__name__,
                                            "message": " | ".join(msg[-3:])[:600]}

    # --- the CUDA post kernel alone over the private suffixes (prefix statistics = empty partial) ---
    def post(i):
        t = sets[i % copies]
        attention_ops.single_query_cached_kv_post_attention(post_out, t["query"], t["key_cache"], t["value_cache"], hm, scale,
                                                            tables, lens, qk_max, exp_sum, b, max_ctx, None)

    post_out = torch.zeros_like(sets[0]["query"])
    qk_max = torch.full((rows, h), -1e30, dtype=torch.float32, device=dev)
    exp_sum = torch.zeros((rows, h), dtype=torch.float32, device=dev)
    try:
        ms = _time(post, steps, warmup, torch, dev)
        post_out.zero_()
        post(0)
        torch.cuda.synchronize(dev)
        rep["post_kernel_suffix_only"] = {"status": "ran", **rate(ms), "max_abs_vs_ours": diff(post_out, "suffix")}
    except Exception as exc:
        rep["post_kernel_suffix_only"] = {"status": "failed", "message": str(exc)[:300]}

    # --- unshared paged attention: every sequence walks prefix ++ suffix ---
    width = npb + tables.shape[1]
    full_tables = torch.zeros((rows, width), dtype=torch.int32, device=dev)
    full_tables[:, :npb] = flash_table
    full_tables[:, npb:] = tables
    full_lens = (lens + plen).to(torch.int32)
    block_lens = torch.zeros((rows, width), dtype=torch.int32, device=dev)   # never read by the kernel
    block_nums = ((full_lens + b - 1) // b).to(torch.int32)                    # table entries the kernel walks
    plain_out = torch.empty_like(sets[0]["query"])

    def plain(i):
        t = sets[i % copies]
        attention_ops.single_query_cached_kv_attention(plain_out, t["query"], t["key_cache"], t["value_cache"], hm, scale, full_tables,
                                                       block_lens, block_nums, full_lens, b, width * b, None)

    try:
        ms = _time(plain, max(3, steps // 4), max(1, warmup // 4), torch, dev)
        plain(0)
        torch.cuda.synchronize(dev)
        # copy 0 was used by the last call: compare on it
        rep["unshared_paged_attention"] = {"status": "ran", **rate(ms), "max_abs_vs_ours": diff(plain_out)}
    except Exception as exc:
        rep["unshared_paged_attention"] = {"status": "failed", "message": str(exc)[:300]}

    # --- KV fill of the step's new tokens ---
    def fill(i):
        t = sets[i % copies]
        cache_ops.reshape_and_cache(t["k_new"], t["v_new"], t["key_cache"], t["value_cache"], slots32)

    slots32 = sets[0]["fill_slots"].to(torch.int32)
    try:
        rep["reshape_and_cache"] = {"status": "ran", "new_tokens": int(slots32.numel()),
                                    "ms_per_call": _time(fill, steps, warmup, torch, dev)}
    except Exception as exc:
        rep["reshape_and_cache"] = {"status": "failed", "message": str(exc)[:300]}
    return rep
