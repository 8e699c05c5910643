"""install() against the REAL ParrotServe package (CPU only; skipped where no checkout is found).

A child process imports the reference with stub modules for the native extensions it cannot load
here (the stubs of tests/golden/make_golden.py), calls ``parrotserve_b200.attn_func.install()``,
resolves the attention function through the reference's own ``BuiltinConfig`` and drives the
reference's own ``IterationState`` (parrot/engine/builtin/iter_state.py:29-48) with real
``BlockContext`` trees that contain Fill jobs. The metadata our builder derives from those real
objects is compared, field by field, with what the reference's
``xFormersFill_SharedPromptsGenerate.init_iteration_state`` (attn_func.py:462-599) produces for
the same jobs. The checkout is looked up in $PARROT_REFERENCE, then beside the repository.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _reference_root():
    for cand in (os.environ.get("PARROT_REFERENCE"), ROOT.parent / "reference"):
        if cand and (Path(cand) / "parrot/engine/builtin/attn_func.py").exists():
            return Path(cand)
    return None


CHILD = r"""
import importlib.util, sys
from pathlib import Path
root, ref = Path(sys.argv[1]), Path(sys.argv[2])
sys.path.insert(0, str(root)); sys.path.insert(0, str(ref))
spec = importlib.util.spec_from_file_location("_mk", root / "tests/golden/make_golden.py")
mk = importlib.util.module_from_spec(spec); spec.loader.exec_module(mk)
mk.install_stubs()
import parrot
parrot.attention_ops = mk._stub("parrot.attention_ops")
import numpy as np
from transformers import PretrainedConfig
from parrot.engine.config import BuiltinConfig
from parrot.engine.context.block_context import BlockContext
from parrot.engine.primitive_job import Fill, Generate
from parrot.sampling_config import SamplingConfig
from parrot.utils import RecyclePool
import parrot.engine.builtin.attn_func as ref_attn
from parrot.engine.builtin.iter_state import IterationState
from parrot.engine.builtin.mem_layout import ATTN_FUNC_LAYOUT_MAP, MemLayout
from parrotserve_b200 import attn_func as af

name = af.install()
assert name == af.ATTN_FUNC_NAME and name in ref_attn.ATTN_FUNCS and ATTN_FUNC_LAYOUT_MAP[name] == MemLayout.VLLM
assert af.install() == name and ref_attn.ATTN_FUNCS.count(name) == 1          # idempotent
cfg = BuiltinConfig(num_kv_cache_blocks=4096, attn_func=name, block_size=16, device="cpu")
assert cfg.attn_func is af.B200SharedPromptsGenerate                           # the reference's own lookup
ref_cfg = BuiltinConfig(num_kv_cache_blocks=4096, attn_func="xformers_fill_shared_prompts_generate", block_size=16, device="cpu")
assert ref_cfg.attn_func is ref_attn.xFormersFill_SharedPromptsGenerate        # and the chain still reaches the old names
hf = PretrainedConfig(num_attention_heads=4, hidden_size=64)

def tree(root_len, fills, children, b=16):
    pool = RecyclePool()
    root = None
    if root_len:
        root = BlockContext(0, None, pool, b); root.allocate(root_len)
    jobs, cid = [], 1
    for cached, n_new in fills:
        ctx = BlockContext(cid, root, pool, b); ctx.allocate(cached)
        job = Fill(session_id=0, task_id=cid, context_id=cid, parent_context_id=0 if root else -1, token_ids=list(range(n_new)))
        job.context = ctx; ctx.allocate(n_new); jobs.append(job); cid += 1
    for extra in children:
        ctx = BlockContext(cid, root, pool, b); ctx.allocate(extra)
        job = Generate(session_id=0, task_id=cid, context_id=cid, parent_context_id=0 if root else -1, sampling_config=SamplingConfig())
        job.context = ctx; ctx.allocate(1); jobs.append(job); cid += 1
    return jobs

checked = 0
for root_len, fills, children in ((40, [(0, 37), (9, 20)], [0, 15, 70]), (64, [(3, 130)], [5, 17, 33, 1]),
                                  (0, [(0, 20)], []), (40, [(13, 20)], []), (64, [], [5, 17])):
    jobs = tree(root_len, fills, children)
    st = IterationState(jobs, hf, ref_cfg)              # the reference's own builder
    meta = af.IterationMetadata(jobs, 16)               # ours, from the same real objects
    b = 16
    lone_fill = len(jobs) == 1 and len(fills) == 1
    if not lone_fill:
        assert meta.flash_context_len == int(st.flash_context_len)
        assert meta.flash_block_table.tolist() == st.flash_block_table.tolist()
        assert meta.paged_context_lens.tolist() == st.paged_context_lens.tolist()
        assert meta.paged_block_tables.tolist() == st.paged_block_tables.tolist()
    counts = [f[1] for f in fills] + [1] * len(children)
    assert meta.slot_mapping.tolist() == [s for row, n in zip(st.slot_mapping.tolist(), counts) for s in row[:n]]
    assert meta.num_fill_tokens == list(st.num_fill_tokens) and meta.num_generation_jobs == st.num_generation_jobs
    if fills:
        bias = st.q_kv_attn_bias
        assert np.diff(meta.seg_row_offsets).tolist() == list(bias.q_seqlen)
        assert (meta.seg_kv_lens + meta.flash_context_len).tolist() == list(bias.kv_seqlen)
        want, off = st.fill_slots.tolist(), 0
        for s_idx, kv in enumerate(bias.kv_seqlen):
            shared = [int(meta.flash_block_table[t // b]) * b + t % b for t in range(meta.flash_context_len)]
            own = [int(meta.seg_tables[s_idx][t // b]) * b + t % b for t in range(int(meta.seg_kv_lens[s_idx]))]
            assert shared + own == want[off:off + kv]
            off += kv
    # the reference's IterationState with OUR function: builds the metadata from the real jobs and
    # stops where the device is needed (there is no CPU path)
    try:
        IterationState(jobs, hf, cfg)
    except RuntimeError as exc:
        assert "CUDA" in str(exc), exc
    else:
        raise AssertionError("the attention call was built without a CUDA device")
    checked += 1
print("OK", checked)
"""


def test_install_and_metadata_against_the_real_reference_package():
    ref = _reference_root()
    if ref is None:
        pytest.skip("no ParrotServe checkout found (set PARROT_REFERENCE)")
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1")
    r = subprocess.run([sys.executable, "-c", CHILD, str(ROOT), str(ref)], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert r.stdout.strip().endswith("OK 5")
