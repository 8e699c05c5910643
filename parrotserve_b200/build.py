"""Builds the CUDA library of this package in-tree for sm_100a, and the torch-extension shim over it.

    python -m parrotserve_b200.build [--force] [--verbose]

Produces ``parrotserve_b200/libparrot_b200_attn.so`` (the C-ABI library declared in
``include/parrot_b200_attn.h``; nvcc cross-compiles without a GPU) and
``parrotserve_b200/b200_torch_ops.so`` (``csrc/torch_shim.cpp``: the pybind surface of the
reference's ``parrot.attention_ops`` and ``vllm.cache_ops`` over that library, compiled against
the installed torch's headers; skipped with a note when they are not there).
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "libparrot_b200_attn.so"
OBJ_DIR = PKG / "build"

SOURCES = ["capi.cu", "plan.cu", "single_query.cu", "single_query_b8.cu", "single_query_b32.cu", "merge.cu", "kv_fill.cu", "prefix_dense.cu", "dense_pair.cu", "static_scratch.cu", "block_ops.cu", "sampler.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    deps = [CSRC / s for s in SOURCES] + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "parrot_b200_attn.h"]
    stamp = OBJ_DIR / "stamp.txt"
    digest = _digest(deps)
    if not force and OUT.exists() and stamp.exists() and stamp.read_text() == digest:
        return OUT
    OBJ_DIR.mkdir(exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: str) -> Path:
        obj = OBJ_DIR / (src + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", str(CSRC / src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(f"$ {' '.join(cmd)}\n{r.stdout}{r.stderr}")
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    # link beside the target and move into place: a process that loads the library while it is being
    # rebuilt sees the old or the new file, never half of one
    tmp = OUT.with_suffix(".so.tmp")
    cmd = [_nvcc(), "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    os.replace(tmp, OUT)
    stamp.write_text(digest)
    return OUT


SHIM_OUT = PKG / "b200_torch_ops.so"


def build_torch_shim(force: bool = False, verbose: bool = False):
    """Compiles csrc/torch_shim.cpp against the installed torch and links it to the in-tree library.
    Returns the path, or None when torch's C++ headers cannot be used here."""
    src = CSRC / "torch_shim.cpp"
    stamp = OBJ_DIR / "shim_stamp.txt"
    try:
        import torch
        from torch.utils import cpp_extension
    except Exception as exc:  # no torch: nothing to bind against
        sys.stderr.write(f"torch shim skipped: {exc}\n")
        return None
    digest = _digest([src, PKG.parent / "include" / "parrot_b200_attn.h"]) + torch.__version__
    if not force and SHIM_OUT.exists() and stamp.exists() and stamp.read_text() == digest:
        return SHIM_OUT
    bdir = OBJ_DIR / "shim"
    bdir.mkdir(parents=True, exist_ok=True)
    try:
        cpp_extension.load(
            name="b200_torch_ops", sources=[str(src)], extra_cflags=["-O2", "-std=c++17"],
            extra_include_paths=[str(Path(cpp_extension.CUDA_HOME or "/usr/local/cuda") / "include")],
            extra_ldflags=[f"-L{PKG}", "-lparrot_b200_attn", "-Wl,-rpath,'$$ORIGIN:$$ORIGIN/../..'"],  # ($$: ninja's escape of $)
            build_directory=str(bdir), is_python_module=False, with_cuda=True, verbose=verbose)
    except Exception as exc:
        sys.stderr.write(f"torch shim not built: {str(exc).strip().splitlines()[-1][:300]}\n")
        return None
    import shutil

    shutil.copy2(bdir / "b200_torch_ops.so", SHIM_OUT.with_suffix(".so.tmp"))
    os.replace(SHIM_OUT.with_suffix(".so.tmp"), SHIM_OUT)
    stamp.write_text(digest)
    return SHIM_OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_torch_shim(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
