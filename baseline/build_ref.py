"""Builds the reference's OWN GPU kernels for this path into ``baseline/_ref/`` (git-ignored), so
that ``bench.py --impl reference-gpu`` can time them beside ours on the same B200.

    python baseline/build_ref.py /path/to/ParrotServe

Nothing of the reference is modified and nothing of it enters the repository's history: the
sources are compiled where they lie, only build products and an unmodified copy of the one Python
file that holds the Triton kernels land in ``baseline/_ref/``:

* ``attention_ops``  <- csrc/attention.cpp + csrc/attention/attention{,_prev,_post}_kernels.cu
  (the extension the reference's setup.py:105-115 builds as ``parrot.attention_ops``)
* ``cache_ops``      <- 3rdparty/vllm/csrc/cache.cpp + cache_kernels.cu (``vllm.cache_ops``)
* ``shared_flash_decoding.py`` <- parrot/engine/builtin/kernels/shared_flash_decoding.py

Compiled for sm_100a with the installed torch's headers (``torch.utils.cpp_extension.load``);
nvcc cross-compiles without a GPU. A source that does not compile against this torch / CUDA is
reported and left out; its arithmetic is never patched.
"""
from __future__ import annotations

import json
import shutil
import sys
from pathlib import Path

OUT = Path(__file__).resolve().parent / "_ref"

NVCC = ["-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
        "-D_GLIBCXX_USE_CXX11_ABI=1"]


def build(ref_root: str) -> dict:
    import torch  # noqa: F401  (headers and ABI of the installed torch)
    from torch.utils import cpp_extension

    ref = Path(ref_root)
    OUT.mkdir(parents=True, exist_ok=True)
    report = {}
    targets = {
        "attention_ops": [ref / "csrc/attention.cpp", ref / "csrc/attention/attention_kernels.cu",
                          ref / "csrc/attention/attention_prev_kernels.cu", ref / "csrc/attention/attention_post_kernels.cu"],
        "cache_ops": [ref / "3rdparty/vllm/csrc/cache.cpp", ref / "3rdparty/vllm/csrc/cache_kernels.cu"],
    }
    for name, srcs in targets.items():
        bdir = OUT / ("build_" + name)
        bdir.mkdir(exist_ok=True)
        try:
            cpp_extension.load(name=name, sources=[str(s) for s in srcs], extra_cflags=["-O2", "-std=c++17"],
                               extra_cuda_cflags=NVCC, build_directory=str(bdir), is_python_module=False, verbose=False)
            so = bdir / (name + ".so")
            shutil.copy2(so, OUT / (name + ".so"))
            report[name] = "built"
        except Exception as exc:  # compiler output is the record of why
            report[name] = "did not build: " + str(exc).strip().splitlines()[-1][:300]
            (OUT / (name + ".build_error.txt")).write_text(str(exc))
    py = ref / "parrot/engine/builtin/kernels/shared_flash_decoding.py"
    shutil.copy2(py, OUT / "shared_flash_decoding.py")
    report["shared_flash_decoding.py"] = "copied unmodified"
    (OUT / "build_report.json").write_text(json.dumps(report, indent=1))
    return report


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(json.dumps(build(sys.argv[1]), indent=1))
