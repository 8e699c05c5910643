"""Loader of the torch-extension shim ``b200_torch_ops.so`` (``csrc/torch_shim.cpp``): the pybind
surface of the reference's two native modules over this library's C ABI.

    from parrotserve_b200 import torch_ops
    attention_ops, cache_ops = torch_ops.load()        # the submodules, named as in the reference
    torch_ops.install_as_reference_modules()           # sys.modules["parrot.attention_ops"], ["vllm.cache_ops"]

``attention_ops`` has the three functions of ``parrot.attention_ops`` (csrc/attention.cpp:49-62),
``cache_ops`` the four of ``vllm.cache_ops`` (3rdparty/vllm/csrc/cache.cpp:30-46), with the
reference's positional argument lists. The shared object is built in-tree by
``python -m parrotserve_b200.build`` and fails loudly when it is missing.
"""
from __future__ import annotations

import importlib.machinery
import importlib.util
import sys
from pathlib import Path

_PATH = Path(__file__).resolve().parent / "b200_torch_ops.so"
_mod = None


def load():
    """(attention_ops, cache_ops) of the compiled shim."""
    global _mod
    if _mod is None:
        if not _PATH.exists():
            raise RuntimeError(f"{_PATH.name} is not built: run `python -m parrotserve_b200.build`")
        import torch  # noqa: F401  (the extension links against torch's libraries)

        loader = importlib.machinery.ExtensionFileLoader("b200_torch_ops", str(_PATH))
        spec = importlib.util.spec_from_loader("b200_torch_ops", loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
        _mod = mod
    return _mod.attention_ops, _mod.cache_ops


def install_as_reference_modules() -> None:
    """Makes ``from parrot import attention_ops`` and ``from vllm import cache_ops`` (the imports of
    parrot/engine/builtin/kernels/shared_flash_decoding.py:26-28 and kernels/vllm/*.py) resolve to the
    shim, for a ParrotServe checkout whose own extensions are not built."""
    attention_ops, cache_ops = load()
    sys.modules["parrot.attention_ops"] = attention_ops
    sys.modules["vllm.cache_ops"] = cache_ops
    for pkg, name, sub in (("parrot", "attention_ops", attention_ops), ("vllm", "cache_ops", cache_ops)):
        if pkg in sys.modules:
            setattr(sys.modules[pkg], name, sub)
