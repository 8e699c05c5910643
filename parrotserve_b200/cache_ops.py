"""Stand-in for the reference's native module ``vllm.cache_ops`` (3rdparty/vllm/csrc/cache.cpp:31-46):
``reshape_and_cache`` and ``gather_cached_kv`` (on the attention path) and the whole-block
``copy_blocks`` / ``swap_blocks`` (no call site in Parrot's builtin engine; provided for engines that
preempt or copy on write).
"""
from .ops import copy_blocks, gather_cached_kv, swap_blocks, vllm_reshape_and_cache as reshape_and_cache

__all__ = ["reshape_and_cache", "gather_cached_kv", "copy_blocks", "swap_blocks"]
