"""Stand-in for the reference's native module ``vllm.cache_ops`` (3rdparty/vllm/csrc/cache.cpp:31-46),
restricted to the two ops on the attention path. ``copy_blocks`` / ``swap_blocks`` have no call
site in Parrot and are not provided.
"""
from .ops import gather_cached_kv, vllm_reshape_and_cache as reshape_and_cache

__all__ = ["reshape_and_cache", "gather_cached_kv"]
