"""B200-native shared-prefix paged attention: the hot path of ParrotServe's builtin engine.

Public surface mirrors ``parrot/engine/builtin/kernels/__init__.py:7-16``.
"""
from .ops import (  # noqa: F401
    AttentionCall,
    HostStep,
    HostStepPipeline,
    discontinuous_move_tokens,
    flash_paged_attention,
    flash_paged_attention_grouped,
    gather_cached_kv,
    move_tokens_from_blocked_k_cache,
    move_tokens_from_blocked_v_cache,
    paged_flash_attention,
    rotary_reshape_and_cache,
    sample_top_p,
    vllm_paged_attention,
    vllm_reshape_and_cache,
    vllm_rotary_emb,
)
from . import attention_ops, cache_ops  # noqa: F401
from .sampler import Sampler  # noqa: F401

__version__ = "0.1.0"
