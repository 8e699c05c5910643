"""ctypes binding of ``libparrot_b200_attn.so`` (the C ABI in ``include/parrot_b200_attn.h``).

The library is the product: there is no Python or CPU fallback. Loading fails loudly when the
shared object has not been built (``python -m parrotserve_b200.build``).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libparrot_b200_attn.so"

PB_F32, PB_F16, PB_BF16 = 0, 1, 2
PB_OK = 0
PB_ERR_INVALID_ARG, PB_ERR_UNSUPPORTED, PB_ERR_WORKSPACE, PB_ERR_LAUNCH, PB_ERR_DEVICE = -1, -2, -3, -4, -5
PB_STATS_NONE, PB_STATS_SAVE, PB_STATS_LOAD, PB_STATS_LOAD_SAVE = 0, 1, 2, 3

STATUS_NAMES = {
    PB_ERR_INVALID_ARG: "invalid argument (null/misaligned pointer, bad size or stride)",
    PB_ERR_UNSUPPORTED: "unsupported head_size/block_size/dtype",
    PB_ERR_WORKSPACE: "workspace missing or too small",
    PB_ERR_LAUNCH: "CUDA launch failed",
    PB_ERR_DEVICE: "kernel recorded a device-side fault",
}


class PbAttnParams(C.Structure):
    """Mirror of ``pb_attn_params``; field order and types must match the header."""

    _fields_ = [
        ("out", C.c_void_p),
        ("query", C.c_void_p),
        ("key_cache", C.c_void_p),
        ("value_cache", C.c_void_p),
        ("head_mapping", C.c_void_p),
        ("scale", C.c_float),
        ("dtype", C.c_int32),
        ("num_rows", C.c_int32),
        ("num_heads", C.c_int32),
        ("num_kv_heads", C.c_int32),
        ("head_size", C.c_int32),
        ("block_size", C.c_int32),
        ("num_blocks", C.c_int64),
        ("q_stride", C.c_int64),
        ("out_stride", C.c_int64),
        ("kv_block_stride", C.c_int64),
        ("kv_head_stride", C.c_int64),
        ("suffix_lens", C.c_void_p),
        ("suffix_tables", C.c_void_p),
        ("suffix_table_stride", C.c_int32),
        ("num_groups", C.c_int32),
        ("group_row_offsets", C.c_void_p),
        ("group_prefix_lens", C.c_void_p),
        ("group_tables", C.c_void_p),
        ("group_table_stride", C.c_int32),
        ("num_segments", C.c_int32),
        ("seg_row_offsets", C.c_void_p),
        ("seg_kv_lens", C.c_void_p),
        ("seg_tables", C.c_void_p),
        ("seg_table_stride", C.c_int32),
        ("num_outer_groups", C.c_int32),
        ("outer_row_offsets", C.c_void_p),
        ("outer_prefix_lens", C.c_void_p),
        ("outer_tables", C.c_void_p),
        ("outer_table_stride", C.c_int32),
        ("slot_mapping", C.c_void_p),
        ("slot_is_i64", C.c_int32),
        ("key_new", C.c_void_p),
        ("value_new", C.c_void_p),
        ("key_new_stride", C.c_int64),
        ("value_new_stride", C.c_int64),
        ("qk_max", C.c_void_p),
        ("exp_sum", C.c_void_p),
        ("stats_mode", C.c_int32),
        ("dense_min_rows", C.c_int32),
        ("suffix_chunk_blocks", C.c_int32),
        ("prefix_chunk_blocks", C.c_int32),
        ("dense_ctas", C.c_int32),
        ("dense_row_tile", C.c_int32),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
    ]


class PbHostStep(C.Structure):
    """Mirror of ``pb_host_step`` (same field order as the header)."""

    _fields_ = [
        ("h_query", C.c_void_p),
        ("h_key_new", C.c_void_p),
        ("h_value_new", C.c_void_p),
        ("h_slot_mapping", C.c_void_p),
        ("num_new_tokens", C.c_int64),
        ("h_suffix_lens", C.c_void_p),
        ("h_suffix_tables", C.c_void_p),
        ("h_out", C.c_void_p),
        ("d_key_new", C.c_void_p),
        ("d_value_new", C.c_void_p),
        ("d_slot_mapping", C.c_void_p),
        ("replan", C.c_int32),
        ("synchronize", C.c_int32),
        ("merge_adjacent", C.c_int32),
        ("direct_out", C.c_int32),
    ]


# name -> (restype, argtypes); every symbol the header declares.
_vp, _i32, _i64, _f32, _sz = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_size_t
_SQ_COMMON_TAIL = [_i32, _i32, _i32, _i32, _i32, _i32, _i32, _i64, _i64, _i64, _i64, _i32, _vp, _sz, _vp]
SIGNATURES = {
    "pb_abi_version": (C.c_int, []),
    "pb_last_cuda_error": (C.c_char_p, []),
    "pb_attn_set_timing_events": (None, [_vp, _vp]),
    "pb_attn_workspace_bytes": (_sz, [C.POINTER(PbAttnParams)]),
    "pb_attn_plan": (C.c_int, [C.POINTER(PbAttnParams), _vp]),
    "pb_shared_prefix_attention_planned": (C.c_int, [C.POINTER(PbAttnParams), _vp]),
    "pb_shared_prefix_attention": (C.c_int, [C.POINTER(PbAttnParams), _vp]),
    "pb_read_status": (C.c_int, [_vp, _vp, C.POINTER(_i32)]),
    "pb_attention_step_host": (C.c_int, [C.POINTER(PbAttnParams), C.POINTER(PbHostStep), _vp]),
    "pb_single_query_cached_kv_attention": (
        C.c_int, [_vp, _vp, _vp, _vp, _vp, _f32, _vp, _vp] + _SQ_COMMON_TAIL),
    "pb_single_query_cached_kv_prev_attention": (
        C.c_int, [_vp, _vp, _vp, _vp, _vp, _f32, _vp, _vp, _vp, _vp] + _SQ_COMMON_TAIL),
    "pb_single_query_cached_kv_post_attention": (
        C.c_int, [_vp, _vp, _vp, _vp, _vp, _f32, _vp, _vp, _vp, _vp] + _SQ_COMMON_TAIL),
    "pb_single_query_workspace_bytes": (_sz, [_i32, _i32, _i32, _i32, _i32]),
    "pb_single_query_cached_kv_attention_static": (
        C.c_int, [_vp, _vp, _vp, _vp, _vp, _f32, _vp, _vp] + _SQ_COMMON_TAIL[:12] + [_vp]),
    "pb_static_scratch_bytes": (_sz, []),
    "pb_static_scratch_status": (C.c_int, [_vp, C.POINTER(_i32)]),
    "pb_reshape_and_cache": (
        C.c_int, [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i32, _i32, _i32, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "pb_rotary_reshape_and_cache": (
        C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _i32, _i64, _i64, _i32, _i32, _i32, _i32,
                  _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _vp]),
    "pb_gather_cached_kv": (
        C.c_int, [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i32, _i32, _i32, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "pb_move_tokens_from_blocked_cache": (
        C.c_int, [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "pb_copy_blocks": (C.c_int, [_vp, _vp, _i32, _vp, _i64, _i64, _i64, _vp]),
    "pb_swap_blocks": (C.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp]),
    "pb_sample_top_p": (C.c_int, [_vp, _i32, _i32, _i32, _i64, _vp, _vp, _vp, _vp, _vp]),
    "pb_discontinuous_move_tokens": (
        C.c_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _vp]),
}

_lib = None


class PbError(RuntimeError):
    """A non-zero pb_status, raised like the reference's TORCH_CHECK failures
    (csrc/attention/attention_post_kernels.cu:448,500,525)."""

    def __init__(self, code: int, where: str, detail: str = ""):
        self.code = code
        msg = f"{where}: {STATUS_NAMES.get(code, 'error')} (pb_status {code})"
        if detail:
            msg += f": {detail}"
        super().__init__(msg)


def lib() -> C.CDLL:
    """Loads the C-ABI library once; raises if it was not built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m parrotserve_b200.build`. "
                "There is no CPU or PyTorch fallback for this path."
            )
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(code: int, where: str) -> None:
    if code != PB_OK:
        detail = ""
        if code == PB_ERR_LAUNCH:
            detail = (lib().pb_last_cuda_error() or b"").decode()
        raise PbError(code, where, detail)
