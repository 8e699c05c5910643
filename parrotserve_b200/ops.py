"""Host-side operators with the names, argument orders and error behaviour of the reference's
kernel wrappers (``parrot/engine/builtin/kernels/__init__.py:7-16``), backed by the C-ABI CUDA
library. Tensors are torch CUDA tensors; torch only provides device memory and streams here.

Function-level boundary (reference file:line each one replaces):

* ``flash_paged_attention`` / ``paged_flash_attention``   kernels/shared_flash_decoding.py:285-376
* ``vllm_paged_attention``                                kernels/vllm/paged_attention.py:12-38
* ``vllm_reshape_and_cache``                              kernels/vllm/reshape_and_cache.py:9-22
* ``discontinuous_move_tokens``                           kernels/tokens_moving.py:67-100
* ``move_tokens_from_blocked_{k,v}_cache``                kernels/tokens_moving.py:163-218, 271-313
* ``flash_paged_attention_grouped``                       the same path for G prefix groups
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from ._lib import PbAttnParams, check, lib

_DTYPES = {torch.float32: _lib.PB_F32, torch.float16: _lib.PB_F16, torch.bfloat16: _lib.PB_BF16}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise RuntimeError(f"unsupported dtype {t.dtype}") from None


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("parrotserve_b200 ops need CUDA tensors; there is no CPU path")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _as_i32(t: torch.Tensor) -> torch.Tensor:
    if t.dtype != torch.int32:
        t = t.to(torch.int32)
    return t.contiguous()


class Workspace:
    """Grow-only scratch buffer per device; the C ABI never allocates."""

    _bufs: Dict[Tuple[str, int], torch.Tensor] = {}

    @classmethod
    def get(cls, device: torch.device, nbytes: int, tag: str = "attn") -> torch.Tensor:
        key = (tag, device.index if device.index is not None else torch.cuda.current_device())
        buf = cls._bufs.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
            cls._bufs[key] = buf
        return buf


def _kv_geometry(key_cache: torch.Tensor, value_cache: torch.Tensor):
    # K [NB, Hkv, D/x, B, x], V [NB, Hkv, D, B]   (parrot/engine/builtin/mem.py:69-82)
    if key_cache.dim() != 5 or value_cache.dim() != 4:
        raise RuntimeError("key_cache must be [NB,H,D/x,B,x] and value_cache [NB,H,D,B]")
    nb, hkv, d, b = value_cache.shape
    x = key_cache.shape[4]
    if key_cache.shape[0] != nb or key_cache.shape[1] != hkv or key_cache.shape[2] * x != d or key_cache.shape[3] != b:
        raise RuntimeError("key_cache / value_cache shapes disagree")
    if x * key_cache.element_size() != 16:
        raise RuntimeError("key_cache innermost dimension must span 16 bytes")
    if key_cache.stride(0) != value_cache.stride(0) or key_cache.stride(1) != value_cache.stride(1):
        raise RuntimeError("key_cache and value_cache must share block and head strides")
    if key_cache[0, 0].is_contiguous() is False or value_cache[0, 0].is_contiguous() is False:
        raise RuntimeError("a (block, head) tile must be contiguous")
    return nb, hkv, d, b, key_cache.stride(0), key_cache.stride(1)


class AttentionCall:
    """One grouped shared-prefix attention problem bound to a parameter block.

    ``plan()`` builds the device-side work lists from the lengths (once per iteration);
    ``run(query, out, key_cache, value_cache)`` enqueues prefix stage, suffix stage and merge
    for one layer. Metadata tensors are kept alive by this object.
    """

    def __init__(
        self,
        *,
        num_rows: int,
        num_heads: int,
        head_size: int,
        block_size: int,
        dtype: torch.dtype,
        device: torch.device,
        suffix_lens: Optional[torch.Tensor],
        suffix_tables: Optional[torch.Tensor],
        group_row_offsets: Optional[torch.Tensor] = None,
        group_prefix_lens: Optional[torch.Tensor] = None,
        group_tables: Optional[torch.Tensor] = None,
        seg_row_offsets: Optional[torch.Tensor] = None,
        seg_kv_lens: Optional[torch.Tensor] = None,
        seg_tables: Optional[torch.Tensor] = None,
        outer_row_offsets: Optional[torch.Tensor] = None,
        outer_prefix_lens: Optional[torch.Tensor] = None,
        outer_tables: Optional[torch.Tensor] = None,
        head_mapping: Optional[torch.Tensor] = None,
        slot_mapping: Optional[torch.Tensor] = None,
        scale: Optional[float] = None,
        dense_min_rows: int = 0,
        suffix_chunk_blocks: int = 0,
        prefix_chunk_blocks: int = 0,
        dense_ctas: int = 0,
        dense_row_tile: int = 0,
        workspace: Optional[torch.Tensor] = None,
        shared_workspace: bool = False,
    ):
        self.device = device
        self.dtype = dtype
        p = PbAttnParams()
        p.scale = float(head_size ** -0.5 if scale is None else scale)
        p.dtype = _DTYPES[dtype]
        p.num_rows = num_rows
        p.num_heads = num_heads
        p.num_kv_heads = num_heads
        p.head_size = head_size
        p.block_size = block_size
        self._keep = []
        if suffix_tables is not None and suffix_tables.numel() > 0 and suffix_tables.shape[-1] > 0:
            suffix_tables = _as_i32(suffix_tables)
            suffix_lens = _as_i32(suffix_lens)
            _require_cuda(suffix_tables, suffix_lens)
            if suffix_tables.dim() != 2 or suffix_tables.shape[0] != num_rows or suffix_lens.numel() != num_rows:
                raise RuntimeError("suffix tables/lens must be [num_rows, max_blocks] / [num_rows]")
            p.suffix_lens = suffix_lens.data_ptr()
            p.suffix_tables = suffix_tables.data_ptr()
            p.suffix_table_stride = suffix_tables.shape[1]
            self._keep += [suffix_tables, suffix_lens]
        else:
            p.suffix_table_stride = 0
        if group_prefix_lens is not None and group_prefix_lens.numel() > 0:
            group_prefix_lens = _as_i32(group_prefix_lens)
            group_row_offsets = _as_i32(group_row_offsets)
            g = group_prefix_lens.numel()
            if group_row_offsets.numel() != g + 1:
                raise RuntimeError("group_row_offsets must have num_groups + 1 entries")
            p.num_groups = g
            p.group_row_offsets = group_row_offsets.data_ptr()
            p.group_prefix_lens = group_prefix_lens.data_ptr()
            self._keep += [group_prefix_lens, group_row_offsets]
            if group_tables is not None and group_tables.numel() > 0:
                group_tables = _as_i32(group_tables)
                if group_tables.dim() == 1:
                    group_tables = group_tables.unsqueeze(0)
                if group_tables.shape[0] != g:
                    raise RuntimeError("group_tables must be [num_groups, max_prefix_blocks]")
                p.group_tables = group_tables.data_ptr()
                p.group_table_stride = group_tables.shape[1]
                self._keep.append(group_tables)
            _require_cuda(*self._keep)
        if seg_kv_lens is not None and seg_kv_lens.numel() > 0:
            # causal segments: the new tokens of prefill requests (see pb_attn_params in the header)
            seg_kv_lens, seg_row_offsets, seg_tables = _as_i32(seg_kv_lens), _as_i32(seg_row_offsets), _as_i32(seg_tables)
            _require_cuda(seg_kv_lens, seg_row_offsets, seg_tables)
            ns = seg_kv_lens.numel()
            if seg_row_offsets.numel() != ns + 1 or seg_tables.dim() != 2 or seg_tables.shape[0] != ns or seg_tables.shape[1] == 0:
                raise RuntimeError("segments need [n+1] row offsets, [n] kv lengths and [n, max_blocks] tables")
            p.num_segments = ns
            p.seg_row_offsets = seg_row_offsets.data_ptr()
            p.seg_kv_lens = seg_kv_lens.data_ptr()
            p.seg_tables = seg_tables.data_ptr()
            p.seg_table_stride = seg_tables.shape[1]
            self._keep += [seg_kv_lens, seg_row_offsets, seg_tables]
        if outer_prefix_lens is not None and outer_prefix_lens.numel() > 0:
            # outer prefix groups: a context shared above the groups (see pb_attn_params in the header)
            outer_prefix_lens, outer_row_offsets, outer_tables = (_as_i32(outer_prefix_lens), _as_i32(outer_row_offsets),
                                                                  _as_i32(outer_tables))
            _require_cuda(outer_prefix_lens, outer_row_offsets, outer_tables)
            no = outer_prefix_lens.numel()
            if outer_tables.dim() == 1:
                outer_tables = outer_tables.unsqueeze(0)
            if outer_row_offsets.numel() != no + 1 or outer_tables.dim() != 2 or outer_tables.shape[0] != no:
                raise RuntimeError("outer groups need [n+1] row offsets, [n] prefix lengths and [n, max_blocks] tables")
            p.num_outer_groups = no
            p.outer_row_offsets = outer_row_offsets.data_ptr()
            p.outer_prefix_lens = outer_prefix_lens.data_ptr()
            p.outer_tables = outer_tables.data_ptr()
            p.outer_table_stride = outer_tables.shape[1]
            self._keep += [outer_prefix_lens, outer_row_offsets, outer_tables]
        if head_mapping is not None:
            head_mapping = _as_i32(head_mapping)
            _require_cuda(head_mapping)
            p.head_mapping = head_mapping.data_ptr()
            self._keep.append(head_mapping)
        if slot_mapping is not None:
            # one cache slot per query row (its new token; negative = none): the call then performs the KV
            # fill itself when run() is given key_new / value_new (see pb_attn_params in the header)
            _require_cuda(slot_mapping)
            if slot_mapping.dtype not in (torch.int32, torch.int64) or slot_mapping.numel() != num_rows:
                raise RuntimeError("slot_mapping must hold one int32/int64 slot per query row")
            slot_mapping = slot_mapping.reshape(-1).contiguous()
            p.slot_mapping = slot_mapping.data_ptr()
            p.slot_is_i64 = 1 if slot_mapping.dtype == torch.int64 else 0
            self._keep.append(slot_mapping)
        self._has_slots = slot_mapping is not None
        p.dense_min_rows = dense_min_rows
        p.suffix_chunk_blocks = suffix_chunk_blocks
        p.prefix_chunk_blocks = prefix_chunk_blocks
        p.dense_ctas = dense_ctas
        p.dense_row_tile = dense_row_tile
        self.params = p
        nbytes = lib().pb_attn_workspace_bytes(C.byref(p))
        if nbytes == 0:
            raise _lib.PbError(_lib.PB_ERR_UNSUPPORTED, "pb_attn_workspace_bytes",
                               f"head_size={head_size} block_size={block_size} dtype={dtype}")
        self.workspace_bytes = nbytes
        # A planned call keeps its work lists in the workspace between plan() and every run(), so it owns
        # its buffer; only the one-shot wrappers (plan + run in one library call) share the per-device one.
        if workspace is not None:
            self.workspace = workspace
        elif shared_workspace:
            self.workspace = Workspace.get(device, nbytes)
        else:
            self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=device)
        if self.workspace.numel() < nbytes:
            raise _lib.PbError(_lib.PB_ERR_WORKSPACE, "AttentionCall")
        p.workspace = self.workspace.data_ptr()
        p.workspace_bytes = self.workspace.numel()
        self._planned = False
        self._bound = {}

    def _bind(self, query, out, key_cache, value_cache, qk_max=None, exp_sum=None, stats_mode=_lib.PB_STATS_NONE):
        p = self.params
        # the same tensors as in an earlier call (every layer of an iteration, every step of a loop):
        # their checks and geometry are remembered, only the pointers are rewritten
        key = (query.data_ptr(), out.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(), query.stride(0), out.stride(0),
               query.shape, out.shape, key_cache.shape, query.dtype, out.dtype, key_cache.dtype)
        hit = self._bound.get(key)
        if hit is not None and stats_mode == _lib.PB_STATS_NONE:
            (p.out, p.query, p.key_cache, p.value_cache, p.num_kv_heads, p.num_blocks, p.q_stride, p.out_stride,
             p.kv_block_stride, p.kv_head_stride) = hit
            p.qk_max = p.exp_sum = None
            p.stats_mode = stats_mode
            return
        _require_cuda(query, out, key_cache, value_cache)
        nb, hkv, d, b, kbs, khs = _kv_geometry(key_cache, value_cache)
        if query.dtype != self.dtype or key_cache.dtype != self.dtype or value_cache.dtype != self.dtype or out.dtype != self.dtype:
            raise RuntimeError("query, caches and out must share the dtype of the call")
        if query.dim() != 3 or query.shape[0] != p.num_rows or query.shape[1] != p.num_heads or query.shape[2] != p.head_size:
            raise RuntimeError(f"query must be [{p.num_rows}, {p.num_heads}, {p.head_size}]")
        if d != p.head_size or b != p.block_size:
            raise RuntimeError("cache head_size/block_size differ from the call's")
        if query.stride(2) != 1 or query.stride(1) != d or out.stride(2) != 1 or out.stride(1) != d:
            raise RuntimeError("query/out must be dense over (head, dim)")
        p.out = out.data_ptr()
        p.query = query.data_ptr()
        p.key_cache = key_cache.data_ptr()
        p.value_cache = value_cache.data_ptr()
        p.num_kv_heads = hkv
        p.num_blocks = nb
        p.q_stride = query.stride(0)
        p.out_stride = out.stride(0)
        p.kv_block_stride = kbs
        p.kv_head_stride = khs
        p.qk_max = _ptr(qk_max)
        p.exp_sum = _ptr(exp_sum)
        p.stats_mode = stats_mode
        if len(self._bound) > 64:
            self._bound.clear()
        # (shapes and dtypes were checked above; a tensor freed and another allocated at the same
        # address with other strides gets a different key through the strides)
        self._bound[key] = (p.out, p.query, p.key_cache, p.value_cache, p.num_kv_heads, p.num_blocks, p.q_stride,
                            p.out_stride, p.kv_block_stride, p.kv_head_stride)

    def plan(self, query, out, key_cache, value_cache) -> None:
        self._bind(query, out, key_cache, value_cache)
        check(lib().pb_attn_plan(C.byref(self.params), _stream(query)), "pb_attn_plan")
        self._planned = True

    def run(self, query, out, key_cache, value_cache, qk_max=None, exp_sum=None, stats_mode=_lib.PB_STATS_NONE,
            key_new=None, value_new=None):
        """One layer. With ``key_new`` / ``value_new`` ([num_rows, kv_heads, head_size], any row stride)
        the call also writes the rows' new tokens into the caches at the ``slot_mapping`` given to the
        constructor: the reference's ``vllm_reshape_and_cache`` followed by its attention, as one call."""
        self._bind(query, out, key_cache, value_cache, qk_max, exp_sum, stats_mode)
        p = self.params
        if key_new is not None:
            if not self._has_slots:
                raise RuntimeError("key_new / value_new need the slot_mapping given to AttentionCall")
            _require_cuda(key_new, value_new)
            shape = (p.num_rows, p.num_kv_heads, p.head_size)
            for x in (key_new, value_new):
                if tuple(x.shape) != shape or x.dtype != self.dtype or x.stride(2) != 1 or x.stride(1) != p.head_size:
                    raise RuntimeError(f"key_new / value_new must be {shape}, dense over (head, dim), of the call's dtype")
            p.key_new, p.value_new = key_new.data_ptr(), value_new.data_ptr()
            p.key_new_stride, p.value_new_stride = key_new.stride(0), value_new.stride(0)
        else:
            p.key_new = p.value_new = None
        if self._planned:
            rc = lib().pb_shared_prefix_attention_planned(C.byref(self.params), _stream(query))
        else:
            rc = lib().pb_shared_prefix_attention(C.byref(self.params), _stream(query))
        check(rc, "pb_shared_prefix_attention")
        return out

    def status(self) -> int:
        """Synchronises and returns the device status word (0 = clean)."""
        word = C.c_int32(0)
        rc = lib().pb_read_status(self.workspace.data_ptr(), torch.cuda.current_stream(self.device).cuda_stream, C.byref(word))
        if rc not in (_lib.PB_OK, _lib.PB_ERR_DEVICE):
            check(rc, "pb_read_status")
        return word.value


class HostStep:
    """One attention layer per call for tensors that live in page-locked HOST memory.

    Owns the device staging buffers of a fixed-shape decode batch and drives
    ``pb_attention_step_host``: upload of query / new K,V / slots / suffix lengths and tables,
    KV fill, planning, attention and download of the result are enqueued by ONE library call, in
    the order the reference's attention function runs them per layer
    (parrot/engine/builtin/attn_func.py:601-696). ``run()`` takes any contiguous host tensors;
    a caller that produces its inputs straight into the page-locked views ``h_query``,
    ``h_key_new``, ``h_value_new``, ``h_slots``, ``h_suffix_tables``, ``h_suffix_lens`` (and reads
    ``h_out``) gets them uploaded in one transfer.
    """

    def __init__(self, *, num_rows: int, num_heads: int, head_size: int, block_size: int, dtype: torch.dtype,
                 device: torch.device, max_suffix_blocks: int, num_new_tokens: int,
                 group_row_offsets: torch.Tensor, group_prefix_lens: torch.Tensor, group_tables: Optional[torch.Tensor],
                 num_kv_heads: Optional[int] = None, **tuning):
        hkv = num_kv_heads or num_heads
        esz = torch.empty((), dtype=dtype).element_size()
        t_new, width = max(num_new_tokens, 1), max(max_suffix_blocks, 1)
        # One staging arena on each side with the same layout: the library merges uploads whose
        # host and device ranges are adjacent, so inputs written into the h_* views below go up in
        # a single transfer.
        fields = [
            ("query", (num_rows, num_heads, head_size), dtype, num_rows * num_heads * head_size * esz),
            ("key_new", (t_new, hkv, head_size), dtype, t_new * hkv * head_size * esz),
            ("value_new", (t_new, hkv, head_size), dtype, t_new * hkv * head_size * esz),
            ("slots", (t_new,), torch.int64, t_new * 8),
            ("suffix_tables", (num_rows, width), torch.int32, num_rows * width * 4),
            ("suffix_lens", (num_rows,), torch.int32, num_rows * 4),
        ]
        total = sum(f[3] for f in fields)
        self.d_arena = torch.zeros((total,), dtype=torch.uint8, device=device)
        self.h_arena = torch.zeros((total,), dtype=torch.uint8).pin_memory()
        off = 0
        for name, shape, dt, nbytes in fields:
            setattr(self, name, self.d_arena[off:off + nbytes].view(dt).view(shape))
            setattr(self, "h_" + name, self.h_arena[off:off + nbytes].view(dt).view(shape))
            off += nbytes
        self.out = torch.empty_like(self.query)
        self.h_out = torch.empty((num_rows, num_heads, head_size), dtype=dtype).pin_memory()
        self.call = AttentionCall(
            num_rows=num_rows, num_heads=num_heads, head_size=head_size, block_size=block_size, dtype=dtype,
            device=device, suffix_lens=self.suffix_lens, suffix_tables=self.suffix_tables,
            group_row_offsets=group_row_offsets, group_prefix_lens=group_prefix_lens, group_tables=group_tables, **tuning)
        io = _lib.PbHostStep()
        io.d_key_new, io.d_value_new, io.d_slot_mapping = self.key_new.data_ptr(), self.value_new.data_ptr(), self.slots.data_ptr()
        io.num_new_tokens = num_new_tokens
        self.io = io
        self.device = device
        self._fn = lib().pb_attention_step_host
        self._params_ref, self._io_ref = C.byref(self.call.params), C.byref(io)
        self._bound = None
        self._graphs = {}

    @staticmethod
    def _host(t: Optional[torch.Tensor], dtype=None) -> Optional[int]:
        if t is None:
            return None
        if t.is_cuda or not t.is_contiguous() or (dtype is not None and t.dtype != dtype):
            raise RuntimeError("host step inputs must be contiguous CPU tensors of the expected dtype")
        return t.data_ptr()

    def run(self, query, key_new, value_new, slot_mapping, suffix_lens, suffix_tables, out_host, key_cache, value_cache,
            *, replan: bool = True, synchronize: bool = True):
        """All tensor arguments except the caches are host tensors; ``suffix_lens`` /
        ``suffix_tables`` may be None when they did not change since the last call."""
        io, call = self.io, self.call
        if tuple(query.shape) != tuple(self.query.shape) or tuple(out_host.shape) != tuple(self.out.shape):
            raise RuntimeError("query/out shape differs from the batch this HostStep was built for")
        if key_new is not None and key_new.shape[0] != io.num_new_tokens:
            raise RuntimeError("number of new tokens differs from the batch this HostStep was built for")
        if suffix_tables is not None and tuple(suffix_tables.shape) != tuple(self.suffix_tables.shape):
            raise RuntimeError("suffix_tables must be [num_rows, max_suffix_blocks]")
        io.h_query = self._host(query, self.query.dtype)
        io.h_key_new = self._host(key_new, self.query.dtype)
        io.h_value_new = self._host(value_new, self.query.dtype)
        io.h_slot_mapping = self._host(slot_mapping, torch.int64)
        io.h_suffix_lens = self._host(suffix_lens, torch.int32)
        io.h_suffix_tables = self._host(suffix_tables, torch.int32)
        io.h_out = self._host(out_host, self.query.dtype)
        io.direct_out = 0
        lo, hi = self.h_arena.data_ptr(), self.h_arena.data_ptr() + self.h_arena.numel()
        ins = (io.h_query, io.h_key_new, io.h_value_new, io.h_slot_mapping, io.h_suffix_lens, io.h_suffix_tables)
        io.merge_adjacent = 1 if all(a is None or lo <= a < hi for a in ins) else 0
        io.replan = 1 if replan else 0
        io.synchronize = 1 if synchronize else 0
        call._bind(self.query, self.out, key_cache, value_cache)
        self._bound = None
        check(self._fn(C.byref(call.params), C.byref(io), _stream(self.query)), "pb_attention_step_host")
        return out_host

    def step_graph(self, key_cache, value_cache, *, replan: bool = True, wait: bool = True):
        """``step()`` replayed from a CUDA graph captured once per (cache pair, replan): upload,
        fill, planner, attention and the result's way back are ONE launch for the host, which then
        waits for the stream. The first call for a cache pair runs ``step()`` itself (lazy one-time
        initialisation must not fall into a capture), the second captures, later ones replay. The
        graph bakes in the addresses of this object's staging views and of the caches. With
        ``wait=False`` a replay returns as soon as it is enqueued on the current stream (the
        caller synchronises before it reads ``h_out`` or rewrites the staging views)."""
        key = (key_cache.data_ptr(), value_cache.data_ptr(), bool(replan))
        state = self._graphs.get(key)
        stream = torch.cuda.current_stream(self.device)
        if state is None:
            self._graphs[key] = "warm"
            return self.step(key_cache, value_cache, replan=replan, synchronize=True)
        if state == "warm":
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(stream)
            with torch.cuda.graph(graph, stream=side):
                self.step(key_cache, value_cache, replan=replan, synchronize=False)
            self._graphs[key] = state = graph
        state.replay()
        if wait:
            stream.synchronize()
        return self.h_out

    def step(self, key_cache, value_cache, *, replan: bool = True, synchronize: bool = True):
        """``run()`` on the step's own page-locked views (``h_query`` ... ``h_out``), with the
        per-call argument checks done once per cache pair: the hot loop of a host-side caller."""
        io, call = self.io, self.call
        key = (key_cache.data_ptr(), value_cache.data_ptr())
        if self._bound != key:
            io.h_query, io.h_key_new, io.h_value_new = self.h_query.data_ptr(), self.h_key_new.data_ptr(), self.h_value_new.data_ptr()
            io.h_slot_mapping, io.h_out = self.h_slots.data_ptr(), self.h_out.data_ptr()
            io.h_suffix_lens, io.h_suffix_tables = self.h_suffix_lens.data_ptr(), self.h_suffix_tables.data_ptr()
            # (direct_out stays off: measured here, the merge kernel's own stores over the bus were never
            # faster than the copy engine's download and up to 20 us slower on some hosts)
            io.merge_adjacent, io.direct_out = 1, 0
            call._bind(self.query, self.out, key_cache, value_cache)
            self._bound = key
        io.replan = 1 if replan else 0
        io.synchronize = 1 if synchronize else 0
        rc = self._fn(self._params_ref, self._io_ref, torch.cuda.current_stream(self.device).cuda_stream)
        if rc != _lib.PB_OK:
            check(rc, "pb_attention_step_host")
        return self.h_out


class HostStepPipeline:
    """``depth`` host steps in flight: a ring of ``HostStep`` objects, each with its own page-locked
    staging views, device staging, workspace and stream, so that the upload and download of one
    step run beside the kernels of another (two independent micro-batches, or a producer that
    prepares step i+1 while step i computes). Every step still uploads its inputs and delivers
    its result to host memory; ``submit`` returns the result of the OLDEST step in flight.

        pipe = HostStepPipeline(depth=2, **host_step_arguments)
        slot = pipe.next_slot()            # write the step's inputs into slot.h_query, ...
        done = pipe.submit(key_cache, value_cache)   # None while the ring fills, then a HostStep whose h_out is ready
        ...
        for slot in pipe.drain(): ...      # the results still in flight, oldest first

    Steps in flight at the same time must not write KV slots another of them reads."""

    def __init__(self, depth: int = 2, **host_step_args):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.slots = [HostStep(**host_step_args) for _ in range(depth)]
        dev = self.slots[0].device
        self.streams = [torch.cuda.Stream(device=dev) for _ in range(depth)]
        self.done = [torch.cuda.Event() for _ in range(depth)]
        self.in_flight = [False] * depth
        self.count = 0

    def next_slot(self) -> "HostStep":
        """The HostStep the next ``submit`` will run; its previous result has been handed out."""
        return self.slots[self.count % len(self.slots)]

    def submit(self, key_cache, value_cache, *, replan: bool = True) -> Optional["HostStep"]:
        depth = len(self.slots)
        s = self.count % depth
        if self.in_flight[s]:
            raise RuntimeError("the slot's previous result was not collected")
        with torch.cuda.stream(self.streams[s]):
            self.slots[s].step_graph(key_cache, value_cache, replan=replan, wait=False)
            self.done[s].record(self.streams[s])
        self.in_flight[s] = True
        self.count += 1
        oldest = self.count % depth
        if not self.in_flight[oldest]:
            return None
        self.done[oldest].synchronize()
        self.in_flight[oldest] = False
        return self.slots[oldest]

    def drain(self):
        """Waits for the steps still in flight; their HostSteps, oldest first."""
        depth, out = len(self.slots), []
        for k in range(depth):
            s = (self.count + k) % depth
            if self.in_flight[s]:
                self.done[s].synchronize()
                self.in_flight[s] = False
                out.append(self.slots[s])
        return out


# small device constants, cached so the single-group wrapper does not upload on every call
_const_cache: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}


def _single_group_meta(device: torch.device, prefix_len: int, num_rows: int):
    key = (device.index, prefix_len, num_rows)
    hit = _const_cache.get(key)
    if hit is None:
        if len(_const_cache) > 256:
            _const_cache.clear()
        hit = (
            torch.tensor([0, num_rows], dtype=torch.int32, device=device),
            torch.tensor([prefix_len], dtype=torch.int32, device=device),
        )
        _const_cache[key] = hit
    return hit


def flash_paged_attention_grouped(
    query: torch.Tensor,  # [num_rows, num_heads, head_size]
    key_cache: torch.Tensor,  # [num_blocks, num_kv_heads, head_size/x, block_size, x]
    value_cache: torch.Tensor,  # [num_blocks, num_kv_heads, head_size, block_size]
    head_mapping: Optional[torch.Tensor],  # [num_heads] or None (identity)
    group_prefix_lens: torch.Tensor,  # [G] int32, true token counts
    group_block_tables: torch.Tensor,  # [G, max_prefix_blocks] int32
    group_row_offsets: torch.Tensor,  # [G + 1] int32 CSR over rows (rows sorted by group)
    paged_context_lens: torch.Tensor,  # [num_rows] int32
    paged_block_tables: torch.Tensor,  # [num_rows, max_blocks] int32
    out: Optional[torch.Tensor] = None,
    **tuning,
) -> torch.Tensor:
    """Shared-prefix decode attention for G prefix groups; the reference supports one
    (a single LCA per batch, parrot/engine/builtin/attn_func.py:441-459)."""
    num_rows, num_heads, head_size = query.shape
    if out is None:
        out = torch.empty((num_rows, num_heads, head_size), dtype=query.dtype, device=query.device)
    if num_rows == 0:
        return out
    call = AttentionCall(
        num_rows=num_rows, num_heads=num_heads, head_size=head_size, block_size=value_cache.shape[3],
        dtype=query.dtype, device=query.device, suffix_lens=paged_context_lens, suffix_tables=paged_block_tables,
        group_row_offsets=group_row_offsets, group_prefix_lens=group_prefix_lens, group_tables=group_block_tables,
        head_mapping=head_mapping, shared_workspace=True, **tuning,
    )
    return call.run(query, out, key_cache, value_cache)


def flash_paged_attention(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    head_mapping: Optional[torch.Tensor],
    flash_context_len: int,
    flash_block_table: torch.Tensor,  # [max_prefix_blocks]
    paged_context_lens: torch.Tensor,  # [num_seqs]
    paged_block_tables: torch.Tensor,  # [num_seqs, max_num_blocks_per_seq]
    **tuning,
) -> torch.Tensor:
    """Same signature as the reference's flash_paged_attention
    (parrot/engine/builtin/kernels/shared_flash_decoding.py:285-329)."""
    num_seqs = query.shape[0]
    offs, plen = _single_group_meta(query.device, int(flash_context_len), num_seqs)
    tables = flash_block_table.reshape(1, -1)
    return flash_paged_attention_grouped(
        query, key_cache, value_cache, head_mapping, plen, tables, offs, paged_context_lens,
        paged_block_tables, **tuning,
    )


# The reference's second variant runs the two stages in the other order
# (shared_flash_decoding.py:332-376); the result is the same attention.
paged_flash_attention = flash_paged_attention


def vllm_paged_attention(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    head_mapping: Optional[torch.Tensor],
    context_lens: torch.Tensor,
    block_tables: torch.Tensor,
) -> torch.Tensor:
    """Unshared paged decode attention (parrot/engine/builtin/kernels/vllm/paged_attention.py:12-38)."""
    num_rows, num_heads, head_size = query.shape
    out = torch.empty((num_rows, num_heads, head_size), dtype=query.dtype, device=query.device)
    if num_rows == 0:
        return out
    call = AttentionCall(
        num_rows=num_rows, num_heads=num_heads, head_size=head_size, block_size=value_cache.shape[3],
        dtype=query.dtype, device=query.device, suffix_lens=context_lens, suffix_tables=block_tables,
        head_mapping=head_mapping, shared_workspace=True,
    )
    return call.run(query, out, key_cache, value_cache)


def _flat_slots(slot_mapping: torch.Tensor, num_tokens: int) -> torch.Tensor:
    # The reference's AttnFunc hands over a 2-D zero-padded [num_jobs, max_new] tensor that the
    # kernel indexes flat (attn_func.py:567,589-593 vs cache_kernels.cu:155-156); that is only
    # meaningful when it has exactly one slot per token.
    if slot_mapping.numel() != num_tokens:
        raise RuntimeError(
            f"slot_mapping has {slot_mapping.numel()} entries for {num_tokens} tokens; pass a flat ragged mapping"
        )
    if slot_mapping.dtype not in (torch.int32, torch.int64):
        slot_mapping = slot_mapping.to(torch.int64)
    return slot_mapping.reshape(-1).contiguous()


def _kv_rows_call(fn_name, key, value, key_cache, value_cache, slot_mapping):
    _require_cuda(key, value, key_cache, value_cache, slot_mapping)
    if key.shape != value.shape or key.dim() != 3:
        raise RuntimeError("key and value must both be [num_tokens, num_heads, head_size]")
    if key.dtype != key_cache.dtype or value.dtype != value_cache.dtype or key.dtype != value.dtype:
        raise RuntimeError("key/value and caches must share a dtype")
    t, h, d = key.shape
    nb, hkv, dc, b, kbs, khs = _kv_geometry(key_cache, value_cache)
    if hkv != h or dc != d:
        raise RuntimeError("cache heads/head_size differ from key's")
    for x in (key, value):
        if x.stride(2) != 1 or x.stride(1) != d:
            raise RuntimeError("key/value must be dense over (head, dim)")
    slots = _flat_slots(slot_mapping, t)
    rc = getattr(lib(), fn_name)(
        key.data_ptr(), value.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(), slots.data_ptr(),
        1 if slots.dtype == torch.int64 else 0, t, h, d, b, key.stride(0), value.stride(0), kbs, khs, nb,
        _dtype_code(key), _stream(key),
    )
    check(rc, fn_name)


def vllm_reshape_and_cache(key_to_cache, value_to_cache, key_cache, value_cache, slot_mapping) -> None:
    """KV fill (parrot/engine/builtin/kernels/vllm/reshape_and_cache.py:9-22)."""
    _kv_rows_call("pb_reshape_and_cache", key_to_cache, value_to_cache, key_cache, value_cache, slot_mapping)


def _rotary_common(positions, query, key, cos_sin_cache, head_size):
    _require_cuda(positions, query, key, cos_sin_cache)
    if positions.dtype != torch.int64:
        positions = positions.to(torch.int64)
    positions = positions.reshape(-1).contiguous()
    t = positions.numel()
    if query.dtype != key.dtype or cos_sin_cache.dtype != query.dtype:
        raise RuntimeError("query, key and cos_sin_cache must share a dtype")
    if cos_sin_cache.dim() != 2 or not cos_sin_cache.is_contiguous():
        raise RuntimeError("cos_sin_cache must be a contiguous [max_position, rot_dim] tensor")

    def rows(x, what):  # [T, H*D] or [T, H, D], dense inside a token, any row stride
        if x.shape[0] != t or x.stride(-1) != 1 or (x.dim() == 3 and x.stride(1) != head_size):
            raise RuntimeError(f"{what} must be [num_tokens, num_heads(*)head_size], dense inside a token")
        width = x.shape[1] if x.dim() == 2 else x.shape[1] * x.shape[2]
        if x.dim() not in (2, 3) or width % head_size:
            raise RuntimeError(f"{what} width is not a multiple of head_size")
        return width // head_size

    return positions, t, rows(query, "query"), rows(key, "key")


def vllm_rotary_emb(positions, query, key, cos_sin_cache, head_size: int) -> None:
    """NeoX rotary embedding of query and key IN PLACE; same signature as the reference's
    vllm_rotary_emb (parrot/engine/builtin/kernels/vllm/rotary_embed.py:10-25)."""
    positions, t, hq, hk = _rotary_common(positions, query, key, cos_sin_cache, head_size)
    rc = lib().pb_rotary_reshape_and_cache(
        query.data_ptr(), key.data_ptr(), None, None, None, None, 1, positions.data_ptr(), cos_sin_cache.data_ptr(),
        cos_sin_cache.shape[1], cos_sin_cache.shape[0], t, hq, hk, head_size, 16, query.stride(0), key.stride(0), 0,
        0, 0, 0, 1, _dtype_code(query), _stream(query))
    check(rc, "pb_rotary_reshape_and_cache")


def rotary_reshape_and_cache(positions, query, key, value, key_cache, value_cache, slot_mapping, cos_sin_cache,
                             head_size: int, write_key_back: bool = False) -> None:
    """The reference's ``vllm_rotary_emb`` followed by ``vllm_reshape_and_cache``
    (parrot/engine/builtin/models/llama.py:123-137) in one pass: query rotated in place, the rotated
    key written straight into the paged cache (and back into ``key`` only on request), value cached."""
    positions, t, hq, hk = _rotary_common(positions, query, key, cos_sin_cache, head_size)
    _require_cuda(value, key_cache, value_cache, slot_mapping)
    nb, hkv, dc, b, kbs, khs = _kv_geometry(key_cache, value_cache)
    if hkv != hk or dc != head_size or value.shape[0] != t or value.stride(-1) != 1:
        raise RuntimeError("cache heads/head_size differ from key's, or value is not [num_tokens, ...]")
    if value.dim() == 3 and value.stride(1) != head_size:
        raise RuntimeError("value must be dense inside a token")
    if key_cache.dtype != key.dtype or value.dtype != key.dtype:
        raise RuntimeError("key/value and caches must share a dtype")
    slots = _flat_slots(slot_mapping, t)
    rc = lib().pb_rotary_reshape_and_cache(
        query.data_ptr(), key.data_ptr(), value.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
        slots.data_ptr(), 1 if slots.dtype == torch.int64 else 0, positions.data_ptr(), cos_sin_cache.data_ptr(),
        cos_sin_cache.shape[1], cos_sin_cache.shape[0], t, hq, hk, head_size, b, query.stride(0), key.stride(0),
        value.stride(0), kbs, khs, nb, 1 if write_key_back else 0, _dtype_code(query), _stream(query))
    check(rc, "pb_rotary_reshape_and_cache")


def gather_cached_kv(key, value, key_cache, value_cache, slot_mapping) -> None:
    """Inverse of the fill (3rdparty/vllm/csrc/cache.cpp:24-29)."""
    _kv_rows_call("pb_gather_cached_kv", key, value, key_cache, value_cache, slot_mapping)


def _move_from_cache(cache, dest, src_slot_indices, dest_indices, is_value: bool):
    if src_slot_indices.shape != dest_indices.shape:
        raise AssertionError("src_indices and dest_indices must have the same shape")
    _require_cuda(cache, dest, src_slot_indices, dest_indices)
    if is_value:
        nb, h, d, b = cache.shape
    else:
        nb, h, dx, b, x = cache.shape
        d = dx * x
    if dest.dim() != 3 or dest.shape[1] != h or dest.shape[2] != d:
        raise AssertionError("storage shape mismatch")
    if dest.shape[0] < dest_indices.shape[0]:
        raise AssertionError("dest_storage is too small")
    if dest.stride(2) != 1 or dest.stride(1) != d:
        raise RuntimeError("dest must be dense over (head, dim)")
    src = src_slot_indices.to(torch.int64).contiguous()
    dst = dest_indices.to(torch.int64).contiguous()
    rc = lib().pb_move_tokens_from_blocked_cache(
        cache.data_ptr(), dest.data_ptr(), src.data_ptr(), dst.data_ptr(), src.numel(), 1 if is_value else 0,
        h, d, b, dest.stride(0), cache.stride(0), cache.stride(1), nb, dest.shape[0], _dtype_code(cache),
        _stream(cache),
    )
    check(rc, "pb_move_tokens_from_blocked_cache")


def move_tokens_from_blocked_k_cache(blocked_k_cache, dest_storage, src_slot_indices, dest_indices) -> None:
    """Paged K -> contiguous rows (parrot/engine/builtin/kernels/tokens_moving.py:163-218)."""
    _move_from_cache(blocked_k_cache, dest_storage, src_slot_indices, dest_indices, False)


def move_tokens_from_blocked_v_cache(blocked_v_cache, dest_storage, src_slot_indices, dest_indices) -> None:
    """Paged V -> contiguous rows (parrot/engine/builtin/kernels/tokens_moving.py:271-313)."""
    _move_from_cache(blocked_v_cache, dest_storage, src_slot_indices, dest_indices, True)


def discontinuous_move_tokens(src_storage, dest_storage, src_indices, dest_indices) -> None:
    """dest[dest_indices[i]] = src[src_indices[i]] (parrot/engine/builtin/kernels/tokens_moving.py:67-100)."""
    if src_indices.shape != dest_indices.shape:
        raise AssertionError("src_indices and dest_indices must have the same shape")
    if src_storage.shape[0] < src_indices.shape[0]:
        raise AssertionError("src_storage is too small")
    if dest_storage.shape[0] < dest_indices.shape[0]:
        raise AssertionError("dest_storage is too small")
    if dest_storage.shape[1:] != src_storage.shape[1:]:
        raise AssertionError("storage shape mismatch")
    _require_cuda(src_storage, dest_storage, src_indices, dest_indices)
    if src_storage.dtype != dest_storage.dtype:
        raise RuntimeError("dtype mismatch")
    if not src_storage[0].is_contiguous() or not dest_storage[0].is_contiguous():
        raise RuntimeError("rows must be contiguous")
    es = src_storage.element_size()
    row_bytes = src_storage[0].numel() * es
    src = src_indices.to(torch.int64).contiguous()
    dst = dest_indices.to(torch.int64).contiguous()
    rc = lib().pb_discontinuous_move_tokens(
        src_storage.data_ptr(), dest_storage.data_ptr(), src.data_ptr(), dst.data_ptr(), src.numel(), row_bytes,
        src_storage.stride(0) * es, dest_storage.stride(0) * es, src_storage.shape[0], dest_storage.shape[0],
        _stream(src_storage),
    )
    check(rc, "pb_discontinuous_move_tokens")


def copy_blocks(key_caches, value_caches, block_mapping) -> None:
    """Copies cache blocks inside every layer's K and V cache: ``block_mapping`` maps a source
    block to the list of its destination blocks. Same signature as the reference extension's
    ``cache_ops.copy_blocks`` (3rdparty/vllm/csrc/cache_kernels.cu:54-138)."""
    if len(key_caches) != len(value_caches):
        raise RuntimeError("key_caches and value_caches must have one tensor per layer each")
    pairs = [(int(src), int(dst)) for src, dsts in block_mapping.items() for dst in dsts]
    if not key_caches or not pairs:
        return
    k0 = key_caches[0]
    _require_cuda(*key_caches, *value_caches)
    for k, v in zip(key_caches, value_caches):
        if k.dtype != k0.dtype or v.dtype != k0.dtype or k.shape != k0.shape or v.shape[0] != k0.shape[0] or v[0].numel() != k0[0].numel():
            raise RuntimeError("all layers must share dtype, block count and block size")
        if not k.is_contiguous() or not v.is_contiguous():
            raise RuntimeError("caches must be contiguous")
    dev = k0.device
    kp = torch.tensor([k.data_ptr() for k in key_caches], dtype=torch.int64, device=dev)
    vp = torch.tensor([v.data_ptr() for v in value_caches], dtype=torch.int64, device=dev)
    pr = torch.tensor(pairs, dtype=torch.int64, device=dev)
    rc = lib().pb_copy_blocks(kp.data_ptr(), vp.data_ptr(), len(key_caches), pr.data_ptr(), len(pairs),
                              k0[0].numel() * k0.element_size(), k0.shape[0], _stream(k0))
    check(rc, "pb_copy_blocks")


def swap_blocks(src: torch.Tensor, dst: torch.Tensor, block_mapping) -> None:
    """Copies blocks ``src[s] -> dst[d]`` for every ``s: d`` of ``block_mapping`` between a GPU cache
    and a host cache or two caches on one GPU. Same signature as the reference extension's
    ``cache_ops.swap_blocks`` (3rdparty/vllm/csrc/cache_kernels.cu:9-50)."""
    if src.dtype != dst.dtype or src[0].numel() != dst[0].numel() or not src.is_contiguous() or not dst.is_contiguous():
        raise RuntimeError("src and dst must be contiguous caches of one dtype and block size")
    if src.is_cuda and dst.is_cuda:
        if src.device != dst.device:
            raise RuntimeError("src and dst must be on the same GPU")
        direction, cuda_t = 0, src
    elif src.is_cuda:
        direction, cuda_t = 1, src
    elif dst.is_cuda:
        direction, cuda_t = 2, dst
    else:
        raise RuntimeError("Invalid device combination")
    pairs = sorted((int(s), int(d)) for s, d in block_mapping.items())
    if not pairs:
        return
    hp = torch.tensor(pairs, dtype=torch.int64)
    rc = lib().pb_swap_blocks(src.data_ptr(), dst.data_ptr(), hp.data_ptr(), len(pairs), src[0].numel() * src.element_size(),
                              src.shape[0], dst.shape[0], direction, _stream(cuda_t))
    check(rc, "pb_swap_blocks")


def sample_top_p(logits: torch.Tensor, temperature=None, top_p=None, uniforms: Optional[torch.Tensor] = None,
                 generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """One token id per row of ``logits`` [rows, vocab]: logits / temperature, nucleus filtering,
    softmax and one draw, in a single kernel that never sorts the row. The part of the reference's
    ``Sampler.forward`` after the logits GEMM (parrot/engine/builtin/models/sampler.py:33-66).
    ``temperature`` / ``top_p``: per-row sequences or float tensors, None = 1.0. ``uniforms``: float32
    [rows] in [0, 1) (drawn from ``generator`` when None); the result is a pure function of them."""
    _require_cuda(logits)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise RuntimeError("logits must be [rows, vocab] with unit stride along the vocabulary")
    rows, vocab = logits.shape
    dev = logits.device

    def per_row(v, name):
        if v is None:
            return None
        if not isinstance(v, torch.Tensor):
            v = [float(t) for t in v]
            if name == "temperature" and any(t <= 0.0 for t in v):
                raise ValueError("temperature must be positive")
            if all(t == 1.0 for t in v):
                return None
            v = torch.tensor(v, dtype=torch.float32, device=dev)
        if v.shape != (rows,) or v.dtype != torch.float32 or v.device != dev or not v.is_contiguous():
            raise RuntimeError(f"{name} must be a contiguous float32 tensor [rows] on the logits' device")
        return v

    temperature, top_p = per_row(temperature, "temperature"), per_row(top_p, "top_p")
    if uniforms is None:
        uniforms = torch.rand(rows, dtype=torch.float32, device=dev, generator=generator)
    uniforms = per_row(uniforms, "uniforms")
    ids = torch.empty(rows, dtype=torch.int64, device=dev)
    if rows == 0:
        return ids
    rc = lib().pb_sample_top_p(logits.data_ptr(), _dtype_code(logits), rows, vocab, logits.stride(0),
                               temperature.data_ptr() if temperature is not None else None,
                               top_p.data_ptr() if top_p is not None else None,
                               uniforms.data_ptr(), ids.data_ptr(), _stream(logits))
    check(rc, "pb_sample_top_p")
    return ids
