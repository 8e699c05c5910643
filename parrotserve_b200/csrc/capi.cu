// extern "C" entry points of the attention path: validation, workspace carve-up, launch order.
// No allocation, no host synchronisation (except pb_read_status), nothing thrown.
#include <mutex>

#include "common.cuh"

namespace pb {

int sm_count() {
  static std::mutex mu;
  static int cached[64] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return kMaxSMs;  // no device to ask (a size query on a machine without a GPU)
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = kMaxSMs;
    }
    cached[dev] = n < kMaxSMs ? n : kMaxSMs;
  }
  return cached[dev];
}

namespace {

// Events a caller asked to have recorded around the next single-query kernel launch of this thread
// (pb_attn_set_timing_events); consumed by that launch.
thread_local cudaEvent_t g_ev_begin = nullptr, g_ev_end = nullptr;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
int elem_bytes(int dtype) { return dtype == PB_F32 ? 4 : 2; }

int pow2_floor(long long v) {
  int r = 1;
  while ((long long)r * 2 <= v) r *= 2;
  return r;
}

bool sq_shape_supported(int head_size, int block_size) {
  return (head_size == 128 || head_size == 64 || head_size == 80 || head_size == 96 || head_size == 112 ||
          head_size == 256) && (block_size == 8 || block_size == 16 || block_size == 32);
}

// Static bounds -> chunking and workspace layout. Returns a pb_status.
int compute_layout(const pb_attn_params* p, WsLayout* L) {
  if (!p) return PB_ERR_INVALID_ARG;
  if (p->num_rows < 0 || p->num_heads <= 0 || p->num_kv_heads <= 0 || p->head_size <= 0 ||
      p->block_size <= 0 || p->num_groups < 0 || p->suffix_table_stride < 0 || p->group_table_stride < 0 ||
      p->num_segments < 0 || p->seg_table_stride < 0 || p->num_outer_groups < 0 || p->outer_table_stride < 0)
    return PB_ERR_INVALID_ARG;
  if (p->dtype != PB_F32 && p->dtype != PB_F16 && p->dtype != PB_BF16) return PB_ERR_UNSUPPORTED;
  if (!sq_shape_supported(p->head_size, p->block_size)) return PB_ERR_UNSUPPORTED;
  if (p->num_heads > 0xffff) return PB_ERR_UNSUPPORTED;  // (head, partial slot) travel as one word
  const long long rows = p->num_rows, H = p->num_heads;
  const int kNumSMs = sm_count();
  const long long total_warps = (long long)kNumSMs * 8;

  // suffix chunk: aim at ~24 work items per resident warp, assuming rows are half full on average
  int cs = p->suffix_chunk_blocks;
  if (cs <= 0) {
    const long long est = rows * H * p->suffix_table_stride / 2;
    cs = pow2_floor(est / (24 * total_warps) > 0 ? est / (24 * total_warps) : 1);
    if (cs < 4) cs = 4;
    if (cs > 32) cs = 32;
  }
  // prefix chunk: aim at >= 4 dense items per SM; a multiple of 8 blocks (one 128-token MMA tile)
  int cp = p->prefix_chunk_blocks;
  if (cp <= 0) {
    const long long tot = (long long)(p->num_groups > 0 ? p->num_groups : 1) * H * p->group_table_stride;
    long long want = tot / (4 * kNumSMs);
    cp = pow2_floor(want > 0 ? want : 1);
    if (cp < 8) cp = 8;
    if (cp > 256) cp = 256;
  }
  L->cs = cs;
  L->cp = cp;
  // prefix partial slots: chunks of the single-query fallback, or one per dense CTA that can
  // touch a (row tile, head): at most its kv tiles and at most the CTA count
  int dense_parts = (p->group_table_stride + kDenseTileBlocks - 1) / kDenseTileBlocks;
  if (dense_parts > kNumSMs) dense_parts = kNumSMs;
  if (!dense_prefix_supported(p->dtype, p->head_size, p->block_size)) dense_parts = 0;
  L->pparts = (p->num_groups > 0) ? (p->group_table_stride + cp - 1) / cp : 0;
  if (p->num_groups > 0 && dense_parts > L->pparts) L->pparts = dense_parts;
  L->sparts = (p->suffix_table_stride + cs - 1) / cs;
  // causal segments: one partial per dense CTA that touches a (row tile, head), or per chunk of the
  // single-query fallback
  L->cparts = 0;
  if (p->num_segments > 0) {
    int dense_c = (p->seg_table_stride + kDenseTileBlocks - 1) / kDenseTileBlocks;
    if (dense_c > kNumSMs) dense_c = kNumSMs;
    if (!dense_prefix_supported(p->dtype, p->head_size, p->block_size)) dense_c = 0;
    L->cparts = (p->seg_table_stride + cs - 1) / cs;
    if (dense_c > L->cparts) L->cparts = dense_c;
  }
  if (p->num_segments > 0 && p->num_groups > 0 && dense_parts > 0) {
    // a prefill request joined with its group: one item spans the prefix and the request's context
    int joined = (p->group_table_stride + kDenseTileBlocks - 1) / kDenseTileBlocks +
                 (p->seg_table_stride + kDenseTileBlocks - 1) / kDenseTileBlocks;
    if (joined > kNumSMs) joined = kNumSMs;
    if (joined > L->pparts) L->pparts = joined;
  }
  // outer prefix groups: sized like the prefix range
  L->oparts = 0;
  if (p->num_outer_groups > 0) {
    int dense_o = (p->outer_table_stride + kDenseTileBlocks - 1) / kDenseTileBlocks;
    if (dense_o > kNumSMs) dense_o = kNumSMs;
    if (!dense_prefix_supported(p->dtype, p->head_size, p->block_size)) dense_o = 0;
    L->oparts = (p->outer_table_stride + cp - 1) / cp;
    if (dense_o > L->oparts) L->oparts = dense_o;
  }
  L->parts = L->pparts + L->cparts + L->sparts + L->oparts;
  if (L->parts < 1) L->parts = 1;
  const long long cap_sq = rows * (L->pparts + L->cparts + L->sparts + L->oparts) + 1;
  // row tiles of groups and segments, plus the partial tiles the gaps around joined segments add
  const long long cap_dn = (long long)p->num_groups + p->num_outer_groups + 2ll * p->num_segments + 3 * ((rows + 127) / 128) + 1;
  if (cap_sq > 0x7fffffffll || cap_dn > 0x7fffffffll || rows * L->parts > 0x7fffffffll || L->parts > 0x7fff)
    return PB_ERR_INVALID_ARG;
  L->cap_sq = (int32_t)cap_sq;
  L->cap_dn = (int32_t)cap_dn;
  L->dense_min_rows = p->dense_min_rows > 0 ? p->dense_min_rows : 4;

  size_t off = align_up(kHdrInts * sizeof(int32_t), 256);
  L->off_rowinfo = off; off = align_up(off + (size_t)rows * sizeof(RowInfo), 256);
  L->off_sq = off;      off = align_up(off + (size_t)cap_sq * sizeof(SqItem), 256);
  L->off_dn = off;      off = align_up(off + (size_t)cap_dn * sizeof(DnItem), 256);
  L->off_ml = off;      off = align_up(off + (size_t)rows * L->parts * H * sizeof(float2), 256);
  L->off_acc = off;     off = align_up(off + (size_t)rows * L->parts * H * p->head_size * sizeof(float), 256);
  L->total = off;
  return PB_OK;
}

int validate_and_bind(const pb_attn_params* p, WsLayout* L, AttnDev* d) {
  int rc = compute_layout(p, L);
  if (rc != PB_OK) return rc;
  if (p->num_rows == 0) return PB_OK;
  if (!p->out || !p->query || !p->key_cache || !p->value_cache) return PB_ERR_INVALID_ARG;
  if (p->suffix_table_stride > 0 && (!p->suffix_lens || !p->suffix_tables)) return PB_ERR_INVALID_ARG;
  if (p->num_groups > 0 && (!p->group_row_offsets || !p->group_prefix_lens)) return PB_ERR_INVALID_ARG;
  if (p->num_groups > 0 && p->group_table_stride > 0 && !p->group_tables) return PB_ERR_INVALID_ARG;
  if (p->num_segments > 0 && (!p->seg_row_offsets || !p->seg_kv_lens || !p->seg_tables || p->seg_table_stride <= 0))
    return PB_ERR_INVALID_ARG;
  if (p->num_outer_groups > 0 && (!p->outer_row_offsets || !p->outer_prefix_lens)) return PB_ERR_INVALID_ARG;
  if (p->num_outer_groups > 0 && p->outer_table_stride > 0 && !p->outer_tables) return PB_ERR_INVALID_ARG;
  if (p->stats_mode < PB_STATS_NONE || p->stats_mode > PB_STATS_LOAD_SAVE) return PB_ERR_INVALID_ARG;
  if (p->dense_row_tile != 0 && p->dense_row_tile != 128 && p->dense_row_tile != 256) return PB_ERR_INVALID_ARG;
  if (p->stats_mode != PB_STATS_NONE && (!p->qk_max || !p->exp_sum)) return PB_ERR_INVALID_ARG;
  const int vec = 16 / elem_bytes(p->dtype);
  if (!aligned16(p->query) || !aligned16(p->key_cache) || !aligned16(p->value_cache)) return PB_ERR_INVALID_ARG;
  if (p->q_stride % vec || p->kv_block_stride % vec || p->kv_head_stride % vec) return PB_ERR_INVALID_ARG;
  if (p->q_stride < (int64_t)p->num_heads * p->head_size || p->out_stride < (int64_t)p->num_heads * p->head_size)
    return PB_ERR_INVALID_ARG;
  if (p->kv_head_stride < (int64_t)p->head_size * p->block_size) return PB_ERR_INVALID_ARG;
  if (p->num_blocks <= 0) return PB_ERR_INVALID_ARG;
  if ((p->key_new != nullptr) != (p->value_new != nullptr)) return PB_ERR_INVALID_ARG;
  if (p->key_new) {
    if (!p->slot_mapping || !aligned16(p->key_new) || !aligned16(p->value_new)) return PB_ERR_INVALID_ARG;
    if (p->key_new_stride % vec || p->value_new_stride % vec) return PB_ERR_INVALID_ARG;
    if (p->key_new_stride < (int64_t)p->num_kv_heads * p->head_size || p->value_new_stride < (int64_t)p->num_kv_heads * p->head_size)
      return PB_ERR_INVALID_ARG;
  }
  if (!p->workspace || !aligned16(p->workspace) || p->workspace_bytes < L->total) return PB_ERR_WORKSPACE;

  uint8_t* ws = static_cast<uint8_t*>(p->workspace);
  d->out = p->out; d->query = p->query; d->key_cache = p->key_cache; d->value_cache = p->value_cache;
  d->head_mapping = p->head_mapping;
  d->suffix_lens = p->suffix_table_stride > 0 ? p->suffix_lens : nullptr;
  d->suffix_tables = p->suffix_tables;
  d->group_row_offsets = p->group_row_offsets;
  d->group_prefix_lens = p->group_prefix_lens;
  d->group_tables = p->group_tables;
  d->seg_row_offsets = p->seg_row_offsets; d->seg_kv_lens = p->seg_kv_lens; d->seg_tables = p->seg_tables;
  d->num_segments = p->num_segments; d->seg_table_stride = p->seg_table_stride; d->cparts = L->cparts;
  d->outer_row_offsets = p->outer_row_offsets; d->outer_prefix_lens = p->outer_prefix_lens; d->outer_tables = p->outer_tables;
  d->num_outer_groups = p->num_outer_groups; d->outer_table_stride = p->outer_table_stride; d->oparts = L->oparts;
  d->qk_max = p->qk_max; d->exp_sum = p->exp_sum;
  d->hdr = reinterpret_cast<int32_t*>(ws);
  d->row_info = reinterpret_cast<RowInfo*>(ws + L->off_rowinfo);
  d->sq_items = reinterpret_cast<SqItem*>(ws + L->off_sq);
  d->dn_items = reinterpret_cast<DnItem*>(ws + L->off_dn);
  d->ml = reinterpret_cast<float2*>(ws + L->off_ml);
  d->acc = reinterpret_cast<float*>(ws + L->off_acc);
  d->scale_log2e = p->scale * kLog2e;
  d->num_rows = p->num_rows; d->num_heads = p->num_heads; d->num_kv_heads = p->num_kv_heads;
  d->num_groups = p->num_groups;
  d->suffix_table_stride = p->suffix_table_stride; d->group_table_stride = p->group_table_stride;
  d->parts = L->parts; d->pparts = L->pparts; d->sparts = L->sparts; d->cs = L->cs; d->cp = L->cp;
  d->cap_sq = L->cap_sq; d->cap_dn = L->cap_dn; d->dense_min_rows = L->dense_min_rows;
  d->stats_mode = p->stats_mode;
  // SMs given to the dense kernel while the suffix kernel runs beside it on the rest: the caller's
  // explicit value, else 0 = the planner decides from the exact amounts of dense and suffix work.
  // Read by the planner only: the split is part of the plan.
  d->num_sms = sm_count();
  d->dense_ctas = p->dense_ctas > 0 ? (p->dense_ctas < d->num_sms ? p->dense_ctas : d->num_sms) : 0;
  // Rows per dense item. Row-tile pairs pay when most of the dense work comes in tiles of 128 rows
  // (prefill, large groups); a decode batch with small groups keeps single row tiles, where the
  // rows of a tile are duplicated so that several threads share a row's exponentials.
  d->dense_row_tile = p->dense_row_tile > 0 ? p->dense_row_tile : 128;
  d->q_stride = p->q_stride; d->out_stride = p->out_stride;
  d->out_vec16 = (aligned16(p->out) && (p->out_stride * elem_bytes(p->dtype)) % 16 == 0) ? 1 : 0;
  d->acc_tma = 0;
  d->kv_block_stride = p->kv_block_stride; d->kv_head_stride = p->kv_head_stride;
  d->num_blocks = p->num_blocks;
  // new tokens: the planner reads the slots; the suffix kernel takes over the fill only for a pure
  // decode batch with identity head mapping (run_stages decides and sets key_new / value_new)
  d->slot_mapping = p->slot_mapping; d->slot_is_i64 = p->slot_is_i64;
  d->key_new = nullptr; d->value_new = nullptr;
  d->key_new_stride = p->key_new_stride; d->value_new_stride = p->value_new_stride;
  return PB_OK;
}

int fail_launch(cudaError_t e) {
  set_cuda_error(e);
  return PB_ERR_LAUNCH;
}

int run_plan(const pb_attn_params* p, const AttnDev& d, cudaStream_t s) {
  const bool dense_ok = dense_prefix_supported(p->dtype, p->head_size, p->block_size);
  cudaError_t e = launch_plan(d, p->block_size, dense_ok, s);
  return e == cudaSuccess ? PB_OK : fail_launch(e);
}

int run_stages(const pb_attn_params* p, const AttnDev& d_in, cudaStream_t s) {
  cudaError_t e;
  AttnDev d = d_in;
  const bool dense = (p->num_groups > 0 || p->num_segments > 0 || p->num_outer_groups > 0) &&
                     dense_prefix_supported(p->dtype, p->head_size, p->block_size);
  d.sq_waits_at_start = dense ? 0 : 1;
  if (p->key_new) {
    // The call performs the KV fill of its rows' new tokens. Pure decode batch: the suffix kernel
    // does it on the fly (the planner marked the items that carry a new token). Otherwise (prefill
    // requests read their own new tokens from the cache, or several query heads share a kv head):
    // the fill kernel first, as a caller of pb_reshape_and_cache would have run it.
    if (p->num_segments == 0 && !p->head_mapping) {
      d.key_new = p->key_new;
      d.value_new = p->value_new;
    } else {
      const int rc = pb_reshape_and_cache(p->key_new, p->value_new, const_cast<void*>(p->key_cache), const_cast<void*>(p->value_cache),
                                          p->slot_mapping, p->slot_is_i64, p->num_rows, p->num_kv_heads, p->head_size, p->block_size,
                                          p->key_new_stride, p->value_new_stride, p->kv_block_stride, p->kv_head_stride,
                                          p->num_blocks, p->dtype, s);
      if (rc != PB_OK) return rc;
    }
  }
  if (dense) {
    e = launch_dense_prefix(d, p->dtype, p->head_size, p->block_size, s);
    if (e != cudaSuccess) return fail_launch(e);
  }
  const cudaEvent_t ev0 = g_ev_begin, ev1 = g_ev_end;
  g_ev_begin = g_ev_end = nullptr;
  if (ev0) cudaEventRecord(ev0, s);
  e = launch_single_query(d, p->dtype, p->head_size, p->block_size, s);
  if (e != cudaSuccess) return fail_launch(e);
  if (ev1) cudaEventRecord(ev1, s);
  e = launch_merge(d, p->dtype, p->head_size, s);
  if (e != cudaSuccess) return fail_launch(e);
  return PB_OK;
}

int single_query_entry(void* out, const void* query, const void* key_cache, const void* value_cache,
                       const int32_t* head_mapping, float scale, const int32_t* block_tables,
                       const int32_t* context_lens, float* qk_maxs, float* exp_sums, int stats_mode,
                       int32_t block_size, int32_t num_seqs, int32_t num_heads, int32_t num_kv_heads,
                       int32_t head_size, int32_t max_num_blocks_per_seq, int64_t q_stride,
                       int64_t kv_block_stride, int64_t kv_head_stride, int64_t num_blocks, int32_t dtype,
                       void* workspace, size_t workspace_bytes, void* stream) {
  pb_attn_params p = {};
  p.out = out; p.query = query; p.key_cache = key_cache; p.value_cache = value_cache;
  p.head_mapping = head_mapping; p.scale = scale; p.dtype = dtype;
  p.num_rows = num_seqs; p.num_heads = num_heads; p.num_kv_heads = num_kv_heads;
  p.head_size = head_size; p.block_size = block_size; p.num_blocks = num_blocks;
  p.q_stride = q_stride; p.out_stride = (int64_t)num_heads * head_size;
  p.kv_block_stride = kv_block_stride; p.kv_head_stride = kv_head_stride;
  p.suffix_lens = context_lens; p.suffix_tables = block_tables;
  p.suffix_table_stride = max_num_blocks_per_seq;
  p.num_groups = 0;
  p.qk_max = qk_maxs; p.exp_sum = exp_sums; p.stats_mode = stats_mode;
  p.workspace = workspace; p.workspace_bytes = workspace_bytes;
  return pb_shared_prefix_attention(&p, stream);
}

}  // namespace
}  // namespace pb

extern "C" {

int pb_abi_version(void) { return 3; }

void pb_attn_set_timing_events(void* begin, void* end) {
  pb::g_ev_begin = static_cast<cudaEvent_t>(begin);
  pb::g_ev_end = static_cast<cudaEvent_t>(end);
}

const char* pb_last_cuda_error(void) { return pb::last_cuda_error(); }

size_t pb_attn_workspace_bytes(const pb_attn_params* p) {
  pb::WsLayout L;
  if (pb::compute_layout(p, &L) != PB_OK) return 0;
  return L.total;
}

int pb_attn_plan(const pb_attn_params* p, void* stream) {
  pb::WsLayout L;
  pb::AttnDev d;
  int rc = pb::validate_and_bind(p, &L, &d);
  if (rc != PB_OK || p->num_rows == 0) return rc;
  return pb::run_plan(p, d, static_cast<cudaStream_t>(stream));
}

int pb_shared_prefix_attention_planned(const pb_attn_params* p, void* stream) {
  pb::WsLayout L;
  pb::AttnDev d;
  int rc = pb::validate_and_bind(p, &L, &d);
  if (rc != PB_OK || p->num_rows == 0) return rc;
  return pb::run_stages(p, d, static_cast<cudaStream_t>(stream));
}

int pb_shared_prefix_attention(const pb_attn_params* p, void* stream) {
  pb::WsLayout L;
  pb::AttnDev d;
  int rc = pb::validate_and_bind(p, &L, &d);
  if (rc != PB_OK || p->num_rows == 0) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  rc = pb::run_plan(p, d, s);
  if (rc != PB_OK) return rc;
  return pb::run_stages(p, d, s);
}

int pb_attention_step_host(const pb_attn_params* p, const pb_host_step* io, void* stream) {
  if (!p || !io || !io->h_query || !io->h_out) return PB_ERR_INVALID_ARG;
  pb::WsLayout L;
  pb::AttnDev d;
  int rc = pb::validate_and_bind(p, &L, &d);
  if (rc != PB_OK) return rc;
  const int64_t row_elems = (int64_t)p->num_heads * p->head_size;
  if (p->q_stride != row_elems || p->out_stride != row_elems) return PB_ERR_INVALID_ARG;
  if (io->num_new_tokens < 0) return PB_ERR_INVALID_ARG;
  const bool fill = io->h_key_new && io->num_new_tokens > 0;
  if (fill && (!io->h_value_new || !io->h_slot_mapping || !io->d_key_new || !io->d_value_new || !io->d_slot_mapping))
    return PB_ERR_INVALID_ARG;
  if ((io->h_suffix_lens && !p->suffix_lens) || (io->h_suffix_tables && !p->suffix_tables)) return PB_ERR_INVALID_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t eb = pb::elem_bytes(p->dtype);
  const int64_t kv_elems = (int64_t)p->num_kv_heads * p->head_size;
  // Every transfer pays a fixed latency of several microseconds, so for a caller that lays its host
  // buffers out like the device staging area, inside one allocation on each side, transfers whose
  // ranges follow one another directly are merged.
  struct Xfer { char* dst; const char* src; size_t bytes; };
  auto upload = [&](Xfer* x, int n, cudaStream_t on) -> cudaError_t {
    for (int i = 1; i < n; ++i)  // insertion sort by host address
      for (int j = i; j > 0 && x[j].src < x[j - 1].src; --j) { Xfer t = x[j]; x[j] = x[j - 1]; x[j - 1] = t; }
    for (int i = 0; i < n;) {
      Xfer run = x[i++];
      while (io->merge_adjacent && i < n && x[i].src == run.src + run.bytes && x[i].dst == run.dst + run.bytes)
        run.bytes += x[i++].bytes;
      const cudaError_t err = cudaMemcpyAsync(run.dst, run.src, run.bytes, cudaMemcpyHostToDevice, on);
      if (err != cudaSuccess) return err;
    }
    return cudaSuccess;
  };
  auto add = [&](Xfer* x, int& n, const void* dst, const void* src, size_t bytes) {
    if (src && dst && bytes) x[n++] = Xfer{static_cast<char*>(const_cast<void*>(dst)), static_cast<const char*>(src), bytes};
  };
  Xfer x[6];
  int n = 0;
  if (p->num_rows > 0) {
    add(x, n, p->suffix_lens, io->h_suffix_lens, (size_t)p->num_rows * 4);
    add(x, n, p->suffix_tables, io->h_suffix_tables, (size_t)p->num_rows * p->suffix_table_stride * 4);
    add(x, n, p->query, io->h_query, (size_t)p->num_rows * row_elems * eb);
  }
  if (fill) {
    const size_t kv_bytes = (size_t)io->num_new_tokens * kv_elems * eb;
    add(x, n, io->d_key_new, io->h_key_new, kv_bytes);
    add(x, n, io->d_value_new, io->h_value_new, kv_bytes);
    add(x, n, io->d_slot_mapping, io->h_slot_mapping, (size_t)io->num_new_tokens * 8);
  }
  cudaError_t e = upload(x, n, s);
  if (e != cudaSuccess) return pb::fail_launch(e);
  // One new token per query row, in row order (every decode batch): the attention call performs the
  // fill itself (see pb_attn_params.slot_mapping); the lists must then be planned with the slots.
  pb_attn_params fused = *p;
  const bool fuse = fill && p->num_rows > 0 && io->num_new_tokens == p->num_rows && io->replan;
  if (fuse) {
    fused.slot_mapping = io->d_slot_mapping; fused.slot_is_i64 = 1;
    fused.key_new = io->d_key_new; fused.value_new = io->d_value_new;
    fused.key_new_stride = fused.value_new_stride = kv_elems;
    if ((rc = pb::validate_and_bind(&fused, &L, &d)) != PB_OK) return rc;
    p = &fused;
  }
  if (fill && !fuse) {
    rc = pb_reshape_and_cache(io->d_key_new, io->d_value_new, const_cast<void*>(p->key_cache), const_cast<void*>(p->value_cache),
                              io->d_slot_mapping, 1, io->num_new_tokens, p->num_kv_heads, p->head_size, p->block_size,
                              kv_elems, kv_elems, p->kv_block_stride, p->kv_head_stride, p->num_blocks, p->dtype, stream);
    if (rc != PB_OK) return rc;
  }
  if (p->num_rows > 0) {
    if (io->replan && (rc = pb::run_plan(p, d, s)) != PB_OK) return rc;
    bool direct = false;
    if (io->direct_out) {
      cudaPointerAttributes attr;
      if (cudaPointerGetAttributes(&attr, io->h_out) == cudaSuccess) {
        if (attr.type == cudaMemoryTypeHost && attr.devicePointer) {
          d.out = attr.devicePointer;  // the merge kernel's stores go over the bus themselves
          direct = true;
        }
      } else {
        (void)cudaGetLastError();  // not a pointer the runtime knows: fall back to the download
      }
    }
    if ((rc = pb::run_stages(p, d, s)) != PB_OK) return rc;
    if (!direct) {
      e = cudaMemcpyAsync(io->h_out, p->out, (size_t)p->num_rows * row_elems * eb, cudaMemcpyDeviceToHost, s);
      if (e != cudaSuccess) return pb::fail_launch(e);
    }
  }
  if (io->synchronize && (e = cudaStreamSynchronize(s)) != cudaSuccess) return pb::fail_launch(e);
  return PB_OK;
}

int pb_read_status(const void* workspace, void* stream, int32_t* detail) {
  if (!workspace) return PB_ERR_INVALID_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) { pb::set_cuda_error(e); return PB_ERR_LAUNCH; }
  int32_t word = 0;
  e = cudaMemcpy(&word, workspace, sizeof(word), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) { pb::set_cuda_error(e); return PB_ERR_LAUNCH; }
  if (detail) *detail = word;
  return word == pb::kStatusOk ? PB_OK : PB_ERR_DEVICE;
}

size_t pb_single_query_workspace_bytes(int32_t num_seqs, int32_t num_heads, int32_t head_size,
                                       int32_t block_size, int32_t max_num_blocks_per_seq) {
  pb_attn_params p = {};
  p.num_rows = num_seqs; p.num_heads = num_heads; p.num_kv_heads = num_heads;
  p.head_size = head_size; p.block_size = block_size;
  p.suffix_table_stride = max_num_blocks_per_seq;
  p.dtype = PB_F16;
  return pb_attn_workspace_bytes(&p);
}

int pb_single_query_cached_kv_attention(
    void* out, const void* query, const void* key_cache, const void* value_cache,
    const int32_t* head_mapping, float scale, const int32_t* block_tables, const int32_t* context_lens,
    int32_t block_size, int32_t max_context_len, int32_t num_seqs, int32_t num_heads,
    int32_t num_kv_heads, int32_t head_size, int32_t max_num_blocks_per_seq, int64_t q_stride,
    int64_t kv_block_stride, int64_t kv_head_stride, int64_t num_blocks, int32_t dtype, void* workspace,
    size_t workspace_bytes, void* stream) {
  (void)max_context_len;
  return pb::single_query_entry(out, query, key_cache, value_cache, head_mapping, scale, block_tables,
                                context_lens, nullptr, nullptr, PB_STATS_NONE, block_size, num_seqs,
                                num_heads, num_kv_heads, head_size, max_num_blocks_per_seq, q_stride,
                                kv_block_stride, kv_head_stride, num_blocks, dtype, workspace,
                                workspace_bytes, stream);
}

int pb_single_query_cached_kv_prev_attention(
    void* out, const void* query, const void* key_cache, const void* value_cache,
    const int32_t* head_mapping, float scale, const int32_t* block_tables, const int32_t* context_lens,
    float* qk_maxs, float* exp_sums, int32_t block_size, int32_t max_context_len, int32_t num_seqs,
    int32_t num_heads, int32_t num_kv_heads, int32_t head_size, int32_t max_num_blocks_per_seq,
    int64_t q_stride, int64_t kv_block_stride, int64_t kv_head_stride, int64_t num_blocks, int32_t dtype,
    void* workspace, size_t workspace_bytes, void* stream) {
  (void)max_context_len;
  return pb::single_query_entry(out, query, key_cache, value_cache, head_mapping, scale, block_tables,
                                context_lens, qk_maxs, exp_sums, PB_STATS_SAVE, block_size, num_seqs,
                                num_heads, num_kv_heads, head_size, max_num_blocks_per_seq, q_stride,
                                kv_block_stride, kv_head_stride, num_blocks, dtype, workspace,
                                workspace_bytes, stream);
}

int pb_single_query_cached_kv_post_attention(
    void* out, const void* query, const void* key_cache, const void* value_cache,
    const int32_t* head_mapping, float scale, const int32_t* block_tables, const int32_t* context_lens,
    float* prev_qk_maxs, float* prev_exp_sums, int32_t block_size, int32_t max_context_len,
    int32_t num_seqs, int32_t num_heads, int32_t num_kv_heads, int32_t head_size,
    int32_t max_num_blocks_per_seq, int64_t q_stride, int64_t kv_block_stride, int64_t kv_head_stride,
    int64_t num_blocks, int32_t dtype, void* workspace, size_t workspace_bytes, void* stream) {
  (void)max_context_len;
  return pb::single_query_entry(out, query, key_cache, value_cache, head_mapping, scale, block_tables,
                                context_lens, prev_qk_maxs, prev_exp_sums, PB_STATS_LOAD, block_size,
                                num_seqs, num_heads, num_kv_heads, head_size, max_num_blocks_per_seq,
                                q_stride, kv_block_stride, kv_head_stride, num_blocks, dtype, workspace,
                                workspace_bytes, stream);
}

}  // extern "C"
