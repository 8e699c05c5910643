// Log-sum-exp merge of the partial results of one (row, head): prefix chunks, suffix chunks and,
// in LOAD mode, the caller's earlier partial held in out / qk_max / exp_sum.
//
// Algebra (base-2 domain): partial i carries (acc_i, m_i, l_i) with acc_i un-normalised;
// M = max m_i, w_i = 2^(m_i - M), out = sum w_i acc_i / sum w_i l_i. Associative, so the order
// of the partials does not matter.
//
// Reference counterparts: _reduce_kernel (parrot/engine/builtin/kernels/shared_flash_decoding.py:137-199)
// and the in-place merge tail of single_query_cached_kv_post_attention_kernel
// (csrc/attention/attention_post_kernels.cu:321-340).
#include "common.cuh"

namespace pb {
namespace {

constexpr int kMergeWarps = 4;
constexpr int kPairLanes = 16;                 // lanes that share one (row, head)
constexpr int kPairsPerWarp = 32 / kPairLanes;  // two (row, head) pairs per warp: twice the loads in flight

template <typename T, int D>
__global__ void __launch_bounds__(kMergeWarps * 32) merge_kernel(const AttnDev d) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % kPairLanes;  // position inside the pair's lane group
  const long long idx = ((long long)blockIdx.x * kMergeWarps + warp) * kPairsPerWarp + lane / kPairLanes;
  const int H = d.num_heads;
  // The planner's output (row_info, dense items, header) is older than the attention kernels of
  // this call, so it is read while they still run; only then wait for their partials.
  const bool active = idx < (long long)d.num_rows * H;
  const int row = active ? (int)(idx / H) : 0, head = active ? (int)(idx - (long long)row * H) : 0;
  const RowInfo info = d.row_info[row];
  // partials of the row: [prefix][causal segment][suffix]; a dense stage leaves one partial per
  // CTA that touched the (row tile, head), the single-query kernel one per chunk
  const long long total = d.hdr[kHdrDnTiles];
  const int dctas = dense_ctas_of(d);
  auto dense_parts = [&](int dn) {
    const DnItem it = d.dn_items[dn];
    const long long g0 = (long long)it.tile_base + (long long)head * it.nt;
    return dense_cta_of_tile(g0 + it.nt - 1, total, dctas) - dense_cta_of_tile(g0, total, dctas) + 1;
  };
  const int np = (info.dn >= 0) ? dense_parts(info.dn) : info.np_sq;
  const int nc = (info.seg_dn >= 0) ? dense_parts(info.seg_dn) : info.nc_sq;
  // rows the dense kernel finished by itself (its only partial, held whole by one CTA): nothing to do
  const int no = (info.odn >= 0) ? dense_parts(info.odn) : info.onp_sq;  // outer-prefix partials
  const bool direct = active && info.dn >= 0 && np == 1 && nc == 0 && info.nsc == 0 && no == 0 &&
                      dense_direct_ok(d, d.dn_items[info.dn]);
  pdl_wait();  // every partial of the prefix and suffix stages is complete and visible
  if (blockIdx.x == 0 && threadIdx.x == 0) d.hdr[kHdrSqCounter] = 0;  // ready for the next layer call
  // A call whose kernels recorded a fault (a wait that ran out, an index outside the cache, a list
  // that did not fit) has results that cannot be trusted: every output row becomes NaN, so that the
  // fault cannot pass unnoticed into the sampler even if nobody reads the status word.
  const bool poison = __ldcg(&d.hdr[kHdrStatus]) != kStatusOk;
  const int n = (active && !direct) ? np + nc + info.nsc + no : 0;
  int n_warp = n;  // the two pairs of a warp walk their partials in lockstep
#pragma unroll
  for (int o = kPairLanes; o < 32; o <<= 1) n_warp = max(n_warp, __shfl_xor_sync(0xffffffffu, n_warp, o));
  constexpr int kVecs = D / 4;                                     // float4 per partial row
  constexpr int kPer = (kVecs + kPairLanes - 1) / kPairLanes;      // float4 per lane
  auto part_of = [&](int j) {  // partial ranges of a row: [prefix][segment][suffix][outer prefix]
    if (j < np) return j;
    if (j < np + nc) return d.pparts + (j - np);
    if (j < np + nc + info.nsc) return d.pparts + d.cparts + (j - np - nc);
    return d.pparts + d.cparts + d.sparts + (j - np - nc - info.nsc);
  };

  const bool load_prev = (d.stats_mode & PB_STATS_LOAD) != 0;
  float m_prev = -INFINITY, l_prev = 0.f;
  if (load_prev && active) {
    m_prev = d.qk_max[idx];
    l_prev = d.exp_sum[idx];
    if (!(l_prev > 0.f)) { l_prev = 0.f; m_prev = -INFINITY; }
  }

  // pass 1: global maximum (lane j of the pair reads the statistics of partial j; with at most
  // kPairLanes partials, the usual case, they stay in registers and are not read again)
  float M = m_prev;
  float2 ml0 = make_float2(-INFINITY, 0.f);
  if (sub < n) ml0 = d.ml[partial_slot(d, row, part_of(sub), head)];
  M = fmaxf(M, ml0.x);
  for (int j = sub + kPairLanes; j < n; j += kPairLanes) M = fmaxf(M, d.ml[partial_slot(d, row, part_of(j), head)].x);
#pragma unroll
  for (int o = kPairLanes / 2; o >= 1; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  // Everything this kernel reads of the planner's output has arrived (the statistics just reduced
  // were addressed with it), so the next kernel in the stream may become resident: an attention
  // kernel or a KV fill waits for this grid's completion before it touches anything, and a planner
  // only overwrites the lists read above and completes after this grid.
  pdl_trigger();

  float4 o4[kPer];
#pragma unroll
  for (int k = 0; k < kPer; ++k) o4[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  float L = 0.f;
  const bool any = M > -INFINITY;

  for (int jb = 0; jb < n_warp; jb += kPairLanes) {
    // weights of up to kPairLanes partials at once, then their accumulators with independent loads
    float w_lane = 0.f;
    if (any && jb + sub < n) {
      const float2 ml = (jb == 0) ? ml0 : d.ml[partial_slot(d, row, part_of(jb + sub), head)];
      w_lane = fast_exp2(ml.x - M);
      L = fmaf(ml.y, w_lane, L);
    }
    const int cnt = any ? min(kPairLanes, n - jb) : 0;          // this pair's partials in the round
    const int cnt_warp = min(kPairLanes, n_warp - jb);
    for (int j0 = 0; j0 < cnt_warp; j0 += 4) {
      // four partials per round: all their loads are issued before the first is used
      float4 a[4][kPer];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const bool live = j0 + u < cnt;
        const float4* ap = reinterpret_cast<const float4*>(
            d.acc + partial_slot(d, row, part_of(jb + (live ? j0 + u : 0)), head) * D);
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
          const int v = sub + kPairLanes * k;
          a[u][k] = (live && v < kVecs) ? __ldcs(ap + v) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float w = __shfl_sync(0xffffffffu, w_lane, (j0 + u) % kPairLanes, kPairLanes);
        if (j0 + u >= cnt) w = 0.f;
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
          o4[k].x = fmaf(a[u][k].x, w, o4[k].x); o4[k].y = fmaf(a[u][k].y, w, o4[k].y);
          o4[k].z = fmaf(a[u][k].z, w, o4[k].z); o4[k].w = fmaf(a[u][k].w, w, o4[k].w);
        }
      }
    }
  }
#pragma unroll
  for (int o = kPairLanes / 2; o >= 1; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
  if (!active || (direct && !poison)) return;
  if (l_prev > 0.f) {
    const float w = fast_exp2(m_prev - M) * l_prev;
    L += w;
    const T* op = reinterpret_cast<const T*>(d.out) + (size_t)row * d.out_stride + (size_t)head * D;
#pragma unroll
    for (int k = 0; k < kPer; ++k) {
      const int v = sub + kPairLanes * k;
      if (v < kVecs) {
        o4[k].x = fmaf(to_float<T>(op[v * 4 + 0]), w, o4[k].x);
        o4[k].y = fmaf(to_float<T>(op[v * 4 + 1]), w, o4[k].y);
        o4[k].z = fmaf(to_float<T>(op[v * 4 + 2]), w, o4[k].z);
        o4[k].w = fmaf(to_float<T>(op[v * 4 + 3]), w, o4[k].w);
      }
    }
  }
  const float inv = poison ? __int_as_float(0x7fc00000) : (L > 0.f) ? 1.f / L : 0.f;
  T* op = reinterpret_cast<T*>(d.out) + (size_t)row * d.out_stride + (size_t)head * D;
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int v = sub + kPairLanes * k;
    if (v < kVecs) {
      op[v * 4 + 0] = from_float<T>(o4[k].x * inv);
      op[v * 4 + 1] = from_float<T>(o4[k].y * inv);
      op[v * 4 + 2] = from_float<T>(o4[k].z * inv);
      op[v * 4 + 3] = from_float<T>(o4[k].w * inv);
    }
  }
  if ((d.stats_mode & PB_STATS_SAVE) && sub == 0) {
    d.qk_max[idx] = M;
    d.exp_sum[idx] = L;
  }
}

template <typename T>
cudaError_t launch_merge_t(const AttnDev& d, int head_size, cudaStream_t s) {
  const long long n = (long long)d.num_rows * d.num_heads;
  if (n == 0) return cudaSuccess;
  const long long per_cta = (long long)kMergeWarps * kPairsPerWarp;
  const unsigned grid = (unsigned)((n + per_cta - 1) / per_cta);
  switch (head_size) {
    case 64: return launch_kernel(merge_kernel<T, 64>, grid, kMergeWarps * 32, 0, s, true, d);
    case 80: return launch_kernel(merge_kernel<T, 80>, grid, kMergeWarps * 32, 0, s, true, d);
    case 96: return launch_kernel(merge_kernel<T, 96>, grid, kMergeWarps * 32, 0, s, true, d);
    case 112: return launch_kernel(merge_kernel<T, 112>, grid, kMergeWarps * 32, 0, s, true, d);
    case 128: return launch_kernel(merge_kernel<T, 128>, grid, kMergeWarps * 32, 0, s, true, d);
    case 256: return launch_kernel(merge_kernel<T, 256>, grid, kMergeWarps * 32, 0, s, true, d);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

cudaError_t launch_merge(const AttnDev& d, int dtype, int head_size, cudaStream_t s) {
  if (dtype == PB_F16) return launch_merge_t<__half>(d, head_size, s);
  if (dtype == PB_BF16) return launch_merge_t<__nv_bfloat16>(d, head_size, s);
  if (dtype == PB_F32) return launch_merge_t<float>(d, head_size, s);
  return cudaErrorInvalidValue;
}

}  // namespace pb
