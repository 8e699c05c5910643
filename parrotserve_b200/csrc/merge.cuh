// Log-sum-exp merge of all partial results of one (row, head), done by ONE WARP: prefix parts,
// causal-segment parts, suffix chunks, outer-prefix parts and, in LOAD mode, the caller's earlier
// partial held in out / qk_max / exp_sum.
//
// There is no merge kernel. Every partial written to the workspace is followed by a decrement of
// the (row, head)'s `remain` counter; the writer that brings it to zero is the last to arrive: if
// it is a warp of the single-query kernel it merges at once (the partials are still in L2), if it
// is a thread of the dense kernel it appends the pair to the todo list, which the single-query
// kernel's CTAs work off after the dense grid has completed. Nobody waits for anybody.
//
// Algebra (base-2 domain): partial i carries (acc_i, m_i, l_i) with acc_i un-normalised;
// M = max m_i, w_i = 2^(m_i - M), out = sum w_i acc_i / sum w_i l_i. Associative, so the order
// of the partials does not matter.
//
// Reference counterparts: _reduce_kernel (parrot/engine/builtin/kernels/shared_flash_decoding.py:137-199)
// and the in-place merge tail of single_query_cached_kv_post_attention_kernel
// (csrc/attention/attention_post_kernels.cu:321-340).
#pragma once

#include "common.cuh"

namespace pb {

// Partials the attention kernels leave for (row, head), by range: prefix, causal segment, suffix,
// outer prefix. A dense stage leaves one partial per CTA that touched the (row tile, head) (the
// planner tabulated that in dn_parts), the single-query kernel one per chunk.
struct PartCounts {
  int np, nc, ns, no;
  __device__ __forceinline__ int total() const { return np + nc + ns + no; }
};
__device__ __forceinline__ PartCounts part_counts(const AttnDev& d, const RowInfo& info, int head) {
  PartCounts c;
  const int H = d.num_heads;
  c.np = (info.dn >= 0) ? d.dn_parts[(size_t)info.dn * H + head] : info.np_sq;
  c.nc = (info.seg_dn >= 0) ? d.dn_parts[(size_t)info.seg_dn * H + head] : info.nc_sq;
  c.ns = info.nsc;
  c.no = (info.odn >= 0) ? d.dn_parts[(size_t)info.odn * H + head] : info.onp_sq;
  return c;
}
// Whether the dense kernel finishes this (row, head) by itself (its only partial, held whole by one
// CTA, written as the normalised output): such pairs are never counted and never merged.
__device__ __forceinline__ bool row_is_direct(const AttnDev& d, const RowInfo& info, const PartCounts& c) {
  return info.dn >= 0 && c.np == 1 && c.nc == 0 && c.ns == 0 && c.no == 0 && dense_direct_ok(d, d.dn_items[info.dn]);
}

// Four consecutive output elements; one vector store when the output rows allow it.
template <typename T>
__device__ __forceinline__ void store_out4(T* p, float x, float y, float z, float w, bool vec) {
  if (vec) {
    if constexpr (sizeof(T) == 4) {
      *reinterpret_cast<float4*>(p) = make_float4(x, y, z, w);
    } else {
      const T a = from_float<T>(x), b = from_float<T>(y), c = from_float<T>(z), e = from_float<T>(w);
      uint2 u;
      u.x = (uint32_t)(*reinterpret_cast<const uint16_t*>(&a)) | ((uint32_t)(*reinterpret_cast<const uint16_t*>(&b)) << 16);
      u.y = (uint32_t)(*reinterpret_cast<const uint16_t*>(&c)) | ((uint32_t)(*reinterpret_cast<const uint16_t*>(&e)) << 16);
      *reinterpret_cast<uint2*>(p) = u;
    }
  } else {
    p[0] = from_float<T>(x); p[1] = from_float<T>(y); p[2] = from_float<T>(z); p[3] = from_float<T>(w);
  }
}

// Merges up to 32 / LP (row, head) pairs at once, LP lanes each (LP = 8: four pairs per warp, so a
// warp that works off a list keeps four times the loads in flight; a warp with a single pair to
// merge passes -1 for the others). Called by all 32 lanes; `pair` = row * heads + head of the
// calling lane's group, or -1. The pairs' last partials must already be visible.
template <typename T, int D, int LP = 8>
__device__ __forceinline__ void merge_pairs(const AttnDev& d, long long pair) {
  static_assert(LP == 8 || LP == 16 || LP == 32, "lanes per pair");
  const int lane = threadIdx.x & 31;
  const int sub = lane % LP;
  const int H = d.num_heads;
  const bool active = pair >= 0;
  const int row = active ? (int)(pair / H) : 0, head = active ? (int)(pair - (long long)row * H) : 0;
  const size_t idx = (size_t)row * H + head;
  const RowInfo info = d.row_info[row];
  const PartCounts pc = part_counts(d, info, head);
  const int n = active ? pc.total() : 0;
  int n_warp = n;  // the pairs of a warp walk their partials in lockstep
#pragma unroll
  for (int o = LP; o < 32; o <<= 1) n_warp = max(n_warp, __shfl_xor_sync(0xffffffffu, n_warp, o));
  auto part_of = [&](int j) {
    if (j < pc.np) return j;
    if (j < pc.np + pc.nc) return d.pparts + (j - pc.np);
    if (j < pc.np + pc.nc + pc.ns) return d.pparts + d.cparts + (j - pc.np - pc.nc);
    return d.pparts + d.cparts + d.sparts + (j - pc.np - pc.nc - pc.ns);
  };
  const bool load_prev = (d.stats_mode & PB_STATS_LOAD) != 0;
  float m_prev = -INFINITY, l_prev = 0.f;
  if (load_prev && active) {
    m_prev = d.qk_max[idx];
    l_prev = d.exp_sum[idx];
    if (!(l_prev > 0.f)) { l_prev = 0.f; m_prev = -INFINITY; }
  }
  // pass 1: statistics (lane j of the group holds those of partials j, j + LP, ...; the first LP stay in registers)
  float M = m_prev;
  float2 ml0 = make_float2(-INFINITY, 0.f);
  if (sub < n) ml0 = __ldcg(&d.ml[partial_slot(d, row, part_of(sub), head)]);
  M = fmaxf(M, ml0.x);
  for (int j = sub + LP; j < n; j += LP) M = fmaxf(M, __ldcg(&d.ml[partial_slot(d, row, part_of(j), head)]).x);
#pragma unroll
  for (int o = LP / 2; o >= 1; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  const bool any = M > -INFINITY;

  constexpr int kVecs = D / 4;                        // float4 per partial row
  constexpr int kPer = (kVecs + LP - 1) / LP;         // float4 per lane
  constexpr int kRound = kPer >= 8 ? 1 : (kPer >= 4 ? 2 : 4);  // partials whose loads are in flight together
  float4 o4[kPer];
#pragma unroll
  for (int k = 0; k < kPer; ++k) o4[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  float L = 0.f;
  for (int jb = 0; jb < n_warp; jb += LP) {
    float w_lane = 0.f;
    if (any && jb + sub < n) {
      const float2 ml = (jb == 0) ? ml0 : __ldcg(&d.ml[partial_slot(d, row, part_of(jb + sub), head)]);
      w_lane = fast_exp2(ml.x - M);
      L = fmaf(ml.y, w_lane, L);
    }
    const int cnt = any ? max(0, min(LP, n - jb)) : 0;  // this pair's partials in the round
    const int cnt_warp = min(LP, n_warp - jb);
    for (int j0 = 0; j0 < cnt_warp; j0 += kRound) {
      float4 a[kRound][kPer];
#pragma unroll
      for (int u = 0; u < kRound; ++u) {
        const bool live = j0 + u < cnt;
        const float4* ap = reinterpret_cast<const float4*>(d.acc + partial_slot(d, row, part_of(jb + (live ? j0 + u : 0)), head) * D);
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
          const int v = sub + LP * k;
          a[u][k] = (live && v < kVecs) ? __ldcg(ap + v) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < kRound; ++u) {
        float w = __shfl_sync(0xffffffffu, w_lane, (j0 + u) % LP, LP);
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
  for (int o = LP / 2; o >= 1; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
  if (!active) return;
  T* op = reinterpret_cast<T*>(d.out) + (size_t)row * d.out_stride + (size_t)head * D;
  if (l_prev > 0.f) {
    const float w = fast_exp2(m_prev - M) * l_prev;
    L += w;
#pragma unroll
    for (int k = 0; k < kPer; ++k) {
      const int v = sub + LP * k;
      if (v < kVecs) {
        o4[k].x = fmaf(to_float<T>(op[v * 4 + 0]), w, o4[k].x);
        o4[k].y = fmaf(to_float<T>(op[v * 4 + 1]), w, o4[k].y);
        o4[k].z = fmaf(to_float<T>(op[v * 4 + 2]), w, o4[k].z);
        o4[k].w = fmaf(to_float<T>(op[v * 4 + 3]), w, o4[k].w);
      }
    }
  }
  const float inv = (L > 0.f) ? 1.f / L : 0.f;
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int v = sub + LP * k;
    if (v < kVecs) store_out4<T>(op + v * 4, o4[k].x * inv, o4[k].y * inv, o4[k].z * inv, o4[k].w * inv, d.out_vec16 != 0);
  }
  if (sub == 0) {
    if (d.stats_mode & PB_STATS_SAVE) {
      d.qk_max[idx] = M;
      d.exp_sum[idx] = L;
    }
    d.remain[idx] = n;  // ready for the next layer call
  }
}

}  // namespace pb
