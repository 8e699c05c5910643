// Work-list builder: turns the device-resident lengths of one iteration into the item lists the
// attention kernels walk. One CTA; the lists depend on lengths only, so one plan serves every
// layer of the iteration.
//
// Reference counterpart: the per-iteration metadata of
// xFormersFill_SharedPromptsGenerate.init_iteration_state (parrot/engine/builtin/attn_func.py:461-599)
// stops at block tables and lengths; the split-KV decomposition there is implicit in the Triton
// grid (parrot/engine/builtin/kernels/shared_flash_decoding.py:240-243).
#include "common.cuh"

namespace pb {
namespace {

constexpr int kPlanThreads = 1024;

// Exclusive scan of one int per thread over the CTA; returns the exclusive prefix, sets total.
__device__ int block_exclusive_scan(int v, int* warp_sums, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  __syncthreads();  // protect warp_sums from the previous use
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = (lane < (kPlanThreads >> 5)) ? warp_sums[lane] : 0;
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += n;
    }
    warp_sums[lane] = wi - w;       // exclusive per warp
    if (lane == 31) warp_sums[32] = wi;  // total
  }
  __syncthreads();
  total = warp_sums[32];
  return warp_sums[warp] + incl - v;
}

// Short chunks carry their block ids inside the item; longer ones point into their table.
__device__ __forceinline__ SqItem make_sq_item(int row, const int32_t* table, int tbl_off, int is_prefix, int nblk,
                                               int ntok, int part) {
  SqItem it;
  it.row = row;
  it.ntok = ntok;
  it.part = part;
  const bool embed = nblk <= kSqEmbedMax;
  it.meta = nblk | (is_prefix << 16) | ((embed ? 1 : 0) << 17);
#pragma unroll
  for (int j = 0; j < kSqEmbedMax; ++j) it.bid[j] = (embed && j < nblk) ? table[tbl_off + j] : 0;
  if (!embed) it.bid[0] = tbl_off;
  return it;
}

struct GroupPlan {
  int n_rows, plen, nblk, npc, dense, n_rt, nt;
};

__device__ __forceinline__ GroupPlan group_plan(const AttnDev& d, int g, int B, bool dense_ok) {
  GroupPlan p;
  const int r0 = d.group_row_offsets[g], r1 = d.group_row_offsets[g + 1];
  p.n_rows = max(r1 - r0, 0);
  p.plen = max(d.group_prefix_lens[g], 0);
  p.nblk = (p.plen + B - 1) / B;
  if (p.nblk > d.group_table_stride) {  // length claims more blocks than the table holds
    p.nblk = d.group_table_stride;
    p.plen = p.nblk * B;
    atomicMax(&d.hdr[kHdrStatus], kStatusBadIndex);
  }
  p.npc = (p.nblk + d.cp - 1) / d.cp;
  if (p.n_rows == 0) p.npc = 0;
  p.dense = (dense_ok && p.npc > 0 && p.n_rows >= d.dense_min_rows) ? 1 : 0;
  p.n_rt = (p.n_rows + 127) / 128;
  p.nt = (p.nblk + kDenseTileBlocks - 1) / kDenseTileBlocks;
  return p;
}

__global__ void __launch_bounds__(kPlanThreads, 1) plan_kernel(const AttnDev d, const int B, const bool dense_ok) {
  __shared__ int warp_sums[33];
  const int tid = threadIdx.x;
  const int S = d.num_rows, G = d.num_groups;

  if (tid == 0) { d.hdr[kHdrStatus] = kStatusOk; d.hdr[kHdrSqCounter] = 0; }
  __syncthreads();

  // ---- groups: dense items and unshared ("single-query") prefix items ----
  const int gper = (G + kPlanThreads - 1) / kPlanThreads;
  const int g_lo = min(tid * gper, G), g_hi = min(g_lo + gper, G);
  int my_dn = 0, my_sqp = 0, my_tiles = 0;
  for (int g = g_lo; g < g_hi; ++g) {
    const GroupPlan p = group_plan(d, g, B, dense_ok);
    if (p.dense) { my_dn += p.n_rt; my_tiles += p.n_rt * p.nt; }
    else my_sqp += p.npc * p.n_rows;
  }
  int total_dn, total_sqp, total_tiles;
  int dn_base = block_exclusive_scan(my_dn, warp_sums, total_dn);
  int sqp_base = block_exclusive_scan(my_sqp, warp_sums, total_sqp);
  int tile_base = block_exclusive_scan(my_tiles, warp_sums, total_tiles);

  // ---- rows: suffix items ----
  const int rper = (S + kPlanThreads - 1) / kPlanThreads;
  const int r_lo = min(tid * rper, S), r_hi = min(r_lo + rper, S);
  int my_sqs = 0;
  for (int r = r_lo; r < r_hi; ++r) {
    int len = d.suffix_lens ? max(d.suffix_lens[r], 0) : 0;
    int nblk = (len + B - 1) / B;
    if (nblk > d.suffix_table_stride) nblk = d.suffix_table_stride;
    my_sqs += (nblk + d.cs - 1) / d.cs;
  }
  int total_sqs;
  int sqs_base = block_exclusive_scan(my_sqs, warp_sums, total_sqs);

  const bool overflow = (total_dn > d.cap_dn) || (total_sqp + total_sqs > d.cap_sq);
  if (tid == 0) {
    d.hdr[kHdrNumSq] = overflow ? 0 : total_sqp + total_sqs;
    d.hdr[kHdrNumDn] = overflow ? 0 : total_dn;
    d.hdr[kHdrDnTiles] = overflow ? 0 : total_tiles * d.num_heads;
    if (overflow) atomicMax(&d.hdr[kHdrStatus], kStatusListOverflow);
  }
  if (overflow) return;

  // ---- emit group items, fill row_info for grouped rows ----
  for (int g = g_lo; g < g_hi; ++g) {
    const GroupPlan p = group_plan(d, g, B, dense_ok);
    const int r0 = d.group_row_offsets[g];
    for (int i = 0; i < p.n_rows; ++i) {
      const int r = r0 + i;
      if (r >= 0 && r < S) d.row_info[r] = make_int4(g, p.dense ? 0 : p.npc, 0, p.dense ? dn_base + i / 128 : -1);
    }
    if (p.npc == 0) continue;
    if (p.dense) {
      for (int rt = 0; rt < p.n_rt; ++rt) {
        DnItem it;
        it.row0 = r0 + rt * 128;
        it.nrows = min(128, p.n_rows - rt * 128);
        it.tbl_off = g * d.group_table_stride;
        it.nblk = p.nblk;
        it.ntok = p.plen;
        it.nt = p.nt;
        it.tile_base = tile_base * d.num_heads;
        it.pad0 = 0;
        tile_base += p.nt;
        d.dn_items[dn_base++] = it;
      }
    } else {
      for (int i = 0; i < p.n_rows; ++i)
        for (int c = 0; c < p.npc; ++c) {
          const int nb = min(d.cp, p.nblk - c * d.cp);
          d.sq_items[sqp_base++] = make_sq_item(r0 + i, d.group_tables, g * d.group_table_stride + c * d.cp, 1, nb,
                                                min(p.plen - c * d.cp * B, nb * B), c);
        }
    }
  }
  __syncthreads();  // row_info group fields are complete before the row pass reads them

  // ---- emit suffix items, finish row_info ----
  int w = total_sqp + sqs_base;
  const int rows_grouped_lo = G > 0 ? d.group_row_offsets[0] : S;
  const int rows_grouped_hi = G > 0 ? d.group_row_offsets[G] : S;
  for (int r = r_lo; r < r_hi; ++r) {
    int len = d.suffix_lens ? max(d.suffix_lens[r], 0) : 0;
    int nblk = (len + B - 1) / B;
    if (nblk > d.suffix_table_stride) {
      nblk = d.suffix_table_stride;
      len = nblk * B;
      atomicMax(&d.hdr[kHdrStatus], kStatusBadIndex);
    }
    const int nsc = (nblk + d.cs - 1) / d.cs;
    int4 info = make_int4(-1, 0, 0, -1);
    if (r >= rows_grouped_lo && r < rows_grouped_hi) info = d.row_info[r];
    info.z = nsc;
    d.row_info[r] = info;
    for (int c = 0; c < nsc; ++c) {
      const int nb = min(d.cs, nblk - c * d.cs);
      d.sq_items[w++] = make_sq_item(r, d.suffix_tables, r * d.suffix_table_stride + c * d.cs, 0, nb,
                                     min(len - c * d.cs * B, nb * B), d.pparts + c);
    }
  }
}

}  // namespace

cudaError_t launch_plan(const AttnDev& d, int block_size, bool dense_supported, cudaStream_t s) {
  plan_kernel<<<1, kPlanThreads, 0, s>>>(d, block_size, dense_supported);
  return cudaGetLastError();
}

}  // namespace pb
