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
constexpr double kDenseTileWeight = 3.5;  // SM time of a dense kv tile relative to streaming it once

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
// table_kind: 0 suffix_tables, 1 group_tables, 2 seg_tables, 3 outer_tables.
__device__ __forceinline__ SqItem make_sq_item(int row, const int32_t* table, int tbl_off, int table_kind, int nblk,
                                               int ntok, int part) {
  SqItem it;
  it.row = row;
  it.ntok = ntok;
  it.part = part;
  const bool embed = nblk <= kSqEmbedMax;
  it.meta = nblk | (table_kind << 18) | ((embed ? 1 : 0) << 17);
#pragma unroll
  for (int j = 0; j < kSqEmbedMax; ++j) it.bid[j] = (embed && j < nblk) ? table[tbl_off + j] : 0;
  if (!embed) it.bid[0] = tbl_off;
  return it;
}

struct GroupPlan {
  int r0, n_rows, plen, nblk, npc, dense, n_rt, nt;
};

__device__ __forceinline__ GroupPlan plan_of(const AttnDev& d, const int32_t* row_offsets, const int32_t* prefix_lens,
                                             int table_stride, int g, int B, bool dense_ok);
__device__ __forceinline__ GroupPlan group_plan(const AttnDev& d, int g, int B, bool dense_ok) {
  return plan_of(d, d.group_row_offsets, d.group_prefix_lens, d.group_table_stride, g, B, dense_ok);
}
__device__ __forceinline__ GroupPlan outer_plan(const AttnDev& d, int g, int B, bool dense_ok) {
  return plan_of(d, d.outer_row_offsets, d.outer_prefix_lens, d.outer_table_stride, g, B, dense_ok);
}
__device__ __forceinline__ GroupPlan plan_of(const AttnDev& d, const int32_t* row_offsets, const int32_t* prefix_lens,
                                             int table_stride, int g, int B, bool dense_ok) {
  GroupPlan p;
  int r0 = row_offsets[g], r1 = row_offsets[g + 1];
  if (r0 < 0 || r1 > d.num_rows) {  // offsets outside the batch
    r0 = max(r0, 0);
    r1 = min(r1, d.num_rows);
    atomicMax(&d.hdr[kHdrStatus], kStatusBadIndex);
  }
  p.r0 = r0;
  p.n_rows = max(r1 - r0, 0);
  p.plen = max(prefix_lens[g], 0);
  p.nblk = (p.plen + B - 1) / B;
  if (p.nblk > table_stride) {  // length claims more blocks than the table holds
    p.nblk = table_stride;
    p.plen = p.nblk * B;
    atomicMax(&d.hdr[kHdrStatus], kStatusBadIndex);
  }
  p.npc = (p.nblk + d.cp - 1) / d.cp;
  if (p.n_rows == 0) p.npc = 0;
  p.dense = (dense_ok && p.npc > 0 && p.n_rows >= d.dense_min_rows) ? 1 : 0;
  p.n_rt = (p.n_rows + d.dense_row_tile - 1) / d.dense_row_tile;
  p.nt = (p.nblk + kDenseTileBlocks - 1) / kDenseTileBlocks;
  return p;
}

// A causal segment: n new tokens (rows) of one request over kv private context tokens.
struct SegPlan {
  int r0, n, kv, n_rt;
};

__device__ __forceinline__ SegPlan seg_plan(const AttnDev& d, int s, int B) {
  SegPlan p;
  p.r0 = d.seg_row_offsets[s];
  int r1 = d.seg_row_offsets[s + 1];
  if (p.r0 < 0 || r1 > d.num_rows) {  // offsets outside the batch
    p.r0 = max(p.r0, 0);
    r1 = min(r1, d.num_rows);
    atomicMax(&d.hdr[kHdrStatus], kStatusBadIndex);
  }
  p.n = max(r1 - p.r0, 0);
  p.kv = max(d.seg_kv_lens[s], 0);
  if (p.kv < p.n || (p.kv + B - 1) / B > d.seg_table_stride) {  // inconsistent lengths
    atomicMax(&d.hdr[kHdrStatus], kStatusBadIndex);
    p.kv = max(p.n, min(p.kv, d.seg_table_stride * B));
    if ((p.kv + B - 1) / B > d.seg_table_stride) { p.n = 0; p.kv = 0; }
  }
  p.n_rt = (p.n + d.dense_row_tile - 1) / d.dense_row_tile;
  return p;
}
// tokens the last row of row tile rt sees = kv tokens the tile's dense item has to cover
__device__ __forceinline__ int seg_tile_visible(const AttnDev& d, const SegPlan& p, int rt) {
  return p.kv - p.n + min(p.n, (rt + 1) * d.dense_row_tile);
}

// Index i in [0, n) with offs[i] <= r < offs[i + 1] of a CSR offsets array, or -1.
__device__ __forceinline__ int csr_find(const int32_t* offs, int n, int r) {
  if (n <= 0 || r < offs[0] || r >= offs[n]) return -1;
  int lo = 0, hi = n - 1;  // last i with offs[i] <= r
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (offs[mid] <= r) lo = mid; else hi = mid - 1;
  }
  return r < offs[lo + 1] ? lo : -1;
}
// Dense item in [lo, hi) (ascending row0) whose rows contain r, or -1.
__device__ __forceinline__ int item_find(const DnItem* items, int lo, int hi, int r) {
  if (lo >= hi) return -1;
  int a = lo, b = hi - 1;  // last item with row0 <= r
  while (a < b) {
    const int mid = (a + b + 1) >> 1;
    if (items[mid].row0 <= r) a = mid; else b = mid - 1;
  }
  const DnItem it = items[a];
  return (r >= it.row0 && r < it.row0 + it.nrows) ? a : -1;
}

// A prefill request whose rows all lie inside one prefix group that runs on the dense kernel is
// planned TOGETHER with that group: its row tiles become two-piece items (the group's prefix, then
// the request's own context under the causal mask) that accumulate both in one pass and leave one
// partial instead of two. Returns the group, or -1 when the segment keeps items of its own.
__device__ __forceinline__ int seg_joined_group(const AttnDev& d, const SegPlan& sp, int B, bool dense_ok) {
  if (!dense_ok || sp.n <= 0 || d.num_groups <= 0) return -1;
  const int g = csr_find(d.group_row_offsets, d.num_groups, sp.r0);
  if (g < 0) return -1;
  const GroupPlan p = group_plan(d, g, B, dense_ok);
  if (!p.dense || p.npc == 0) return -1;
  return (sp.r0 >= p.r0 && sp.r0 + sp.n <= p.r0 + p.n_rows) ? g : -1;
}
// kv tiles of a segment's row tile rt (its own context only)
__device__ __forceinline__ int seg_tiles(const AttnDev& d, const SegPlan& sp, int rt, int B) {
  return ((seg_tile_visible(d, sp, rt) + B - 1) / B + kDenseTileBlocks - 1) / kDenseTileBlocks;
}
// Walks the rows of a dense group in ascending order: gap(r_lo, r_hi) for every run of rows outside
// joined segments, joined(s, sp) for every joined segment.
template <typename GapFn, typename SegFn>
__device__ __forceinline__ void walk_group_rows(const AttnDev& d, int g, const GroupPlan& p, int B, bool dense_ok,
                                                GapFn gap, SegFn joined) {
  int cursor = p.r0;
  const int r_end = p.r0 + p.n_rows;
  const int NS = d.num_segments;
  if (NS > 0) {
    // first segment whose rows end after the group's first row
    int lo = 0, hi = NS;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (d.seg_row_offsets[mid + 1] <= p.r0) lo = mid + 1; else hi = mid;
    }
    for (int s = lo; s < NS && d.seg_row_offsets[s] < r_end; ++s) {
      const SegPlan sp = seg_plan(d, s, B);
      if (sp.n <= 0 || sp.r0 < cursor || seg_joined_group(d, sp, B, dense_ok) != g) continue;
      if (sp.r0 > cursor) gap(cursor, sp.r0);
      joined(s, sp);
      cursor = sp.r0 + sp.n;
    }
  }
  if (cursor < r_end) gap(cursor, r_end);
}

__global__ void __launch_bounds__(kPlanThreads, 1) plan_kernel(const AttnDev d, const int B, const bool dense_ok) {
  __shared__ int warp_sums[33];
  __shared__ unsigned long long sq_blocks;  // blocks all single-query items stream, per head
  const int tid = threadIdx.x;
  const int S = d.num_rows, G = d.num_groups, NS = d.num_segments;
  const int RT = d.dense_row_tile;  // rows per dense item: 128, or 256 when the dense kernel works on row-tile pairs

  if (tid == 0) {
    d.hdr[kHdrStatus] = kStatusOk; d.hdr[kHdrSqCounter] = 0; sq_blocks = 0;
    d.hdr[kHdrPlannedSlots] = (d.slot_mapping && NS == 0 && !d.head_mapping) ? 1 : 0;
  }
  __syncthreads();

  // ---- counts: groups (dense items / single-query prefix items) ----
  const int gper = (G + kPlanThreads - 1) / kPlanThreads;
  const int g_lo = min(tid * gper, G), g_hi = min(g_lo + gper, G);
  int my_dng = 0, my_dns = 0, my_sq = 0, my_tiles_g = 0, my_tiles_s = 0;
  long long my_blocks = 0;
  for (int g = g_lo; g < g_hi; ++g) {
    const GroupPlan p = group_plan(d, g, B, dense_ok);
    if (p.dense) {
      walk_group_rows(d, g, p, B, dense_ok,
                      [&](int r_lo, int r_hi) {
                        const int n_rt = (r_hi - r_lo + RT - 1) / RT;
                        my_dng += n_rt;
                        my_tiles_g += n_rt * p.nt;
                      },
                      [&](int, const SegPlan& sp) {
                        my_dng += sp.n_rt;
                        for (int rt = 0; rt < sp.n_rt; ++rt) my_tiles_g += p.nt + seg_tiles(d, sp, rt, B);
                      });
    } else {
      my_sq += p.npc * p.n_rows;
      my_blocks += (long long)p.nblk * p.n_rows;
    }
  }
  // ---- counts: causal segments (dense items per row tile / single-query items per row) ----
  const int sper = (NS + kPlanThreads - 1) / kPlanThreads;
  const int s_lo = min(tid * sper, NS), s_hi = min(s_lo + sper, NS);
  for (int s = s_lo; s < s_hi; ++s) {
    const SegPlan p = seg_plan(d, s, B);
    if (seg_joined_group(d, p, B, dense_ok) >= 0) continue;  // counted with its group
    if (dense_ok) {
      my_dns += p.n_rt;
      for (int rt = 0; rt < p.n_rt; ++rt) my_tiles_s += seg_tiles(d, p, rt, B);
    } else {
      for (int i = 0; i < p.n; ++i) {
        const int nb = (p.kv - p.n + i + 1 + B - 1) / B;
        my_sq += (nb + d.cs - 1) / d.cs;
        my_blocks += nb;
      }
    }
  }
  // ---- counts: outer prefix groups (dense items per row tile / single-query items per row) ----
  const int NO = d.num_outer_groups;
  const int oper = (NO + kPlanThreads - 1) / kPlanThreads;
  const int o_lo = min(tid * oper, NO), o_hi = min(o_lo + oper, NO);
  int my_dno = 0, my_tiles_o = 0;
  for (int o = o_lo; o < o_hi; ++o) {
    const GroupPlan p = outer_plan(d, o, B, dense_ok);
    if (p.dense) { my_dno += p.n_rt; my_tiles_o += p.n_rt * p.nt; }
    else { my_sq += p.npc * p.n_rows; my_blocks += (long long)p.nblk * p.n_rows; }
  }
  // ---- counts: rows (suffix items) ----
  const int rper = (S + kPlanThreads - 1) / kPlanThreads;
  const int r_lo = min(tid * rper, S), r_hi = min(r_lo + rper, S);
  int my_sqs = 0;
  for (int r = r_lo; r < r_hi; ++r) {
    int len = d.suffix_lens ? max(d.suffix_lens[r], 0) : 0;
    int nblk = (len + B - 1) / B;
    if (nblk > d.suffix_table_stride) nblk = d.suffix_table_stride;
    my_sqs += (nblk + d.cs - 1) / d.cs;
    my_blocks += nblk;
  }
  if (my_blocks) atomicAdd(&sq_blocks, (unsigned long long)my_blocks);
  // Dense items: all group items first (ascending rows), then all segment items (ascending rows),
  // so that a row finds its items by binary search and tile_base grows with the item index.
  int total_dng, total_dns, total_sq, total_tiles_g, total_tiles_s, total_sqs;
  int dng_base = block_exclusive_scan(my_dng, warp_sums, total_dng);
  int dns_base = block_exclusive_scan(my_dns, warp_sums, total_dns) + total_dng;
  int sq_base = block_exclusive_scan(my_sq, warp_sums, total_sq);
  int tile_g_base = block_exclusive_scan(my_tiles_g, warp_sums, total_tiles_g);
  int tile_s_base = block_exclusive_scan(my_tiles_s, warp_sums, total_tiles_s) + total_tiles_g;
  const int sqs_base = block_exclusive_scan(my_sqs, warp_sums, total_sqs);
  int total_dno, total_tiles_o;
  const int total_dn_inner = total_dng + total_dns;
  int dno_base = block_exclusive_scan(my_dno, warp_sums, total_dno) + total_dn_inner;
  int tile_o_base = block_exclusive_scan(my_tiles_o, warp_sums, total_tiles_o) + total_tiles_g + total_tiles_s;
  const int total_dn = total_dn_inner + total_dno, total_tiles = total_tiles_g + total_tiles_s + total_tiles_o;

  const bool overflow = (total_dn > d.cap_dn) || (total_sq + total_sqs > d.cap_sq);
  if (tid == 0) {
    d.hdr[kHdrNumSq] = overflow ? 0 : total_sq + total_sqs;
    d.hdr[kHdrNumDn] = overflow ? 0 : total_dn;
    d.hdr[kHdrDnTiles] = overflow ? 0 : total_tiles * d.num_heads;
    if (overflow) atomicMax(&d.hdr[kHdrStatus], kStatusListOverflow);
    // Split of the SMs between the dense kernel and the single-query kernel that runs beside it:
    // proportional to their work in units of one 128-token kv tile of one head (64 KiB of KV for
    // the streaming kernel). A dense tile is weighted: giving the dense kernel too many SMs costs
    // little, because its CTAs retire early and the single-query kernel takes their SMs over, while
    // too few make it the long pole.
    const double td = kDenseTileWeight * (double)total_tiles * d.num_heads * (RT / 128);  // a pair item's kv tile is two tiles of work
    const double ts = (double)sq_blocks * d.num_heads / kDenseTileBlocks;
    const int sms = d.num_sms;
    int c = sms;
    if (td > 0 && ts > 0) {
      c = (int)(sms * td / (td + ts) + 0.5);
      c = (c >= sms * 4 / 5) ? sms : max(4, c);
    }
    if (d.dense_ctas > 0) c = min(d.dense_ctas, sms);  // the caller's choice
    d.hdr[kHdrDenseCtas] = c;
  }
  if (overflow) { pdl_wait(); return; }

  // ---- groups: dense items (whole prefix per row tile) or single-query prefix items per row ----
  for (int g = g_lo; g < g_hi; ++g) {
    const GroupPlan p = group_plan(d, g, B, dense_ok);
    const int r0 = p.r0;
    if (p.npc == 0) continue;
    if (p.dense) {
      walk_group_rows(
          d, g, p, B, dense_ok,
          [&](int r_lo, int r_hi) {  // rows outside joined segments: the prefix alone
            for (int rr = r_lo; rr < r_hi; rr += RT) {
              DnItem it;
              it.row0 = rr;
              it.nrows = min(RT, r_hi - rr);
              it.tbl_off = g * d.group_table_stride;
              it.nblk = p.nblk;
              it.ntok = p.plen;
              it.nt = p.nt;
              it.tile_base = tile_g_base * d.num_heads;
              it.causal_base = 0;
              it.nt1 = it.nblk1 = it.ntok1 = it.tbl2_off = 0;
              it.flags = 0; it.pad[0] = it.pad[1] = it.pad[2] = 0;
              tile_g_base += it.nt;
              d.dn_items[dng_base++] = it;
            }
          },
          [&](int sidx, const SegPlan& sp) {  // a joined prefill request: prefix, then its own context
            for (int rt = 0; rt < sp.n_rt; ++rt) {
              const int vis = seg_tile_visible(d, sp, rt);
              DnItem it;
              it.row0 = sp.r0 + rt * RT;
              it.nrows = min(RT, sp.n - rt * RT);
              it.tbl_off = g * d.group_table_stride;
              it.nt1 = p.nt;
              it.nblk1 = p.nblk;
              it.ntok1 = p.plen;
              it.tbl2_off = sidx * d.seg_table_stride;
              it.flags = kDnDirect;  // withdrawn below if a row of the tile turns out to have a suffix
              it.pad[0] = it.pad[1] = it.pad[2] = 0;
              it.nblk = (vis + B - 1) / B;
              it.ntok = vis;
              it.nt = p.nt + seg_tiles(d, sp, rt, B);
              it.tile_base = tile_g_base * d.num_heads;
              it.causal_base = sp.kv - sp.n + rt * RT + 1;  // own tokens row 0 of the tile sees
              tile_g_base += it.nt;
              d.dn_items[dng_base++] = it;
            }
          });
    } else {
      for (int i = 0; i < p.n_rows; ++i)
        for (int c = 0; c < p.npc; ++c) {
          const int nb = min(d.cp, p.nblk - c * d.cp);
          d.sq_items[sq_base++] = make_sq_item(r0 + i, d.group_tables, g * d.group_table_stride + c * d.cp, 1, nb,
                                               min(p.plen - c * d.cp * B, nb * B), c);
        }
    }
  }

  // ---- causal segments: one dense item per row tile, covering the kv tokens its last row
  //      sees; without a tensor-core path every row becomes single-query items over its own view ----
  for (int s = s_lo; s < s_hi; ++s) {
    const SegPlan p = seg_plan(d, s, B);
    if (seg_joined_group(d, p, B, dense_ok) >= 0) continue;  // emitted with its group
    if (dense_ok) {
      for (int rt = 0; rt < p.n_rt; ++rt) {
        const int vis = seg_tile_visible(d, p, rt);
        DnItem it;
        it.nt1 = it.nblk1 = it.ntok1 = it.tbl2_off = 0;
        it.flags = 0; it.pad[0] = it.pad[1] = it.pad[2] = 0;
        it.row0 = p.r0 + rt * RT;
        it.nrows = min(RT, p.n - rt * RT);
        it.tbl_off = s * d.seg_table_stride;
        it.nblk = (vis + B - 1) / B;
        it.ntok = vis;
        it.nt = (it.nblk + kDenseTileBlocks - 1) / kDenseTileBlocks;
        it.tile_base = tile_s_base * d.num_heads;
        it.causal_base = p.kv - p.n + rt * RT + 1;  // tokens row 0 of the tile sees
        tile_s_base += it.nt;
        d.dn_items[dns_base++] = it;
      }
    } else {
      for (int i = 0; i < p.n; ++i) {
        const int r = p.r0 + i, vis = p.kv - p.n + i + 1;
        const int nblk = (vis + B - 1) / B, nc = (nblk + d.cs - 1) / d.cs;
        for (int c = 0; c < nc; ++c) {
          const int nb = min(d.cs, nblk - c * d.cs);
          d.sq_items[sq_base++] = make_sq_item(r, d.seg_tables, s * d.seg_table_stride + c * d.cs, 2, nb,
                                               min(vis - c * d.cs * B, nb * B), d.pparts + c);
        }
      }
    }
  }
  // ---- outer prefix groups: like plain groups, in their own item and partial ranges ----
  for (int o = o_lo; o < o_hi; ++o) {
    const GroupPlan p = outer_plan(d, o, B, dense_ok);
    if (p.npc == 0) continue;
    if (p.dense) {
      for (int rr = p.r0; rr < p.r0 + p.n_rows; rr += RT) {
        DnItem it;
        it.row0 = rr;
        it.nrows = min(RT, p.r0 + p.n_rows - rr);
        it.tbl_off = o * d.outer_table_stride;
        it.nblk = p.nblk;
        it.ntok = p.plen;
        it.nt = p.nt;
        it.tile_base = tile_o_base * d.num_heads;
        it.causal_base = 0;
        it.nt1 = it.nblk1 = it.ntok1 = it.tbl2_off = 0;
        it.flags = kDnOuter; it.pad[0] = it.pad[1] = it.pad[2] = 0;
        tile_o_base += it.nt;
        d.dn_items[dno_base++] = it;
      }
    } else {
      for (int i = 0; i < p.n_rows; ++i)
        for (int c = 0; c < p.npc; ++c) {
          const int nb = min(d.cp, p.nblk - c * d.cp);
          d.sq_items[sq_base++] = make_sq_item(p.r0 + i, d.outer_tables, o * d.outer_table_stride + c * d.cp, 3, nb,
                                               min(p.plen - c * d.cp * B, nb * B), d.pparts + d.cparts + d.sparts + c);
        }
    }
  }
  __syncthreads();  // the dense items are in place; rows look theirs up below

  // ---- rows: row_info (group, segment and dense items of the row) and the suffix items ----
  int w = total_sq + sqs_base;
  for (int r = r_lo; r < r_hi; ++r) {
    int len = d.suffix_lens ? max(d.suffix_lens[r], 0) : 0;
    int nblk = (len + B - 1) / B;
    if (nblk > d.suffix_table_stride) {
      nblk = d.suffix_table_stride;
      len = nblk * B;
      atomicMax(&d.hdr[kHdrStatus], kStatusBadIndex);
    }
    const int nsc = (nblk + d.cs - 1) / d.cs;
    RowInfo info;
    info.group = -1; info.np_sq = 0; info.nsc = nsc; info.dn = -1; info.seg_dn = -1; info.nc_sq = 0;
    info.odn = -1; info.onp_sq = 0;
    if (NO > 0) {
      const int o = csr_find(d.outer_row_offsets, NO, r);
      if (o >= 0) {
        const GroupPlan p = outer_plan(d, o, B, dense_ok);
        if (p.dense) info.odn = item_find(d.dn_items, total_dn_inner, total_dn, r);
        else info.onp_sq = p.npc;
      }
    }
    const int g = csr_find(d.group_row_offsets, G, r);
    if (g >= 0) {
      const GroupPlan p = group_plan(d, g, B, dense_ok);
      info.group = g;
      info.np_sq = p.dense ? 0 : p.npc;
      info.dn = (p.dense && p.npc > 0) ? item_find(d.dn_items, 0, total_dng, r) : -1;
    }
    if (NS > 0) {
      if (dense_ok) {
        info.seg_dn = item_find(d.dn_items, total_dng, total_dn_inner, r);
      } else {
        const int s = csr_find(d.seg_row_offsets, NS, r);
        if (s >= 0) {
          const SegPlan p = seg_plan(d, s, B);
          if (r - p.r0 < p.n) info.nc_sq = (((p.kv - p.n + (r - p.r0) + 1 + B - 1) / B) + d.cs - 1) / d.cs;
        }
      }
    }
    d.row_info[r] = info;
    if ((nsc > 0 || info.odn >= 0 || info.onp_sq > 0) && info.dn >= 0 && (d.dn_items[info.dn].flags & kDnDirect))
      atomicAnd(&d.dn_items[info.dn].flags, ~kDnDirect);  // this row needs the merge: so does its tile
    // The row's new token (a pure decode batch whose fill the suffix kernel performs itself): it must be
    // the last token of the row's suffix, so that the item of the last chunk can carry it.
    bool carries_new = false;
    if (d.slot_mapping && NS == 0 && !d.head_mapping) {
      const long long slot = d.slot_is_i64 ? reinterpret_cast<const long long*>(d.slot_mapping)[r]
                                           : (long long)reinterpret_cast<const int*>(d.slot_mapping)[r];
      if (slot >= 0) {
        const long long want = (len > 0 && nsc > 0)
            ? (long long)d.suffix_tables[(size_t)r * d.suffix_table_stride + (len - 1) / B] * B + (len - 1) % B : -1;
        if (slot == want) carries_new = true;
        else atomicMax(&d.hdr[kHdrStatus], kStatusBadIndex);
      }
    }
    for (int c = 0; c < nsc; ++c) {
      const int nb = min(d.cs, nblk - c * d.cs);
      SqItem it = make_sq_item(r, d.suffix_tables, r * d.suffix_table_stride + c * d.cs, 0, nb,
                               min(len - c * d.cs * B, nb * B), d.pparts + d.cparts + c);
      if (carries_new && c == nsc - 1) it.meta |= 1 << 20;
      d.sq_items[w++] = it;
    }
  }
  // The planner reads nothing the kernel before it writes (a KV fill, which lets its dependents
  // start early), so it runs beside that kernel; it still must not COMPLETE before it, because the
  // attention kernels wait only for their direct predecessor, the planner.
  pdl_wait();
}

}  // namespace

cudaError_t launch_plan(const AttnDev& d, int block_size, bool dense_supported, cudaStream_t s) {
  return launch_kernel(plan_kernel, 1, kPlanThreads, 0, s, true, d, block_size, dense_supported);
}

}  // namespace pb
