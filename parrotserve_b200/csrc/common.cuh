// Shared device/host helpers of the B200 shared-prefix paged attention library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/parrot_b200_attn.h"

namespace pb {

constexpr int kMaxSMs = 148;   // a B200 has 148 SMs; bound of the per-CTA partial ranges
constexpr float kLog2e = 1.4426950408889634f;

// ---------------------------------------------------------------------------------------------
// Workspace layout. Everything a call needs beyond its inputs and outputs lives here.
//
//   header   int32[64]   [0] status word, [1] number of single-query work items,
//                        [2] number of dense (tensor-core) work items, [3] dense kv tiles * heads,
//                        [4] next unclaimed single-query work item (reset by the planner and the merge),
//                        [5] CTAs of the dense kernel that take work (the planner's split of the SMs, or
//                        the caller's dense_ctas as it was when the lists were built),
//                        [6] 1 when the lists were built with the rows' new-token slots (the items that
//                        carry a new token are marked: the suffix kernel may perform the KV fill)
//   row_info RowInfo[rows]  where each row's partials live (see RowInfo)
//   sq_items SqItem[]    work list of the single-query (suffix) kernel
//   dn_items DnItem[]    work list of the dense prefix kernel
//   ml       float2[rows * parts * heads]        (max, sum) of every partial, base-2 domain
//   acc      float [rows * parts * heads * D]    un-normalised partial outputs
//
// Partial (row r, part j, head h) lives at index (j * heads + h) * rows + r (partial_slot below);
// prefix partial c uses j = c, partial c of the
// row's causal segment uses j = pparts + c, suffix chunk c uses j = pparts + cparts + c.
//
// Dense tile order ("stream-K"): item i, head h, kv tile t has index tile_base_i + h * nt_i + t;
// CTA c of the dense kernel owns [c * total / ctas, (c + 1) * total / ctas). A (item, head) that
// several CTAs touch gets one partial per CTA, numbered in CTA order (dense_first_cta below).
// ---------------------------------------------------------------------------------------------
struct SqItem {       // one (row, kv chunk); the kernel multiplies the list by the heads
  int32_t row;
  int32_t meta;       // nblk (>= 1) | embedded << 17 | table kind << 18 | carries the row's new token << 20
  int32_t ntok;       // tokens in the chunk (>= 1)
  int32_t part;       // partial slot index j
  int32_t bid[4];     // embedded: the chunk's (<= 4) physical block ids, so the kernel needs no
                      // dependent table read; else bid[0] = offset of the first id in its table
};
constexpr int kSqEmbedMax = 4;
static_assert(sizeof(SqItem) == 32, "SqItem must be 32 bytes");

struct RowInfo {      // 32 bytes
  int32_t group;      // prefix group or -1
  int32_t np_sq;      // prefix partials written by the single-query kernel (0 if dense or none)
  int32_t nsc;        // suffix partials
  int32_t dn;         // dense item of the row's prefix, or -1
  int32_t seg_dn;     // dense item of the row's causal segment tile, or -1
  int32_t nc_sq;      // causal-segment partials written by the single-query kernel
  int32_t odn;        // dense item of the row's OUTER prefix group, or -1
  int32_t onp_sq;     // outer-prefix partials written by the single-query kernel
};
static_assert(sizeof(RowInfo) == 32, "RowInfo must be 32 bytes");

struct DnItem {       // one tile of query rows and the kv tokens they attend in the dense kernel
  int32_t row0;       // first row of the tile
  int32_t nrows;      // rows in the tile (1..dense_row_tile: 128, or 256 = two row tiles that share their K/V)
  int32_t tbl_off;    // offset of the first block id of the (first) piece inside its table
  int32_t nblk;       // blocks of the last piece
  int32_t ntok;       // tokens of the last piece
  int32_t nt;         // 128-token kv tiles of the whole item (both pieces)
  int32_t tile_base;  // index of (this item, head 0, kv tile 0) in the global dense tile order
  int32_t causal_base;  // 0: every row sees all tokens of the last piece;
                        // > 0: row i of the tile sees its first causal_base + i tokens (causal segment)
  // Two-piece items (a prefill request inside a prefix group): kv tiles [0, nt1) walk the group's
  // prefix (group_tables + tbl_off, nblk1 blocks, ntok1 tokens, no mask), tiles [nt1, nt) the
  // request's own context (seg_tables + tbl2_off, nblk/ntok/causal_base above). nt1 == 0: one piece,
  // in group_tables (causal_base == 0) or seg_tables (causal_base > 0) at tbl_off.
  int32_t nt1, nblk1, ntok1, tbl2_off;
  int32_t flags;  // kDnDirect: none of the item's rows has any other partial (no suffix, no item of
                  // its own), so a CTA that holds ALL kv tiles of (item, head) writes the finished,
                  // normalised output rows itself and the merge skips them
  int32_t pad[3];
};
static_assert(sizeof(DnItem) == 64, "DnItem must be 64 bytes");
constexpr int32_t kDnDirect = 1;
constexpr int32_t kDnOuter = 2;   // the item walks an outer prefix group (outer_tables, outer partial range)

struct WsLayout {
  size_t off_rowinfo, off_sq, off_dn, off_ml, off_acc, total;
  int32_t parts;        // partial slots per row
  int32_t pparts;       // prefix partial slots per row (first `pparts` slots)
  int32_t sparts;       // suffix partial slots per row
  int32_t cparts;       // causal-segment partial slots per row
  int32_t oparts;       // outer-prefix partial slots per row (the last `oparts` slots)
  int32_t cs;           // suffix chunk, blocks
  int32_t cp;           // prefix chunk, blocks
  int32_t cap_sq, cap_dn;
  int32_t dense_min_rows;
};

enum : int32_t {
  kStatusOk = 0,
  kStatusWaitExpired = 1,   // a bounded mbarrier wait ran out
  kStatusBadIndex = 2,      // block id or slot outside the cache
  kStatusListOverflow = 3,  // a work list did not fit its capacity
};

constexpr int kHdrStatus = 0, kHdrNumSq = 1, kHdrNumDn = 2, kHdrDnTiles = 3, kHdrSqCounter = 4, kHdrDenseCtas = 5,
              kHdrPlannedSlots = 6, kHdrInts = 64;
constexpr int kDenseTileBlocks = 8;  // kv tile of the dense kernel: 8 blocks

// CTA that owns global dense tile g when `total` tiles are split over `ctas` CTAs. With fewer
// tiles than CTAs only the first `total` CTAs work, so every working CTA owns a non-empty range
// and the CTAs that touch one (item, head) are consecutive.
__host__ __device__ inline int dense_active_ctas(long long total, int ctas) {
  return total < ctas ? (int)total : ctas;
}
__host__ __device__ inline int dense_cta_of_tile(long long g, long long total, int ctas) {
  const int c = dense_active_ctas(total, ctas);
  return (int)(((g + 1) * c + total - 1) / total) - 1;
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---------------------------------------------------------------------------------------------
// element helpers
// ---------------------------------------------------------------------------------------------
template <typename T> struct ElemTraits;
template <> struct ElemTraits<float> { static constexpr int kVec = 4; };
template <> struct ElemTraits<__half> { static constexpr int kVec = 8; };
template <> struct ElemTraits<__nv_bfloat16> { static constexpr int kVec = 8; };

// Unpacks one 16-byte vector into ElemTraits<T>::kVec floats.
template <typename T> __device__ __forceinline__ void unpack16(const uint4& v, float* f);
template <> __device__ __forceinline__ void unpack16<float>(const uint4& v, float* f) {
  f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
  f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}
template <> __device__ __forceinline__ void unpack16<__half>(const uint4& v, float* f) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <typename T> __device__ __forceinline__ T from_float(float f);
template <> __device__ __forceinline__ float from_float<float>(float f) { return f; }
template <> __device__ __forceinline__ __half from_float<__half>(float f) { return __float2half_rn(f); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float f) { return __float2bfloat16_rn(f); }

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// ---------------------------------------------------------------------------------------------
// PTX wrappers (mbarrier + bulk async copies). Every wait is bounded.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking test (try_wait may suspend the thread for a while when the phase is not complete).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Waits for the phase with the given parity. Gives up after about two seconds and returns false.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 0xffu) == 0xffu) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > 2000000000ull) return false;
    }
  }
}
// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// The same copy with an L2 eviction policy (createpolicy): data that is read once should not push
// out lines that are read again soon.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}

// Programmatic dependent launch: a kernel launched with the stream-serialization attribute may
// start while its predecessor still runs; it must not touch the predecessor's results before
// pdl_wait(). pdl_trigger() lets the NEXT kernel in the stream start launching.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---------------------------------------------------------------------------------------------
// kernel parameter blocks
// ---------------------------------------------------------------------------------------------
struct AttnDev {            // what the attention kernels read
  void* out;
  const void* query;
  const void* key_cache;
  const void* value_cache;
  const int32_t* head_mapping;
  const int32_t* suffix_lens;
  const int32_t* suffix_tables;
  const int32_t* group_row_offsets;
  const int32_t* group_prefix_lens;
  const int32_t* group_tables;
  const int32_t* seg_row_offsets;
  const int32_t* seg_kv_lens;
  const int32_t* seg_tables;
  float* qk_max;
  float* exp_sum;
  int32_t* hdr;
  RowInfo* row_info;
  SqItem* sq_items;
  DnItem* dn_items;
  float2* ml;
  float* acc;
  float scale_log2e;
  int32_t num_rows, num_heads, num_kv_heads, num_groups;
  int32_t suffix_table_stride, group_table_stride, num_segments, seg_table_stride, cparts;
  int32_t parts, pparts, sparts, oparts, cs, cp, cap_sq, cap_dn, dense_min_rows, stats_mode, dense_ctas, num_sms;
  const int32_t* outer_row_offsets;
  const int32_t* outer_prefix_lens;
  const int32_t* outer_tables;
  int32_t num_outer_groups, outer_table_stride;
  int32_t sq_waits_at_start;  // 1: no dense kernel precedes the single-query kernel in this call
  int32_t dense_row_tile;     // rows per dense item: 128 (one row tile per CTA pass) or 256 (row-tile pairs)
  int32_t acc_tma;            // 1: the dense kernel may write full row tiles of partials with TMA tiled stores
  // new tokens of the step (see pb_attn_params): slot_mapping is the planner's input; key_new /
  // value_new are set only when the suffix kernel itself performs the fill (pure decode batch)
  const void* slot_mapping;
  const void* key_new;
  const void* value_new;
  int64_t key_new_stride, value_new_stride;
  int32_t slot_is_i64;
  int32_t out_vec16;          // 1: output rows may be written with 16-byte stores (base and row stride aligned)
  int64_t q_stride, out_stride, kv_block_stride, kv_head_stride, num_blocks;
};

// Index of the partial of (row, part, head) in the ml / acc arrays. Rows are innermost so the 128
// rows a dense tile writes for one head are contiguous (64 KiB) and a prefill batch of thousands of
// rows does not scatter its partials over the whole workspace.
__device__ __forceinline__ size_t partial_slot(const AttnDev& d, int row, int part, int head) {
  return ((size_t)part * d.num_heads + head) * d.num_rows + row;
}

// CTAs of the dense kernel that take work: fixed when the lists are built (the planner's split of
// the SMs, or the caller's dense_ctas), because the partials a (row, head) receives depend on it.
__device__ __forceinline__ int dense_ctas_of(const AttnDev& d) { return d.hdr[kHdrDenseCtas]; }

// What kv tile t of a dense item covers: where its block ids are, how many blocks and tokens it
// holds, and the causal limit of row 0 inside the tile (tokens of this tile row 0 may attend;
// row i adds i) or a negative value when the tile is not masked.
struct DenseTileView {
  const int32_t* table;
  int nb, ntok, causal0;
  bool causal;
};
__device__ __forceinline__ DenseTileView dense_tile_view(const AttnDev& d, const DnItem& it, int t) {
  DenseTileView v;
  if (t < it.nt1) {
    v.table = d.group_tables + it.tbl_off + t * kDenseTileBlocks;
    v.nb = min(kDenseTileBlocks, it.nblk1 - t * kDenseTileBlocks);
    v.ntok = min(kDenseTileBlocks * 16, it.ntok1 - t * kDenseTileBlocks * 16);
    v.causal = false;
    v.causal0 = 0;
  } else {
    const int t2 = t - it.nt1;
    const int32_t* base = (it.nt1 > 0) ? d.seg_tables + it.tbl2_off
                          : ((it.flags & kDnOuter) ? d.outer_tables : it.causal_base > 0 ? d.seg_tables : d.group_tables) + it.tbl_off;
    v.table = base + t2 * kDenseTileBlocks;
    v.nb = min(kDenseTileBlocks, it.nblk - t2 * kDenseTileBlocks);
    v.ntok = min(kDenseTileBlocks * 16, it.ntok - t2 * kDenseTileBlocks * 16);
    v.causal = it.causal_base > 0;
    v.causal0 = it.causal_base - t2 * kDenseTileBlocks * 16;
  }
  return v;
}
// Whether the rows of a dense item may be finished by the dense kernel itself (by the CTA that holds
// all kv tiles of the (item, head)); the dense kernel and the merge must agree on this.
__device__ __forceinline__ bool dense_direct_ok(const AttnDev& d, const DnItem& it) {
  return (it.flags & kDnDirect) && it.nrows > 64 && d.out_vec16 && d.stats_mode == 0;
}
// first partial slot of a dense item: causal segments on their own use the segment range
__device__ __forceinline__ int dense_part_base(const AttnDev& d, const DnItem& it) {
  if (it.flags & kDnOuter) return d.pparts + d.cparts + d.sparts;  // outer prefixes use the last range
  return (it.causal_base > 0 && it.nt1 == 0) ? d.pparts : 0;
}

// last CUDA runtime error text, per thread
void set_cuda_error(cudaError_t e);
const char* last_cuda_error();

// Launch with (pdl = true) or without programmatic stream serialization.
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl,
                          Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// SMs of the current device (queried once per device); 148 when no device can be asked.
int sm_count();

// launchers implemented in the .cu files (host side, return cudaError_t)
cudaError_t launch_plan(const AttnDev& d, int block_size, bool dense_supported, cudaStream_t s);
cudaError_t launch_single_query(const AttnDev& d, int dtype, int head_size, int block_size, cudaStream_t s);
cudaError_t launch_single_query_b8(const AttnDev& d, int dtype, int head_size, cudaStream_t s);
cudaError_t launch_single_query_b32(const AttnDev& d, int dtype, int head_size, cudaStream_t s);
cudaError_t launch_merge(const AttnDev& d, int dtype, int head_size, cudaStream_t s);
// Dense prefix stage; `supported` reports whether this (dtype, head, block) has a tensor-core path.
bool dense_prefix_supported(int dtype, int head_size, int block_size);
cudaError_t launch_dense_prefix(const AttnDev& d, int dtype, int head_size, int block_size, cudaStream_t s);

}  // namespace pb
