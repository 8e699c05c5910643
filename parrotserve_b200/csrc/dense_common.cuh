// Device helpers shared by the two tensor-core kernels of the prefix / prefill stage
// (prefix_dense.cu: one row tile per pass; dense_pair.cu: row-tile pairs): tcgen05, TMEM and TMA
// wrappers, operand descriptors, bounded waits, and the stream-K walk over the dense work list.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace pb {
namespace dense {

constexpr int kD = 128, kB = 16;
constexpr int kTileBlocks = kDenseTileBlocks;   // 128 tokens per softmax round
constexpr int kTileTok = kTileBlocks * kB;
constexpr int kBlkBytes = kD * kB * 2;          // 4096: one K or V tile of a (block, head)
constexpr int kStages = 2;
constexpr int kQBytes = 128 * kD * 2;           // 32 KiB: the Q operand of one row tile
constexpr int kRingBytes = kTileBlocks * kBlkBytes;  // one K (or V) slot: 32 KiB
constexpr int kPrefetchTiles = 4;               // L2 prefetch distance of the K and V tiles, in tiles
constexpr float kTau = 8.f;                     // lazy-rescale threshold, log2 units

#ifdef PB_PAIR_TRACE
// debug build only: clock stamps of lane 0 of every warp, read back with pb_debug_trace_read
static __device__ unsigned long long g_trace[148 * 12 * 256];  // one per translation unit
__device__ __forceinline__ void pb_trace(int* trace_n, int code) {  // trace_n: 12 counters in shared memory
  const unsigned long long t = clock64();
  if ((threadIdx.x & 31) == 0) {
    const int w = threadIdx.x >> 5;
    if (code < 0) { trace_n[w] = 0; return; }
    const int n = trace_n[w];
    if (n < 256) {
      g_trace[(blockIdx.x * 12 + w) * 256 + n] = ((unsigned long long)code << 48) | (t & 0xffffffffffffull);
      trace_n[w] = n + 1;
    }
  }
}
#define PB_TRACE(code) pb_trace(trace_ctr, code)
#else
#define PB_TRACE(code)
#endif

// ---- tcgen05 / TMA wrappers ----
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Per-thread 16-byte async copy global -> shared (LSU path, any destination address).
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// Arrives on `bar` once all earlier cp.async of this thread have completed (does not count as pending).
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Asks L2 to fetch `bytes` (a multiple of 16) at a 16-byte aligned global address; no destination.
__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// TMA tiled load of one V tile: box {16 tok, 128 d, 1 head, 1 block}; no multicast.
__device__ __forceinline__ void tma_load_v(uint32_t dst, const CUtensorMap* map, uint32_t bar, int kvh, int blk) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(0), "r"(0), "r"(kvh), "r"(blk)
      : "memory");
}

// TMA tiled load of 32 query rows x 64 elements of one head (128-byte swizzle); no multicast.
__device__ __forceinline__ void tma_load_q(uint32_t dst, const CUtensorMap* map, uint32_t bar, int col, int head, int row) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(col), "r"(head), "r"(row)
      : "memory");
}

// TMA tiled store of [128 rows][32 floats] (128-byte swizzle in shared memory) into the partial
// accumulators, as part of the calling thread's current bulk group.
__device__ __forceinline__ void tma_store_acc(const CUtensorMap* map, uint32_t src, int col, int row) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(col), "r"(row) : "memory");
}
// TMA tiled store of [128 rows][64 elements] of one head (128-byte swizzle in shared memory) into
// the output tensor [rows, heads, 128].
__device__ __forceinline__ void tma_store_out(const CUtensorMap* map, uint32_t src, int col, int head, int row) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(col), "r"(head), "r"(row) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Shared-memory matrix descriptor (K-major). layout: 0 = no swizzle, 2 = 128-byte swizzle, 6 = 32-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version of this architecture
  d |= (uint64_t)layout << 61;
  return d;
}
// Instruction descriptor, kind::f16: fp32 accumulate, A and B K-major, fp16 or bf16 inputs.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool bf16) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

// Bounded, abort-aware wait; the outcome is made uniform across the calling warp.
// `backoff_ns` > 0 makes a waiting warp sleep between polls so it does not take issue slots from the
// softmax warps that share its scheduler (used by the copy producers, which are never latency critical).
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status,
                                              uint32_t backoff_ns = 0) {
  bool ok = mbar_try_wait(bar, parity);
  if (!ok) {
    uint64_t t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
      if (backoff_ns) __nanosleep(backoff_ns);
      if (mbar_try_wait(bar, parity)) { ok = true; break; }
      if ((spin & 63u) == 63u) {
        if (*abort_flag) break;
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > 2000000000ull) {
          *abort_flag = 1;
          atomicMax(status, kStatusWaitExpired);
          break;
        }
      }
    }
  }
  return __all_sync(0xffffffffu, ok);
}

template <typename T> struct Pack;
template <> struct Pack<__half> {
  static __device__ __forceinline__ uint32_t two(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static constexpr bool kBf16 = false;
};
template <> struct Pack<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t two(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static constexpr bool kBf16 = true;
};

// One contiguous run of kv tiles of one (item, head), as cut out by a CTA's share of the global
// dense tile order.
struct Segment {
  DnItem it;
  int head, t0, t1, part;
};

// Walks the segments of this CTA; all roles call it with the same arguments and see the same list.
// The item under the cursor and the first tile of the one after it stay in registers, so a step
// inside an item (the common case: one segment per head) reads no memory.
struct SegmentWalker {
  const AttnDev& d;
  long long g, g_end, total, next_base;
  int n_dn, H, ctas, idx;
  DnItem cur;
  __device__ SegmentWalker(const AttnDev& dd, int cta, int nctas) : d(dd) {
    H = d.num_heads;
    n_dn = d.hdr[kHdrNumDn];
    total = d.hdr[kHdrDnTiles];
    ctas = nctas;
    const int active = dense_active_ctas(total, nctas);
    g = (cta < active) ? total * cta / active : 0;
    g_end = (cta < active) ? total * (cta + 1) / active : 0;
    idx = -1;
    next_base = 0;
    if (g < g_end) {
      int lo = 0, hi = n_dn - 1;  // last item with tile_base <= g
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if ((long long)d.dn_items[mid].tile_base <= g) lo = mid; else hi = mid - 1;
      }
      load(lo);
    }
  }
  __device__ void load(int i) {
    idx = i;
    cur = d.dn_items[i];
    next_base = (i + 1 < n_dn) ? (long long)d.dn_items[i + 1].tile_base : total;
  }
  __device__ bool next(Segment& sg) {
    if (g >= g_end) return false;
    while (g >= next_base && idx + 1 < n_dn) load(idx + 1);
    sg.it = cur;
    const long long rel = g - sg.it.tile_base;
    sg.head = (int)(rel / sg.it.nt);
    sg.t0 = (int)(rel - (long long)sg.head * sg.it.nt);
    const long long room = g_end - g;
    sg.t1 = (int)min((long long)sg.it.nt, sg.t0 + room);
    const long long g0 = (long long)sg.it.tile_base + (long long)sg.head * sg.it.nt;
    sg.part = dense_cta_of_tile(g, total, ctas) - dense_cta_of_tile(g0, total, ctas);
    g += sg.t1 - sg.t0;
    return true;
  }
};

// A from tensor memory (lane = row, 16-bit elements packed two per 32-bit column, K-major), B from
// shared memory through a descriptor.
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---- K and V producers (used by dense_pair.cu; prefix_dense.cu keeps the same loops inline: as functions
//      they measured 1-2 % slower there) ----
// Barriers of the two K/V rings sit at the same indices in both kernels.
enum { kBarFullK = 0, kBarEmptyK = 2, kBarFullV = 4, kBarEmptyV = 6 };

// K producer (warp pw of kWarps): per-thread 16-byte async copies with re-pack.
// The 256-byte row of d-chunk c of block j goes to [c][j][16 tok][16 B]: the 8-token groups of ALL
// blocks of the tile then sit 128 bytes apart and one MMA spans the whole tile. A warp instruction
// moves 512 contiguous source bytes (two chunk rows). Each thread signals the slot's mbarrier when
// its own copies have landed (cp.async.mbarrier.arrive.noinc).
template <int kWarps>
__device__ __forceinline__ void k_producer(const AttnDev& d, SegmentWalker& walk, int pw, int lane, uint32_t sK0, uint32_t bars0,
                                           volatile int* abort_flag, int32_t* status) {
  const uint8_t* kc = reinterpret_cast<const uint8_t*>(d.key_cache);
  uint32_t tc = 0;
  bool ok = true;
  Segment sg;
  while (ok && walk.next(sg)) {
    const int kvh = d.head_mapping ? d.head_mapping[sg.head] : sg.head;
    for (int t = sg.t0; t < sg.t1; ++t, ++tc) {
      const int s = tc & 1;
      const uint32_t ph = (tc >> 1) & 1;
      const DenseTileView tv = dense_tile_view(d, sg.it, t);
      const int nb = tv.nb;
      int blk = (lane < nb) ? tv.table[lane] : 0;
      if (blk < 0 || blk >= d.num_blocks) {
        atomicMax(status, kStatusBadIndex);
        blk = 0;
      }
      if (!wait_or_abort(bars0 + (kBarEmptyK + s) * 8, ph ^ 1, abort_flag, status, 100)) { ok = false; break; }
      const uint32_t slot = sK0 + s * kRingBytes;
      for (int j = pw; j < kTileBlocks; j += kWarps) {
        const int bj = __shfl_sync(0xffffffffu, blk, j);
        if (j < nb) {
          const uint8_t* src = kc + ((size_t)bj * d.kv_block_stride + (size_t)kvh * d.kv_head_stride) * 2 + lane * 16;
          const uint32_t dst = slot + (lane >> 4) * (kTileBlocks * 256) + j * 256 + (lane & 15) * 16;
#pragma unroll
          for (int k = 0; k < 8; ++k)
            cp_async16(dst + k * 2 * (kTileBlocks * 256), src + k * 512);
        }
      }
      cp_async_arrive_noinc(bars0 + (kBarFullK + s) * 8);
    }
  }
  cp_async_wait_all();
}

// V producer, the tiles of one segment: TMA tiled loads with the 32-byte swizzle into the V ring,
// and L2 prefetches of the K and V tiles kPrefetchTiles ahead (the two-slot rings hide little
// latency when another kernel saturates HBM beside this one; lane j: block j of the tile, K in the
// lower half-warp, V in the upper). `tc` is the ring index of the segment's first tile and is
// advanced. Returns false when a wait gave up.
__device__ __forceinline__ bool v_tiles(const AttnDev& d, const Segment& sg, const CUtensorMap* vmap, int lane, uint32_t sV0,
                                        uint32_t bars0, uint32_t& tc, volatile int* abort_flag, int32_t* status) {
  const int kvh = d.head_mapping ? d.head_mapping[sg.head] : sg.head;
  auto prefetch_tile = [&](int tp) {
    if (tp >= sg.t1) return;
    const int j = lane & 15;
    const DenseTileView pv = dense_tile_view(d, sg.it, tp);
    if (j < pv.nb) {
      const int b = pv.table[j];
      if (b >= 0 && b < d.num_blocks) {
        const uint8_t* base = reinterpret_cast<const uint8_t*>(lane < 16 ? d.key_cache : d.value_cache);
        prefetch_l2(base + ((size_t)b * d.kv_block_stride + (size_t)kvh * d.kv_head_stride) * 2, kBlkBytes);
      }
    }
  };
  for (int tp = sg.t0 + 1; tp < sg.t0 + kPrefetchTiles; ++tp) prefetch_tile(tp);
  for (int t = sg.t0; t < sg.t1; ++t, ++tc) {
    const int s = tc & 1;
    const uint32_t ph = (tc >> 1) & 1;
    const DenseTileView tv = dense_tile_view(d, sg.it, t);
    const int nb = tv.nb;
    int blk = (lane < nb) ? tv.table[lane] : 0;
    if (blk < 0 || blk >= d.num_blocks) {
      atomicMax(status, kStatusBadIndex);
      blk = 0;
    }
    prefetch_tile(t + kPrefetchTiles);
    if (!wait_or_abort(bars0 + (kBarEmptyV + s) * 8, ph ^ 1, abort_flag, status, 100)) return false;
    if (lane == 0) mbar_arrive_expect_tx(bars0 + (kBarFullV + s) * 8, nb * kBlkBytes);
    __syncwarp();
    for (int j = 0; j < nb; ++j) {
      const int bj = __shfl_sync(0xffffffffu, blk, j);
      if (lane == 0) tma_load_v(sV0 + s * kRingBytes + j * kBlkBytes, vmap, bars0 + (kBarFullV + s) * 8, kvh, bj);
    }
  }
  return true;
}

}  // namespace dense

// Row-tile-pair kernel (dense_pair.cu); the tensor maps are those launch_dense_prefix builds.
cudaError_t launch_dense_pair(const AttnDev& d, int dtype, const CUtensorMap& vmap, const CUtensorMap& qmap,
                              const CUtensorMap& amap, const CUtensorMap& omap, cudaStream_t s);

}  // namespace pb
