// Tensor-core prefix / prefill stage on ROW-TILE PAIRS (tcgen05 + TMEM + TMA).
//
// Same work, lists and results as prefix_dense.cu, for batches whose dense work comes in tiles of
// 128 query rows (prefill requests, large prefix groups). A work item here holds up to 256 rows of
// one group or request: two row tiles that attend the SAME keys. Each K/V tile is brought into
// shared memory once and used by both row tiles, and the two tiles run half a period apart: while
// the tensor pipe computes P.V and the next Q.K^T of one tile, the softmax threads of the other
// tile are at work. Per row tile x (0, 1):
//     S_x[128 x 128] = Q_x . K^T         (A and B from shared memory)
//     O_x[128 x D]  += P_x . V           (A = P_x from TENSOR MEMORY, B from shared memory)
// Tensor memory (512 columns): S_0 [0,128), S_1 [128,256), O_0 [256,384), O_1 [384,512). P_x is
// written by the softmax threads with tcgen05.st as packed 16-bit pairs into the first 64 columns
// of S_x (behind the columns already read), so it never passes through shared memory;
// the next Q_x.K^T is issued behind P_x.V and the tensor pipe executes them in order.
//
// One softmax thread owns one row (TMEM lane = row): it finds the row maximum without any exchange
// with other threads, keeps (m, l) in registers and rescales its O row only when the maximum grows
// by more than 2^8. Warps 0-3 serve row tile 0, warps 4-7 row tile 1; warp 8 produces K, warp 9
// V and Q, warps 10 and 11 issue the MMAs of row tile 0 and 1. An item with at most 128 rows uses
// row tile 0 alone. Every mbarrier wait is bounded; on expiry the CTA records a status, drains and returns.
//
// Reference counterparts: _fwd_kernel_v2 (parrot/engine/builtin/kernels/shared_flash_decoding.py:34-134)
// for the shared prefix, and the gather + xformers FMHA of the Fill path
// (parrot/engine/builtin/attn_func.py:631-675) for causal segments.
#include "common.cuh"
#include "dense_common.cuh"

namespace pb {
namespace {

using namespace dense;

constexpr int kStageBytes = 16384;                       // epilogue staging of one softmax group
constexpr int kOffQ = 0;                                 // Q_0, Q_1
constexpr int kOffK = 2 * kQBytes;
constexpr int kOffV = kOffK + kStages * kRingBytes;
constexpr int kOffStage = kOffV + kStages * kRingBytes;
constexpr int kOffBars = kOffStage + 2 * kStageBytes;
constexpr int kSmemBytes = kOffBars + 512;
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
constexpr int kThreads = 384;                           // 8 softmax warps, K producer, V/Q producer, 2 MMA issuers
constexpr uint32_t kTmemCols = 512;
constexpr int kGroupThreads = 128;                       // softmax threads of one row tile

// barriers 0-7: the K and V rings (dense_common.cuh); per row tile x the index is base + x
enum {
  kBarS = 8,         // S_x of a kv tile is in tensor memory
  kBarP = 10,        // P_x of a kv tile is in tensor memory (all 128 rows)
  kBarPV = 12,       // P_x.V of a kv tile has retired: O_x holds it, S_x / P_x may be overwritten
  kBarQ = 14,        // Q_x of a segment has landed
  kBarQFree = 16,    // every Q_x.K^T of a segment has retired: Q_x may be overwritten
  kBarODrained = 18, // the epilogue of a segment has read O_x out of tensor memory
  kBarGroup = 20,    // meeting point of the 128 softmax threads of row tile x (bounded, unlike bar.sync)
  kBarTurn = 22,     // the warps of row tile x have finished the exponentials of a kv tile (pair items only)
  kNumBars = 24
};


__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}

// Maximum of 32 scores; kMasked: only the first `nvalid` columns count.
template <bool kMasked>
__device__ __forceinline__ float row_max32(const uint32_t* v, int nvalid) {
  float m0 = -INFINITY, m1 = -INFINITY;
  if (!kMasked) {
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      m0 = max3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
      m1 = max3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      m0 = fmaxf(m0, i < nvalid ? __uint_as_float(v[i]) : -INFINITY);
      m1 = fmaxf(m1, i + 1 < nvalid ? __uint_as_float(v[i + 1]) : -INFINITY);
    }
  }
  return fmaxf(m0, m1);
}

// p = 2^(s * scale - m) of 32 scores, packed to 16 words of the model's type; adds them to sum[4].
template <typename T, bool kMasked>
__device__ __forceinline__ void exp_pack32(const uint32_t* v, int nvalid, float scale, float m, float* sum, uint32_t* out) {
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float e0 = fast_exp2(fmaf(__uint_as_float(v[i]), scale, -m));
    float e1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), scale, -m));
    if (kMasked) {
      e0 = (i < nvalid) ? e0 : 0.f;
      e1 = (i + 1 < nvalid) ? e1 : 0.f;
    }
    sum[(i >> 1) & 3] += e0 + e1;
    out[i >> 1] = Pack<T>::two(e0, e1);
  }
}

// State of one softmax thread = one query row: reference maximum and sum (base-2 domain), the
// exact maximum seen.
struct RowState {
  float m_run, l_run, m_true;
};

// The two passes of one softmax thread over its row of S (128 scores in tensor memory, read in
// chunks of 32 columns, the next chunk in flight while one is worked on; the chunk loops are kept
// rolled so that the hot code stays small enough for the instruction cache of a scheduler that
// runs one or two of these warps).
template <bool kMasked>
__device__ __forceinline__ float row_max128(uint32_t tmem_s, int vis) {
  uint32_t a[32], b[32];
  float mx = -INFINITY;
  tmem_ld32(tmem_s, a);
#pragma unroll 1
  for (int c = 0; c < 4; c += 2) {
    tmem_wait_ld();
    tmem_ld32(tmem_s + 32 * (c + 1), b);
    mx = fmaxf(mx, row_max32<kMasked>(a, vis - 32 * c));
    tmem_wait_ld();
    if (c == 0) tmem_ld32(tmem_s + 64, a);
    mx = fmaxf(mx, row_max32<kMasked>(b, vis - 32 * (c + 1)));
  }
  return mx;
}
// P chunk c (tokens [32c, 32c + 32)) goes to columns [16c, 16c + 16) of the row's S columns, which
// the chunks read so far cover; the chunk in flight lies above them. Returns the row sum.
template <typename T, bool kMasked>
__device__ __forceinline__ float row_exp128(uint32_t tmem_s, int vis, float scale, float m) {
  uint32_t a[32], b[32], pk[16];
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
  tmem_ld32(tmem_s, a);
#pragma unroll 1
  for (int c = 0; c < 4; c += 2) {
    tmem_wait_ld();
    tmem_ld32(tmem_s + 32 * (c + 1), b);
    exp_pack32<T, kMasked>(a, vis - 32 * c, scale, m, sum, pk);
    tmem_st16(tmem_s + 16 * c, pk);
    tmem_wait_ld();
    if (c == 0) tmem_ld32(tmem_s + 64, a);
    exp_pack32<T, kMasked>(b, vis - 32 * (c + 1), scale, m, sum, pk);
    tmem_st16(tmem_s + 16 * (c + 1), pk);
  }
  return (sum[0] + sum[1]) + (sum[2] + sum[3]);
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
dense_pair_kernel(const AttnDev d, const __grid_constant__ CUtensorMap vmap, const __grid_constant__ CUtensorMap qmap,
                  const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap omap) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef PB_PAIR_TRACE
  int* trace_ctr = reinterpret_cast<int*>(smem + kOffBars + 256);
  pb_trace(trace_ctr, -1);
#endif
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffBars + kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffBars + kNumBars * 8 + 8);
  int32_t* status = &d.hdr[kHdrStatus];
  const uint32_t bars0 = smem_u32(bars);
  auto bar = [&](int i) { return bars0 + i * 8; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar(kBarFullK + s), 32);  // every thread of the K producer warp arrives
      mbar_init(bar(kBarEmptyK + s), 2);  // one release per MMA issuer
      mbar_init(bar(kBarFullV + s), 1);
      mbar_init(bar(kBarEmptyV + s), 2);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(bar(kBarS + x), 1);
      mbar_init(bar(kBarP + x), kGroupThreads);
      mbar_init(bar(kBarPV + x), 1);
      mbar_init(bar(kBarQ + x), 1);
      mbar_init(bar(kBarQFree + x), 1);
      mbar_init(bar(kBarODrained + x), kGroupThreads);
      mbar_init(bar(kBarGroup + x), kGroupThreads);
      mbar_init(bar(kBarTurn + x), 4);  // one arrival per warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == 11) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // Everything above overlapped the previous kernel in the stream; from here on its results (new
  // KV in the cache, the work lists) are read. Then let the suffix kernel start on the other SMs.
  pdl_wait();
  pdl_trigger();
  const uint32_t tmem_base = *tmem_slot;

  const uint32_t sQ = smem_u32(smem + kOffQ), sK0 = smem_u32(smem + kOffK), sV0 = smem_u32(smem + kOffV);
  // CTAs beyond the planner's share own no tiles and fall straight through to the teardown
  SegmentWalker walk(d, blockIdx.x, min(dense_ctas_of(d), (int)gridDim.x));
  Segment sg;

  if (warp == 8) {
    k_producer<1>(d, walk, 0, lane, sK0, bars0, abort_flag, status);
  } else if (warp == 9) {
    // ============ V producer; also the Q operands of every segment ============
    // Q_x: [2 halves of d][128 rows][128 B], 128-byte swizzle, as eight boxes of 32 rows x 64
    // elements. Rows beyond the batch read as zero; rows beyond the item are other queries whose
    // results are never stored.
    uint32_t tc = 0, segx[2] = {0, 0};
    bool ok = true;
    while (ok && walk.next(sg)) {
      const int nsub = sg.it.nrows > 128 ? 2 : 1;
      for (int x = 0; x < nsub && ok; ++x) {
        if (segx[x] > 0 && !wait_or_abort(bar(kBarQFree + x), (segx[x] - 1) & 1, abort_flag, status, 100)) { ok = false; break; }
        if (lane == 0) {
          mbar_arrive_expect_tx(bar(kBarQ + x), kQBytes);
#pragma unroll
          for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tma_load_q(sQ + x * kQBytes + a * 16384 + j * 4096, &qmap, bar(kBarQ + x), a * 64, sg.head,
                         sg.it.row0 + x * 128 + j * 32);
        }
        ++segx[x];
        __syncwarp();
      }
      if (ok) ok = v_tiles(d, sg, &vmap, lane, sV0, bars0, tc, abort_flag, status);
    }
    if (!ok) {
      // drain: give copies already issued a bounded chance to land before shared memory goes away
      for (uint32_t c = (tc >= 2 ? tc - 2 : 0); c < tc; ++c)
        (void)mbar_wait_bounded(bar(kBarFullV + (c & 1)), (c >> 1) & 1);
      for (int x = 0; x < 2; ++x)
        if (segx[x] > 0) (void)mbar_wait_bounded(bar(kBarQ + x), (segx[x] - 1) & 1);
    }
  } else if (warp == 10 || warp == 11) {
    // ======================= MMA issuer of row tile x =======================
    // A straight chain per kv tile i of a segment:
    //   P_x.V(i)       once P_x(i) is written and V(i) has landed (i = 0: the last epilogue has drained O_x)
    //   Q_x.K^T(i + 1) once K(i + 1) has landed; it overwrites S_x / P_x, and follows P_x.V(i) in this
    //                  thread's program order, which the tensor pipe keeps
    // Two issuers, one per row tile: their chains are independent (disjoint tensor memory) and the
    // instruction stream of one thread cannot feed the pipe for both. A K (V) slot is released by
    // the second of the two commits on it.
    // The operand descriptors are built once; an MMA adds its offset to the address field. (Built per
    // MMA, the descriptor arithmetic of the issuing thread costs more than the MMA itself.)
    //   Q_x: [64-element half][row][128 B], 128-byte swizzle -> SBO 1024 (8-row groups)
    //   K:   [16-byte d chunk][blk][tok][16 B], no swizzle   -> SBO 128 (8-token groups), LBO 2048 (d chunks)
    //   V:   per block [d][16 tok], 32-byte rows, 32-byte swizzle -> SBO 256 (8-row groups)
    //   P_x: tensor memory, lane = row, tokens packed two per column -> block j = columns [8j, 8j + 8)
    const int x = warp - 10;
    constexpr uint32_t kIdescPV = make_idesc(128, kD, Pack<T>::kBf16);
    const uint64_t desc_q = smem_desc(sQ + x * kQBytes, 16, 1024, 2);
    const uint64_t desc_k0 = smem_desc(sK0, 2048, 128, 0), desc_k1 = smem_desc(sK0 + kRingBytes, 2048, 128, 0);
    const uint64_t desc_v0 = smem_desc(sV0, 16, 256, 6), desc_v1 = smem_desc(sV0 + kRingBytes, 16, 256, 6);
    const uint32_t tmem_s = tmem_base + x * 128, tmem_o = tmem_base + 256 + x * 128;
    uint32_t tc = 0, tcx = 0, segx = 0;
    bool ok = true;
    while (ok && walk.next(sg)) {
      const int n = sg.t1 - sg.t0;
      if (x == 1 && sg.it.nrows <= 128) {
        // a lone row tile: nothing to compute here, but every ring slot still takes this issuer's release
        for (int i = 0; i < n && ok; ++i, ++tc) {
          const int s = tc & 1;
          const uint32_t ph = (tc >> 1) & 1;
          if (!wait_or_abort(bar(kBarFullK + s), ph, abort_flag, status, 100)) { ok = false; break; }
          if (lane == 0) mbar_arrive(bar(kBarEmptyK + s));
          if (!wait_or_abort(bar(kBarFullV + s), ph, abort_flag, status, 100)) { ok = false; break; }
          if (lane == 0) mbar_arrive(bar(kBarEmptyV + s));
        }
        continue;
      }
      // S_x = Q_x . K(i)^T (the caller has seen K(i) land); lane 0 only
      auto qk_mmas = [&](int i) {
        const int s = (tc + i) & 1;
        const uint32_t idesc = make_idesc(128, dense_tile_view(d, sg.it, sg.t0 + i).nb * kB, Pack<T>::kBf16);
        const uint64_t bk = s ? desc_k1 : desc_k0;
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)  // a k-step: 32 bytes inside Q's swizzle atom, two d chunks of K
          mma_f16(tmem_s, desc_q + (((kk >> 2) * 16384 + (kk & 3) * 32) >> 4), bk + ((kk * 2 * 2048) >> 4), idesc, kk > 0 ? 1u : 0u);
        mma_commit(bar(kBarS + x));
      };
      auto qk_release = [&](int i) {
        mma_commit(bar(kBarEmptyK + ((tc + i) & 1)));
        if (i == n - 1) mma_commit(bar(kBarQFree + x));
      };
      if (!wait_or_abort(bar(kBarQ + x), segx & 1, abort_flag, status)) { ok = false; break; }
      if (!wait_or_abort(bar(kBarFullK + (tc & 1)), (tc >> 1) & 1, abort_flag, status)) { ok = false; break; }
      fence_proxy_async_smem();  // K was written by per-thread async copies (generic proxy)
      tc_fence_after();
      if (lane == 0) {
        qk_mmas(0);
        qk_release(0);
        PB_TRACE(10 + x);
      }
      __syncwarp();
      for (int i = 0; i < n; ++i) {
        const uint32_t c = tc + i;
        const int s = c & 1;
        const bool more = i + 1 < n;
        // what arrives early first: V(i), K(i + 1), the drained O_x; then P_x(i), which the chain hangs on
        if (!wait_or_abort(bar(kBarFullV + s), (c >> 1) & 1, abort_flag, status)) { ok = false; break; }
        if (more && !wait_or_abort(bar(kBarFullK + (s ^ 1)), ((c + 1) >> 1) & 1, abort_flag, status)) { ok = false; break; }
        if (i == 0 && segx > 0 && !wait_or_abort(bar(kBarODrained + x), (segx - 1) & 1, abort_flag, status)) { ok = false; break; }
        fence_proxy_async_smem();
        if (!wait_or_abort(bar(kBarP + x), (tcx + i) & 1, abort_flag, status)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          PB_TRACE(30 + x);
          const int nb = dense_tile_view(d, sg.it, sg.t0 + i).nb;
          const uint64_t bv = s ? desc_v1 : desc_v0;
#pragma unroll
          for (int j = 0; j < kTileBlocks; ++j)
            if (j < nb) mma_f16_ts(tmem_o, tmem_s + j * 8, bv + j * (kBlkBytes >> 4), kIdescPV, (i > 0 || j > 0) ? 1u : 0u);
          if (more) qk_mmas(i + 1);  // behind P_x.V(i) in the pipe: it overwrites S_x / P_x
          PB_TRACE(32 + x);
          mma_commit(bar(kBarPV + x));
          mma_commit(bar(kBarEmptyV + s));
          if (more) qk_release(i + 1);
          PB_TRACE(20 + x);
        }
        __syncwarp();
      }
      if (!ok) break;
      tc += n;
      tcx += n;
      ++segx;
    }
  } else {
    // ======================= softmax + epilogue: one thread per row =======================
    const int x = warp >> 2;                      // row tile of this thread's group
    const int r = (warp & 3) * 32 + lane;         // row inside the tile = TMEM lane
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem_base + x * 128 + lane_base;
    const uint32_t tmem_o = tmem_base + 256 + x * 128 + lane_base;
    uint8_t* const stage = smem + kOffStage + x * kStageBytes;
    const bool issuer = (r == 0);                 // issues the group's TMA stores
    uint32_t tc = 0, tcx = 0, segx = 0, group_use = 0, pair_tiles = 0;  // pair_tiles: kv tiles of pair items so far
    bool ok = true, store_pending = false;
    auto group_sync = [&]() -> bool {
      mbar_arrive(bar(kBarGroup + x));
      return wait_or_abort(bar(kBarGroup + x), (group_use++) & 1, abort_flag, status);
    };
    // the staging buffer may be written: the TMA store that read it last has done so
    auto stage_begin = [&]() -> bool {
      if (issuer && store_pending) {
        bulk_wait_read();
        store_pending = false;
      }
      return group_sync();
    };
    while (ok && walk.next(sg)) {
      const DnItem& it = sg.it;
      if (x == 1 && it.nrows <= 128) {  // a lone row tile: nothing for this group
        tc += sg.t1 - sg.t0;
        continue;
      }
      const int qrow = x * 128 + r;     // row inside the item
      const bool pair = it.nrows > 128;
      RowState st = {-INFINITY, 0.f, -INFINITY};
      for (int t = sg.t0; t < sg.t1; ++t, ++tc, ++tcx) {
        const int s = tc & 1;
        const DenseTileView tv = dense_tile_view(d, it, t);
        // columns this row may attend: all of the tile's tokens, or (causal tile) the first causal0 + row
        const int vis = tv.causal ? min(tv.ntok, tv.causal0 + qrow) : tv.ntok;
        const bool all_valid = __all_sync(0xffffffffu, vis >= kTileTok);
        if (!wait_or_abort(bar(kBarS + x), tcx & 1, abort_flag, status)) { ok = false; break; }
        tc_fence_after();
        PB_TRACE(1);
        // ---- row maximum ----
        const float mx = (all_valid ? row_max128<false>(tmem_s, vis) : row_max128<true>(tmem_s, vis)) * d.scale_log2e;
        PB_TRACE(2);
        // Lazy reference maximum: the row keeps its reference m_run until a tile exceeds it by more
        // than 2^kTau; P then holds values up to 2^kTau instead of 1, which fp16/bf16 and the fp32
        // accumulators absorb, and O in TMEM is rescaled only on those rare jumps. (m, l, O) stay
        // mutually consistent, which is all the merge needs.
        st.m_true = fmaxf(st.m_true, mx);
        const bool grow = mx > st.m_run + kTau;  // true on the first tile a row sees a token in
        const float alpha = grow ? fast_exp2(st.m_run - mx) : 1.f;
        if (t > sg.t0 && __any_sync(0xffffffffu, grow && st.l_run > 0.f)) {
          // rescale this warp's O rows in TMEM (the previous tile's P.V, which accumulated into
          // them, retired before this tile's S was produced)
          if (!wait_or_abort(bar(kBarPV + x), (tcx - 1) & 1, abort_flag, status)) { ok = false; break; }
          tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < kD; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(tmem_o + c0, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tmem_o + c0, o);
          }
        }
        st.l_run *= alpha;
        st.m_run = grow ? mx : st.m_run;
        // The two row tiles of a pair item take turns at the exponentials (0, 1, 0, 1, ...): that keeps
        // them half a period apart, so that the MMAs of one tile run under the softmax of the other
        // instead of both tiles computing, then both waiting for the tensor pipe.
        if (pair) {
          const bool must_wait = (x == 1) || pair_tiles > 0;
          const uint32_t want = (x == 1) ? pair_tiles : pair_tiles - 1;  // completion of the other tile's turn
          if (must_wait && !wait_or_abort(bar(kBarTurn + (x ^ 1)), want & 1, abort_flag, status)) { ok = false; break; }
        }
        // ---- P = 2^(s - m) into the row's P columns, and the row sum ----
        st.l_run += all_valid ? row_exp128<T, false>(tmem_s, vis, d.scale_log2e, st.m_run)
                              : row_exp128<T, true>(tmem_s, vis, d.scale_log2e, st.m_run);
        if (pair) {
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(kBarTurn + x));
          ++pair_tiles;
        }
        PB_TRACE(3);
        if (tv.ntok & 15) {
          // ragged last block: zero the V columns beyond the length so 0 * (stale bytes) stays 0
          // (both groups do it, each before its own P is announced; row d of the V tile per thread)
          if (!wait_or_abort(bar(kBarFullV + s), (tc >> 1) & 1, abort_flag, status)) { ok = false; break; }
          uint8_t* vt = smem + kOffV + s * kRingBytes + (tv.ntok / 16) * kBlkBytes;
          for (int tk = tv.ntok & 15; tk < 16; ++tk) {
            uint32_t o = (uint32_t)r * 32 + tk * 2;
            o ^= ((o >> 7) & 1u) << 4;  // 32-byte swizzle: 16-byte halves swap in rows 4..7 of every 8
            *reinterpret_cast<uint16_t*>(vt + o) = 0;
          }
          fence_proxy_async_smem();
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar(kBarP + x));
        PB_TRACE(4);
      }
      if (!ok) break;
      // ---- epilogue: O_x rows -> un-normalised partials, or the finished output rows ----
      if (!wait_or_abort(bar(kBarPV + x), (tcx - 1) & 1, abort_flag, status)) { ok = false; break; }
      tc_fence_after();
      const int nrows_x = min(128, it.nrows - x * 128);
      const bool row_ok = r < nrows_x;
      const int row = it.row0 + qrow;
      const size_t slot = partial_slot(d, row_ok ? row : it.row0, dense_part_base(d, it) + sg.part, sg.head);
      // re-base the partial on the exact row maximum; a row that saw no token in this CTA's tiles
      // (causal items) leaves the empty partial (-inf, 0, 0)
      const float fix = (st.m_true == -INFINITY) ? 0.f : fast_exp2(st.m_run - st.m_true);
      // Finished rows: this CTA holds every kv tile of (item, head) and the rows have no other
      // partial, so O / l IS the attention output; it goes out in the model's type and the merge
      // skips these rows (same test on its side: one dense partial, no suffix, the item's flag).
      const bool direct = dense_direct_ok(d, it) && sg.t0 == 0 && sg.t1 == it.nt;
      const bool by_tma = (nrows_x == 128) && d.acc_tma;
      if (direct) {
        const float inv = (st.l_run > 0.f) ? 1.f / st.l_run : 0.f;
        T* orow = reinterpret_cast<T*>(d.out) + (size_t)(row_ok ? row : it.row0) * d.out_stride + (size_t)sg.head * kD;
#pragma unroll 1
        for (int c0 = 0; c0 < kD; c0 += 64) {
          uint32_t v[64];
          tmem_ld32(tmem_o + c0, v);
          tmem_ld32(tmem_o + c0 + 32, v + 32);
          tmem_wait_ld();
          uint32_t h[32];
#pragma unroll
          for (int i = 0; i < 32; ++i)
            h[i] = Pack<T>::two(__uint_as_float(v[2 * i]) * inv, __uint_as_float(v[2 * i + 1]) * inv);
          if (by_tma) {
            // staging: [128 rows][128 B], 16-byte chunks swizzled by the row; one tiled store per half
            if (!stage_begin()) { ok = false; break; }
            uint8_t* rowp = stage + r * 128;
#pragma unroll
            for (int i = 0; i < 8; ++i)
              *reinterpret_cast<uint4*>(rowp + ((i ^ (r & 7)) << 4)) = make_uint4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
            fence_proxy_async_smem();
            if (!group_sync()) { ok = false; break; }
            if (issuer) {
              tma_store_out(&omap, smem_u32(stage), c0, sg.head, it.row0 + x * 128);
              bulk_commit_group();
              store_pending = true;
            }
          } else if (row_ok) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              *reinterpret_cast<uint4*>(orow + c0 + 8 * i) = make_uint4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
          }
        }
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < kD; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_o + c0, v);
          tmem_wait_ld();
          if (by_tma) {
            // Full row tile: its 128 partial rows are contiguous in the workspace. Staged as
            // [128 rows][32 floats] in the 128-byte-swizzled layout and written by one tiled store;
            // a thread's own stores would touch 32 separate lines per instruction.
            if (!stage_begin()) { ok = false; break; }
            uint8_t* rowp = stage + r * 128;
#pragma unroll
            for (int i = 0; i < 8; ++i)
              *reinterpret_cast<float4*>(rowp + ((i ^ (r & 7)) << 4)) =
                  make_float4(__uint_as_float(v[4 * i]) * fix, __uint_as_float(v[4 * i + 1]) * fix,
                              __uint_as_float(v[4 * i + 2]) * fix, __uint_as_float(v[4 * i + 3]) * fix);
            fence_proxy_async_smem();
            if (!group_sync()) { ok = false; break; }
            if (issuer) {
              const size_t slot0 = partial_slot(d, it.row0 + x * 128, dense_part_base(d, it) + sg.part, sg.head);
              tma_store_acc(&amap, smem_u32(stage), c0, (int)slot0);
              bulk_commit_group();
              store_pending = true;
            }
          } else if (row_ok) {
            float4* dst = reinterpret_cast<float4*>(d.acc + slot * kD + c0);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              dst[i] = make_float4(__uint_as_float(v[4 * i]) * fix, __uint_as_float(v[4 * i + 1]) * fix,
                                   __uint_as_float(v[4 * i + 2]) * fix, __uint_as_float(v[4 * i + 3]) * fix);
          }
        }
        if (ok && row_ok) d.ml[slot] = make_float2(st.m_true, st.l_run * fix);
      }
      if (!ok) break;
      tc_fence_before();
      mbar_arrive(bar(kBarODrained + x));
      PB_TRACE(5);
      ++segx;
    }
    if (issuer) bulk_wait_all();  // stores of the last segment have left shared memory and landed
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 11) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

#ifdef PB_PAIR_TRACE
extern "C" int pb_debug_trace_read(void* dst, size_t bytes) {
  return (int)cudaMemcpyFromSymbol(dst, dense::g_trace, bytes < sizeof(dense::g_trace) ? bytes : sizeof(dense::g_trace));
}
#endif

cudaError_t launch_dense_pair(const AttnDev& d, int dtype, const CUtensorMap& vmap, const CUtensorMap& qmap,
                              const CUtensorMap& amap, const CUtensorMap& omap, cudaStream_t s) {
  cudaError_t e;
  if (dtype == PB_F16) {
    auto kfn = dense_pair_kernel<__half>;
    e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    e = launch_kernel(kfn, d.num_sms, kThreads, kSmemBytes, s, true, d, vmap, qmap, amap, omap);
  } else {
    auto kfn = dense_pair_kernel<__nv_bfloat16>;
    e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    e = launch_kernel(kfn, d.num_sms, kThreads, kSmemBytes, s, true, d, vmap, qmap, amap, omap);
  }
  return e;
}

}  // namespace pb
