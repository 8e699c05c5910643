// Dense shared-prefix stage on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// One work item = (tile of up to 128 query rows of one prefix group, head, chunk of the group's
// prefix). All rows of the tile attend to the SAME keys, so the chunk's K/V is read from HBM
// once and both contractions run as MMAs:
//     S[128 x 128] = Q[128 x D] . K^T          (N = 128 tokens = 8 physical blocks, 8 K-steps)
//     O[128 x D]  += P[128 x 128] . V          (per 16-token physical block: K = 16)
// Operand layouts come straight from the paged cache:
//   * a K tile [D/8][16 tok][8] is already made of canonical no-swizzle K-major core matrices
//     (8 tokens x 16 bytes contiguous); its 16 d-chunk rows (256 B) are copied to
//     [d chunk][block][256 B] with per-thread 16-byte async copies, which gives the 8 blocks of
//     a kv tile ONE uniform operand layout (bulk copies of 256 B proved request-rate bound);
//   * a V tile [D][16 tok] has 32-byte rows: it is fetched through a TMA tensor map with the
//     32-byte swizzle, which is the K-major SWIZZLE_32B operand layout.
//   * Q rows come through a TMA tensor map over [rows, heads, D] as 32-row x 64-element boxes in
//     the 128-byte-swizzled K-major layout, loaded by the V producer warp as soon as the previous
//     segment's last Q.K^T has retired.
// S and O accumulate in TMEM (fp32); the 256 softmax threads (two per row and column half) keep
// the running max/sum in registers, write P to shared memory as the next A operand and rescale
// O in TMEM only when a row maximum grows by more than 2^8. Un-normalised partials go to the
// workspace (full row tiles through shared memory and TMA tiled stores); a CTA that holds every
// kv tile of a (row tile, head) whose rows have no other partial writes the normalised output
// itself.
//
// Work is cut "stream-K" style: all (item, head, 128-token kv tile) triples form one global
// order and every CTA takes an equal contiguous share, so CTAs finish together and a head whose
// tiles span several CTAs yields one partial per CTA. S is double-buffered in TMEM, so the
// Q.K^T of tile t+1 runs while the softmax threads work on tile t.
//
// Warp roles: warps 0-7 softmax/epilogue (TMEM lane = row; warps w and w+4 share a lane quarter and
// split the columns), warps 8-9 K producers, warp 10 V producer, warp 11 MMA issuer.
// Every mbarrier wait is bounded; on expiry the CTA records a status, drains and returns.
//
// The same kernel runs prefill: a causal item is a tile of up to 128 NEW tokens of one request over
// that request's private context; row i of the tile then sees the first causal_base + i tokens
// (bottom-right aligned causal mask), which only changes the column mask of the softmax threads.
// A request inside a prefix group is a two-piece item: the kv tiles of the group's prefix first,
// then those of its own context (dense_tile_view in common.cuh says what each tile covers).
// It replaces the gather + xformers FMHA of the reference's Fill path
// (parrot/engine/builtin/attn_func.py:631-675).
//
// Reference counterpart: _fwd_kernel_v2 (parrot/engine/builtin/kernels/shared_flash_decoding.py:34-134),
// a Triton kernel with compiler-chosen mma that re-reads the prefix once per 16..128-row tile
// and gathers K through a pointer tensor.
#include <cuda.h>
#include <string.h>

#include "common.cuh"
#include "dense_common.cuh"

namespace pb {
namespace {

using namespace dense;

constexpr int kPBytes = 128 * kTileTok * 2;     // 32 KiB
constexpr int kOffQ = 0, kOffP = kQBytes, kOffK = kQBytes + 2 * kPBytes, kOffV = kOffK + kStages * kRingBytes;
constexpr int kOffBars = kOffV + kStages * kRingBytes;
constexpr int kOffLsum = kOffBars + 256;            // first exchange buffer (row maxima per tile, row sums per segment)
constexpr int kOffPmax = kOffLsum + 1024;           // second exchange buffer ([2 halves][128 rows] floats each)
constexpr int kSmemBytes = kOffPmax + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
constexpr int kSoftmaxThreads = 256;            // warps 0-7: two column halves x four TMEM lane quarters
constexpr int kThreads = 384;                   // + warps 8, 9: K producers, warp 10: V producer, warp 11: MMA issuer
constexpr uint32_t kTmemCols = 512;             // S0: [0,128)  S1: [128,256)  O: [256,384)

enum {
  // barriers 0-7: the K and V rings (dense_common.cuh)
  kBarS = 8, kBarP = 10, kBarQ = 12, kBarO = 13,
  kBarX = 14, kBarY = 15,  // exchange points of the softmax threads (bounded, unlike bar.sync)
  kBarQFree = 16,         // every Q.K^T of a segment has retired: the Q operand may be overwritten
  kNumBars = 17
};

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
dense_prefix_kernel(const AttnDev d, const __grid_constant__ CUtensorMap vmap, const __grid_constant__ CUtensorMap qmap,
                    const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap omap) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef PB_PAIR_TRACE
  int* trace_ctr = reinterpret_cast<int*>(smem + kOffBars + 200);
  pb_trace(trace_ctr, -1);
#endif
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffBars + kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffBars + kNumBars * 8 + 8);
  int32_t* status = &d.hdr[kHdrStatus];
  auto bar = [&](int i) { return smem_u32(&bars[i]); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar(kBarFullK + s), 64);  // every thread of the two K producer warps arrives
      mbar_init(bar(kBarEmptyK + s), 1);
      mbar_init(bar(kBarFullV + s), 1);
      mbar_init(bar(kBarEmptyV + s), 1);
      mbar_init(bar(kBarS + s), 1);
      mbar_init(bar(kBarP + s), kSoftmaxThreads);
    }
    mbar_init(bar(kBarQ), 1);
    mbar_init(bar(kBarQFree), 1);
    mbar_init(bar(kBarO), 1);
    mbar_init(bar(kBarX), kSoftmaxThreads);
    mbar_init(bar(kBarY), kSoftmaxThreads);
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
  const uint32_t tmem_o = tmem_base + 256;

  const uint32_t sQ = smem_u32(smem + kOffQ), sP = smem_u32(smem + kOffP);
  auto sK = [&](int s) { return smem_u32(smem + kOffK + s * kRingBytes); };
  auto sV = [&](int s) { return smem_u32(smem + kOffV + s * kRingBytes); };
  // CTAs beyond the planner's share own no tiles and fall straight through to the teardown
  SegmentWalker walk(d, blockIdx.x, min(dense_ctas_of(d), (int)gridDim.x));
  Segment sg;

  if (warp == 8 || warp == 9) {
    // ============ K producers (2 warps): per-thread 16-byte async copies with re-pack ============
    // The 256-byte row of d-chunk c of block j goes to [c][j][16 tok][16 B]: the 8-token groups of
    // ALL blocks of the tile then sit 128 bytes apart and one MMA spans the whole tile. A warp
    // instruction moves 512 contiguous source bytes (two chunk rows). Each thread signals the
    // slot's mbarrier when its own copies have landed (cp.async.mbarrier.arrive.noinc).
    const int pw = warp - 8;
    const uint8_t* kc = reinterpret_cast<const uint8_t*>(d.key_cache);
    uint32_t tc = 0;
    bool ok = true;
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
        if (!wait_or_abort(bar(kBarEmptyK + s), ph ^ 1, abort_flag, status, 100)) { ok = false; break; }
        for (int j = pw; j < kTileBlocks; j += 2) {
          const int bj = __shfl_sync(0xffffffffu, blk, j);
          if (j < nb) {
            const uint8_t* src = kc + ((size_t)bj * d.kv_block_stride + (size_t)kvh * d.kv_head_stride) * 2 + lane * 16;
            const uint32_t dst = sK(s) + (lane >> 4) * (kTileBlocks * 256) + j * 256 + (lane & 15) * 16;
#pragma unroll
            for (int k = 0; k < 8; ++k)
              cp_async16(dst + k * 2 * (kTileBlocks * 256), src + k * 512);
          }
        }
        cp_async_arrive_noinc(bar(kBarFullK + s));
      }
    }
    cp_async_wait_all();
  } else if (warp == 10) {
    // ============ V producer: TMA tiled loads with the 32-byte swizzle ============
    uint32_t tc = 0, seg_idx = 0;
    bool ok = true;
    while (ok && walk.next(sg)) {
      const int kvh = d.head_mapping ? d.head_mapping[sg.head] : sg.head;
      // ---- Q operand of the segment: [2 halves of d][128 rows][128 B], 128-byte swizzle, as eight
      //      boxes of 32 rows x 64 elements. With at most 64 (32) query rows the boxes repeat, so the
      //      rows appear twice (four times) in the operand. Rows beyond the batch read as zero; rows
      //      beyond the item are other queries whose results are never stored. ----
      if (seg_idx > 0 && !wait_or_abort(bar(kBarQFree), (seg_idx - 1) & 1, abort_flag, status, 100)) { ok = false; break; }
      if (lane == 0) {
        const int rows_per = (sg.it.nrows <= 32) ? 32 : (sg.it.nrows <= 64) ? 64 : 128;
        mbar_arrive_expect_tx(bar(kBarQ), kQBytes);
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            tma_load_q(sQ + a * 16384 + j * 4096, &qmap, bar(kBarQ), a * 64, sg.head, sg.it.row0 + ((j * 32) & (rows_per - 1)));
      }
      ++seg_idx;
      __syncwarp();

      // The two-slot rings hide little latency when the single-query kernel saturates HBM beside
      // this one: ask L2 for the K and V tiles of the blocks kPrefetchTiles tiles ahead (lane j:
      // block j of the tile; K in the lower half-warp, V in the upper).
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
        if (!wait_or_abort(bar(kBarEmptyV + s), ph ^ 1, abort_flag, status, 100)) { ok = false; break; }
        if (lane == 0) mbar_arrive_expect_tx(bar(kBarFullV + s), nb * kBlkBytes);
        __syncwarp();
        for (int j = 0; j < nb; ++j) {
          const int bj = __shfl_sync(0xffffffffu, blk, j);
          if (lane == 0) tma_load_v(sV(s) + j * kBlkBytes, &vmap, bar(kBarFullV + s), kvh, bj);
        }
      }
    }
    if (!ok && (tc > 0 || seg_idx > 0)) {
      // drain: give copies already issued a bounded chance to land before shared memory goes away
      for (uint32_t c = (tc >= 2 ? tc - 2 : 0); c < tc; ++c)
        (void)mbar_wait_bounded(bar(kBarFullV + (c & 1)), (c >> 1) & 1);
      if (seg_idx > 0) (void)mbar_wait_bounded(bar(kBarQ), (seg_idx - 1) & 1);
    }
  } else if (warp == 11) {
    // ======================= MMA issuer =======================
    // Polls two independent conditions so neither contraction waits behind the other's inputs:
    //   K(next) landed              -> issue S(next) = Q.K^T   (at most one tile ahead of P.V)
    //   P(cur) written, V(cur) here -> issue O += P.V
    constexpr uint32_t kIdescPV = make_idesc(128, kD, Pack<T>::kBf16);
    uint32_t tc0 = 0, seg_ctr = 0;
    bool ok = true;
    while (ok && walk.next(sg)) {
      const int n = sg.t1 - sg.t0;
      auto nb_of = [&](int i) { return dense_tile_view(d, sg.it, sg.t0 + i).nb; };
      if (!wait_or_abort(bar(kBarQ), seg_ctr & 1, abort_flag, status)) { ok = false; break; }
      tc_fence_after();
      int qk_next = 0, pv_next = 0;
      uint64_t t_start = 0;
      uint32_t spin = 0;
      while (pv_next < n) {
        bool progress = false;
        if (qk_next < n && qk_next <= pv_next + 1) {
          const uint32_t c = tc0 + qk_next;
          bool ready = mbar_test_wait(bar(kBarFullK + (c & 1)), (c >> 1) & 1);
          ready = __all_sync(0xffffffffu, ready);
          if (ready) {
            fence_proxy_async_smem();  // K was written by per-thread async copies (generic proxy)
            tc_fence_after();
            if (lane == 0) {
              const int s = c & 1;
              const uint32_t idesc = make_idesc(128, nb_of(qk_next) * kB, Pack<T>::kBf16);
#pragma unroll
              for (int kk = 0; kk < kD / 16; ++kk) {
                // Q: [64-element half][row][128 B], 128-byte swizzle -> SBO 1024 (8-row groups); a k-step
                //    of 16 elements is 32 bytes further inside the swizzle atom
                // K: [16-byte d chunk][blk][tok][16 B]  -> SBO 128 (8-token groups), LBO 2048 (d chunks)
                const uint64_t a = smem_desc(sQ + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024, 2);
                const uint64_t b = smem_desc(sK(s) + kk * 2 * 2048, 2048, 128, 0);
                mma_f16(tmem_base + s * 128, a, b, idesc, kk > 0 ? 1u : 0u);
              }
              mma_commit(bar(kBarS + s));
              mma_commit(bar(kBarEmptyK + s));
              PB_TRACE(10);
              if (qk_next == n - 1) mma_commit(bar(kBarQFree));
            }
            __syncwarp();
            ++qk_next;
            progress = true;
          }
        }
        if (pv_next < qk_next) {
          const uint32_t c = tc0 + pv_next;
          const int s = c & 1;
          const uint32_t ph = (c >> 1) & 1;
          bool ready = mbar_test_wait(bar(kBarP + s), ph) && mbar_test_wait(bar(kBarFullV + s), ph);
          ready = __all_sync(0xffffffffu, ready);
          if (ready) {
            tc_fence_after();
            if (lane == 0) {
              const int nb = nb_of(pv_next);
              for (int j = 0; j < nb; ++j) {
                // P: [8-token chunk][row][16 B] -> SBO 128, LBO 2048; block j = chunks 2j, 2j+1
                const uint64_t a = smem_desc(sP + s * kPBytes + j * 2 * 2048, 2048, 128, 0);
                // V tile: [d][16 tok] 32-byte rows, 32-byte swizzle -> SBO 256 (8-row groups)
                const uint64_t b = smem_desc(sV(s) + j * kBlkBytes, 16, 256, 6);
                mma_f16(tmem_o, a, b, kIdescPV, (pv_next > 0 || j > 0) ? 1u : 0u);
              }
              mma_commit(bar(kBarEmptyV + s));
              if (pv_next == n - 1) mma_commit(bar(kBarO));
              PB_TRACE(20);
            }
            __syncwarp();
            ++pv_next;
            progress = true;
          }
        }
        if (progress) {
          spin = 0;
          t_start = 0;
        } else if (__nanosleep(40), (++spin & 255u) == 0) {
          bool give_up = (*abort_flag != 0);
          const uint64_t now = global_timer_ns();
          if (t_start == 0) t_start = now;
          else if (now - t_start > 2000000000ull) give_up = true;
          if (__any_sync(0xffffffffu, give_up)) {
            *abort_flag = 1;
            atomicMax(status, kStatusWaitExpired);
            ok = false;
            break;
          }
        }
      }
      tc0 += n;
      ++seg_ctr;
    }
  } else {
    // ======================= softmax + epilogue =======================
    // 256 threads. Thread (r, ch): TMEM lane r = (warp & 3) * 32 + lane, column half ch = warp >> 2.
    // With at most 64 (32) query rows in the tile the rows are loaded twice (four times) into the
    // 128-row Q operand, so lanes r, r + 64 (r + 32, ...) hold the same S row and split its columns
    // further: a row's exponentials are shared by 2, 4 or 8 threads on different schedulers.
    const int r = (warp & 3) * 32 + lane;
    const int ch = warp >> 2;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    // two exchange buffers of [2 halves][128 rows] floats, used alternately by the tiles (row
    // maxima) and, at the end of a segment, the one the last tile did not use (row sums)
    float* const xbuf[2] = {reinterpret_cast<float*>(smem + kOffPmax), reinterpret_cast<float*>(smem + kOffLsum)};
    uint32_t tc = 0, seg_ctr = 0, x_use = 0, y_use = 0;
    bool ok = true, store_pending = false;
    // barrier among the 256 softmax threads; bounded like every other wait of this kernel
    auto sync_x = [&]() -> bool {
      mbar_arrive(bar(kBarX));
      return wait_or_abort(bar(kBarX), (x_use++) & 1, abort_flag, status);
    };
    auto sync_y = [&]() -> bool {
      mbar_arrive(bar(kBarY));
      return wait_or_abort(bar(kBarY), (y_use++) & 1, abort_flag, status);
    };
    Segment sg_next;
    bool have = walk.next(sg);
    while (ok && have) {
      const bool have_next = walk.next(sg_next);
      const DnItem& it = sg.it;
      const int dup_log = (it.nrows <= 32) ? 2 : (it.nrows <= 64) ? 1 : 0;
      const int rows_per = 128 >> dup_log;         // distinct query rows in the operand
      const int qrow = r & (rows_per - 1);         // the query row this lane computes
      const int part = r >> (7 - dup_log);         // which share of the half's columns (warp-uniform)
      const int gshift = 3 - dup_log;              // 16-byte P chunks per share = 1 << gshift
      const bool owner = (ch == 0 && part == 0);   // the thread that owns the row's O and (m, l)
      float m_run = -INFINITY, l_run = 0.f, m_true = -INFINITY;
      for (int t = sg.t0; t < sg.t1; ++t, ++tc) {
        const int s = tc & 1;
        const uint32_t ph = (tc >> 1) & 1;
        const uint32_t tmem_s = tmem_base + s * 128 + ch * 64;
        const DenseTileView tv = dense_tile_view(d, it, t);
        const int ntok_tile = tv.ntok;  // tokens of the item in this tile
        // columns this row may attend: all of them, or (causal tile) the first causal0 + row
        const int vis = tv.causal ? min(ntok_tile, tv.causal0 + qrow) : ntok_tile;
        const int ntok = vis - ch * 64;  // valid columns of this half (may be <= 0)
        if (!wait_or_abort(bar(kBarS + s), ph, abort_flag, status)) { ok = false; break; }
        tc_fence_after();
        PB_TRACE(1);
        // this half of the S row (64 fp32) in registers: two back-to-back TMEM loads, one wait
        uint32_t v[64];
        tmem_ld32(tmem_s + lane_base + 0, v);
        tmem_ld32(tmem_s + lane_base + 32, v + 32);
        tmem_wait_ld();
        // four independent chains: a single running maximum would be 64 dependent operations
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (ntok >= 64) {
#pragma unroll
          for (int i = 0; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (i < ntok) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // row maximum = max of the two halves, exchanged through shared memory
        if (store_pending) {  // the previous segment's partials are still being read out of the P buffers
          bulk_wait_read();
          store_pending = false;
        }
        // (the next tile writes the other buffer, whose readers all passed this tile's barrier)
        float* pmax = xbuf[tc & 1];
        pmax[ch * 128 + r] = mx;
        PB_TRACE(2);
        if (!sync_x()) { ok = false; break; }
        PB_TRACE(3);
        mx = fmaxf(mx, pmax[(ch ^ 1) * 128 + r]);
        // Lazy reference maximum: the row keeps its reference m_run until a tile exceeds it by more
        // than 2^kTau; P then holds values up to 2^kTau instead of 1, which fp16/bf16 and the fp32
        // accumulators absorb, and O in TMEM is rescaled only on those rare jumps. (m, l, O) stay
        // mutually consistent, which is all the merge needs.
        const float m_cand = mx * d.scale_log2e;
        m_true = fmaxf(m_true, m_cand);
        const bool grow = m_cand > m_run + kTau;  // always true on a row's first tile (m_run = -inf)
        const float m_new = grow ? m_cand : m_run;
        const float alpha = grow ? fast_exp2(m_run - m_new) : 1.f;
        if (t > sg.t0 && owner && __any_sync(0xffffffffu, grow)) {
          // rescale the O rows of this warp in TMEM, once the previous tile's P.V (which
          // accumulates into them) has retired
          if (!wait_or_abort(bar(kBarEmptyV + ((tc - 1) & 1)), ((tc - 1) >> 1) & 1, abort_flag, status)) { ok = false; break; }
          tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < kD; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(tmem_o + lane_base + c0, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tmem_o + lane_base + c0, o);
          }
          tmem_wait_st();
        }
        l_run *= alpha;
        m_run = m_new;
        // P = 2^(s - m) for this thread's share of the columns, row sum, P -> shared memory as the
        // A operand of P.V (buffer tile & 1; its previous reader, P.V of tile - 2, retired before
        // this tile's S could be produced)
        float lsum4[4] = {0.f, 0.f, 0.f, 0.f};
        uint8_t* prow = smem + kOffP + s * kPBytes + (ch * 8) * 2048 + qrow * 16;
        if (ntok >= 64) {
          // every column of this half is visible (all tiles but an item's last and the causal ones):
          // no per-column test; the exponentials section is bound by instruction issue, not by the
          // special-function unit
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            if ((g >> gshift) == part) {
              float p[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                p[i] = fast_exp2(fmaf(__uint_as_float(v[g * 8 + i]), d.scale_log2e, -m_run));
                lsum4[i & 3] += p[i];
              }
              uint4 w;
              w.x = Pack<T>::two(p[0], p[1]);
              w.y = Pack<T>::two(p[2], p[3]);
              w.z = Pack<T>::two(p[4], p[5]);
              w.w = Pack<T>::two(p[6], p[7]);
              *reinterpret_cast<uint4*>(prow + g * 2048) = w;
            }
          }
        } else {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            if ((g >> gshift) == part) {
              float p[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float e = fast_exp2(fmaf(__uint_as_float(v[g * 8 + i]), d.scale_log2e, -m_run));
                p[i] = (g * 8 + i < ntok) ? e : 0.f;
                lsum4[i & 3] += p[i];
              }
              uint4 w;
              w.x = Pack<T>::two(p[0], p[1]);
              w.y = Pack<T>::two(p[2], p[3]);
              w.z = Pack<T>::two(p[4], p[5]);
              w.w = Pack<T>::two(p[6], p[7]);
              *reinterpret_cast<uint4*>(prow + g * 2048) = w;
            }
          }
        }
        l_run += (lsum4[0] + lsum4[1]) + (lsum4[2] + lsum4[3]);
        PB_TRACE(4);
        if ((ntok_tile & 15) && ch == 0) {
          // ragged last block: zero the V columns beyond the length so 0 * (stale bytes) stays 0
          if (!wait_or_abort(bar(kBarFullV + s), ph, abort_flag, status)) { ok = false; break; }
          const int j = ntok_tile / 16;
          uint8_t* vt = smem + kOffV + s * kRingBytes + j * kBlkBytes;
          for (int tk = ntok_tile & 15; tk < 16; ++tk) {
            uint32_t o = (uint32_t)r * 32 + tk * 2;
            o ^= ((o >> 7) & 1u) << 4;  // 32-byte swizzle: 16-byte halves swap in rows 4..7 of every 8
            *reinterpret_cast<uint16_t*>(vt + o) = 0;
          }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(bar(kBarP + s));
        PB_TRACE(5);
      }
      if (!ok) break;
      // ---- row sums of the helper threads -> the thread that owns the row ----
      float* lsh = xbuf[tc & 1];  // not the buffer of the segment's last tile
      if (!owner) lsh[ch * 128 + r] = l_run;
      if (!sync_x()) { ok = false; break; }
      if (owner) {
        for (int k = 0; k < (1 << dup_log); ++k) {
          if (k > 0) l_run += lsh[r + k * rows_per];
          l_run += lsh[128 + r + k * rows_per];
        }
      }
      if (!sync_y()) { ok = false; break; }
      // ---- epilogue: O rows -> un-normalised partials (each column half by one thread) ----
      if (!wait_or_abort(bar(kBarO), seg_ctr & 1, abort_flag, status)) { ok = false; break; }
      tc_fence_after();
      const size_t slot = partial_slot(d, it.row0 + r, dense_part_base(d, it) + sg.part, sg.head);
      // re-base the partial on the exact row maximum; a row that saw no token in this CTA's tiles
      // (causal items) leaves the empty partial (-inf, 0, 0)
      const float fix = (m_true == -INFINITY) ? 0.f : fast_exp2(m_run - m_true);
      // Finished rows: this CTA holds every kv tile of (item, head) and the rows have no other
      // partial, so O / l IS the attention output; it goes out in the model's type and the merge
      // skips these rows (same test on its side: one dense partial, no suffix, the item's flag).
      const bool direct = dense_direct_ok(d, it) && sg.t0 == 0 && sg.t1 == it.nt;
      if (direct) {
        // the row sum lives with the row's owner: hand it to the thread of the other column half
        if (owner) lsh[r] = l_run;
        if (!sync_x()) { ok = false; break; }
        const float l_row = lsh[r];
        const float inv = (l_row > 0.f) ? 1.f / l_row : 0.f;
        const bool full = (it.nrows == 128) && d.acc_tma;
        T* orow = reinterpret_cast<T*>(d.out) + (size_t)(it.row0 + r) * d.out_stride + (size_t)sg.head * kD + ch * 64;
#pragma unroll 1
        for (int c0 = 0; c0 < 64; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_o + lane_base + ch * 64 + c0, v);
          tmem_wait_ld();
          uint32_t h[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            h[i] = Pack<T>::two(__uint_as_float(v[2 * i]) * inv, __uint_as_float(v[2 * i + 1]) * inv);
          if (full) {
            // staging: [column half ch][128 rows][128 B], 16-byte chunks swizzled by the row
            uint8_t* rowp = smem + kOffP + ch * 16384 + r * 128;
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<uint4*>(rowp + ((((c0 >> 3) + i) ^ (r & 7)) << 4)) =
                  make_uint4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
          } else if (r < it.nrows) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<uint4*>(orow + c0 + 8 * i) = make_uint4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
          }
        }
        if (full) {
          fence_proxy_async_smem();
          if (!sync_y()) { ok = false; break; }
          if (threadIdx.x == 0) {
            tma_store_out(&omap, smem_u32(smem + kOffP), 0, sg.head, it.row0);
            tma_store_out(&omap, smem_u32(smem + kOffP + 16384), 64, sg.head, it.row0);
            bulk_commit_group();
            store_pending = true;
          }
        } else if (!sync_y()) { ok = false; break; }  // keeps the two exchange barriers in step
      } else if (it.nrows == 128 && d.acc_tma) {
        // Full row tile: its 128 partial rows are contiguous in the workspace. Stage them in the P
        // buffers (free: every P.V of the segment has retired) in the 128-byte-swizzled layout, four
        // column groups of [128 rows][32 floats], and let TMA write each group with one tiled store;
        // a thread's own stores would touch 32 separate lines per instruction.
#pragma unroll 1
        for (int c0 = ch * 64; c0 < ch * 64 + 64; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_o + lane_base + c0, v);
          tmem_wait_ld();
          uint8_t* rowp = smem + kOffP + (c0 >> 5) * 16384 + r * 128;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(rowp + ((i ^ (r & 7)) << 4)) =
                make_float4(__uint_as_float(v[4 * i]) * fix, __uint_as_float(v[4 * i + 1]) * fix,
                            __uint_as_float(v[4 * i + 2]) * fix, __uint_as_float(v[4 * i + 3]) * fix);
        }
        fence_proxy_async_smem();
        if (!sync_x()) { ok = false; break; }
        if (threadIdx.x == 0) {
          const size_t slot0 = partial_slot(d, it.row0, dense_part_base(d, it) + sg.part, sg.head);
#pragma unroll
          for (int g = 0; g < 4; ++g) tma_store_acc(&amap, smem_u32(smem + kOffP + g * 16384), g * 32, (int)slot0);
          bulk_commit_group();
          store_pending = true;
        }
      } else {
#pragma unroll 1
        for (int c0 = ch * 64; c0 < ch * 64 + 64; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_o + lane_base + c0, v);
          tmem_wait_ld();
          if (r < it.nrows) {
            float4* dst = reinterpret_cast<float4*>(d.acc + slot * kD + c0);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              dst[i] = make_float4(__uint_as_float(v[4 * i]) * fix, __uint_as_float(v[4 * i + 1]) * fix,
                                   __uint_as_float(v[4 * i + 2]) * fix, __uint_as_float(v[4 * i + 3]) * fix);
          }
        }
      }
      if (!direct && r < it.nrows && ch == 0) d.ml[slot] = make_float2(m_true, l_run * fix);
      tc_fence_before();
      ++seg_ctr;
      sg = sg_next;
      have = have_next;
    }
    if (threadIdx.x == 0) bulk_wait_all();  // stores of the last segment have left shared memory and landed
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 11) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// cuTensorMapEncodeTiled is a pure function of its arguments; a layer call needs four maps and a
// model runs the same shapes over a handful of buffers layer after layer, so the encoded maps of
// the last calls of this thread are kept and looked up by their arguments.
struct MapKey {
  int type, rank, swizzle, promo;
  const void* base;
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4];
};
struct MapSlot { MapKey key; CUtensorMap map; bool used; };
constexpr int kMapSlots = 64;

CUresult encode_cached(EncodeTiledFn enc, CUtensorMap* out, CUtensorMapDataType type, int rank, const void* base,
                       const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box,
                       CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promo) {
  thread_local MapSlot slots[kMapSlots] = {};
  thread_local int next = 0;
  MapKey k;
  memset(&k, 0, sizeof(k));
  k.type = (int)type; k.rank = rank; k.swizzle = (int)swizzle; k.promo = (int)promo; k.base = base;
  for (int i = 0; i < rank; ++i) { k.dims[i] = dims[i]; k.box[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) k.strides[i] = strides[i];
  for (int i = 0; i < kMapSlots; ++i)
    if (slots[i].used && memcmp(&slots[i].key, &k, sizeof(k)) == 0) { *out = slots[i].map; return CUDA_SUCCESS; }
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(out, type, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) {
    MapSlot& sl = slots[next];
    next = (next + 1) % kMapSlots;
    sl.key = k; sl.map = *out; sl.used = true;
  }
  return r;
}

}  // namespace

#ifdef PB_PAIR_TRACE
extern "C" int pb_debug_trace_read_single(void* dst, size_t bytes) {
  return (int)cudaMemcpyFromSymbol(dst, dense::g_trace, bytes < sizeof(dense::g_trace) ? bytes : sizeof(dense::g_trace));
}
#endif

bool dense_prefix_supported(int dtype, int head_size, int block_size) {
  return (dtype == PB_F16 || dtype == PB_BF16) && head_size == kD && block_size == kB;
}

cudaError_t launch_dense_prefix(const AttnDev& d, int dtype, int head_size, int block_size, cudaStream_t s) {
  if (!dense_prefix_supported(dtype, head_size, block_size)) return cudaErrorInvalidValue;
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return cudaErrorNotSupported;
  CUtensorMap vmap;
  const cuuint64_t dims[4] = {(cuuint64_t)kB, (cuuint64_t)kD, (cuuint64_t)d.num_kv_heads, (cuuint64_t)d.num_blocks};
  const cuuint64_t strides[3] = {(cuuint64_t)kB * 2, (cuuint64_t)d.kv_head_stride * 2, (cuuint64_t)d.kv_block_stride * 2};
  const cuuint32_t box[4] = {(cuuint32_t)kB, (cuuint32_t)kD, 1, 1};
  const CUtensorMapDataType elem = dtype == PB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUresult r = encode_cached(enc, &vmap, elem, 4, d.value_cache, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_32B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  // queries: [num_rows][num_heads][128] with row stride q_stride; box = 32 rows x 64 elements of one head
  CUtensorMap qmap;
  const cuuint64_t qdims[3] = {(cuuint64_t)kD, (cuuint64_t)d.num_heads, (cuuint64_t)d.num_rows};
  const cuuint64_t qstrides[2] = {(cuuint64_t)kD * 2, (cuuint64_t)d.q_stride * 2};
  const cuuint32_t qbox[3] = {64, 1, 32};
  const CUresult rq = encode_cached(enc, &qmap, elem, 3, d.query, qdims, qstrides, qbox, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
  if (rq != CUDA_SUCCESS) return cudaErrorInvalidValue;
  // partial accumulators: [parts * heads * rows][128] fp32; box = 128 rows x 32 floats
  AttnDev dd = d;
  CUtensorMap amap;
  const unsigned long long acc_rows = (unsigned long long)d.parts * d.num_heads * d.num_rows;
  dd.acc_tma = 0;
  if (acc_rows <= 0x7fffffffull) {
    const cuuint64_t adims[2] = {(cuuint64_t)kD, (cuuint64_t)acc_rows};
    const cuuint64_t astrides[1] = {(cuuint64_t)kD * 4};
    const cuuint32_t abox[2] = {32, 128};
    const CUresult ra = encode_cached(enc, &amap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, d.acc, adims, astrides, abox,
                                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE);
    if (ra != CUDA_SUCCESS) return cudaErrorInvalidValue;
    dd.acc_tma = 1;
  } else {
    amap = qmap;  // never used: the kernel keeps to its own stores
  }
  // outputs: [num_rows][num_heads][128] with row stride out_stride; box = 128 rows x 64 elements of one head
  CUtensorMap omap;
  {
    const cuuint64_t odims[3] = {(cuuint64_t)kD, (cuuint64_t)d.num_heads, (cuuint64_t)d.num_rows};
    const cuuint64_t ostrides[2] = {(cuuint64_t)kD * 2, (cuuint64_t)d.out_stride * 2};
    const cuuint32_t obox[3] = {64, 1, 128};
    const bool aligned = (reinterpret_cast<uintptr_t>(d.out) & 15u) == 0 && (d.out_stride * 2) % 16 == 0;
    const CUresult ro = aligned ? encode_cached(enc, &omap, elem, 3, d.out, odims, ostrides, obox, CU_TENSOR_MAP_SWIZZLE_128B,
                                                CU_TENSOR_MAP_L2_PROMOTION_NONE)
                                : CUDA_ERROR_INVALID_VALUE;
    if (ro != CUDA_SUCCESS) {  // an output the tensor map cannot describe: keep to partials and per-thread stores
      omap = qmap;
      dd.acc_tma = 0;
    }
  }
  if (d.dense_row_tile == 256) return launch_dense_pair(dd, dtype, vmap, qmap, amap, omap, s);
  cudaError_t e;
  if (dtype == PB_F16) {
    auto kfn = dense_prefix_kernel<__half>;
    e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    e = launch_kernel(kfn, d.num_sms, kThreads, kSmemBytes, s, true, dd, vmap, qmap, amap, omap);
  } else {
    auto kfn = dense_prefix_kernel<__nv_bfloat16>;
    e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    e = launch_kernel(kfn, d.num_sms, kThreads, kSmemBytes, s, true, dd, vmap, qmap, amap, omap);
  }
  return e;
}

}  // namespace pb
