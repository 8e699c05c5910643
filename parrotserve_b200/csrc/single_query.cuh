// Single-query paged attention over ragged KV chunks: the bandwidth-bound "suffix" stage.
//
// Each WARP is an independent streaming pipeline. It walks its share of the work list
// (row, head, kv chunk), pulls every physical block's K tile and V tile (one contiguous
// head_size*block_size*sizeof(T) run each in the paged layout) into its private shared-memory
// ring with 1-D bulk async copies that complete on an mbarrier, and consumes the ring with
// 128-bit shared loads, fp32 FMAs and warp shuffles. Loads for the next items are issued while
// the current one is being reduced, so a warp's copy queue never drains between items.
// The un-normalised partial (acc, max, sum) of every item goes to the workspace; the merge
// kernel combines them.
//
// Reference counterparts: single_query_cached_kv_post_attention_kernel
// (csrc/attention/attention_post_kernels.cu:69-341), ..._prev_attention_kernel
// (attention_prev_kernels.cu:69-338) and single_query_cached_kv_attention_kernel
// (attention_kernels.cu:75-374), which run one CTA per (head, sequence) with the whole
// sequence's logits staged in shared memory.
#pragma once

#include "common.cuh"

namespace pb {
namespace {

template <typename T, int D, int B>
struct SqCfg {
  static constexpr int kVec = ElemTraits<T>::kVec;          // elements per 16 bytes
  static constexpr int kTileBytes = D * B * (int)sizeof(T);  // one K or V tile of a (block, head)
  static constexpr int kQBytes = D * (int)sizeof(T);
  // K tile, V tile, q row, and the row's new key and value rows (items that carry the new token)
  static constexpr int kStageBytes = (2 * kTileBytes + 3 * kQBytes + 127) / 128 * 128;
  static constexpr int kDSplit = 32 / B;                     // lanes that share one token in QK
  static constexpr int kChunks = D / kVec;                   // 16-byte chunks of one K row
  // lane (tok, dq) takes the chunks dq, dq + kDSplit, ... of its token; lane (lr, lt) the V rows
  // lr, lr + kRowsPerPass, ...; where the counts do not divide, the last round is partly idle
  static constexpr int kKChunks = (kChunks + kDSplit - 1) / kDSplit;  // 16-byte K chunks per lane
  static constexpr bool kKExact = kChunks % kDSplit == 0;
  static constexpr int kQRegs = kKChunks * kVec;             // q values per lane
  static constexpr int kLanesPerRow = B / kVec;              // lanes that share one V row
  static constexpr int kRowsPerPass = 32 / kLanesPerRow;
  static constexpr int kAcc = (D + kRowsPerPass - 1) / kRowsPerPass;  // output rows per lane
  static constexpr bool kVExact = D % kRowsPerPass == 0;
  static_assert(B == 8 || B == 16 || B == 32, "block size");
  static_assert(kStageBytes % 128 == 0, "stage alignment");
  static_assert(kKChunks >= 1 && kAcc >= 1, "shape");
  static constexpr int warp_bytes(int ns) { return ns * kStageBytes + 128 /*p*/ + ns * 16 /*meta*/ + 64 /*bars*/ ; }
};

struct ItemState {
  int row, head, kvh, part, nblk, ntok, has_new;
  const int32_t* tbl;  // first block id of the chunk
};

// Work queue of a CTA: a helper warp claims items from the global counter in batches, reads their
// descriptors and first block ids, and publishes them here; the streaming warps pop finished
// entries from shared memory, so no global-memory round trip sits between two of their items.
constexpr int kQueueDepth = 8;   // entries
constexpr int kQueueBatch = 4;   // items claimed with one atomic
struct QueueEntry {
  int row, head, kvh, part, nblk, ntok, table_kind, tbl_off;
  int has_new;  // the item's last block ends with the row's new token, to be taken from key_new / value_new
  int ids[32];  // the first 32 block ids of the chunk
};
struct WorkQueue {
  QueueEntry e[kQueueDepth];
  int free_at[kQueueDepth];  // slot i may be written for entry index free_at[i] (i, i + depth, ...)
  int tail;   // entries published (helper)
  int head;   // entries reserved (streaming warps)
  int final;  // total number of entries there will ever be; -1 while unknown
};
__device__ __forceinline__ int ld_volatile_shared(const int* p) { return *reinterpret_cast<const volatile int*>(p); }

// ---- warp-level tensor-core helpers of the MMA consumer (16-bit element types) ----
template <typename T> struct MmaOps;
template <> struct MmaOps<__half> {
  static __device__ __forceinline__ void mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  // (hi, lo) split of two floats: hi = rounded pair, lo = rounded remainders
  static __device__ __forceinline__ void split(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(x, y);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
  }
};
template <> struct MmaOps<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ void split(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
  }
};
template <> struct MmaOps<float> {  // never instantiated with MMA = true
  static __device__ __forceinline__ void mma(float*, const uint32_t*, uint32_t, uint32_t) {}
  static __device__ __forceinline__ void split(float, float, uint32_t&, uint32_t&) {}
};
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// MMA == false: fp32 FMA consumer (any element type).
// MMA == true : warp-level tensor-core consumer for 16-bit types, B == 16. The single query row is
//   row 0 of the 16-row A operand of  S = q.K^T  (B operand = the K tile, read with ldmatrix exactly
//   as it lies in the cache layout); lanes 0-3 then hold the 16 logits in the very register layout
//   the B operand of  O = V.p  needs, so P never moves between lanes. p enters as an exact
//   (hi + lo) pair of 16-bit values. This cuts the instruction stream per 8 KiB of KV about 5x,
//   which is what kept the FMA consumer from saturating HBM.
template <typename T, int D, int B, int WARPS, int NS, bool MMA>
__global__ void __launch_bounds__((WARPS + 1) * 32, 1) sq_attn_kernel(const AttnDev d) {
  using C = SqCfg<T, D, B>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kWarpBytes = (C::warp_bytes(NS) + 127) / 128 * 128;
  WorkQueue* wq = reinterpret_cast<WorkQueue*>(smem_raw + WARPS * kWarpBytes);
  uint8_t* wbase = smem_raw + (warp < WARPS ? warp : 0) * kWarpBytes;
  float* pbuf = reinterpret_cast<float*>(wbase + NS * C::kStageBytes);
  int4* meta = reinterpret_cast<int4*>(wbase + NS * C::kStageBytes + 128);
  uint64_t* bars = reinterpret_cast<uint64_t*>(wbase + NS * C::kStageBytes + 128 + NS * 16);

  if (lane == 0 && warp < WARPS) {
#pragma unroll
    for (int s = 0; s < NS; ++s) mbar_init(smem_u32(&bars[s]), 1);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (threadIdx.x == 0) { wq->tail = 0; wq->head = 0; wq->final = -1; }
  if (threadIdx.x < kQueueDepth) wq->free_at[threadIdx.x] = threadIdx.x;
  __syncthreads();

  // Launched with programmatic stream serialization. When a dense prefix kernel precedes this
  // one it has already waited for the KV fill and the planner, and the two kernels are independent
  // (disjoint partial slots): this kernel starts at once on the SMs the dense kernel leaves free
  // and only waits for it at the very end, so the merge sees both complete.
  if (d.sq_waits_at_start) pdl_wait();
  pdl_trigger();
  const int H = d.num_heads;
  const long long n_items = (long long)d.hdr[kHdrNumSq] * H;
  // Asked to perform the KV fill, but the lists were built without the new-token slots: no item
  // carries a token, the fill would silently not happen. Recorded as a fault (NaN output).
  if (blockIdx.x == 0 && threadIdx.x == 0 && d.key_new != nullptr && d.hdr[kHdrPlannedSlots] == 0)
    atomicMax(&d.hdr[kHdrStatus], kStatusBadIndex);
  if (warp == WARPS) {
    // ------------------------------ helper warp: fills the queue ------------------------------
    // Claims kQueueBatch items with one atomic (so CTAs that become resident late, after the dense
    // kernel's CTAs retire, simply take what is left), lane e reads the descriptor of item e, then
    // all lanes read each item's block ids, and the batch is published with one store.
    int tail = 0;
    int want = kQueueBatch;  // items per claim; smaller near the end of the list (see below)
    bool ok = true;
    while (ok) {
      // every slot of the next batch has been copied out by the warp that popped its previous entry;
      // near the end of the list, moreover, at most two published items wait unstarted
      for (uint32_t spin = 0;; ++spin) {
        bool mine = lane >= want || ld_volatile_shared(&wq->free_at[(tail + lane) % kQueueDepth]) == tail + lane;
        if (want < kQueueBatch) mine = mine && (tail - ld_volatile_shared(&wq->head) <= 2);
        if (__all_sync(0xffffffffu, mine)) break;
        __nanosleep(64);
        if (spin > (1u << 24)) { ok = false; break; }  // about a second: the consumers are gone
      }
      if (!ok) break;
      int v = 0;
      if (lane == 0) v = atomicAdd(&d.hdr[kHdrSqCounter], want);
      // the first item of every streaming warp of the grid is assigned statically (below): the
      // counter hands out the items behind them
      const long long base = (long long)__shfl_sync(0xffffffffu, v, 0) + (long long)gridDim.x * WARPS;
      if (base >= n_items) break;
      const int cnt = (int)min((long long)want, n_items - base);
      // What a CTA has queued nobody else can take: once less than one full batch per SM is left,
      // claim half batches and keep the queue short, so the CTAs run dry within a few items of
      // each other.
      if (n_items - (base + cnt) < (long long)gridDim.x * kQueueBatch) want = kQueueBatch / 2;
      int4 a = make_int4(0, 0, 0, 0), b = make_int4(0, 0, 0, 0);
      int head = 0;
      if (lane < cnt) {
        const long long id = base + lane;
        const int sc = (int)(id / H);
        head = (int)(id - (long long)sc * H);
        a = *reinterpret_cast<const int4*>(&d.sq_items[sc]);        // row, meta, ntok, part
        b = *(reinterpret_cast<const int4*>(&d.sq_items[sc]) + 1);  // bid[4]
      }
      const int kvh = d.head_mapping ? d.head_mapping[head] : head;
      int ids[kQueueBatch];
#pragma unroll
      for (int e = 0; e < kQueueBatch; ++e) {  // independent loads, all in flight together
        const int meta = __shfl_sync(0xffffffffu, a.y, e);
        const int bx = __shfl_sync(0xffffffffu, b.x, e), by = __shfl_sync(0xffffffffu, b.y, e);
        const int bz = __shfl_sync(0xffffffffu, b.z, e), bw = __shfl_sync(0xffffffffu, b.w, e);
        const int nblk = meta & 0xffff;
        ids[e] = 0;
        if (e < cnt) {
          if (meta & (1 << 17)) {
            ids[e] = (lane == 0) ? bx : (lane == 1) ? by : (lane == 2) ? bz : bw;
          } else if (lane < nblk) {
            const int kind = (meta >> 18) & 3;  // 0 suffix, 1 group prefix, 2 causal segment, 3 outer prefix
            ids[e] = (kind == 1 ? d.group_tables : kind == 2 ? d.seg_tables : kind == 3 ? d.outer_tables : d.suffix_tables)[bx + lane];
          }
        }
      }
#pragma unroll
      for (int e = 0; e < kQueueBatch; ++e)
        if (e < cnt) wq->e[(tail + e) % kQueueDepth].ids[lane] = ids[e];
      if (lane < cnt) {
        QueueEntry& q = wq->e[(tail + lane) % kQueueDepth];
        q.row = a.x; q.head = head; q.kvh = kvh; q.part = a.w; q.nblk = a.y & 0xffff; q.ntok = a.z;
        q.table_kind = (a.y & (1 << 17)) ? -1 : ((a.y >> 18) & 3);
        q.tbl_off = b.x;
        q.has_new = (a.y >> 20) & 1;
      }
      __threadfence_block();  // the slots were seen free (acquire) and are now complete (release)
      __syncwarp();
      tail += cnt;
      if (lane == 0) *reinterpret_cast<volatile int*>(&wq->tail) = tail;
      if (base + cnt >= n_items) break;
    }
    __threadfence_block();
    if (lane == 0) *reinterpret_cast<volatile int*>(&wq->final) = tail;
  } else {
  // ------------------------------ streaming warps ------------------------------
  // Next item of this CTA: a finished queue entry (descriptor and block ids from shared memory),
  // or nblk == 0 when the list is exhausted (or the helper gave up).
  bool failed = false;
  auto pop = [&](int& bid) -> ItemState {
    ItemState it;
    it.nblk = 0; it.row = 0; it.head = 0; it.kvh = 0; it.part = 0; it.ntok = 0; it.has_new = 0; it.tbl = nullptr;
    bid = 0;
    int idx = 0;
    if (lane == 0) idx = atomicAdd(&wq->head, 1);
    idx = __shfl_sync(0xffffffffu, idx, 0);
    for (uint32_t spin = 0;; ++spin) {
      if (ld_volatile_shared(&wq->tail) > idx) break;
      const int fin = ld_volatile_shared(&wq->final);
      if (fin >= 0 && idx >= fin) return it;
      __nanosleep(32);
      if (spin > (1u << 25)) {  // about a second without a publisher
        if (lane == 0) atomicMax(&d.hdr[kHdrStatus], kStatusWaitExpired);
        failed = true;
        return it;
      }
    }
    __threadfence_block();
    const QueueEntry& q = wq->e[idx % kQueueDepth];
    it.row = q.row; it.head = q.head; it.kvh = q.kvh; it.part = q.part; it.nblk = q.nblk; it.ntok = q.ntok;
    it.has_new = q.has_new;
    if (q.table_kind >= 0)
      it.tbl = (q.table_kind == 1 ? d.group_tables : q.table_kind == 2 ? d.seg_tables
                : q.table_kind == 3 ? d.outer_tables : d.suffix_tables) + q.tbl_off;
    bid = q.ids[lane];
    __syncwarp();
    if (lane == 0) {
      __threadfence_block();
      *reinterpret_cast<volatile int*>(&wq->free_at[idx % kQueueDepth]) = idx + kQueueDepth;
    }
    return it;
  };

  // First item of this warp: item (CTA, warp) of the list, read straight from the planner's output,
  // so that every warp of the grid has copies in flight one memory round trip after the kernel
  // starts instead of waiting for the helper's first claims (an atomic, the descriptors, the block
  // ids, four items at a time). Everything after it comes through the queue.
  int cur_bid = 0;
  ItemState cur;
  {
    const long long id0 = (long long)blockIdx.x * WARPS + warp;
    if (id0 < n_items) {
      const int sc = (int)(id0 / H);
      const int head = (int)(id0 - (long long)sc * H);
      const int4 a = *reinterpret_cast<const int4*>(&d.sq_items[sc]);        // row, meta, ntok, part
      const int4 b = *(reinterpret_cast<const int4*>(&d.sq_items[sc]) + 1);  // bid[4]
      cur.row = a.x; cur.head = head; cur.kvh = d.head_mapping ? d.head_mapping[head] : head;
      cur.part = a.w; cur.nblk = a.y & 0xffff; cur.ntok = a.z; cur.has_new = (a.y >> 20) & 1;
      cur.tbl = nullptr;
      if (a.y & (1 << 17)) {
        cur_bid = (lane == 0) ? b.x : (lane == 1) ? b.y : (lane == 2) ? b.z : b.w;
      } else {
        const int kind = (a.y >> 18) & 3;  // 0 suffix, 1 group prefix, 2 causal segment, 3 outer prefix
        cur.tbl = (kind == 1 ? d.group_tables : kind == 2 ? d.seg_tables : kind == 3 ? d.outer_tables : d.suffix_tables) + b.x;
        cur_bid = (lane < cur.nblk) ? cur.tbl[lane] : 0;
      }
    } else {
      cur = pop(cur_bid);
    }
  }
  int p_blk = 0;
  uint32_t issued = 0, consumed = 0;

  const size_t esz = sizeof(T);
  const uint64_t kv_policy = l2_policy_evict_first();
  const uint8_t* kc = reinterpret_cast<const uint8_t*>(d.key_cache);
  const uint8_t* vc = reinterpret_cast<const uint8_t*>(d.value_cache);
  const uint8_t* qg = reinterpret_cast<const uint8_t*>(d.query);

  // consumer state
  constexpr int kKSteps = D / 16;                       // MMA consumer: k-steps of q.K^T, m-tiles of V.p
  constexpr int kQN = MMA ? 1 : C::kQRegs, kAccN = MMA ? 1 : C::kAcc;
  float q[kQN];
  float acc[kAccN];
  uint32_t qa[MMA ? kKSteps : 1][2];                    // q as A fragments (row 0 only)
  float oacc[MMA ? kKSteps : 1][4];                     // O^T accumulators, column 0 is the output
  float m_run = -INFINITY, l_run = 0.f;
  float m_true = -INFINITY;                             // MMA consumer: exact running maximum
#pragma unroll
  for (int i = 0; i < kQN; ++i) q[i] = 0.f;
#pragma unroll
  for (int i = 0; i < kAccN; ++i) acc[i] = 0.f;
  const int quad_t = lane & 3;
  const bool row0 = lane < 4;                           // lanes that hold row 0 / column 0 of B
  const uint32_t ldm_k_off = (uint32_t)((((lane >> 3) & 1) * 16 + (lane >> 4) * 8 + (lane & 7)) * 16);
  const uint32_t ldm_v_off = (uint32_t)((((lane >> 3) & 1) * 8 + (lane & 7)) * 32 + (lane >> 4) * 16);

  const int tok = lane % B, dq = lane / B;
  const int lr = lane / C::kLanesPerRow, lt = lane % C::kLanesPerRow;

  while (true) {
    // ------------------------------ producer ------------------------------
    while (issued - consumed < (uint32_t)NS && cur.nblk > 0) {
      const int s = issued % NS;
      if (p_blk > 0 && (p_blk & 31) == 0)  // chunks longer than 32 blocks: next window of ids
        cur_bid = (p_blk + lane < cur.nblk) ? cur.tbl[p_blk + lane] : 0;
      int blk = __shfl_sync(0xffffffffu, cur_bid, p_blk & 31);
      if (blk < 0 || blk >= d.num_blocks) {
        if (lane == 0) atomicMax(&d.hdr[kHdrStatus], kStatusBadIndex);
        blk = 0;
      }
      if (lane == 0) {
        const bool first = (p_blk == 0), last = (p_blk == cur.nblk - 1);
        const bool nw = last && cur.has_new && d.key_new != nullptr;  // this block ends with the row's new token
        const int ntok_blk = min(B, cur.ntok - p_blk * B);
        meta[s] = make_int4(cur.row, cur.head | (cur.part << 16), blk,
                            ntok_blk | (first ? 256 : 0) | (last ? 512 : 0) | (nw ? 1024 : 0));
        const uint32_t bar = smem_u32(&bars[s]);
        const uint32_t dst = smem_u32(wbase + s * C::kStageBytes);
        const size_t off = ((size_t)blk * d.kv_block_stride + (size_t)cur.kvh * d.kv_head_stride) * esz;
        mbar_arrive_expect_tx(bar, 2 * C::kTileBytes + (first ? C::kQBytes : 0) + (nw ? 2 * C::kQBytes : 0));
        // the K and V tiles are read once per call: first out of L2, so that the partials and tables stay
        bulk_g2s_hint(dst, kc + off, C::kTileBytes, bar, kv_policy);
        bulk_g2s_hint(dst + C::kTileBytes, vc + off, C::kTileBytes, bar, kv_policy);
        if (first)
          bulk_g2s(dst + 2 * C::kTileBytes,
                   qg + ((size_t)cur.row * d.q_stride + (size_t)cur.head * D) * esz, C::kQBytes, bar);
        if (nw) {  // the new key and value rows of (row, head) ride along with the block they belong in
          bulk_g2s(dst + 2 * C::kTileBytes + C::kQBytes,
                   reinterpret_cast<const uint8_t*>(d.key_new) + ((size_t)cur.row * d.key_new_stride + (size_t)cur.head * D) * esz,
                   C::kQBytes, bar);
          bulk_g2s(dst + 2 * C::kTileBytes + 2 * C::kQBytes,
                   reinterpret_cast<const uint8_t*>(d.value_new) + ((size_t)cur.row * d.value_new_stride + (size_t)cur.head * D) * esz,
                   C::kQBytes, bar);
        }
      }
      ++issued;
      ++p_blk;
      if (p_blk == cur.nblk) {
        cur = pop(cur_bid);
        p_blk = 0;
      }
    }
    if (consumed == issued) break;
    __syncwarp();

    // ------------------------------ consumer ------------------------------
    const int s = consumed % NS;
    if (!mbar_wait_bounded(smem_u32(&bars[s]), (consumed / NS) & 1)) {
      if (lane == 0) atomicMax(&d.hdr[kHdrStatus], kStatusWaitExpired);
      failed = true;
      break;
    }
    const int4 mt = meta[s];
    const int ntok_blk = mt.w & 255;
    const int it_row = mt.x, it_head = mt.y & 0xffff, it_part = mt.y >> 16;
    const uint8_t* stage = wbase + s * C::kStageBytes;

    if (mt.w & 1024) {
      // KV fill of the row's new token, fused: its key and value rows arrived with the block. They
      // replace the (not yet written) last token of this copy of the block and go into the cache
      // itself, where later calls find them (with identity head mapping this warp is the only one
      // that holds (row, kv head)). K tile [D/x][B tok][x], V tile [D][B tok].
      const int t = ntok_blk - 1;
      uint8_t* st = const_cast<uint8_t*>(stage);
      const uint8_t* kn = stage + 2 * C::kTileBytes + C::kQBytes;
      const uint8_t* vn = kn + C::kQBytes;
      const size_t goff = ((size_t)mt.z * d.kv_block_stride + (size_t)it_head * d.kv_head_stride) * esz;
      uint8_t* kg = const_cast<uint8_t*>(kc) + goff;
      uint8_t* vg = const_cast<uint8_t*>(vc) + goff;
      for (int c = lane; c < D / C::kVec; c += 32) {
        const uint4 v16 = *reinterpret_cast<const uint4*>(kn + c * 16);
        *reinterpret_cast<uint4*>(st + (c * B + t) * 16) = v16;
        *reinterpret_cast<uint4*>(kg + (c * B + t) * 16) = v16;
      }
      for (int dd = lane; dd < D; dd += 32) {
        const T ve = *reinterpret_cast<const T*>(vn + dd * sizeof(T));
        *reinterpret_cast<T*>(st + C::kTileBytes + ((size_t)dd * B + t) * sizeof(T)) = ve;
        *reinterpret_cast<T*>(vg + ((size_t)dd * B + t) * sizeof(T)) = ve;
      }
      fence_proxy_async_smem();  // generic stores into a stage that a later bulk copy refills
      __syncwarp();
    }

    if constexpr (MMA) {
      const uint32_t st_addr = smem_u32(stage);
      if (mt.w & 256) {  // first block of an item: fresh accumulators, q as row 0 of the A fragments
        const uint32_t* qs = reinterpret_cast<const uint32_t*>(stage + 2 * C::kTileBytes);
#pragma unroll
        for (int kk = 0; kk < kKSteps; ++kk) {
          qa[kk][0] = row0 ? qs[kk * 8 + quad_t] : 0u;      // q[16kk + 2t], q[16kk + 2t + 1]
          qa[kk][1] = row0 ? qs[kk * 8 + 4 + quad_t] : 0u;  // q[16kk + 8 + 2t], q[16kk + 9 + 2t]
        }
        m_run = m_true = -INFINITY;
        l_run = 0.f;
#pragma unroll
        for (int j = 0; j < kKSteps; ++j) oacc[j][0] = oacc[j][1] = oacc[j][2] = oacc[j][3] = 0.f;
      }
      // S = q.K^T: B operand = K tile [d chunk][16 tok][16 B]; one ldmatrix.x4 per k-step feeds the
      // two 8-token n-tiles. Lanes 0-3 end with the logits of tokens 2t, 2t+1, 8+2t, 9+2t.
      float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < kKSteps; ++kk) {
        uint32_t kb[4];
        ldmatrix_x4(kb, st_addr + ldm_k_off + kk * 512);
        const uint32_t a[4] = {qa[kk][0], 0u, qa[kk][1], 0u};
        MmaOps<T>::mma(sa, a, kb[0], kb[1]);
        MmaOps<T>::mma(sb, a, kb[2], kb[3]);
      }
      float lg[4] = {sa[0] * d.scale_log2e, sa[1] * d.scale_log2e, sb[0] * d.scale_log2e, sb[1] * d.scale_log2e};
      if (ntok_blk < B) {
        if (2 * quad_t >= ntok_blk) lg[0] = -INFINITY;
        if (2 * quad_t + 1 >= ntok_blk) lg[1] = -INFINITY;
        if (8 + 2 * quad_t >= ntok_blk) lg[2] = -INFINITY;
        if (9 + 2 * quad_t >= ntok_blk) lg[3] = -INFINITY;
      }
      float bm = fmaxf(fmaxf(lg[0], lg[1]), fmaxf(lg[2], lg[3]));
      bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
      bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
      bm = __shfl_sync(0xffffffffu, bm, 0);  // the block maximum, from the quad that holds row 0
      m_true = fmaxf(m_true, bm);
      if (bm > m_run + 8.f) {  // lazy reference maximum: rescale only on jumps of more than 2^8
        const float alpha = fast_exp2(m_run - bm);
        l_run *= alpha;
#pragma unroll
        for (int j = 0; j < kKSteps; ++j) { oacc[j][0] *= alpha; oacc[j][1] *= alpha; oacc[j][2] *= alpha; oacc[j][3] *= alpha; }
        m_run = bm;
      }
      float p[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) p[i] = row0 ? fast_exp2(lg[i] - m_run) : 0.f;
      l_run += (p[0] + p[1]) + (p[2] + p[3]);
      uint32_t hi0, lo0, hi1, lo1;
      MmaOps<T>::split(p[0], p[1], hi0, lo0);  // B fragment rows 2t, 2t+1   (column 0 in lanes 0-3)
      MmaOps<T>::split(p[2], p[3], hi1, lo1);  // B fragment rows 8+2t, 9+2t
      if (ntok_blk < B) {
        // ragged last block: zero the V columns beyond the length so 0 * (stale bytes) stays 0
        uint16_t* vz = reinterpret_cast<uint16_t*>(const_cast<uint8_t*>(stage) + C::kTileBytes);
        for (int dd = lane; dd < D; dd += 32)
          for (int tk = ntok_blk; tk < B; ++tk) vz[dd * B + tk] = 0;
        fence_proxy_async_smem();  // these generic stores come before the bulk copy that refills the stage
        __syncwarp();
      }
      // O^T += V.p: A operand = V tile [d][16 tok] read with ldmatrix as it lies; column 0 of the
      // result (lanes with lane % 4 == 0) is the output. p = hi + lo keeps the weights exact.
#pragma unroll
      for (int j = 0; j < kKSteps; ++j) {
        uint32_t va[4];
        ldmatrix_x4(va, st_addr + C::kTileBytes + ldm_v_off + j * 512);
        MmaOps<T>::mma(oacc[j], va, hi0, hi1);
        MmaOps<T>::mma(oacc[j], va, lo0, lo1);
      }
      __syncwarp();  // stage s may be overwritten from here on
      if (mt.w & 512) {  // last block of the item: emit the partial, re-based on the exact maximum
        const float fix = fast_exp2(m_run - m_true);  // <= 1; the reference point lagged by < 2^8
        float l = l_run * fix;
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const size_t slot = partial_slot(d, it_row, it_part, it_head);
        if (quad_t == 0) {
          float* ap = d.acc + slot * D + (lane >> 2);
#pragma unroll
          for (int j = 0; j < kKSteps; ++j) {
            ap[16 * j] = oacc[j][0] * fix;
            ap[16 * j + 8] = oacc[j][2] * fix;
          }
        }
        if (lane == 0) d.ml[slot] = make_float2(m_true, l);
      }
    } else {
    if (mt.w & 256) {  // first block of an item: fresh accumulators, load q
      const uint4* qs = reinterpret_cast<const uint4*>(stage + 2 * C::kTileBytes) + dq;
#pragma unroll
      for (int i = 0; i < C::kKChunks; ++i) {
        float f[C::kVec];
        const bool live = C::kKExact || dq + i * C::kDSplit < C::kChunks;
        unpack16<T>(live ? qs[i * C::kDSplit] : make_uint4(0u, 0u, 0u, 0u), f);
#pragma unroll
        for (int j = 0; j < C::kVec; ++j) q[i * C::kVec + j] = f[j] * d.scale_log2e;
      }
      m_run = -INFINITY;
      l_run = 0.f;
#pragma unroll
      for (int i = 0; i < C::kAcc; ++i) acc[i] = 0.f;
    }

    // logits of the block's B tokens: lane (tok, dq) covers the 16-byte chunks dq, dq + kDSplit, ... of its token
    float s4[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const uint4* kt = reinterpret_cast<const uint4*>(stage) + dq * B + tok;
#pragma unroll
      for (int i = 0; i < C::kKChunks; ++i) {
        float f[C::kVec];
        const bool live = C::kKExact || dq + i * C::kDSplit < C::kChunks;  // (q is zero in the idle slots)
        unpack16<T>(live ? kt[i * C::kDSplit * B] : make_uint4(0u, 0u, 0u, 0u), f);
#pragma unroll
        for (int j = 0; j < C::kVec; ++j) s4[j & 3] = fmaf(q[i * C::kVec + j], f[j], s4[j & 3]);
      }
    }
    float logit = (s4[0] + s4[1]) + (s4[2] + s4[3]);
#pragma unroll
    for (int o = B; o < 32; o <<= 1) logit += __shfl_xor_sync(0xffffffffu, logit, o);
    if (tok >= ntok_blk) logit = -INFINITY;

    if (__any_sync(0xffffffffu, logit > m_run)) {
      float bm = logit;
#pragma unroll
      for (int o = B / 2; o >= 1; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
      const float m_new = fmaxf(m_run, bm);
      const float alpha = fast_exp2(m_run - m_new);  // m_run = -inf -> 0
      l_run *= alpha;
#pragma unroll
      for (int i = 0; i < C::kAcc; ++i) acc[i] *= alpha;
      m_run = m_new;
    }
    const float p = fast_exp2(logit - m_run);
    l_run += p;
    if (dq == 0) pbuf[tok] = p;
    __syncwarp();

    // out[d] += sum_t p[t] * V[d][t]; lane (lr, lt) covers rows lr + i*kRowsPerPass, tokens lt*kVec..
    {
      float pv[C::kVec];
#pragma unroll
      for (int j = 0; j < C::kVec; j += 4) {
        const float4 t4 = *reinterpret_cast<const float4*>(pbuf + lt * C::kVec + j);
        pv[j] = t4.x; pv[j + 1] = t4.y; pv[j + 2] = t4.z; pv[j + 3] = t4.w;
      }
      const uint4* vt = reinterpret_cast<const uint4*>(stage + C::kTileBytes) + lr * C::kLanesPerRow + lt;
      if (ntok_blk == B) {
#pragma unroll
        for (int i = 0; i < C::kAcc; ++i) {
          float f[C::kVec];
          const bool live = C::kVExact || lr + i * C::kRowsPerPass < D;
          unpack16<T>(live ? vt[i * C::kRowsPerPass * C::kLanesPerRow] : make_uint4(0u, 0u, 0u, 0u), f);
#pragma unroll
          for (int j = 0; j < C::kVec; ++j) acc[i] = fmaf(pv[j], f[j], acc[i]);
        }
      } else {  // ragged last block: never touch cache bytes beyond the length
#pragma unroll
        for (int i = 0; i < C::kAcc; ++i) {
          float f[C::kVec];
          const bool live = C::kVExact || lr + i * C::kRowsPerPass < D;
          unpack16<T>(live ? vt[i * C::kRowsPerPass * C::kLanesPerRow] : make_uint4(0u, 0u, 0u, 0u), f);
#pragma unroll
          for (int j = 0; j < C::kVec; ++j)
            if (lt * C::kVec + j < ntok_blk) acc[i] = fmaf(pv[j], f[j], acc[i]);
        }
      }
    }
    __syncwarp();  // stage s and pbuf may be overwritten from here on

    if (mt.w & 512) {  // last block of the item: emit the partial
#pragma unroll
      for (int i = 0; i < C::kAcc; ++i) {
#pragma unroll
        for (int o = 1; o < C::kLanesPerRow; o <<= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
      }
      float l = l_run;
#pragma unroll
      for (int o = B / 2; o >= 1; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
      const size_t slot = partial_slot(d, it_row, it_part, it_head);
      if (lt == 0) {
        float* ap = d.acc + slot * D + lr;
#pragma unroll
        for (int i = 0; i < C::kAcc; ++i)
          if (C::kVExact || lr + i * C::kRowsPerPass < D) ap[i * C::kRowsPerPass] = acc[i];
      }
      if (lane == 0) d.ml[slot] = make_float2(m_run, l);
    }
    }  // !MMA
    ++consumed;
  }
  if (failed) {
    // Give the copies still in flight one more bounded chance to land before the CTA's shared
    // memory is released.
    for (uint32_t c = consumed + 1; c < issued; ++c)
      (void)mbar_wait_bounded(smem_u32(&bars[c % NS]), (c / NS) & 1);
  }
  }  // streaming warps

  if (!d.sq_waits_at_start) pdl_wait();  // the dense prefix kernel has completed
}

template <typename T, int D, int B, int WARPS, int NS, bool MMA>
cudaError_t launch_sq(const AttnDev& d, cudaStream_t s) {
  using C = SqCfg<T, D, B>;
  constexpr int kWarpBytes = (C::warp_bytes(NS) + 127) / 128 * 128;
  constexpr int smem = WARPS * kWarpBytes + (int)sizeof(WorkQueue);
  static_assert(smem <= 227 * 1024, "shared memory budget");
  auto kfn = sq_attn_kernel<T, D, B, WARPS, NS, MMA>;
  cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  return launch_kernel(kfn, d.num_sms, (WARPS + 1) * 32, smem, s, true, d);
}


// Warps that fit the shared-memory budget with NS stages each (at most 8 streaming warps).
template <typename T, int D, int B, int NS>
constexpr int sq_auto_warps() {
  using C = SqCfg<T, D, B>;
  const int wb = (C::warp_bytes(NS) + 127) / 128 * 128;
  const int w = (227 * 1024 - (int)sizeof(WorkQueue)) / wb;
  return w > 8 ? 8 : w;
}
// The fp32-FMA consumer for any (type, head size, block size), warps chosen to fit.
template <typename T, int D, int B>
cudaError_t launch_sq_fma_auto(const AttnDev& d, cudaStream_t s) {
  constexpr int NS = 3;
  constexpr int W = sq_auto_warps<T, D, B, NS>();
  static_assert(W >= 1, "one warp's stages must fit shared memory");
  return launch_sq<T, D, B, W, NS, false>(d, s);
}
// All head sizes of the reference's kernels for one block size other than 16.
template <int B>
cudaError_t launch_sq_other_block(const AttnDev& d, int dtype, int head_size, cudaStream_t s) {
#define PB_SQ_B(DD)                                                                   \
  if (head_size == DD) {                                                              \
    if (dtype == PB_F16) return launch_sq_fma_auto<__half, DD, B>(d, s);              \
    if (dtype == PB_BF16) return launch_sq_fma_auto<__nv_bfloat16, DD, B>(d, s);      \
    if (dtype == PB_F32) return launch_sq_fma_auto<float, DD, B>(d, s);               \
  }
  PB_SQ_B(64) PB_SQ_B(80) PB_SQ_B(96) PB_SQ_B(112) PB_SQ_B(128) PB_SQ_B(256)
#undef PB_SQ_B
  return cudaErrorInvalidValue;
}

}  // namespace
}  // namespace pb
