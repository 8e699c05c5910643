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
#include "common.cuh"

namespace pb {
namespace {

template <typename T, int D, int B>
struct SqCfg {
  static constexpr int kVec = ElemTraits<T>::kVec;          // elements per 16 bytes
  static constexpr int kTileBytes = D * B * (int)sizeof(T);  // one K or V tile of a (block, head)
  static constexpr int kQBytes = D * (int)sizeof(T);
  static constexpr int kStageBytes = 2 * kTileBytes + kQBytes;
  static constexpr int kDSplit = 32 / B;                     // lanes that share one token in QK
  static constexpr int kKChunks = D / kVec / kDSplit;        // 16-byte K chunks per lane
  static constexpr int kQRegs = D / kDSplit;                 // q values per lane
  static constexpr int kLanesPerRow = B / kVec;              // lanes that share one V row
  static constexpr int kRowsPerPass = 32 / kLanesPerRow;
  static constexpr int kAcc = D / kRowsPerPass;              // output rows per lane
  static_assert(B == 8 || B == 16 || B == 32, "block size");
  static_assert(kStageBytes % 128 == 0, "stage alignment");
  static_assert(kKChunks >= 1 && kAcc >= 1, "shape");
  static constexpr int warp_bytes(int ns) { return ns * kStageBytes + 128 /*p*/ + ns * 16 /*meta*/ + 64 /*bars*/ ; }
};

struct ItemState {
  int row, head, kvh, part, nblk, ntok;
  const int32_t* tbl;  // first block id of the chunk
};

template <typename T, int D, int B, int WARPS, int NS>
__global__ void __launch_bounds__(WARPS * 32, 1) sq_attn_kernel(const AttnDev d) {
  using C = SqCfg<T, D, B>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kWarpBytes = (C::warp_bytes(NS) + 127) / 128 * 128;
  uint8_t* wbase = smem_raw + warp * kWarpBytes;
  float* pbuf = reinterpret_cast<float*>(wbase + NS * C::kStageBytes);
  int4* meta = reinterpret_cast<int4*>(wbase + NS * C::kStageBytes + 128);
  uint64_t* bars = reinterpret_cast<uint64_t*>(wbase + NS * C::kStageBytes + 128 + NS * 16);

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NS; ++s) mbar_init(smem_u32(&bars[s]), 1);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  __syncthreads();

  const int H = d.num_heads;
  const long long n_items = (long long)d.hdr[kHdrNumSq] * H;
  const long long W = (long long)gridDim.x * WARPS;
  const long long gw = (long long)blockIdx.x * WARPS + warp;

  auto load_item = [&](long long id) -> ItemState {
    ItemState it;
    it.nblk = 0; it.row = 0; it.head = 0; it.kvh = 0; it.part = 0; it.ntok = 0; it.tbl = nullptr;
    if (id < n_items) {
      const int sc = (int)(id / H);
      it.head = (int)(id - (long long)sc * H);
      const int4 a = *reinterpret_cast<const int4*>(&d.sq_items[sc]);         // row, tbl_off, is_prefix, nblk
      const int2 b = *(reinterpret_cast<const int2*>(&d.sq_items[sc]) + 2);   // ntok, part
      it.row = a.x;
      it.tbl = (a.z ? d.group_tables : d.suffix_tables) + a.y;
      it.nblk = a.w;
      it.ntok = b.x;
      it.part = b.y;
      it.kvh = d.head_mapping ? d.head_mapping[it.head] : it.head;
    }
    return it;
  };
  auto load_bid = [&](const ItemState& it) -> int {
    return (lane < it.nblk) ? it.tbl[lane] : 0;
  };

  ItemState cur = load_item(gw), nxt = load_item(gw + W), nx2 = load_item(gw + 2 * W);
  long long nx2_id = gw + 2 * W;
  int cur_bid = load_bid(cur), nxt_bid = load_bid(nxt);
  int p_blk = 0;
  uint32_t issued = 0, consumed = 0;

  const size_t esz = sizeof(T);
  const uint8_t* kc = reinterpret_cast<const uint8_t*>(d.key_cache);
  const uint8_t* vc = reinterpret_cast<const uint8_t*>(d.value_cache);
  const uint8_t* qg = reinterpret_cast<const uint8_t*>(d.query);

  // consumer state
  float q[C::kQRegs];
  float acc[C::kAcc];
  float m_run = -INFINITY, l_run = 0.f;
#pragma unroll
  for (int i = 0; i < C::kQRegs; ++i) q[i] = 0.f;
#pragma unroll
  for (int i = 0; i < C::kAcc; ++i) acc[i] = 0.f;

  const int tok = lane % B, dq = lane / B;
  const int lr = lane / C::kLanesPerRow, lt = lane % C::kLanesPerRow;
  bool failed = false;

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
        const int ntok_blk = min(B, cur.ntok - p_blk * B);
        meta[s] = make_int4(cur.row, cur.head, cur.part, ntok_blk | (first ? 256 : 0) | (last ? 512 : 0));
        const uint32_t bar = smem_u32(&bars[s]);
        const uint32_t dst = smem_u32(wbase + s * C::kStageBytes);
        const size_t off = ((size_t)blk * d.kv_block_stride + (size_t)cur.kvh * d.kv_head_stride) * esz;
        mbar_arrive_expect_tx(bar, 2 * C::kTileBytes + (first ? C::kQBytes : 0));
        bulk_g2s(dst, kc + off, C::kTileBytes, bar);
        bulk_g2s(dst + C::kTileBytes, vc + off, C::kTileBytes, bar);
        if (first)
          bulk_g2s(dst + 2 * C::kTileBytes,
                   qg + ((size_t)cur.row * d.q_stride + (size_t)cur.head * D) * esz, C::kQBytes, bar);
      }
      ++issued;
      ++p_blk;
      if (p_blk == cur.nblk) {
        cur = nxt; cur_bid = nxt_bid;
        nxt = nx2; nxt_bid = load_bid(nxt);
        nx2_id += W; nx2 = load_item(nx2_id);
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
    const uint8_t* stage = wbase + s * C::kStageBytes;

    if (mt.w & 256) {  // first block of an item: fresh accumulators, load q
      const uint4* qs = reinterpret_cast<const uint4*>(stage + 2 * C::kTileBytes) + dq * C::kKChunks;
#pragma unroll
      for (int i = 0; i < C::kKChunks; ++i) {
        float f[C::kVec];
        unpack16<T>(qs[i], f);
#pragma unroll
        for (int j = 0; j < C::kVec; ++j) q[i * C::kVec + j] = f[j] * d.scale_log2e;
      }
      m_run = -INFINITY;
      l_run = 0.f;
#pragma unroll
      for (int i = 0; i < C::kAcc; ++i) acc[i] = 0.f;
    }

    // logits of the block's B tokens: lane (tok, dq) covers d in [dq*kQRegs, (dq+1)*kQRegs)
    float s4[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const uint4* kt = reinterpret_cast<const uint4*>(stage) + (dq * C::kKChunks) * B + tok;
#pragma unroll
      for (int i = 0; i < C::kKChunks; ++i) {
        float f[C::kVec];
        unpack16<T>(kt[i * B], f);
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
          unpack16<T>(vt[i * C::kRowsPerPass * C::kLanesPerRow], f);
#pragma unroll
          for (int j = 0; j < C::kVec; ++j) acc[i] = fmaf(pv[j], f[j], acc[i]);
        }
      } else {  // ragged last block: never touch cache bytes beyond the length
#pragma unroll
        for (int i = 0; i < C::kAcc; ++i) {
          float f[C::kVec];
          unpack16<T>(vt[i * C::kRowsPerPass * C::kLanesPerRow], f);
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
      const size_t slot = ((size_t)mt.x * d.parts + mt.z) * H + mt.y;
      if (lt == 0) {
        float* ap = d.acc + slot * D + lr;
#pragma unroll
        for (int i = 0; i < C::kAcc; ++i) ap[i * C::kRowsPerPass] = acc[i];
      }
      if (lane == 0) d.ml[slot] = make_float2(m_run, l);
    }
    ++consumed;
  }

  if (failed) {
    // Give the copies still in flight one more bounded chance to land before the CTA's shared
    // memory is released.
    for (uint32_t c = consumed + 1; c < issued; ++c)
      (void)mbar_wait_bounded(smem_u32(&bars[c % NS]), (c / NS) & 1);
  }
}

template <typename T, int D, int B, int WARPS, int NS>
cudaError_t launch_sq(const AttnDev& d, cudaStream_t s) {
  using C = SqCfg<T, D, B>;
  constexpr int kWarpBytes = (C::warp_bytes(NS) + 127) / 128 * 128;
  constexpr int smem = WARPS * kWarpBytes;
  static_assert(smem <= 227 * 1024, "shared memory budget");
  auto kfn = sq_attn_kernel<T, D, B, WARPS, NS>;
  cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  kfn<<<kNumSMs, WARPS * 32, smem, s>>>(d);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_single_query(const AttnDev& d, int dtype, int head_size, int block_size, cudaStream_t s) {
  if (head_size == 128 && block_size == 16) {
    if (dtype == PB_F16) return launch_sq<__half, 128, 16, 8, 3>(d, s);
    if (dtype == PB_BF16) return launch_sq<__nv_bfloat16, 128, 16, 8, 3>(d, s);
    if (dtype == PB_F32) return launch_sq<float, 128, 16, 4, 3>(d, s);
  }
  if (head_size == 64 && block_size == 16) {
    if (dtype == PB_F16) return launch_sq<__half, 64, 16, 8, 4>(d, s);
    if (dtype == PB_BF16) return launch_sq<__nv_bfloat16, 64, 16, 8, 4>(d, s);
    if (dtype == PB_F32) return launch_sq<float, 64, 16, 8, 3>(d, s);
  }
  return cudaErrorInvalidValue;
}

}  // namespace pb
