// Token sampling on the device: temperature, nucleus (top-p) filtering and one draw per row of a
// [rows, vocab] logits matrix, without sorting the row.
//
// Reference counterpart: Sampler.forward (parrot/engine/builtin/models/sampler.py:19-66), which sorts
// every row, takes a softmax and a cumulative sum of the sorted row, masks, un-sorts, takes a second
// softmax and calls torch.multinomial. Here one CTA owns one row and makes a few passes over it
// (the row stays in L2 after the first):
//   1. max of logit / temperature;
//   2. every token's un-normalised probability exp(x - max) as a 2^-40 fixed-point integer, summed into a
//      2048-bin histogram keyed by (max - x) * 64: integer sums do not depend on the order of the atomics,
//      so the result is the same on every run; the bin in which the mass sorted before a token first
//      exceeds top_p * total holds the edge of the nucleus;
//   3. that bin's tokens (usually a few dozen) are collected into a list in shared memory and the bin is
//      refined twice by 2048 (resolution 2^-28 in the logit): tokens before the final bin are kept, tokens
//      after it dropped, tokens inside it (ties) are kept in index order while the mass before them allows
//      it, which is what a stable descending sort does. Bins of more than 2048 tokens and tie classes of
//      more than 32 are refined by passes over the row instead;
//   4. the draw is the inverse CDF over the kept tokens in index order for the caller's uniform number.
// Rows without top-p need passes 1, a plain sum, and 4.
#include "common.cuh"

namespace pb {
namespace {

constexpr int kSampThreads = 1024;
constexpr int kSampWarps = kSampThreads / 32;
constexpr int kPerThread = 8;                       // consecutive tokens of one thread in a tile
constexpr int kTile = kSampThreads * kPerThread;    // tokens per pass step
constexpr int kBins = 2048;
constexpr int kBinsPerThread = kBins / kSampThreads;
constexpr int kListCap = 2048;
constexpr float kFixedOne = 1099511627776.f;  // 2^40
typedef unsigned long long u64;

struct SampShared {
  // bin mass = hist_hi * 2^32 + hist_lo: two native 32-bit atomics per token, the carry out of the low
  // word is seen by exactly the thread whose add wrapped it
  uint32_t hist_lo[kBins];
  uint32_t hist_hi[kBins];
  u64 warp_tot[kSampWarps + 1];
  float warp_max[kSampWarps];
  u64 budget_next;
  u64 tie_mass;
  int cross;
  int last_kept_tie;
  int found;
  // tokens of the first-level bin the nucleus edge falls in (usually a few dozen): when they fit, the two
  // refinements and the tie handling run over this list instead of over the row
  int list_n, tie_n;
  float list_d[kListCap];
  int list_i[kListCap];
  u64 tie_q[32];
  int tie_i[32];
};

// exclusive prefix of v over the CTA in thread order; `total` = the CTA's sum
__device__ __forceinline__ u64 block_excl_scan(u64 v, SampShared& sh, u64& total) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  u64 incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const u64 n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) sh.warp_tot[wid] = incl;
  __syncthreads();
  if (wid == 0) {
    const u64 t = lane < kSampWarps ? sh.warp_tot[lane] : 0;
    u64 it = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const u64 n = __shfl_up_sync(0xffffffffu, it, o);
      if (lane >= o) it += n;
    }
    if (lane < kSampWarps) sh.warp_tot[lane] = it - t;
    if (lane == 31) sh.warp_tot[kSampWarps] = it;
  }
  __syncthreads();
  const u64 excl = sh.warp_tot[wid] + incl - v;
  total = sh.warp_tot[kSampWarps];
  __syncthreads();  // warp_tot is reused by the next call
  return excl;
}

__device__ __forceinline__ void hist_add(SampShared& sh, int bin, u64 q) {
  const uint32_t lo = (uint32_t)q;
  const uint32_t old = atomicAdd(&sh.hist_lo[bin], lo);
  const uint32_t hi = (uint32_t)(q >> 32) + (old > ~lo ? 1u : 0u);
  if (hi) atomicAdd(&sh.hist_hi[bin], hi);
}

// The thread's kPerThread consecutive logits of the tile at `base`, times 1 / temperature;
// -inf beyond the row (weight 0, never drawn). 16-byte loads when the row allows it.
template <typename T>
__device__ __forceinline__ void load_tokens(const T* __restrict__ row, int vocab, bool vec, int base, float inv_temp,
                                            float (&x)[kPerThread]) {
  const int i0 = base + threadIdx.x * kPerThread;
  if (vec && i0 + kPerThread <= vocab) {
    constexpr int kV = ElemTraits<T>::kVec;
#pragma unroll
    for (int v = 0; v < kPerThread / kV; ++v) unpack16<T>(*reinterpret_cast<const uint4*>(row + i0 + v * kV), &x[v * kV]);
  } else {
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) x[j] = i0 + j < vocab ? to_float<T>(row[i0 + j]) : -INFINITY;
  }
#pragma unroll
  for (int j = 0; j < kPerThread; ++j) x[j] *= inv_temp;
}

// One token, from d = max - x >= 0: the fixed-point weight exp(-d) * 2^40, the first-level bin, and the
// 33-bit three-level key (smaller key = larger logit). Most tokens are decided by the first level alone.
__device__ __forceinline__ u64 token_weight(float d) {
  float w;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(w) : "f"(-d * 1.4426950408889634f));
  return __float2ull_rd(w * kFixedOne);
}
__device__ __forceinline__ int token_bin1(float d) { return min(max(__float2int_rz(d * 64.f), 0), kBins - 1); }
__device__ __forceinline__ u64 token_key(float d) {
  const float t0 = d * 64.f;
  const int k1 = min(max(__float2int_rz(t0), 0), kBins - 1);
  const float t1 = (t0 - (float)k1) * (float)kBins;
  const int k2 = min(max(__float2int_rz(t1), 0), kBins - 1);
  const float t2 = (t1 - (float)k2) * (float)kBins;
  const int k3 = min(max(__float2int_rz(t2), 0), kBins - 1);
  return ((u64)k1 << 22) | ((u64)k2 << 11) | (u64)k3;
}
// Whether the token's first-level bin is `f1`, by comparisons instead of a conversion (same rounding:
// the bin is trunc(d * 64) clamped to the last bin).
__device__ __forceinline__ bool token_in_bin1(float d, int f1) {
  const float t0 = d * 64.f;
  return t0 >= (float)f1 && (f1 == kBins - 1 || t0 < (float)(f1 + 1));
}
// -1: sorted before the tie class (kept), 0: in it, +1: after it (dropped)
__device__ __forceinline__ int token_side(float d, u64 final_key) {
  const int f1 = (int)(final_key >> 22);
  if (!token_in_bin1(d, f1)) return d * 64.f < (float)f1 ? -1 : 1;
  const u64 key = token_key(d);
  return key < final_key ? -1 : (key == final_key ? 0 : 1);
}

// After a histogram level is complete: the first bin whose mass, added to the mass of the bins before it,
// exceeds the budget (kBins if none). Moves the mass before that bin from `budget` to `kept_before`.
// With `p_keep` >= 0 (first level) the budget is first set to p_keep * total mass.
__device__ __forceinline__ int settle_level(SampShared& sh, float p_keep, u64& budget, u64& kept_before, u64& total) {
  const int tid = threadIdx.x;
  if (tid == 0) sh.cross = kBins;
  u64 h[kBinsPerThread], mine = 0;
#pragma unroll
  for (int b = 0; b < kBinsPerThread; ++b) {
    h[b] = ((u64)sh.hist_hi[kBinsPerThread * tid + b] << 32) + sh.hist_lo[kBinsPerThread * tid + b];
    mine += h[b];
  }
  u64 run = block_excl_scan(mine, sh, total);  // its barriers also publish sh.cross = kBins
  // a token is dropped when the mass sorted before it exceeds top_p * total
  if (p_keep >= 0.f) budget = (u64)((double)p_keep * (double)total);
  u64 before_cross = 0;
  int my_cross = kBins;
#pragma unroll
  for (int b = 0; b < kBinsPerThread; ++b) {
    if (my_cross == kBins && run + h[b] > budget) my_cross = kBinsPerThread * tid + b, before_cross = run;
    run += h[b];
  }
  if (my_cross != kBins) atomicMin(&sh.cross, my_cross);
  __syncthreads();
  const int cross = sh.cross;
  if (cross == kBins) return cross;
  if (my_cross == cross) sh.budget_next = budget - before_cross;
  __syncthreads();
  kept_before += budget - sh.budget_next;
  budget = sh.budget_next;
  __syncthreads();
  return cross;
}

// Adds one token to the histogram of refinement level 1 or 2 if its key matches `final_key` above that level.
__device__ __forceinline__ void refine_add(SampShared& sh, float d, int level, u64 final_key) {
  const int shift = 22 - 11 * level;
  const u64 key = token_key(d);
  if ((key >> (shift + 11)) != (final_key >> (shift + 11))) return;
  const u64 q = token_weight(d);
  if (q) hist_add(sh, (int)((key >> shift) & (kBins - 1)), q);  // weightless tokens change no sum
}

template <typename T>
__global__ void __launch_bounds__(kSampThreads) sample_top_p_kernel(
    const T* __restrict__ logits, const int vocab, const long long row_stride, const float* __restrict__ temperature,
    const float* __restrict__ top_p, const float* __restrict__ uniforms, long long* __restrict__ ids) {
  __shared__ SampShared sh;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const T* row = logits + (long long)blockIdx.x * row_stride;
  const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
  const float temp = temperature ? __fdiv_rn(1.f, temperature[blockIdx.x]) : 1.f;  // 1 / temperature
  const float p_keep = top_p ? fmaxf(top_p[blockIdx.x], 0.f) : 1.f;

  // Every pass walks the row in tiles of kTile tokens; the next tile's loads are issued before the
  // current tile is processed.
#define PB_FOR_TILES(cond, ...)                                              \
  {                                                                          \
    float cur[kPerThread];                                                   \
    load_tokens<T>(row, vocab, vec, 0, temp, cur);                           \
    for (int base = 0; base < vocab && (cond); base += kTile) {              \
      float nxt[kPerThread];                                                 \
      if (base + kTile < vocab) load_tokens<T>(row, vocab, vec, base + kTile, temp, nxt); \
      __VA_ARGS__                                                            \
      _Pragma("unroll") for (int j = 0; j < kPerThread; ++j) cur[j] = nxt[j]; \
    }                                                                        \
  }

  // pass 1: max of the scaled row
  float mx = -INFINITY;
  PB_FOR_TILES(true, {
    _Pragma("unroll") for (int j = 0; j < kPerThread; ++j) mx = fmaxf(mx, cur[j]);
  })
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) sh.warp_max[wid] = mx;
  __syncthreads();
  mx = lane < kSampWarps ? sh.warp_max[lane] : -INFINITY;
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));

  // `final_key` ends as the key of the tie class at the nucleus edge
  u64 final_key = ~0ull;   // ~0: every token is kept
  u64 budget = 0, total_mass = 0, kept_before = 0;  // kept_before: mass of the tokens with key < final_key
  u64 kept_mass = 0;
  int last_tie = -1;
  if (p_keep >= 1.f) {  // no nucleus: only the total weight is needed
    u64 mine = 0;
    PB_FOR_TILES(true, {
      _Pragma("unroll") for (int j = 0; j < kPerThread; ++j) mine += token_weight(mx - cur[j]);
    })
    block_excl_scan(mine, sh, total_mass);
    kept_mass = total_mass;
  } else {
    // pass 2: first histogram level over the whole row
    for (int b = tid; b < kBins; b += kSampThreads) sh.hist_lo[b] = 0, sh.hist_hi[b] = 0;
    if (tid == 0) sh.list_n = 0, sh.tie_n = 0, sh.last_kept_tie = -1, sh.tie_mass = 0;
    __syncthreads();
    PB_FOR_TILES(true, {
      _Pragma("unroll") for (int j = 0; j < kPerThread; ++j) {
        const float d = mx - cur[j];
        const u64 q = token_weight(d);
        if (q) hist_add(sh, token_bin1(d), q);
      }
    })
    __syncthreads();
    int cross = settle_level(sh, p_keep, budget, kept_before, total_mass);
    kept_mass = total_mass;
    if (cross != kBins) {
      final_key = ((u64)cross << 22) | ((1ull << 22) - 1);
      // pass 3: the tokens of that bin, into the list if they fit
      PB_FOR_TILES(true, {
        _Pragma("unroll") for (int j = 0; j < kPerThread; ++j) {
          const float d = mx - cur[j];
          if (token_in_bin1(d, cross) && token_weight(d)) {
            const int slot = atomicAdd(&sh.list_n, 1);
            if (slot < kListCap) sh.list_d[slot] = d, sh.list_i[slot] = base + tid * kPerThread + j;
          }
        }
      })
      __syncthreads();
      const int list_n = sh.list_n;
      const bool listed = list_n <= kListCap;
      bool ties_done = false;
      for (int level = 1; level < 3; ++level) {
        const int shift = 22 - 11 * level;
        for (int b = tid; b < kBins; b += kSampThreads) sh.hist_lo[b] = 0, sh.hist_hi[b] = 0;
        __syncthreads();
        if (listed) {
          for (int e = tid; e < list_n; e += kSampThreads) refine_add(sh, sh.list_d[e], level, final_key);
        } else {
          PB_FOR_TILES(true, {
            _Pragma("unroll") for (int j = 0; j < kPerThread; ++j) {
              const float d = mx - cur[j];
              if (token_in_bin1(d, (int)(final_key >> 22))) refine_add(sh, d, level, final_key);
            }
          })
        }
        __syncthreads();
        u64 unused;
        cross = settle_level(sh, -1.f, budget, kept_before, unused);
        if (cross == kBins) break;  // cannot happen: the bin's mass exceeded the budget one level up
        final_key = (final_key >> (shift + 11) << (shift + 11)) | ((u64)cross << shift) | ((1ull << shift) - 1);
      }
      // the tie class in index order: kept while the mass of the ties before a token fits the budget
      if (listed) {
        for (int e = tid; e < list_n; e += kSampThreads) {
          const float d = sh.list_d[e];
          if (token_key(d) == final_key) {
            const int slot = atomicAdd(&sh.tie_n, 1);
            if (slot < 32) sh.tie_q[slot] = token_weight(d), sh.tie_i[slot] = sh.list_i[e];
          }
        }
        __syncthreads();
        const int tie_n = sh.tie_n;
        if (tie_n <= 32) {  // one warp: mass of the ties with a smaller index, by exchange
          if (wid == 0) {
            const u64 q = lane < tie_n ? sh.tie_q[lane] : 0;
            const int idx = lane < tie_n ? sh.tie_i[lane] : 0x7fffffff;
            u64 before = 0;
            for (int m = 0; m < tie_n; ++m) {
              const u64 qm = __shfl_sync(0xffffffffu, q, m);
              const int im = __shfl_sync(0xffffffffu, idx, m);
              if (im < idx) before += qm;
            }
            const bool kept = lane < tie_n && before <= budget;
            u64 mass = kept ? q : 0;
            int last = kept ? idx : -1;
            for (int o = 16; o; o >>= 1) {
              mass += __shfl_xor_sync(0xffffffffu, mass, o);
              last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
            }
            if (lane == 0) sh.tie_mass = mass, sh.last_kept_tie = last;
          }
          __syncthreads();
          kept_mass = kept_before + sh.tie_mass;
          last_tie = sh.last_kept_tie;
          ties_done = true;
        }
      }
      if (!ties_done) {  // many ties (or no list): an index-ordered scan of the tie class over the row
        u64 carry = 0, mine = 0;
        PB_FOR_TILES(carry <= budget, {
          u64 tq[kPerThread], local = 0;
          _Pragma("unroll") for (int j = 0; j < kPerThread; ++j) {
            const float d = mx - cur[j];
            tq[j] = token_side(d, final_key) == 0 ? token_weight(d) : 0;
            local += tq[j];
          }
          u64 total;
          u64 before = carry + block_excl_scan(local, sh, total);
          if (local) {
            _Pragma("unroll") for (int j = 0; j < kPerThread; ++j) {
              if (tq[j] && before <= budget) {
                mine += tq[j];
                atomicMax(&sh.last_kept_tie, base + tid * kPerThread + j);
              }
              before += tq[j];
            }
          }
          carry += total;
        })
        u64 tie_mass;
        block_excl_scan(mine, sh, tie_mass);   // its barriers also order the atomicMax before the read
        last_tie = sh.last_kept_tie;
        kept_mass = kept_before + tie_mass;
      }
    }
  }

  // pass 5b: inverse CDF over the kept tokens in index order
  const float u = uniforms[blockIdx.x];
  u64 target = (u64)((double)fminf(fmaxf(u, 0.f), 1.f) * (double)kept_mass);
  if (kept_mass > 0 && target >= kept_mass) target = kept_mass - 1;
  if (tid == 0) sh.found = 0x7fffffff;
  __syncthreads();
  {
    u64 carry = 0;
    PB_FOR_TILES(carry <= target, {
      u64 w[kPerThread], local = 0;
      _Pragma("unroll") for (int j = 0; j < kPerThread; ++j) {
        const float d = mx - cur[j];
        bool kept = true;
        if (final_key != ~0ull) {
          const int side = token_side(d, final_key);
          kept = side < 0 || (side == 0 && base + tid * kPerThread + j <= last_tie);
        }
        w[j] = kept ? token_weight(d) : 0;
        local += w[j];
      }
      u64 total;
      u64 before = carry + block_excl_scan(local, sh, total);
      if (local && before <= target && before + local > target) {  // exactly one thread, exactly one token
        _Pragma("unroll") for (int j = 0; j < kPerThread; ++j) {
          if (w[j] && before <= target && before + w[j] > target) sh.found = base + tid * kPerThread + j;
          before += w[j];
        }
      }
      carry += total;
    })
  }
#undef PB_FOR_TILES
  __syncthreads();
  if (tid == 0) ids[blockIdx.x] = sh.found == 0x7fffffff ? (long long)(vocab - 1) : (long long)sh.found;
}

}  // namespace
}  // namespace pb

extern "C" int pb_sample_top_p(const void* logits, int32_t dtype, int32_t num_rows, int32_t vocab, int64_t row_stride,
                               const float* temperature, const float* top_p, const float* uniforms, int64_t* ids,
                               void* stream) {
  if (num_rows < 0 || vocab <= 0 || row_stride < vocab) return PB_ERR_INVALID_ARG;
  if (num_rows == 0) return PB_OK;
  if (!logits || !uniforms || !ids) return PB_ERR_INVALID_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  long long* out = reinterpret_cast<long long*>(ids);
  switch (dtype) {
    case PB_F32:
      pb::sample_top_p_kernel<float><<<num_rows, pb::kSampThreads, 0, s>>>(
          static_cast<const float*>(logits), vocab, row_stride, temperature, top_p, uniforms, out);
      break;
    case PB_F16:
      pb::sample_top_p_kernel<__half><<<num_rows, pb::kSampThreads, 0, s>>>(
          static_cast<const __half*>(logits), vocab, row_stride, temperature, top_p, uniforms, out);
      break;
    case PB_BF16:
      pb::sample_top_p_kernel<__nv_bfloat16><<<num_rows, pb::kSampThreads, 0, s>>>(
          static_cast<const __nv_bfloat16*>(logits), vocab, row_stride, temperature, top_p, uniforms, out);
      break;
    default:
      return PB_ERR_UNSUPPORTED;
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { pb::set_cuda_error(e); return PB_ERR_LAUNCH; }
  return PB_OK;
}
