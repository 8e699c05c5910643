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
//      so the result is the same on every run;
//   3. the bin in which the mass sorted before a token first exceeds top_p * total is refined twice by
//      2048 (resolution 2^-28 in the logit): tokens before that point are kept, tokens after it dropped,
//      tokens inside the last bin (ties) are kept in index order while the mass before them allows it,
//      which is what a stable descending sort does;
//   4. the draw is the inverse CDF over the kept tokens in index order for the caller's uniform number.
#include "common.cuh"

namespace pb {
namespace {

constexpr int kSampThreads = 1024;
constexpr int kSampWarps = kSampThreads / 32;
constexpr int kBins = 2048;  // two per thread
constexpr float kFixedOne = 1099511627776.f;  // 2^40
typedef unsigned long long u64;

struct SampShared {
  u64 hist[kBins];
  u64 warp_tot[kSampWarps + 1];
  float warp_max[kSampWarps];
  u64 budget_next;
  int cross;
  int last_kept_tie;
  int found;
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
    const u64 t = sh.warp_tot[lane];
    u64 it = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const u64 n = __shfl_up_sync(0xffffffffu, it, o);
      if (lane >= o) it += n;
    }
    sh.warp_tot[lane] = it - t;
    if (lane == 31) sh.warp_tot[kSampWarps] = it;
  }
  __syncthreads();
  const u64 excl = sh.warp_tot[wid] + incl - v;
  total = sh.warp_tot[kSampWarps];
  __syncthreads();  // warp_tot is reused by the next call
  return excl;
}

// One token of the row: fixed-point weight and the 33-bit three-level key (smaller key = larger logit).
template <typename T>
__device__ __forceinline__ void token(const T* __restrict__ row, int i, float temp, float mx, u64& q, u64& key) {
  const float x = __fdiv_rn(to_float<T>(row[i]), temp);
  const float d = mx - x;
  q = __float2ull_rd(exp2f(-d * 1.4426950408889634f) * kFixedOne);
  const float t0 = d * 64.f;
  const int k1 = min(__float2int_rz(t0), kBins - 1);
  const float t1 = (t0 - (float)k1) * (float)kBins;
  const int k2 = min(max(__float2int_rz(t1), 0), kBins - 1);
  const float t2 = (t1 - (float)k2) * (float)kBins;
  const int k3 = min(max(__float2int_rz(t2), 0), kBins - 1);
  key = ((u64)max(k1, 0) << 22) | ((u64)k2 << 11) | (u64)k3;
}

template <typename T>
__global__ void __launch_bounds__(kSampThreads) sample_top_p_kernel(
    const T* __restrict__ logits, const int vocab, const long long row_stride, const float* __restrict__ temperature,
    const float* __restrict__ top_p, const float* __restrict__ uniforms, long long* __restrict__ ids) {
  __shared__ SampShared sh;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const T* row = logits + (long long)blockIdx.x * row_stride;
  const float temp = temperature ? temperature[blockIdx.x] : 1.f;
  const float p_keep = top_p ? top_p[blockIdx.x] : 1.f;

  // pass 1: max of the scaled row
  float mx = -INFINITY;
  for (int i = tid; i < vocab; i += kSampThreads) mx = fmaxf(mx, __fdiv_rn(to_float<T>(row[i]), temp));
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) sh.warp_max[wid] = mx;
  __syncthreads();
  mx = sh.warp_max[lane];
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));

  // passes 2-4: three histogram levels; `final_key` ends as the key of the tie class at the nucleus edge
  u64 final_key = ~0ull;   // ~0: every token is kept
  u64 budget = 0, total_mass = 0, kept_before = 0;  // kept_before: mass of the tokens with key < final_key
  for (int level = 0; level < 3; ++level) {
    const int shift = 22 - 11 * level;  // bits of the key below this level's bin
    for (int b = tid; b < kBins; b += kSampThreads) sh.hist[b] = 0;
    if (tid == 0) sh.cross = kBins;
    __syncthreads();
    for (int base = 0; base < vocab; base += kSampThreads) {
      const int i = base + tid;
      u64 q = 0, key = 0;
      bool match = false;
      if (i < vocab) {
        token<T>(row, i, temp, mx, q, key);
        match = level == 0 || (key >> (shift + 11)) == (final_key >> (shift + 11));
      }
      const unsigned ballot = __ballot_sync(0xffffffffu, match);
      if (ballot == 0) continue;
      const int bin = (int)((key >> shift) & (kBins - 1));
      const int ref_bin = __shfl_sync(0xffffffffu, bin, __ffs(ballot) - 1);
      if (__all_sync(0xffffffffu, !match || bin == ref_bin)) {  // one bin for the whole warp: one atomic
        u64 s = match ? q : 0;
#pragma unroll
        for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) atomicAdd(&sh.hist[ref_bin], s);
      } else if (match) {
        atomicAdd(&sh.hist[bin], q);
      }
    }
    __syncthreads();
    const u64 h0 = sh.hist[2 * tid], h1 = sh.hist[2 * tid + 1];
    u64 total;
    const u64 excl = block_excl_scan(h0 + h1, sh, total);
    if (level == 0) {
      total_mass = total;
      // a token is dropped when the mass sorted before it exceeds top_p * total
      budget = p_keep >= 1.f ? total : (u64)((double)p_keep * (double)total);
    }
    if (excl + h0 > budget) atomicMin(&sh.cross, 2 * tid);
    else if (excl + h0 + h1 > budget) atomicMin(&sh.cross, 2 * tid + 1);
    __syncthreads();
    const int cross = sh.cross;
    if (cross == kBins) break;  // (level 0 only) nothing exceeds the budget: keep everything
    if (tid == cross / 2) sh.budget_next = budget - ((cross & 1) ? excl + h0 : excl);
    __syncthreads();
    kept_before += budget - sh.budget_next;
    budget = sh.budget_next;
    final_key = (level == 0 ? 0ull : (final_key >> (shift + 11) << (shift + 11))) | ((u64)cross << shift);
    if (level < 2) final_key |= (1ull << shift) - 1;  // lower levels still open
    __syncthreads();
  }

  // pass 5a: the tie class in index order: kept while the mass of the ties before a token fits the budget
  u64 kept_mass = total_mass;
  int last_tie = -1;
  if (final_key != ~0ull) {
    if (tid == 0) sh.last_kept_tie = -1;
    __syncthreads();
    u64 carry = 0, mine = 0;
    for (int base = 0; base < vocab && carry <= budget; base += kSampThreads) {
      const int i = base + tid;
      u64 q = 0, key = 0;
      if (i < vocab) token<T>(row, i, temp, mx, q, key);
      const bool tie = i < vocab && key == final_key;
      u64 total;
      const u64 before = carry + block_excl_scan(tie ? q : 0, sh, total);
      if (tie && before <= budget) {
        mine += q;
        atomicMax(&sh.last_kept_tie, i);
      }
      carry += total;
    }
    u64 tie_mass;
    block_excl_scan(mine, sh, tie_mass);   // its barriers also order the atomicMax before the read
    last_tie = sh.last_kept_tie;
    kept_mass = kept_before + tie_mass;
  }

  // pass 5b: inverse CDF over the kept tokens in index order
  const float u = uniforms[blockIdx.x];
  u64 target = (u64)((double)fminf(fmaxf(u, 0.f), 1.f) * (double)kept_mass);
  if (kept_mass > 0 && target >= kept_mass) target = kept_mass - 1;
  if (tid == 0) sh.found = 0x7fffffff;
  __syncthreads();
  u64 carry = 0;
  for (int base = 0; base < vocab && carry <= target; base += kSampThreads) {
    const int i = base + tid;
    u64 q = 0, key = 0;
    if (i < vocab) token<T>(row, i, temp, mx, q, key);
    const bool kept = i < vocab && (key < final_key || (key == final_key && i <= last_tie));
    const u64 w = kept ? q : 0;
    u64 total;
    const u64 before = carry + block_excl_scan(w, sh, total);
    if (w > 0 && before <= target && before + w > target) sh.found = i;  // exactly one token satisfies this
    carry += total;
  }
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
