// Whole-block copies of the paged KV caches: copy-on-write inside the caches of all layers, and
// swaps between a GPU cache and a host (or second GPU) cache. Pure byte movement.
//
// Reference counterparts: copy_blocks / swap_blocks of the vendored cache extension
// (3rdparty/vllm/csrc/cache_kernels.cu:9-138); Parrot's builtin engine does not call them (no
// preemption, no copy-on-write in parrot/engine/context/block_context.py), they complete the cache
// operator set for engines that do.
#include "common.cuh"

namespace pb {
namespace {

constexpr int kCopyThreads = 256;
constexpr int kCopySlices = 8;  // CTAs that share one (pair, layer, K|V) block

// grid (pairs, 2 * layers, slices): block pair p of layer y / 2, K cache (y even) or V cache (y odd)
__global__ void __launch_bounds__(kCopyThreads) copy_blocks_kernel(
    const long long* __restrict__ key_ptrs, const long long* __restrict__ value_ptrs,
    const long long* __restrict__ pairs, const long long block_bytes, const long long num_blocks) {
  const long long src = pairs[2 * blockIdx.x], dst = pairs[2 * blockIdx.x + 1];
  if (src < 0 || src >= num_blocks || dst < 0 || dst >= num_blocks || src == dst) return;  // never touch memory outside the cache
  const int layer = blockIdx.y >> 1;
  uint8_t* base = reinterpret_cast<uint8_t*>((blockIdx.y & 1) ? value_ptrs[layer] : key_ptrs[layer]);
  const uint4* s = reinterpret_cast<const uint4*>(base + src * block_bytes);
  uint4* t = reinterpret_cast<uint4*>(base + dst * block_bytes);
  const long long n = block_bytes / 16;
  for (long long i = (long long)blockIdx.z * kCopyThreads + threadIdx.x; i < n; i += (long long)gridDim.z * kCopyThreads)
    t[i] = s[i];
}

}  // namespace
}  // namespace pb

extern "C" {

int pb_copy_blocks(const int64_t* key_cache_ptrs, const int64_t* value_cache_ptrs, int32_t num_layers,
                   const int64_t* block_pairs, int64_t num_pairs, int64_t block_bytes, int64_t num_blocks,
                   void* stream) {
  if (num_layers < 0 || num_pairs < 0 || block_bytes <= 0 || num_blocks <= 0) return PB_ERR_INVALID_ARG;
  if (num_layers == 0 || num_pairs == 0) return PB_OK;
  if (!key_cache_ptrs || !value_cache_ptrs || !block_pairs) return PB_ERR_INVALID_ARG;
  if (block_bytes % 16 != 0) return PB_ERR_UNSUPPORTED;  // every cache layout of this library has 16-byte rows
  if (num_pairs > 0x7fffffffll || num_layers > 32767) return PB_ERR_INVALID_ARG;
  const dim3 grid((unsigned)num_pairs, (unsigned)(2 * num_layers), pb::kCopySlices);
  pb::copy_blocks_kernel<<<grid, pb::kCopyThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const long long*>(key_cache_ptrs), reinterpret_cast<const long long*>(value_cache_ptrs),
      reinterpret_cast<const long long*>(block_pairs), block_bytes, num_blocks);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { pb::set_cuda_error(e); return PB_ERR_LAUNCH; }
  return PB_OK;
}

int pb_swap_blocks(const void* src, void* dst, const int64_t* host_block_pairs, int64_t num_pairs,
                   int64_t block_bytes, int64_t src_blocks, int64_t dst_blocks, int32_t direction, void* stream) {
  if (num_pairs < 0 || block_bytes <= 0 || src_blocks <= 0 || dst_blocks <= 0) return PB_ERR_INVALID_ARG;
  if (num_pairs == 0) return PB_OK;
  if (!src || !dst || !host_block_pairs) return PB_ERR_INVALID_ARG;
  cudaMemcpyKind kind;
  switch (direction) {
    case 0: kind = cudaMemcpyDeviceToDevice; break;
    case 1: kind = cudaMemcpyDeviceToHost; break;
    case 2: kind = cudaMemcpyHostToDevice; break;
    default: return PB_ERR_INVALID_ARG;
  }
  for (int64_t i = 0; i < num_pairs; ++i)
    if (host_block_pairs[2 * i] < 0 || host_block_pairs[2 * i] >= src_blocks || host_block_pairs[2 * i + 1] < 0 ||
        host_block_pairs[2 * i + 1] >= dst_blocks)
      return PB_ERR_INVALID_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // one asynchronous copy per RUN of pairs whose source and destination blocks are both consecutive
  for (int64_t i = 0; i < num_pairs;) {
    int64_t j = i + 1;
    while (j < num_pairs && host_block_pairs[2 * j] == host_block_pairs[2 * (j - 1)] + 1 &&
           host_block_pairs[2 * j + 1] == host_block_pairs[2 * (j - 1) + 1] + 1)
      ++j;
    const cudaError_t e = cudaMemcpyAsync(static_cast<uint8_t*>(dst) + host_block_pairs[2 * i + 1] * block_bytes,
                                          static_cast<const uint8_t*>(src) + host_block_pairs[2 * i] * block_bytes,
                                          (size_t)((j - i) * block_bytes), kind, s);
    if (e != cudaSuccess) { pb::set_cuda_error(e); return PB_ERR_LAUNCH; }
    i = j;
  }
  return PB_OK;
}

}  // extern "C"
