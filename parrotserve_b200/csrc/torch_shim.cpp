// Torch-extension shim: the pybind11 surface of the reference's two native modules, forwarding to the
// C ABI of this library (include/parrot_b200_attn.h).
//
//   attention_ops  = parrot.attention_ops   (csrc/attention.cpp:49-62)
//       single_query_cached_kv_attention / _prev_attention / _post_attention
//   cache_ops      = vllm.cache_ops         (3rdparty/vllm/csrc/cache.cpp:30-46)
//       swap_blocks / copy_blocks / reshape_and_cache / gather_cached_kv
//
// Same function names, argument lists and types (torch::Tensor&, float scale, int block_size,
// int max_context_len, c10::optional<Tensor> alibi_slopes; std::map block mappings), same behaviour
// at the edge: void functions that write in place, launch on the current CUDA stream and raise a
// Python RuntimeError through TORCH_CHECK on anything unsupported
// (csrc/attention/attention_post_kernels.cu:448,500,525). The one thing the reference's kernels do
// not need and ours do is scratch memory: the shim keeps one grow-only torch buffer per device.
//
// Built as ONE shared object with two submodules; the package's torch_ops.py loads it and can
// install the submodules under the reference's import names.
#include <ATen/cuda/CUDAContext.h>
#include <c10/util/Optional.h>
#include <torch/extension.h>

#include <cstdarg>
#include <cstdio>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/parrot_b200_attn.h"

namespace {

// Error texts are formatted here and handed to TORCH_CHECK as one string.
std::string text(const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  return std::string(buf);
}

int dtype_code(const torch::Tensor& t) {
  switch (t.scalar_type()) {
    case at::ScalarType::Float: return PB_F32;
    case at::ScalarType::Half: return PB_F16;
    case at::ScalarType::BFloat16: return PB_BF16;
    default: TORCH_CHECK(false, text("Unsupported data type: %s", c10::toString(t.scalar_type()))); return -1;
  }
}

void check_rc(int rc, const char* what) {
  if (rc == PB_OK) return;
  TORCH_CHECK(rc != PB_ERR_UNSUPPORTED, text("%s: unsupported head size, block size or data type", what));
  TORCH_CHECK(rc != PB_ERR_LAUNCH, text("%s: CUDA launch failed: %s", what, pb_last_cuda_error()));
  TORCH_CHECK(false, text("%s: invalid argument (pb_status %d)", what, rc));
}

// grow-only scratch per device (the C ABI never allocates)
torch::Tensor& workspace(const torch::Tensor& like, size_t bytes) {
  static std::mutex mu;
  static std::map<int, torch::Tensor> bufs;
  std::lock_guard<std::mutex> lock(mu);
  torch::Tensor& b = bufs[like.get_device()];
  if (!b.defined() || (size_t)b.numel() < bytes)
    b = torch::empty({(int64_t)std::max<size_t>(bytes, 1 << 20)}, like.options().dtype(torch::kUInt8));
  return b;
}

struct Geometry {
  int num_seqs, num_heads, head_size, num_kv_heads, max_blocks;
  int64_t q_stride, kv_block_stride, kv_head_stride, num_blocks;
};

Geometry geometry(const torch::Tensor& out, const torch::Tensor& query, const torch::Tensor& key_cache,
                  const torch::Tensor& value_cache, const torch::Tensor& head_mapping, const torch::Tensor& block_tables,
                  const torch::Tensor& context_lens, int block_size, const c10::optional<torch::Tensor>& alibi_slopes) {
  TORCH_CHECK(!alibi_slopes.has_value(), "alibi_slopes is not supported (the reference always passes None)");
  TORCH_CHECK(query.is_cuda() && out.is_cuda() && key_cache.is_cuda() && value_cache.is_cuda(), "CUDA tensors expected");
  TORCH_CHECK(query.dim() == 3 && key_cache.dim() == 5 && value_cache.dim() == 4, "unexpected tensor ranks");
  TORCH_CHECK(value_cache.size(3) == block_size, text("Unsupported block size: %d", block_size));
  TORCH_CHECK(out.is_contiguous(), "out must be contiguous");
  TORCH_CHECK(block_tables.scalar_type() == at::ScalarType::Int && context_lens.scalar_type() == at::ScalarType::Int &&
                  head_mapping.scalar_type() == at::ScalarType::Int,
              "block_tables, context_lens and head_mapping must be int32");
  TORCH_CHECK(block_tables.is_contiguous() && context_lens.is_contiguous() && head_mapping.is_contiguous(),
              "index tensors must be contiguous");
  Geometry g;
  g.num_seqs = (int)query.size(0);
  g.num_heads = (int)query.size(1);
  g.head_size = (int)query.size(2);
  g.num_kv_heads = (int)value_cache.size(1);
  g.max_blocks = block_tables.dim() == 2 ? (int)block_tables.size(1) : 0;
  g.q_stride = query.stride(0);
  g.kv_block_stride = key_cache.stride(0);
  g.kv_head_stride = key_cache.stride(1);
  g.num_blocks = key_cache.size(0);
  TORCH_CHECK(value_cache.size(2) == g.head_size, text("Unsupported head size: %d", g.head_size));
  return g;
}

typedef int (*StatsFn)(void*, const void*, const void*, const void*, const int32_t*, float, const int32_t*, const int32_t*,
                       float*, float*, int32_t, int32_t, int32_t, int32_t, int32_t, int32_t, int32_t, int64_t, int64_t,
                       int64_t, int64_t, int32_t, void*, size_t, void*);

void run_stats(StatsFn fn, const char* name, torch::Tensor& out, torch::Tensor& query, torch::Tensor& key_cache,
               torch::Tensor& value_cache, torch::Tensor& head_mapping, float scale, torch::Tensor& block_tables,
               torch::Tensor& context_lens, torch::Tensor& qk_maxs, torch::Tensor& exp_sums, int block_size,
               int max_context_len, const c10::optional<torch::Tensor>& alibi_slopes) {
  const Geometry g = geometry(out, query, key_cache, value_cache, head_mapping, block_tables, context_lens, block_size, alibi_slopes);
  TORCH_CHECK(qk_maxs.scalar_type() == at::ScalarType::Float && exp_sums.scalar_type() == at::ScalarType::Float &&
                  qk_maxs.is_contiguous() && exp_sums.is_contiguous(),
              "qk_maxs and exp_sums must be contiguous float32 tensors");
  const size_t need = pb_single_query_workspace_bytes(g.num_seqs, g.num_heads, g.head_size, block_size, g.max_blocks);
  TORCH_CHECK(need > 0, text("%s: unsupported head size %d or block size %d", name, g.head_size, block_size));
  torch::Tensor& ws = workspace(query, need);
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  check_rc(fn(out.data_ptr(), query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(), head_mapping.data_ptr<int32_t>(),
              scale, block_tables.data_ptr<int32_t>(), context_lens.data_ptr<int32_t>(), qk_maxs.data_ptr<float>(),
              exp_sums.data_ptr<float>(), block_size, max_context_len, g.num_seqs, g.num_heads, g.num_kv_heads, g.head_size,
              g.max_blocks, g.q_stride, g.kv_block_stride, g.kv_head_stride, g.num_blocks, dtype_code(query), ws.data_ptr(),
              (size_t)ws.numel(), stream),
           name);
}

// ---- parrot.attention_ops (csrc/attention.cpp:4-47) ----
void single_query_cached_kv_attention(torch::Tensor& out, torch::Tensor& query, torch::Tensor& key_cache,
                                      torch::Tensor& value_cache, torch::Tensor& head_mapping, float scale,
                                      torch::Tensor& block_tables, torch::Tensor& block_lens, torch::Tensor& block_nums,
                                      torch::Tensor& context_lens, int block_size, int max_context_len,
                                      const c10::optional<torch::Tensor>& alibi_slopes) {
  // block_lens is never read by the reference kernel and block_nums only bounds the blocks it walks
  // (csrc/attention/attention_kernels.cu:159-162): the attention is the one over context_lens tokens.
  (void)block_lens;
  (void)block_nums;
  const Geometry g = geometry(out, query, key_cache, value_cache, head_mapping, block_tables, context_lens, block_size, alibi_slopes);
  const size_t need = pb_single_query_workspace_bytes(g.num_seqs, g.num_heads, g.head_size, block_size, g.max_blocks);
  TORCH_CHECK(need > 0, text("single_query_cached_kv_attention: unsupported head size %d or block size %d", g.head_size, block_size));
  torch::Tensor& ws = workspace(query, need);
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  check_rc(pb_single_query_cached_kv_attention(
               out.data_ptr(), query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(), head_mapping.data_ptr<int32_t>(),
               scale, block_tables.data_ptr<int32_t>(), context_lens.data_ptr<int32_t>(), block_size, max_context_len,
               g.num_seqs, g.num_heads, g.num_kv_heads, g.head_size, g.max_blocks, g.q_stride, g.kv_block_stride,
               g.kv_head_stride, g.num_blocks, dtype_code(query), ws.data_ptr(), (size_t)ws.numel(), stream),
           "single_query_cached_kv_attention");
}

void single_query_cached_kv_prev_attention(torch::Tensor& out, torch::Tensor& query, torch::Tensor& key_cache,
                                           torch::Tensor& value_cache, torch::Tensor& head_mapping, float scale,
                                           torch::Tensor& block_tables, torch::Tensor& context_lens, torch::Tensor& qk_maxs,
                                           torch::Tensor& exp_sums, int block_size, int max_context_len,
                                           const c10::optional<torch::Tensor>& alibi_slopes) {
  run_stats(pb_single_query_cached_kv_prev_attention, "single_query_cached_kv_prev_attention", out, query, key_cache,
            value_cache, head_mapping, scale, block_tables, context_lens, qk_maxs, exp_sums, block_size, max_context_len,
            alibi_slopes);
}

void single_query_cached_kv_post_attention(torch::Tensor& out, torch::Tensor& query, torch::Tensor& key_cache,
                                           torch::Tensor& value_cache, torch::Tensor& head_mapping, float scale,
                                           torch::Tensor& block_tables, torch::Tensor& context_lens,
                                           torch::Tensor& prev_qk_maxs, torch::Tensor& prev_exp_sums, int block_size,
                                           int max_context_len, const c10::optional<torch::Tensor>& alibi_slopes) {
  run_stats(pb_single_query_cached_kv_post_attention, "single_query_cached_kv_post_attention", out, query, key_cache,
            value_cache, head_mapping, scale, block_tables, context_lens, prev_qk_maxs, prev_exp_sums, block_size,
            max_context_len, alibi_slopes);
}

// ---- vllm.cache_ops (3rdparty/vllm/csrc/cache.cpp:6-28) ----
void kv_rows(bool fill, torch::Tensor& key, torch::Tensor& value, torch::Tensor& key_cache, torch::Tensor& value_cache,
             torch::Tensor& slot_mapping) {
  TORCH_CHECK(key.is_cuda() && value.is_cuda() && key_cache.is_cuda() && value_cache.is_cuda() && slot_mapping.is_cuda(),
              "CUDA tensors expected");
  TORCH_CHECK(key.dim() == 3 && value.dim() == 3 && key_cache.dim() == 5 && value_cache.dim() == 4, "unexpected tensor ranks");
  const auto st = slot_mapping.scalar_type();
  TORCH_CHECK(st == at::ScalarType::Int || st == at::ScalarType::Long, "slot_mapping must be int32 or int64");
  TORCH_CHECK(slot_mapping.is_contiguous() && slot_mapping.numel() == key.size(0), "one slot per token expected");
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const int rc = fill
      ? pb_reshape_and_cache(key.data_ptr(), value.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
                             slot_mapping.data_ptr(), st == at::ScalarType::Long ? 1 : 0, key.size(0), (int)key.size(1),
                             (int)key.size(2), (int)value_cache.size(3), key.stride(0), value.stride(0), key_cache.stride(0),
                             key_cache.stride(1), key_cache.size(0), dtype_code(key), stream)
      : pb_gather_cached_kv(key.data_ptr(), value.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
                            slot_mapping.data_ptr(), st == at::ScalarType::Long ? 1 : 0, key.size(0), (int)key.size(1),
                            (int)key.size(2), (int)value_cache.size(3), key.stride(0), value.stride(0), key_cache.stride(0),
                            key_cache.stride(1), key_cache.size(0), dtype_code(key), stream);
  check_rc(rc, fill ? "reshape_and_cache" : "gather_cached_kv");
}

void reshape_and_cache(torch::Tensor& key, torch::Tensor& value, torch::Tensor& key_cache, torch::Tensor& value_cache,
                       torch::Tensor& slot_mapping) {
  kv_rows(true, key, value, key_cache, value_cache, slot_mapping);
}

void gather_cached_kv(torch::Tensor& key, torch::Tensor& value, torch::Tensor& key_cache, torch::Tensor& value_cache,
                      torch::Tensor& slot_mapping) {
  kv_rows(false, key, value, key_cache, value_cache, slot_mapping);
}

void copy_blocks(std::vector<torch::Tensor>& key_caches, std::vector<torch::Tensor>& value_caches,
                 const std::map<int64_t, std::vector<int64_t>>& block_mapping) {
  const int num_layers = (int)key_caches.size();
  TORCH_CHECK(num_layers == (int)value_caches.size(), "one key cache and one value cache per layer expected");
  if (num_layers == 0) return;
  std::vector<int64_t> kp(num_layers), vp(num_layers), pairs;
  for (int i = 0; i < num_layers; ++i) {
    TORCH_CHECK(key_caches[i].is_cuda() && key_caches[i].is_contiguous() && value_caches[i].is_contiguous(),
                "contiguous CUDA caches expected");
    kp[i] = reinterpret_cast<int64_t>(key_caches[i].data_ptr());
    vp[i] = reinterpret_cast<int64_t>(value_caches[i].data_ptr());
  }
  for (const auto& kv : block_mapping)
    for (int64_t dst : kv.second) { pairs.push_back(kv.first); pairs.push_back(dst); }
  if (pairs.empty()) return;
  const auto dev = key_caches[0].device();
  const auto i64 = torch::TensorOptions().dtype(torch::kInt64);
  torch::Tensor kd = torch::from_blob(kp.data(), {num_layers}, i64).to(dev);
  torch::Tensor vd = torch::from_blob(vp.data(), {num_layers}, i64).to(dev);
  torch::Tensor pd = torch::from_blob(pairs.data(), {(int64_t)pairs.size()}, i64).to(dev);
  const int64_t block_bytes = key_caches[0][0].numel() * key_caches[0].element_size();
  check_rc(pb_copy_blocks(kd.data_ptr<int64_t>(), vd.data_ptr<int64_t>(), num_layers, pd.data_ptr<int64_t>(),
                          (int64_t)pairs.size() / 2, block_bytes, key_caches[0].size(0),
                          at::cuda::getCurrentCUDAStream()),
           "copy_blocks");
}

void swap_blocks(torch::Tensor& src, torch::Tensor& dst, const std::map<int64_t, int64_t>& block_mapping) {
  int direction;
  if (src.is_cuda() && dst.is_cuda()) {
    TORCH_CHECK(src.get_device() == dst.get_device(), "src and dst must be on the same GPU");
    direction = 0;
  } else if (src.is_cuda() && dst.is_cpu()) {
    direction = 1;
  } else if (src.is_cpu() && dst.is_cuda()) {
    direction = 2;
  } else {
    TORCH_CHECK(false, "Invalid device combination");
  }
  TORCH_CHECK(src.is_contiguous() && dst.is_contiguous() && src.scalar_type() == dst.scalar_type() &&
                  src[0].numel() == dst[0].numel(),
              "src and dst must be contiguous caches of one data type and block size");
  std::vector<int64_t> pairs;
  for (const auto& kv : block_mapping) { pairs.push_back(kv.first); pairs.push_back(kv.second); }
  if (pairs.empty()) return;
  check_rc(pb_swap_blocks(src.data_ptr(), dst.data_ptr(), pairs.data(), (int64_t)pairs.size() / 2,
                          src[0].numel() * src.element_size(), src.size(0), dst.size(0), direction,
                          at::cuda::getCurrentCUDAStream()),
           "swap_blocks");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "pybind surface of parrot.attention_ops and vllm.cache_ops over the B200 attention library";
  auto a = m.def_submodule("attention_ops", "parrot.attention_ops (csrc/attention.cpp:49-62)");
  a.def("single_query_cached_kv_attention", &single_query_cached_kv_attention,
        "Compute the attention between an input query and the cached key/value tensors");
  a.def("single_query_cached_kv_prev_attention", &single_query_cached_kv_prev_attention,
        "Compute the attention between an input query and the cached key/value tensors and log middle results");
  a.def("single_query_cached_kv_post_attention", &single_query_cached_kv_post_attention,
        "Compute the attention between an input query and the cached key/value tensors based on previous results");
  auto c = m.def_submodule("cache_ops", "vllm.cache_ops (3rdparty/vllm/csrc/cache.cpp:30-46)");
  c.def("swap_blocks", &swap_blocks, "Swap in (out) the cache blocks from src to dst");
  c.def("copy_blocks", &copy_blocks, "Copy the cache blocks from src to dst");
  c.def("reshape_and_cache", &reshape_and_cache, "Reshape the key and value tensors and cache them");
  c.def("gather_cached_kv", &gather_cached_kv, "Gather key and value from the cache into contiguous QKV tensors");
}
