// Paged KV cache fill / gather / row moves. Pure byte movement: bit-exact by construction.
//
//   fill   : new K/V rows [T, H, D]  ->  K [NB, H, D/x, B, x], V [NB, H, D, B] at slot_mapping[t]
//   gather : the inverse
//   move   : dest[dest_idx[i]] = row of slot src_slots[i] (K or V)
//   rows   : dest[dest_idx[i]] = src[src_idx[i]] over plain rows
//
// A run of tokens whose slots are consecutive inside one physical block (prefill) is handled
// by one warp per head: K moves as 16-byte chunks, V is transposed through shared memory so a
// full block is written with 16-byte stores; a lone decode token degenerates to the scattered
// element writes the layout forces.
//
// Reference counterparts: reshape_and_cache_kernel / gather_cached_kv_kernel
// (3rdparty/vllm/csrc/cache_kernels.cu:142-182, 229-344) and the Triton movers
// (parrot/engine/builtin/kernels/tokens_moving.py:25-64, 104-160, 222-268).
#include "common.cuh"

namespace pb {
namespace {

constexpr int kFillWarps = 4;

__device__ __forceinline__ long long load_slot(const void* slots, int is64, long long t) {
  return is64 ? reinterpret_cast<const long long*>(slots)[t]
              : (long long)reinterpret_cast<const int*>(slots)[t];
}

template <int E> struct ElemOf;
template <> struct ElemOf<2> { using type = uint16_t; };
template <> struct ElemOf<4> { using type = uint32_t; };

// FILL == true : scatter rows into the cache.   FILL == false : gather rows out of the cache.
template <int E, bool FILL>
__global__ void __launch_bounds__(kFillWarps * 32) kv_run_kernel(
    uint8_t* __restrict__ key, uint8_t* __restrict__ value, uint8_t* __restrict__ kcache,
    uint8_t* __restrict__ vcache, const void* __restrict__ slots, const int is64,
    const long long T, const int H, const int D, const int B, const long long key_stride,
    const long long value_stride, const long long kbs, const long long khs,
    const long long num_blocks, int* __restrict__ status) {
  using elem_t = typename ElemOf<E>::type;
  extern __shared__ __align__(16) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t = blockIdx.x;
  // Launched with programmatic stream serialization, so the CTAs are resident while the kernel
  // before this one drains: wait for it before reading anything, then let the next kernel (an
  // attention kernel or the planner) set itself up; those wait before they read the cache.
  pdl_wait();
  pdl_trigger();
  // the three slot reads do not depend on each other: issue them together
  const long long slot = load_slot(slots, is64, t);
  const long long prev = (t > 0) ? load_slot(slots, is64, t - 1) : -2;
  const long long next = (lane > 0 && lane < B && t + lane < T) ? load_slot(slots, is64, t + lane) : -3;
  if (slot < 0) return;
  const long long blk = slot / B;
  const int off0 = (int)(slot - blk * B);
  if (blk >= num_blocks) {
    if (threadIdx.x == 0 && status) atomicMax(status, kStatusBadIndex);
    return;
  }
  const bool leader = (t == 0) || (prev + 1 != slot) || (off0 == 0);
  if (!leader) return;
  // run length: tokens t+i with slot+i, staying inside the block
  bool ok = (lane == 0);
  if (lane > 0 && lane < B && off0 + lane < B && t + lane < T) ok = (next == slot + lane);
  const unsigned mask = __ballot_sync(0xffffffffu, ok);
  const int n = __ffs(~mask) - 1;  // trailing ones; mask bit 0 is always set, n in 1..B (32 -> ~mask==0)
  const int run = (~mask == 0u) ? 32 : n;

  constexpr int kVec = 16 / E;
  const int nch = D / kVec;  // 16-byte chunks per (token, head) row
  uint8_t* tile = smem + (size_t)warp * B * D * E;

  for (int h = blockIdx.y * kFillWarps + warp; h < H; h += gridDim.y * kFillWarps) {
    uint8_t* kt = kcache + ((size_t)blk * kbs + (size_t)h * khs) * E;
    uint8_t* vt = vcache + ((size_t)blk * kbs + (size_t)h * khs) * E;
    // ---- K: 16-byte chunk (token i, chunk c) <-> tile[(c*B + off0+i)] ----
    // (four chunks per lane are read before the first is written: a run of a whole block is 8 chunks
    // per lane, and one dependent load-store pair per trip to memory made the copy latency-bound)
    for (int base = 0; base < run * nch; base += 4 * 32) {
      uint4 tmp[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * 32 + lane;
        if (idx < run * nch) {
          const int i = idx / nch, c = idx - i * nch;
          const uint4* row = reinterpret_cast<const uint4*>(key + ((size_t)(t + i) * key_stride + (size_t)h * D) * E) + c;
          const uint4* cell = reinterpret_cast<const uint4*>(kt) + (size_t)c * B + off0 + i;
          tmp[u] = FILL ? *row : *cell;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * 32 + lane;
        if (idx < run * nch) {
          const int i = idx / nch, c = idx - i * nch;
          uint4* row = reinterpret_cast<uint4*>(key + ((size_t)(t + i) * key_stride + (size_t)h * D) * E) + c;
          uint4* cell = reinterpret_cast<uint4*>(kt) + (size_t)c * B + off0 + i;
          if (FILL) *cell = tmp[u]; else *row = tmp[u];
        }
      }
    }
    // ---- V: element (token i, d) <-> tile[d*B + off0+i], transposed through shared memory ----
    if (FILL) {
      for (int base = 0; base < run * nch; base += 4 * 32) {  // four loads in flight per lane, as for K
        uint4 tmp[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = base + u * 32 + lane;
          if (idx < run * nch) {
            const int i = idx / nch, c = idx - i * nch;
            tmp[u] = *(reinterpret_cast<const uint4*>(value + ((size_t)(t + i) * value_stride + (size_t)h * D) * E) + c);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = base + u * 32 + lane;
          if (idx < run * nch) reinterpret_cast<uint4*>(tile)[idx] = tmp[u];  // idx == i * nch + c
        }
      }
      __syncwarp();
      const elem_t* ts = reinterpret_cast<const elem_t*>(tile);
      for (int dd = lane; dd < D; dd += 32) {
        elem_t* dst = reinterpret_cast<elem_t*>(vt) + (size_t)dd * B + off0;
        if (run == B) {  // a full block (off0 == 0): 16-byte stores
          for (int v = 0; v < B / kVec; ++v) {
            elem_t tmp[kVec];
#pragma unroll
            for (int j = 0; j < kVec; ++j) tmp[j] = ts[(size_t)(v * kVec + j) * D + dd];
            reinterpret_cast<uint4*>(dst)[v] = *reinterpret_cast<const uint4*>(tmp);
          }
        } else {
          for (int i = 0; i < run; ++i) dst[i] = ts[(size_t)i * D + dd];
        }
      }
      __syncwarp();
    } else {
      elem_t* ts = reinterpret_cast<elem_t*>(tile);
      for (int dd = lane; dd < D; dd += 32) {
        const elem_t* src = reinterpret_cast<const elem_t*>(vt) + (size_t)dd * B + off0;
        if (run == B) {
          for (int v = 0; v < B / kVec; ++v) {
            const uint4 u = reinterpret_cast<const uint4*>(src)[v];
            const elem_t* tmp = reinterpret_cast<const elem_t*>(&u);
#pragma unroll
            for (int j = 0; j < kVec; ++j) ts[(size_t)(v * kVec + j) * D + dd] = tmp[j];
          }
        } else {
          for (int i = 0; i < run; ++i) ts[(size_t)i * D + dd] = src[i];
        }
      }
      __syncwarp();
      for (int idx = lane; idx < run * nch; idx += 32) {
        const int i = idx / nch, c = idx - i * nch;
        uint4* row = reinterpret_cast<uint4*>(value + ((size_t)(t + i) * value_stride + (size_t)h * D) * E) + c;
        *row = reinterpret_cast<const uint4*>(tile)[i * nch + c];
      }
      __syncwarp();
    }
  }
}

// ---- NeoX rotary embedding fused with the KV fill ----
// q and k rows are rotated at their token's position (first rot_dim elements of every head:
// x = d < rot_dim/2 pairs with y = d + rot_dim/2; out_x = x cos - y sin, out_y = y cos + x sin,
// cos/sin from cos_sin_cache[pos] = [cos(rot_dim/2) | sin(rot_dim/2)]); q is rewritten in place,
// the rotated k goes straight into its cache cell (and back into `key` only if asked), v is
// scattered as in the plain fill. One pass over q, k and v instead of rotary (read+write q, k)
// followed by the fill (read k, v again). Products are formed in fp32 and rounded once.
//
// Reference counterparts: rotary_embedding_neox_kernel (3rdparty/vllm/csrc/pos_encoding_kernels.cu:7-60;
// called from parrot/engine/builtin/models/llama.py:123-129 through kernels/vllm/rotary_embed.py:10-25)
// followed by reshape_and_cache_kernel (3rdparty/vllm/csrc/cache_kernels.cu:142-182).
template <typename T> struct BitsOf { using type = uint16_t; };
template <> struct BitsOf<float> { using type = uint32_t; };

template <typename T>
__device__ __forceinline__ uint4 pack16(const float* f) {
  constexpr int kVec = ElemTraits<T>::kVec;
  uint4 out;
  T* o = reinterpret_cast<T*>(&out);
#pragma unroll
  for (int j = 0; j < kVec; ++j) o[j] = from_float<T>(f[j]);
  return out;
}

// Rotates the chunk pair (cx, cy = cx + half) of one head row; cs points at the token's cos/sin row.
template <typename T>
__device__ __forceinline__ void rotate_pair(const uint4& x, const uint4& y, const uint8_t* cs, int cx, int half_chunks,
                                            uint4& ox, uint4& oy) {
  constexpr int kVec = ElemTraits<T>::kVec;
  float fx[kVec], fy[kVec], fc[kVec], fs[kVec], rx[kVec], ry[kVec];
  unpack16<T>(x, fx);
  unpack16<T>(y, fy);
  unpack16<T>(reinterpret_cast<const uint4*>(cs)[cx], fc);
  unpack16<T>(reinterpret_cast<const uint4*>(cs)[half_chunks + cx], fs);
#pragma unroll
  for (int j = 0; j < kVec; ++j) {
    rx[j] = fx[j] * fc[j] - fy[j] * fs[j];
    ry[j] = fy[j] * fc[j] + fx[j] * fs[j];
  }
  ox = pack16<T>(rx);
  oy = pack16<T>(ry);
}

template <typename T>
__global__ void __launch_bounds__(kFillWarps * 32) rotary_fill_kernel(
    uint8_t* __restrict__ query, uint8_t* __restrict__ key, const uint8_t* __restrict__ value,
    uint8_t* __restrict__ kcache, uint8_t* __restrict__ vcache, const void* __restrict__ slots, const int is64,
    const long long* __restrict__ positions, const uint8_t* __restrict__ cos_sin, const int rot_dim,
    const long long max_pos, const long long T_tok, const int Hq, const int H, const int D, const int B,
    const long long q_stride, const long long key_stride, const long long value_stride, const long long kbs,
    const long long khs, const long long num_blocks, const int write_key_back) {
  constexpr int E = (int)sizeof(T);
  constexpr int kVec = 16 / E;
  using elem_t = typename BitsOf<T>::type;
  extern __shared__ __align__(16) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t = blockIdx.x;
  pdl_wait();
  pdl_trigger();
  const int nch = D / kVec;             // 16-byte chunks per head row
  const int half = rot_dim / kVec / 2;  // chunks in each half of the rotated part
  const int units = nch - half;         // chunk pairs of the rotated part + pass-through chunks
  auto cs_row = [&](long long tok) {
    long long pos = positions[tok];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);  // clamped: never read outside the table
    return cos_sin + (size_t)pos * rot_dim * E;
  };

  // ---- q of this token, in place (every token, whether or not it leads a run of slots) ----
  {
    const uint8_t* cs = cs_row(t);
    for (int h = blockIdx.y * kFillWarps + warp; h < Hq; h += gridDim.y * kFillWarps) {
      uint4* row = reinterpret_cast<uint4*>(query + ((size_t)t * q_stride + (size_t)h * D) * E);
      for (int u = lane; u < half; u += 32) {
        uint4 ox, oy;
        rotate_pair<T>(row[u], row[u + half], cs, u, half, ox, oy);
        row[u] = ox;
        row[u + half] = oy;
      }
    }
  }

  if (kcache == nullptr) {
    // rotation only (the reference's rotary_embedding_neox): k of this token in place, no cache
    const uint8_t* cs = cs_row(t);
    for (int h = blockIdx.y * kFillWarps + warp; h < H; h += gridDim.y * kFillWarps) {
      uint4* row = reinterpret_cast<uint4*>(key + ((size_t)t * key_stride + (size_t)h * D) * E);
      for (int u = lane; u < half; u += 32) {
        uint4 ox, oy;
        rotate_pair<T>(row[u], row[u + half], cs, u, half, ox, oy);
        row[u] = ox;
        row[u + half] = oy;
      }
    }
    return;
  }

  // ---- k and v: the warp of a run's first token moves the whole run (as in the plain fill) ----
  const long long slot = load_slot(slots, is64, t);
  const long long prev = (t > 0) ? load_slot(slots, is64, t - 1) : -2;
  const long long next = (lane > 0 && lane < B && t + lane < T_tok) ? load_slot(slots, is64, t + lane) : -3;
  if (slot < 0) return;
  const long long blk = slot / B;
  const int off0 = (int)(slot - blk * B);
  if (blk >= num_blocks) return;
  const bool leader = (t == 0) || (prev + 1 != slot) || (off0 == 0);
  if (!leader) return;
  bool ok = (lane == 0);
  if (lane > 0 && lane < B && off0 + lane < B && t + lane < T_tok) ok = (next == slot + lane);
  const unsigned mask = __ballot_sync(0xffffffffu, ok);
  const int n = __ffs(~mask) - 1;
  const int run = (~mask == 0u) ? 32 : n;
  uint8_t* tile = smem + (size_t)warp * B * D * E;

  for (int h = blockIdx.y * kFillWarps + warp; h < H; h += gridDim.y * kFillWarps) {
    uint8_t* kt = kcache + ((size_t)blk * kbs + (size_t)h * khs) * E;
    uint8_t* vt = vcache + ((size_t)blk * kbs + (size_t)h * khs) * E;
    // K: chunk pair (token i, cx, cx + half) rotated, or pass-through chunk c >= 2 * half
    for (int idx = lane; idx < run * units; idx += 32) {
      const int i = idx / units, u = idx - i * units;
      uint4* row = reinterpret_cast<uint4*>(key + ((size_t)(t + i) * key_stride + (size_t)h * D) * E);
      uint4* cell = reinterpret_cast<uint4*>(kt) + off0 + i;
      if (u < half) {
        uint4 ox, oy;
        rotate_pair<T>(row[u], row[u + half], cs_row(t + i), u, half, ox, oy);
        cell[(size_t)u * B] = ox;
        cell[(size_t)(u + half) * B] = oy;
        if (write_key_back) { row[u] = ox; row[u + half] = oy; }
      } else {
        const int c = u + half;
        cell[(size_t)c * B] = row[c];
      }
    }
    // V: transposed through shared memory, full blocks written with 16-byte stores
    for (int idx = lane; idx < run * nch; idx += 32) {
      const int i = idx / nch, c = idx - i * nch;
      const uint4* row = reinterpret_cast<const uint4*>(value + ((size_t)(t + i) * value_stride + (size_t)h * D) * E) + c;
      reinterpret_cast<uint4*>(tile)[i * nch + c] = *row;
    }
    __syncwarp();
    const elem_t* ts = reinterpret_cast<const elem_t*>(tile);
    for (int dd = lane; dd < D; dd += 32) {
      elem_t* dst = reinterpret_cast<elem_t*>(vt) + (size_t)dd * B + off0;
      if (run == B) {
        for (int v = 0; v < B / kVec; ++v) {
          elem_t tmp[kVec];
#pragma unroll
          for (int j = 0; j < kVec; ++j) tmp[j] = ts[(size_t)(v * kVec + j) * D + dd];
          reinterpret_cast<uint4*>(dst)[v] = *reinterpret_cast<const uint4*>(tmp);
        }
      } else {
        for (int i = 0; i < run; ++i) dst[i] = ts[(size_t)i * D + dd];
      }
    }
    __syncwarp();
  }
}

// dest[dest_idx[i]] = cache row at slot src_slots[i]; one warp per (token, head).
template <int E, bool IS_V>
__global__ void __launch_bounds__(128) move_from_cache_kernel(
    const uint8_t* __restrict__ cache, uint8_t* __restrict__ dest, const long long* __restrict__ src_slots,
    const long long* __restrict__ dest_idx, const long long n, const int H, const int D, const int B,
    const long long dest_stride, const long long kbs, const long long khs, const long long num_blocks,
    const long long dest_rows, int* __restrict__ status) {
  using elem_t = typename ElemOf<E>::type;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * 4 + warp;
  if (gw >= n * H) return;
  const long long i = gw / H;
  const int h = (int)(gw - i * H);
  const long long slot = src_slots[i], di = dest_idx[i];
  const long long blk = slot / B;
  const int off = (int)(slot - blk * B);
  if (slot < 0 || blk >= num_blocks || di < 0 || di >= dest_rows) {
    if (lane == 0 && status) atomicMax(status, kStatusBadIndex);
    return;
  }
  constexpr int kVec = 16 / E;
  const uint8_t* tile = cache + ((size_t)blk * kbs + (size_t)h * khs) * E;
  uint8_t* row = dest + ((size_t)di * dest_stride + (size_t)h * D) * E;
  if (IS_V) {
    for (int dd = lane; dd < D; dd += 32)
      reinterpret_cast<elem_t*>(row)[dd] = reinterpret_cast<const elem_t*>(tile)[(size_t)dd * B + off];
  } else {
    for (int c = lane; c < D / kVec; c += 32)
      reinterpret_cast<uint4*>(row)[c] = reinterpret_cast<const uint4*>(tile)[(size_t)c * B + off];
  }
}

// dest[dest_idx[i]] = src[src_idx[i]] over rows of row_bytes bytes; one warp per row.
template <bool VEC16>
__global__ void __launch_bounds__(128) move_rows_kernel(
    const uint8_t* __restrict__ src, uint8_t* __restrict__ dest, const long long* __restrict__ src_idx,
    const long long* __restrict__ dest_idx, const long long n, const long long row_bytes,
    const long long src_stride, const long long dest_stride, const long long src_rows,
    const long long dest_rows, int* __restrict__ status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long i = (long long)blockIdx.x * 4 + warp;
  if (i >= n) return;
  const long long si = src_idx[i], di = dest_idx[i];
  if (si < 0 || si >= src_rows || di < 0 || di >= dest_rows) {
    if (lane == 0 && status) atomicMax(status, kStatusBadIndex);
    return;
  }
  const uint8_t* s = src + (size_t)si * src_stride;
  uint8_t* t = dest + (size_t)di * dest_stride;
  if (VEC16) {
    for (long long b = lane; b < row_bytes / 16; b += 32)
      reinterpret_cast<uint4*>(t)[b] = reinterpret_cast<const uint4*>(s)[b];
  } else {
    for (long long b = lane; b < row_bytes; b += 32) t[b] = s[b];
  }
}

thread_local char g_err[256] = "";

}  // namespace

void set_cuda_error(cudaError_t e) {
  const char* s = cudaGetErrorString(e);
  int i = 0;
  for (; s && s[i] && i < 255; ++i) g_err[i] = s[i];
  g_err[i] = 0;
}
const char* last_cuda_error() { return g_err; }

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int kv_run_launch(bool fill, void* key, void* value, void* kcache, void* vcache, const void* slots,
                         int is64, long long T, int H, int D, int B, long long ks, long long vs,
                         long long kbs, long long khs, long long num_blocks, int dtype, cudaStream_t s) {
  if (T < 0 || H <= 0 || D <= 0 || num_blocks < 0) return PB_ERR_INVALID_ARG;
  if (T == 0) return PB_OK;
  if (!key || !value || !kcache || !vcache || !slots) return PB_ERR_INVALID_ARG;
  if (dtype != PB_F32 && dtype != PB_F16 && dtype != PB_BF16) return PB_ERR_UNSUPPORTED;
  const int E = (dtype == PB_F32) ? 4 : 2;
  const int vec = 16 / E;
  if (B != 8 && B != 16 && B != 32) return PB_ERR_UNSUPPORTED;
  if (D % vec != 0 || D > 256) return PB_ERR_UNSUPPORTED;
  if (!aligned16(key) || !aligned16(value) || !aligned16(kcache) || !aligned16(vcache)) return PB_ERR_INVALID_ARG;
  if (ks % vec || vs % vec || kbs % vec || khs % vec) return PB_ERR_INVALID_ARG;
  if (T > 0x7fffffffll) return PB_ERR_INVALID_ARG;
  const size_t smem = (size_t)kFillWarps * B * D * E;
  // few tokens (decode): spread the heads over more CTAs; many tokens (prefill): at most four CTAs per token
  unsigned hgroups = (unsigned)((H + kFillWarps - 1) / kFillWarps);
  if (T >= 2048 && hgroups > 4) hgroups = 4;
  cudaError_t e = cudaSuccess;
#define PB_KV_RUN(EE, FF)                                                                              \
  do {                                                                                                 \
    auto kfn = kv_run_kernel<EE, FF>;                                                                  \
    if (smem > 48 * 1024) e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e == cudaSuccess) {                                                                            \
      e = launch_kernel(kfn, dim3((unsigned)T, hgroups), dim3(kFillWarps * 32), smem, s, FF,                       \
                        (uint8_t*)key, (uint8_t*)value, (uint8_t*)kcache, (uint8_t*)vcache, slots, is64, T, H, D, B, \
                        ks, vs, kbs, khs, num_blocks, (int*)nullptr);                                  \
    }                                                                                                  \
  } while (0)
  if (E == 2) { if (fill) PB_KV_RUN(2, true); else PB_KV_RUN(2, false); }
  else { if (fill) PB_KV_RUN(4, true); else PB_KV_RUN(4, false); }
#undef PB_KV_RUN
  if (e != cudaSuccess) { set_cuda_error(e); return PB_ERR_LAUNCH; }
  return PB_OK;
}

template <typename T>
static cudaError_t rotary_fill_launch_t(void* q, void* k, const void* v, void* kc, void* vc, const void* slots, int is64,
                                        const int64_t* positions, const void* cos_sin, int rot_dim, long long max_pos,
                                        long long T_tok, int Hq, int H, int D, int B, long long qs, long long ks,
                                        long long vs, long long kbs, long long khs, long long num_blocks, int write_back,
                                        cudaStream_t s) {
  const size_t smem = (size_t)kFillWarps * B * D * sizeof(T);
  auto kfn = rotary_fill_kernel<T>;
  cudaError_t e = cudaSuccess;
  if (smem > 48 * 1024) e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int hmax = Hq > H ? Hq : H;
  unsigned hgroups = (unsigned)((hmax + kFillWarps - 1) / kFillWarps);
  if (T_tok >= 2048 && hgroups > 4) hgroups = 4;  // many tokens: four CTAs per token measured best (1, 2, 4, 8 tried)
  return launch_kernel(kfn, dim3((unsigned)T_tok, hgroups), dim3(kFillWarps * 32), smem, s, true,
                       (uint8_t*)q, (uint8_t*)k, (const uint8_t*)v, (uint8_t*)kc, (uint8_t*)vc, slots, is64,
                       (const long long*)positions, (const uint8_t*)cos_sin, rot_dim, max_pos, T_tok, Hq, H, D, B, qs, ks,
                       vs, kbs, khs, num_blocks, write_back);
}

}  // namespace pb

extern "C" {

int pb_reshape_and_cache(const void* key, const void* value, void* key_cache, void* value_cache,
                         const void* slot_mapping, int32_t slot_is_i64, int64_t num_tokens,
                         int32_t num_heads, int32_t head_size, int32_t block_size, int64_t key_stride,
                         int64_t value_stride, int64_t kv_block_stride, int64_t kv_head_stride,
                         int64_t num_blocks, int32_t dtype, void* stream) {
  return pb::kv_run_launch(true, const_cast<void*>(key), const_cast<void*>(value), key_cache, value_cache,
                           slot_mapping, slot_is_i64, num_tokens, num_heads, head_size, block_size,
                           key_stride, value_stride, kv_block_stride, kv_head_stride, num_blocks, dtype,
                           static_cast<cudaStream_t>(stream));
}

int pb_rotary_reshape_and_cache(void* query, void* key, const void* value, void* key_cache, void* value_cache,
                                const void* slot_mapping, int32_t slot_is_i64, const int64_t* positions,
                                const void* cos_sin_cache, int32_t rot_dim, int64_t max_position, int64_t num_tokens,
                                int32_t num_heads, int32_t num_kv_heads, int32_t head_size, int32_t block_size,
                                int64_t query_stride, int64_t key_stride, int64_t value_stride,
                                int64_t kv_block_stride, int64_t kv_head_stride, int64_t num_blocks,
                                int32_t write_key_back, int32_t dtype, void* stream) {
  if (num_tokens == 0) return PB_OK;
  const bool rotate_only = (key_cache == nullptr);  // q and k rotated in place, nothing cached
  if (!query || !key || !positions || !cos_sin_cache) return PB_ERR_INVALID_ARG;
  if (!rotate_only && (!value || !value_cache || !slot_mapping)) return PB_ERR_INVALID_ARG;
  if (num_tokens < 0 || num_tokens > 0x7fffffffll || num_heads <= 0 || num_kv_heads <= 0 || max_position <= 0)
    return PB_ERR_INVALID_ARG;
  if (dtype != PB_F32 && dtype != PB_F16 && dtype != PB_BF16) return PB_ERR_UNSUPPORTED;
  const int E = (dtype == PB_F32) ? 4 : 2;
  const int vec = 16 / E;
  if (block_size != 8 && block_size != 16 && block_size != 32) return PB_ERR_UNSUPPORTED;
  if (head_size % vec != 0 || head_size > 256) return PB_ERR_UNSUPPORTED;
  // both halves of the rotated part must be whole 16-byte chunks
  if (rot_dim <= 0 || rot_dim > head_size || rot_dim % (2 * vec) != 0) return PB_ERR_UNSUPPORTED;
  if (!pb::aligned16(query) || !pb::aligned16(key) || !pb::aligned16(cos_sin_cache)) return PB_ERR_INVALID_ARG;
  if (query_stride % vec || key_stride % vec) return PB_ERR_INVALID_ARG;
  if (!rotate_only) {
    if (!pb::aligned16(value) || !pb::aligned16(key_cache) || !pb::aligned16(value_cache)) return PB_ERR_INVALID_ARG;
    if (value_stride % vec || kv_block_stride % vec || kv_head_stride % vec || num_blocks <= 0) return PB_ERR_INVALID_ARG;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
#define PB_ROT(TT)                                                                                              \
  e = pb::rotary_fill_launch_t<TT>(query, key, value, key_cache, value_cache, slot_mapping, slot_is_i64, positions, \
                                   cos_sin_cache, rot_dim, max_position, num_tokens, num_heads, num_kv_heads,   \
                                   head_size, block_size, query_stride, key_stride, value_stride, kv_block_stride, \
                                   kv_head_stride, num_blocks, write_key_back, s)
  if (dtype == PB_F16) PB_ROT(__half);
  else if (dtype == PB_BF16) PB_ROT(__nv_bfloat16);
  else PB_ROT(float);
#undef PB_ROT
  if (e != cudaSuccess) { pb::set_cuda_error(e); return PB_ERR_LAUNCH; }
  return PB_OK;
}

int pb_gather_cached_kv(void* key, void* value, const void* key_cache, const void* value_cache,
                        const void* slot_mapping, int32_t slot_is_i64, int64_t num_tokens,
                        int32_t num_heads, int32_t head_size, int32_t block_size, int64_t key_stride,
                        int64_t value_stride, int64_t kv_block_stride, int64_t kv_head_stride,
                        int64_t num_blocks, int32_t dtype, void* stream) {
  return pb::kv_run_launch(false, key, value, const_cast<void*>(key_cache), const_cast<void*>(value_cache),
                           slot_mapping, slot_is_i64, num_tokens, num_heads, head_size, block_size,
                           key_stride, value_stride, kv_block_stride, kv_head_stride, num_blocks, dtype,
                           static_cast<cudaStream_t>(stream));
}

int pb_move_tokens_from_blocked_cache(const void* cache, void* dest, const int64_t* src_slots,
                                      const int64_t* dest_indices, int64_t num_tokens, int32_t is_value,
                                      int32_t num_heads, int32_t head_size, int32_t block_size,
                                      int64_t dest_stride, int64_t kv_block_stride, int64_t kv_head_stride,
                                      int64_t num_blocks, int64_t dest_rows, int32_t dtype, void* stream) {
  using namespace pb;
  if (num_tokens < 0 || num_heads <= 0 || head_size <= 0) return PB_ERR_INVALID_ARG;
  if (num_tokens == 0) return PB_OK;
  if (!cache || !dest || !src_slots || !dest_indices) return PB_ERR_INVALID_ARG;
  if (dtype != PB_F32 && dtype != PB_F16 && dtype != PB_BF16) return PB_ERR_UNSUPPORTED;
  const int E = (dtype == PB_F32) ? 4 : 2;
  const int vec = 16 / E;
  if (block_size <= 0 || head_size % vec) return PB_ERR_UNSUPPORTED;
  if (!aligned16(cache) || !aligned16(dest) || dest_stride % vec || kv_block_stride % vec ||
      kv_head_stride % vec)
    return PB_ERR_INVALID_ARG;
  const long long warps = (long long)num_tokens * num_heads;
  const unsigned grid = (unsigned)((warps + 3) / 4);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define PB_MOVE(EE, VV)                                                                               \
  move_from_cache_kernel<EE, VV><<<grid, 128, 0, s>>>(                                                \
      (const uint8_t*)cache, (uint8_t*)dest, (const long long*)src_slots, (const long long*)dest_indices, \
      num_tokens, num_heads, head_size, block_size, dest_stride, kv_block_stride, kv_head_stride,     \
      num_blocks, dest_rows, nullptr)
  if (E == 2) { if (is_value) PB_MOVE(2, true); else PB_MOVE(2, false); }
  else { if (is_value) PB_MOVE(4, true); else PB_MOVE(4, false); }
#undef PB_MOVE
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_cuda_error(e); return PB_ERR_LAUNCH; }
  return PB_OK;
}

int pb_discontinuous_move_tokens(const void* src, void* dest, const int64_t* src_indices,
                                 const int64_t* dest_indices, int64_t num_tokens, int64_t row_bytes,
                                 int64_t src_stride_bytes, int64_t dest_stride_bytes, int64_t src_rows,
                                 int64_t dest_rows, void* stream) {
  using namespace pb;
  if (num_tokens < 0 || row_bytes < 0) return PB_ERR_INVALID_ARG;
  if (num_tokens == 0 || row_bytes == 0) return PB_OK;
  if (!src || !dest || !src_indices || !dest_indices) return PB_ERR_INVALID_ARG;
  const bool vec = aligned16(src) && aligned16(dest) && row_bytes % 16 == 0 && src_stride_bytes % 16 == 0 &&
                   dest_stride_bytes % 16 == 0;
  const unsigned grid = (unsigned)((num_tokens + 3) / 4);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (vec)
    move_rows_kernel<true><<<grid, 128, 0, s>>>((const uint8_t*)src, (uint8_t*)dest, (const long long*)src_indices,
                                                (const long long*)dest_indices, num_tokens, row_bytes,
                                                src_stride_bytes, dest_stride_bytes, src_rows, dest_rows, nullptr);
  else
    move_rows_kernel<false><<<grid, 128, 0, s>>>((const uint8_t*)src, (uint8_t*)dest, (const long long*)src_indices,
                                                 (const long long*)dest_indices, num_tokens, row_bytes,
                                                 src_stride_bytes, dest_stride_bytes, src_rows, dest_rows, nullptr);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_cuda_error(e); return PB_ERR_LAUNCH; }
  return PB_OK;
}

}  // extern "C"
