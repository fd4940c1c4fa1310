// Memory-bound sm_100a kernels: RMSNorm / fused add+RMSNorm, LayerNorm, gated
// activations, embedding gather, the fused per-head QK-norm + rotary + KV-cache
// write, the stand-alone KV write, per-token int8 quantisation and greedy argmax.
//
// All of them move 16 bytes per thread per access and touch every byte once
// (the norm kernels keep a row in registers between the reduction and the
// scaling pass), so their ceiling is HBM bandwidth.
#include <atomic>
#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"
#include "kernels.h"

namespace mb200 {

static std::atomic<uint64_t> g_launches{0};
uint64_t launch_count() { return g_launches.load(); }
void note_launch(int n) { g_launches.fetch_add(n); }
bool pdl_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("MLLM_B200_PDL");
    return !(v != nullptr && v[0] == '0');
  }();
  return on;
}

cudaError_t ensure_dynamic_smem(const void* kernel, int bytes) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, int> set_to;  // (kernel, device) -> bytes granted
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  std::lock_guard<std::mutex> lock(mu);
  auto it = set_to.find({kernel, dev});
  if (it != set_to.end() && it->second >= bytes) return cudaSuccess;
  err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (err == cudaSuccess) set_to[{kernel, dev}] = bytes;
  return err;
}

void ensure_max_carveout(const void* kernel) {
  static const bool on = [] {
    // opt-in: measured neutral on the decode step (5.38 ms with, 5.34 ms without), so the default leaves every
    // kernel's carve-out to the driver
    const char* v = std::getenv("MLLM_B200_MAX_CARVEOUT");
    return v != nullptr && v[0] == '1';
  }();
  if (!on) return;
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, bool> done;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  std::lock_guard<std::mutex> lock(mu);
  auto& d = done[{kernel, dev}];
  if (d) return;
  d = true;
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  cudaGetLastError();   // a kernel that cannot take the hint keeps its default
}

namespace {

template <typename T>
struct Vec8 {
  uint4 raw;
};

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]);
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& raw, float (&f)[8]) {
  const uint32_t* u = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 p = unpack_bf16x2(u[i]);
    f[2 * i] = p.x;
    f[2 * i + 1] = p.y;
  }
}
template <>
__device__ __forceinline__ void unpack8<__half>(const uint4& raw, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 p = __half22float2(h[i]);
    f[2 * i] = p.x;
    f[2 * i + 1] = p.y;
  }
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]);
template <>
__device__ __forceinline__ uint4 pack8<__nv_bfloat16>(const float (&f)[8]) {
  uint4 r;
  uint32_t* u = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) u[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
  return r;
}
template <>
__device__ __forceinline__ uint4 pack8<__half>(const float (&f)[8]) {
  uint4 r;
  __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  return r;
}
template <typename T>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
template <>
__device__ __forceinline__ float round_to<__half>(float v) {
  return __half2float(__float2half_rn(v));
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane_id() == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (lane_id() == 0) red[32] = t;
  }
  __syncthreads();
  float out = red[32];
  __syncthreads();
  return out;
}

constexpr int kMaxVecPerThread = 4;  // row cache: hidden <= 4 * 8 * blockDim

// ---------------------------------------------------------------------------
// RMSNorm and fused residual-add + RMSNorm. One CTA per row.
// ---------------------------------------------------------------------------
template <typename T, bool kAdd>
__global__ void rmsnorm_kernel(T* __restrict__ x, T* __restrict__ residual, const T* __restrict__ w,
                               T* __restrict__ out, int hidden, int64_t x_stride, int64_t out_stride, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int row = blockIdx.x;
  const int nvec = hidden >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * x_stride);
  uint4* rr = kAdd ? reinterpret_cast<uint4*>(residual + row * x_stride) : nullptr;
  uint4* orow = reinterpret_cast<uint4*>(out + row * out_stride);
  const uint4* wr = reinterpret_cast<const uint4*>(w);

  float cache[kMaxVecPerThread][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kMaxVecPerThread; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
      float f[8];
      unpack8<T>(xr[v], f);
      if (kAdd) {
        float g[8];
        unpack8<T>(rr[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = round_to<T>(f[i] + g[i]);
        rr[v] = pack8<T>(f);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        cache[it][i] = f[i];
        ss += f[i] * f[i];
      }
    }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int it = 0; it < kMaxVecPerThread; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
      float g[8], o[8];
      unpack8<T>(wr[v], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = cache[it][i] * rstd * g[i];
      orow[v] = pack8<T>(o);
    }
  }
}

template <typename T>
__global__ void layernorm_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                                 T* __restrict__ out, int hidden, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int row = blockIdx.x;
  const int nvec = hidden >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(row) * hidden);
  uint4* orow = reinterpret_cast<uint4*>(out + static_cast<int64_t>(row) * hidden);
  float cache[kMaxVecPerThread][8];
  float s = 0.f;
#pragma unroll
  for (int it = 0; it < kMaxVecPerThread; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
      unpack8<T>(xr[v], cache[it]);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += cache[it][i];
    }
  }
  const float mean = block_sum(s, red) / static_cast<float>(hidden);
  float q = 0.f;
#pragma unroll
  for (int it = 0; it < kMaxVecPerThread; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = cache[it][i] - mean;
        q += d * d;
      }
    }
  }
  const float rstd = rsqrtf(block_sum(q, red) / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int it = 0; it < kMaxVecPerThread; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
      float g[8], bb[8], o[8];
      unpack8<T>(reinterpret_cast<const uint4*>(w)[v], g);
      if (b != nullptr) unpack8<T>(reinterpret_cast<const uint4*>(b)[v], bb);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = (cache[it][i] - mean) * rstd * g[i] + (b != nullptr ? bb[i] : 0.f);
      orow[v] = pack8<T>(o);
    }
  }
}

// ---------------------------------------------------------------------------
// gated activations
// ---------------------------------------------------------------------------
__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }
__device__ __forceinline__ float gelu_tanh_f(float v) {
  const float k = 0.7978845608028654f;
  return 0.5f * v * (1.f + tanhf(k * (v + 0.044715f * v * v * v)));
}

template <typename T, int kAct>
__global__ void act_and_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int rows, int inter) {
  pdl_launch_dependents();
  pdl_wait();
  const int vec_per_row = inter >> 3;
  const int64_t total = static_cast<int64_t>(rows) * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int v = static_cast<int>(i - r * vec_per_row);
    const uint4* row = reinterpret_cast<const uint4*>(x + r * 2 * inter);
    float g[8], u[8], o[8];
    unpack8<T>(row[v], g);
    unpack8<T>(row[vec_per_row + v], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = (kAct == 0 ? silu_f(g[j]) : gelu_tanh_f(g[j])) * u[j];
    reinterpret_cast<uint4*>(out + r * inter)[v] = pack8<T>(o);
  }
}

template <typename T>
__global__ void gelu_tanh_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t nvec) {
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float f[8];
    unpack8<T>(reinterpret_cast<const uint4*>(x)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = gelu_tanh_f(f[j]);
    reinterpret_cast<uint4*>(out)[i] = pack8<T>(f);
  }
}

// ---------------------------------------------------------------------------
// embedding gather: one CTA per token
// ---------------------------------------------------------------------------
__global__ void embedding_kernel(const int64_t* __restrict__ ids, const uint4* __restrict__ table,
                                 uint4* __restrict__ out, int vec_per_row, int vocab, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int64_t id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, kStatusBadIndex);
    id = 0;
  }
  const uint4* src = table + id * vec_per_row;
  uint4* dst = out + static_cast<int64_t>(t) * vec_per_row;
  for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) dst[v] = src[v];
}

// ---------------------------------------------------------------------------
// fused per-head RMSNorm (q,k) + NeoX RoPE (q,k) + KV-cache write. head_dim = 128.
// A warp owns one token and every `hsplit`-th head of it; lane l owns features 4l..4l+3, its rotation
// partner (feature +-64) lives in lane l^16.  The sines and cosines depend on the token and the feature
// only, so the warp computes its four pairs once and reuses them for all its heads (with one warp per
// (token, head) the kernel was bound by sincosf: 355 us for 16384 tokens of 48 heads, against 60 us of
// memory traffic).  The host picks hsplit = all heads for a handful of tokens (decode: parallelism
// matters) and a few for long prefills.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void qk_norm_rope_kv_write_kernel(T* __restrict__ qkv, const T* __restrict__ q_w,
                                             const T* __restrict__ k_w, const int64_t* __restrict__ positions,
                                             int pos_rows, const int8_t* __restrict__ axis_map,
                                             const float* __restrict__ inv_freq,
                                             const int64_t* __restrict__ cache_loc, void* __restrict__ k_cache,
                                             void* __restrict__ v_cache, int kv_fmt, int64_t kv_tok_stride,
                                             int64_t kv_head_stride, int tokens, int hq, int hkv, int hsplit,
                                             int64_t qkv_stride, int64_t num_slots, float eps, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int D = 128;
  const int heads = hq + 2 * hkv;
  const int64_t warp = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  if (warp >= static_cast<int64_t>(tokens) * hsplit) return;
  const int t = static_cast<int>(warp / hsplit);
  const int h_first = static_cast<int>(warp - static_cast<int64_t>(t) * hsplit);
  const int lane = lane_id();

  const int64_t slot = cache_loc[t];
  const bool slot_ok = slot >= 0 && slot < num_slots;
  if (!slot_ok && h_first == 0 && lane == 0 && status != nullptr) atomicExch(status, kStatusBadIndex);

  float cs[4], sn[4];
  if (h_first < hq + hkv) {   // this warp has at least one head to rotate
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int fi = (lane * 4 + i) & 63;
      const int ax = (axis_map != nullptr && pos_rows > 1) ? axis_map[fi] : 0;
      const float ang = static_cast<float>(positions[static_cast<int64_t>(ax) * tokens + t]) * inv_freq[fi];
      sincosf(ang, &sn[i], &cs[i]);
      if (lane < 16) sn[i] = -sn[i];   // first half: x cos - partner sin; second half: x cos + partner sin
    }
  }
  float wq[4], wk[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) wq[i] = wk[i] = 1.f;
  if (q_w != nullptr) {
    const uint2 wr = *reinterpret_cast<const uint2*>(q_w + lane * 4);
    const T* we = reinterpret_cast<const T*>(&wr);
#pragma unroll
    for (int i = 0; i < 4; ++i) wq[i] = to_f32(we[i]);
  }
  if (k_w != nullptr) {
    const uint2 wr = *reinterpret_cast<const uint2*>(k_w + lane * 4);
    const T* we = reinterpret_cast<const T*>(&wr);
#pragma unroll
    for (int i = 0; i < 4; ++i) wk[i] = to_f32(we[i]);
  }

  T* row = qkv + t * qkv_stride + lane * 4;
#pragma unroll 4
  for (int h = h_first; h < heads; h += hsplit) {
    T* src = row + h * D;
    uint2 raw = *reinterpret_cast<const uint2*>(src);
    const bool is_q = h < hq, is_k = !is_q && h < hq + hkv;
    if (is_q || is_k) {
      float f[4];
      {
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = to_f32(e[i]);
      }
      if ((is_q ? q_w : k_w) != nullptr) {
        const float ss = f[0] * f[0] + f[1] * f[1] + f[2] * f[2] + f[3] * f[3];
        const float rstd = rsqrtf(warp_sum(ss) / static_cast<float>(D) + eps);
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = round_to<T>(f[i] * rstd * (is_q ? wq[i] : wk[i]));
      }
      T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float partner = __shfl_xor_sync(0xffffffffu, f[i], 16);
        e[i] = from_f32<T>(f[i] * cs[i] + partner * sn[i]);
      }
      *reinterpret_cast<uint2*>(src) = raw;
    }
    if (!is_q && slot_ok) {
      void* cache = is_k ? k_cache : v_cache;
      const int kvh = is_k ? h - hq : h - hq - hkv;
      const int64_t at = slot * kv_tok_stride + kvh * kv_head_stride + lane * 4;
      if (kv_fmt == kKvSame) {
        *reinterpret_cast<uint2*>(static_cast<T*>(cache) + at) = raw;
      } else {   // 8-bit cache: the 16-bit values that attention would have read, rounded once more
        const T* e = reinterpret_cast<const T*>(&raw);
        const uint32_t packed = pack_fp8x2(to_f32(e[0]), to_f32(e[1]), kv_fmt) | (pack_fp8x2(to_f32(e[2]), to_f32(e[3]), kv_fmt) << 16);
        *reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(cache) + at) = packed;
      }
    }
  }
}

// rows of `row_elems` = heads x head_elems elements (head_elems a multiple of 8) copied to the slot rows of both
// caches; a cache row of head h of slot s starts at s * kv_tok_stride + h * kv_head_stride
template <typename T>
__global__ void kv_write_kernel(const T* __restrict__ k, const T* __restrict__ v, const int64_t* __restrict__ loc,
                                void* __restrict__ k_cache, void* __restrict__ v_cache, int kv_fmt, int64_t kv_tok_stride,
                                int64_t kv_head_stride, int head_elems, int tokens, int row_elems,
                                int64_t k_stride, int64_t v_stride, int64_t num_slots, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int vec = row_elems >> 3;
  const int64_t total = static_cast<int64_t>(tokens) * vec;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / vec;
    const int c = static_cast<int>(i - t * vec);
    const int64_t slot = loc[t];
    if (slot < 0 || slot >= num_slots) {
      if (status != nullptr) atomicExch(status, kStatusBadIndex);
      continue;
    }
    const int head = (c << 3) / head_elems;
    const int64_t dst = slot * kv_tok_stride + head * kv_head_stride + ((c << 3) - head * head_elems);
    const uint4 kr = reinterpret_cast<const uint4*>(k + t * k_stride)[c];
    const uint4 vr = reinterpret_cast<const uint4*>(v + t * v_stride)[c];
    if (kv_fmt == kKvSame) {
      *reinterpret_cast<uint4*>(static_cast<T*>(k_cache) + dst) = kr;
      *reinterpret_cast<uint4*>(static_cast<T*>(v_cache) + dst) = vr;
    } else {
      const T* ke = reinterpret_cast<const T*>(&kr);
      const T* ve = reinterpret_cast<const T*>(&vr);
      uint2 ko, vo;
      ko.x = pack_fp8x2(to_f32(ke[0]), to_f32(ke[1]), kv_fmt) | (pack_fp8x2(to_f32(ke[2]), to_f32(ke[3]), kv_fmt) << 16);
      ko.y = pack_fp8x2(to_f32(ke[4]), to_f32(ke[5]), kv_fmt) | (pack_fp8x2(to_f32(ke[6]), to_f32(ke[7]), kv_fmt) << 16);
      vo.x = pack_fp8x2(to_f32(ve[0]), to_f32(ve[1]), kv_fmt) | (pack_fp8x2(to_f32(ve[2]), to_f32(ve[3]), kv_fmt) << 16);
      vo.y = pack_fp8x2(to_f32(ve[4]), to_f32(ve[5]), kv_fmt) | (pack_fp8x2(to_f32(ve[6]), to_f32(ve[7]), kv_fmt) << 16);
      *reinterpret_cast<uint2*>(static_cast<uint8_t*>(k_cache) + dst) = ko;
      *reinterpret_cast<uint2*>(static_cast<uint8_t*>(v_cache) + dst) = vo;
    }
  }
}

// ---------------------------------------------------------------------------
// per-token symmetric int8 quantisation: scale = absmax / 127
// ---------------------------------------------------------------------------
template <typename T>
__global__ void per_token_quant_int8_kernel(const T* __restrict__ x, int8_t* __restrict__ q,
                                            float* __restrict__ scale, int k) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int row = blockIdx.x;
  const int nvec = k >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(row) * k);
  float cache[kMaxVecPerThread][8];
  float amax = 0.f;
#pragma unroll
  for (int it = 0; it < kMaxVecPerThread; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
      unpack8<T>(xr[v], cache[it]);
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(cache[it][i]));
    }
  }
  amax = warp_max(amax);
  if (lane_id() == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = (threadIdx.x < ((blockDim.x + 31) >> 5)) ? red[threadIdx.x] : 0.f;
    t = warp_max(t);
    if (threadIdx.x == 0) red[32] = t;
  }
  __syncthreads();
  amax = fmaxf(red[32], 1e-10f);
  const float sc = amax / 127.f;
  if (threadIdx.x == 0) scale[row] = sc;
#pragma unroll
  for (int it = 0; it < kMaxVecPerThread; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
      int8_t o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float r = rintf(cache[it][i] / sc);
        r = fminf(fmaxf(r, -128.f), 127.f);
        o[i] = static_cast<int8_t>(r);
      }
      reinterpret_cast<uint2*>(q + static_cast<int64_t>(row) * k)[v] = *reinterpret_cast<uint2*>(o);
    }
  }
}

// ---------------------------------------------------------------------------
// greedy argmax: one CTA per row, lowest index wins ties
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float load_as_float(const T* p) {
  return to_f32(*p);
}

template <typename T>
__global__ void argmax_kernel(const T* __restrict__ logits, int64_t* __restrict__ out, int vocab, int64_t stride) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sval[32];
  __shared__ int sidx[32];
  const T* row = logits + blockIdx.x * stride;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = load_as_float(row + i);
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if (lane_id() == 0) {
    sval[threadIdx.x >> 5] = best;
    sidx[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = (blockDim.x + 31) >> 5;
    best = threadIdx.x < nw ? sval[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? sidx[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
  }
}

inline int norm_threads(int hidden) {
  int t = ((hidden >> 3) + 31) / 32 * 32;
  if (t > 1024) t = 1024;
  if (t < 32) t = 32;
  return t;
}

constexpr int kArgmaxChunks = 32;

template <typename T>
__global__ void argmax_partial_kernel(const T* __restrict__ logits, float* __restrict__ part_val, int* __restrict__ part_idx,
                                      int vocab, int64_t stride) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sval[32];
  __shared__ int sidx[32];
  const T* row = logits + blockIdx.y * stride;
  const int per = (vocab + kArgmaxChunks - 1) / kArgmaxChunks;
  const int lo = blockIdx.x * per, hi = min(vocab, lo + per);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = load_as_float(row + i);
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if (lane_id() == 0) {
    sval[threadIdx.x >> 5] = best;
    sidx[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = (blockDim.x + 31) >> 5;
    best = threadIdx.x < nw ? sval[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? sidx[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (threadIdx.x == 0) {
      part_val[blockIdx.y * kArgmaxChunks + blockIdx.x] = best;
      part_idx[blockIdx.y * kArgmaxChunks + blockIdx.x] = bi;
    }
  }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx,
                                    int64_t* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  float best = part_val[blockIdx.x * kArgmaxChunks + threadIdx.x];
  int bi = part_idx[blockIdx.x * kArgmaxChunks + threadIdx.x];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if (threadIdx.x == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
}

}  // namespace


void launch_rmsnorm(const void* x, const void* w, void* out, int rows, int hidden, int64_t x_stride,
                    int64_t out_stride, float eps, DType dt, cudaStream_t s) {
  if (rows == 0) return;
  const int threads = norm_threads(hidden);
  MB200_DISPATCH_HALF(dt, (launch_pdl(rmsnorm_kernel<T, false>, dim3(rows), dim3(threads), 0, s, 
                              const_cast<T*>(static_cast<const T*>(x)), nullptr, static_cast<const T*>(w),
                              static_cast<T*>(out), hidden, x_stride, out_stride, eps)));
  note_launch();
}

void launch_fused_add_rmsnorm(void* x, void* residual, const void* w, int rows, int hidden, float eps, DType dt,
                              cudaStream_t s) {
  if (rows == 0) return;
  const int threads = norm_threads(hidden);
  MB200_DISPATCH_HALF(dt, (launch_pdl(rmsnorm_kernel<T, true>, dim3(rows), dim3(threads), 0, s, 
                              static_cast<T*>(x), static_cast<T*>(residual), static_cast<const T*>(w),
                              static_cast<T*>(x), hidden, hidden, hidden, eps)));
  note_launch();
}

void launch_layernorm(const void* x, const void* w, const void* b, void* out, int rows, int hidden, float eps,
                      DType dt, cudaStream_t s) {
  if (rows == 0) return;
  const int threads = norm_threads(hidden);
  MB200_DISPATCH_HALF(dt, (launch_pdl(layernorm_kernel<T>, dim3(rows), dim3(threads), 0, s, static_cast<const T*>(x),
                                                                         static_cast<const T*>(w),
                                                                         static_cast<const T*>(b),
                                                                         static_cast<T*>(out), hidden, eps)));
  note_launch();
}

void launch_act_and_mul(const void* x, void* out, int rows, int inter, int act, DType dt, cudaStream_t s) {
  if (rows == 0) return;
  const int64_t total = static_cast<int64_t>(rows) * (inter >> 3);
  const int threads = 256;
  const int blocks = static_cast<int>(std::min<int64_t>((total + threads - 1) / threads, 148 * 16));
  if (act == 0) {
    MB200_DISPATCH_HALF(dt, (launch_pdl(act_and_mul_kernel<T, 0>, dim3(blocks), dim3(threads), 0, s, static_cast<const T*>(x),
                                                                                  static_cast<T*>(out), rows, inter)));
  } else {
    MB200_DISPATCH_HALF(dt, (launch_pdl(act_and_mul_kernel<T, 1>, dim3(blocks), dim3(threads), 0, s, static_cast<const T*>(x),
                                                                                  static_cast<T*>(out), rows, inter)));
  }
  note_launch();
}

void launch_gelu_tanh(const void* x, void* out, int64_t n, DType dt, cudaStream_t s) {
  if (n == 0) return;
  const int64_t nvec = n >> 3;
  const int threads = 256;
  const int blocks = static_cast<int>(std::min<int64_t>((nvec + threads - 1) / threads, 148 * 16));
  MB200_DISPATCH_HALF(dt, (launch_pdl(gelu_tanh_kernel<T>, dim3(blocks), dim3(threads), 0, s, static_cast<const T*>(x),
                                                                           static_cast<T*>(out), nvec)));
  note_launch();
}

void launch_embedding(const int64_t* ids, const void* table, void* out, int tokens, int hidden, int vocab,
                      DType dt, int* status, cudaStream_t s) {
  if (tokens == 0) return;
  (void)dt;  // 16-bit element types share the copy
  const int vec = hidden >> 3;
  const int threads = vec >= 256 ? 256 : ((vec + 31) / 32 * 32);
  launch_pdl(embedding_kernel, dim3(tokens), dim3(threads), 0, s, ids, static_cast<const uint4*>(table), static_cast<uint4*>(out), vec,
                                              vocab, status);
  note_launch();
}

// One decode step's bookkeeping for a static batch in a single launch: request b takes KV slot
// own[b, used] for its next token, the slot is entered into the request table at position seq_lens[b], the
// length grows by one, and the step's inputs (token ids, request rows, lengths, slots, positions) are written
// where the captured decode graph reads them.
__global__ void decode_prepare_kernel(const int64_t* __restrict__ last_ids, const int32_t* __restrict__ req_rows,
                                      const int64_t* __restrict__ own, int64_t own_stride, int used,
                                      int32_t* __restrict__ seq_lens, int32_t* __restrict__ req_to_token,
                                      int64_t rtt_stride, int64_t* __restrict__ g_input_ids,
                                      int32_t* __restrict__ g_req_rows, int32_t* __restrict__ g_seq_lens,
                                      int64_t* __restrict__ g_out_loc, int64_t* __restrict__ g_positions, int batch) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const int64_t slot = own[b * own_stride + used];
  const int32_t len = seq_lens[b];          // tokens so far; the new token's position
  const int32_t row = req_rows[b];
  req_to_token[row * rtt_stride + len] = static_cast<int32_t>(slot);
  seq_lens[b] = len + 1;
  g_input_ids[b] = last_ids[b];
  g_req_rows[b] = row;
  g_seq_lens[b] = len + 1;
  g_out_loc[b] = slot;
  g_positions[b] = len;
}

void launch_decode_prepare(const int64_t* last_ids, const int32_t* req_rows, const int64_t* own, int64_t own_stride,
                           int used, int32_t* seq_lens, int32_t* req_to_token, int64_t rtt_stride,
                           int64_t* g_input_ids, int32_t* g_req_rows, int32_t* g_seq_lens, int64_t* g_out_loc,
                           int64_t* g_positions, int batch, cudaStream_t s) {
  if (batch <= 0) return;
  launch_pdl(decode_prepare_kernel, dim3((batch + 127) / 128), dim3(128), 0, s, last_ids, req_rows, own, own_stride,
             used, seq_lens, req_to_token, rtt_stride, g_input_ids, g_req_rows, g_seq_lens, g_out_loc, g_positions,
             batch);
  note_launch();
}

void launch_qk_norm_rope_kv_write(void* qkv, const void* q_w, const void* k_w, const int64_t* positions,
                                  int pos_rows, const int8_t* axis_map, const float* inv_freq,
                                  const int64_t* cache_loc, void* k_cache, void* v_cache, int64_t kv_tok_stride,
                                  int64_t kv_head_stride, int tokens,
                                  int num_q_heads, int num_kv_heads, int head_dim, int64_t qkv_stride,
                                  int64_t num_slots, float eps, DType dt, int kv_fmt, int* status, cudaStream_t s) {
  if (tokens == 0 || head_dim != 128) return;
  // warps per token: every head its own warp for a few tokens, a handful of warps per token for long prefills
  // (each then amortises its sines and cosines over heads / hsplit heads)
  const int heads = num_q_heads + 2 * num_kv_heads;
  const int hsplit = static_cast<int>(std::min<int64_t>(heads, std::max<int64_t>(1, 32768 / tokens)));
  const int64_t warps = static_cast<int64_t>(tokens) * hsplit;
  const int threads = 128;
  const int blocks = static_cast<int>((warps * 32 + threads - 1) / threads);
  MB200_DISPATCH_HALF(dt, (launch_pdl(qk_norm_rope_kv_write_kernel<T>, dim3(blocks), dim3(threads), 0, s, 
                              static_cast<T*>(qkv), static_cast<const T*>(q_w), static_cast<const T*>(k_w),
                              positions, pos_rows, axis_map, inv_freq, cache_loc, k_cache,
                              v_cache, kv_fmt, kv_tok_stride, kv_head_stride, tokens, num_q_heads,
                              num_kv_heads, hsplit, qkv_stride, num_slots, eps, status)));
  note_launch();
}

void launch_kv_write(const void* k, const void* v, const int64_t* loc, void* k_cache, void* v_cache,
                     int64_t kv_tok_stride, int64_t kv_head_stride, int head_elems, int tokens,
                     int row_elems, int64_t k_stride, int64_t v_stride, int64_t num_slots, DType dt, int kv_fmt, int* status,
                     cudaStream_t s) {
  if (tokens == 0) return;
  const int64_t total = static_cast<int64_t>(tokens) * (row_elems >> 3);
  const int threads = 256;
  const int blocks = static_cast<int>(std::min<int64_t>((total + threads - 1) / threads, 148 * 16));
  MB200_DISPATCH_HALF(dt, (launch_pdl(kv_write_kernel<T>, dim3(blocks), dim3(threads), 0, s, 
                              static_cast<const T*>(k), static_cast<const T*>(v), loc, k_cache,
                              v_cache, kv_fmt, kv_tok_stride, kv_head_stride, head_elems, tokens, row_elems,
                              k_stride, v_stride, num_slots, status)));
  note_launch();
}

void launch_per_token_quant_int8(const void* x, int8_t* q, float* scale, int rows, int k, DType dt,
                                 cudaStream_t s) {
  if (rows == 0) return;
  const int threads = norm_threads(k);
  MB200_DISPATCH_HALF(dt, (launch_pdl(per_token_quant_int8_kernel<T>, dim3(rows), dim3(threads), 0, s, static_cast<const T*>(x), q,
                                                                                    scale, k)));
  note_launch();
}

void launch_argmax(const void* logits, int64_t* out, int rows, int vocab, int64_t stride, DType dt,
                   cudaStream_t s) {
  if (rows == 0) return;
  if (dt == kF32) {
    launch_pdl(argmax_kernel<float>, dim3(rows), dim3(1024), 0, s, static_cast<const float*>(logits), out, vocab, stride);
  } else {
    MB200_DISPATCH_HALF(dt, (launch_pdl(argmax_kernel<T>, dim3(rows), dim3(1024), 0, s, static_cast<const T*>(logits), out, vocab,
                                                                     stride)));
  }
  note_launch();
}

// Wide vocabularies, few rows: kArgmaxChunks CTAs per row reduce a slice each, a second tiny kernel
// picks the winner (lowest index wins ties in both stages, so the result equals the one-kernel path).
int launch_argmax_split(const void* logits, int64_t* out, float* part_val, int* part_idx, int rows, int vocab,
                        int64_t stride, DType dt, cudaStream_t s) {
  if (rows == 0) return 0;
  if (dt == kF32) {
    launch_pdl(argmax_partial_kernel<float>, dim3(kArgmaxChunks, rows), dim3(512), 0, s, static_cast<const float*>(logits),
               part_val, part_idx, vocab, stride);
  } else {
    MB200_DISPATCH_HALF(dt, (launch_pdl(argmax_partial_kernel<T>, dim3(kArgmaxChunks, rows), dim3(512), 0, s,
                                        static_cast<const T*>(logits), part_val, part_idx, vocab, stride)));
  }
  launch_pdl(argmax_final_kernel, dim3(rows), dim3(32), 0, s, static_cast<const float*>(part_val),
             static_cast<const int*>(part_idx), out);
  note_launch(2);
  return kArgmaxChunks;
}

}  // namespace mb200
