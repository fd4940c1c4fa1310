// Vision-tower helpers (Qwen3-VL ViT): the 2-D rotary embedding fused with the q/k/v split and the
// zero padding of the head dimension to the 128 columns the tcgen05 attention kernel works on,
// the bilinear position-embedding interpolation fused with its add, and exact (erf) GELU.
// The heavy parts of the tower (patch embedding, qkv / proj / MLP / merger projections, attention)
// run on the tensor-core GEMM and attention kernels.
#include "common.cuh"
#include "kernels.h"

namespace mb200 {
namespace {

// one warp per (token, head); lane handles elements lane, lane + 32, ... of the output row, which is out_dim wide
// (the head size itself, or a wider row whose tail is zero)
template <typename T>
__global__ void vision_rope_split_pad_kernel(const T* __restrict__ qkv, const float* __restrict__ cos,
                                             const float* __restrict__ sin, T* __restrict__ q, T* __restrict__ k,
                                             T* __restrict__ v, int tokens, int heads, int head_dim, int out_dim) {
  pdl_wait();
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= tokens * heads) return;
  const int t = w / heads, h = w % heads;
  const int lane = threadIdx.x & 31;
  const int half = head_dim >> 1;
  const T* src = qkv + (static_cast<int64_t>(t) * 3 * heads + h) * head_dim;
  const int64_t plane = static_cast<int64_t>(heads) * head_dim;
  const int64_t dst = (static_cast<int64_t>(t) * heads + h) * out_dim;
  for (int i = lane; i < out_dim; i += 32) {
    float oq = 0.f, ok = 0.f, ov = 0.f;
    if (i < head_dim) {
      const int f = i < half ? i : i - half;
      const float c = cos[static_cast<int64_t>(t) * half + f], sn = sin[static_cast<int64_t>(t) * half + f];
      const int other = i < half ? i + half : i - half;
      const float sign = i < half ? -1.f : 1.f;
      oq = to_f32(src[i]) * c + sign * to_f32(src[other]) * sn;
      ok = to_f32(src[plane + i]) * c + sign * to_f32(src[plane + other]) * sn;
      ov = to_f32(src[2 * plane + i]);
    }
    q[dst + i] = from_f32<T>(oq);
    k[dst + i] = from_f32<T>(ok);
    v[dst + i] = from_f32<T>(ov);
  }
}

template <typename T>
__global__ void vision_pos_embed_add_kernel(T* __restrict__ x, const T* __restrict__ table, const int64_t* __restrict__ idx,
                                            const float* __restrict__ w, int tokens, int hidden) {
  pdl_wait();
  const int t = blockIdx.x;
  int64_t id[4];
  float wt[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    id[i] = idx[static_cast<int64_t>(i) * tokens + t];
    wt[i] = w[static_cast<int64_t>(i) * tokens + t];
  }
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc += to_f32(from_f32<T>(wt[i] * to_f32(table[id[i] * hidden + c])));
    T* px = x + static_cast<int64_t>(t) * hidden + c;
    *px = from_f32<T>(to_f32(*px) + to_f32(from_f32<T>(acc)));
  }
}

template <typename T>
__global__ void gelu_erf_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t n) {
  pdl_wait();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = to_f32(x[i]);
  out[i] = from_f32<T>(0.5f * v * (1.f + erff(v * 0.70710678118654752f)));
}

}  // namespace

void launch_vision_rope_split_pad(const void* qkv, const float* cos, const float* sin, void* q, void* k, void* v,
                                  int tokens, int heads, int head_dim, int out_dim, DType dt, cudaStream_t s) {
  if (tokens == 0) return;
  const int warps = 8;
  const dim3 grid((tokens * heads + warps - 1) / warps), block(warps * 32);
  MB200_DISPATCH_HALF(dt, (launch_pdl(vision_rope_split_pad_kernel<T>, grid, block, 0, s, static_cast<const T*>(qkv), cos, sin,
                                      static_cast<T*>(q), static_cast<T*>(k), static_cast<T*>(v), tokens, heads, head_dim,
                                      out_dim)));
  note_launch();
}

void launch_vision_pos_embed_add(void* x, const void* table, const int64_t* idx, const float* w, int tokens, int hidden,
                                 DType dt, cudaStream_t s) {
  if (tokens == 0) return;
  MB200_DISPATCH_HALF(dt, (launch_pdl(vision_pos_embed_add_kernel<T>, dim3(tokens), dim3(256), 0, s, static_cast<T*>(x),
                                      static_cast<const T*>(table), idx, w, tokens, hidden)));
  note_launch();
}

void launch_gelu_erf(const void* x, void* out, int64_t n, DType dt, cudaStream_t s) {
  if (n == 0) return;
  const dim3 grid(static_cast<unsigned>((n + 255) / 256)), block(256);
  MB200_DISPATCH_HALF(dt, (launch_pdl(gelu_erf_kernel<T>, grid, block, 0, s, static_cast<const T*>(x), static_cast<T*>(out), n)));
  note_launch();
}

}  // namespace mb200
