// Gated-delta-net kernels of the hybrid (Qwen3.5) models: depth-wise causal convolution + SiLU over
// ragged sequences with per-request history, the recurrent gated delta rule with the state matrix held
// in registers, and the gated RMSNorm that follows it.  Every kernel takes its per-request metadata
// (state row, new-token count, "has history" flag, first token row) from device arrays, so a decode
// step needs no host synchronisation and can be captured in a CUDA graph.
//
//   conv:  y[t, c] = silu(sum_j w[c, j] * in[t - (K-1) + j, c]),  inputs before the first new token come
//          from conv_state[slot, c, :] (or are zero); afterwards conv_state keeps the last K-1 inputs.
//   rule:  S *= exp(g_t);  S += k_t (x) ((v_t - S^T k_t) * beta_t);  o_t = S^T q_t
//          with q, k l2-normalised and q scaled by Dk^-0.5; S is [Dk, Dv] fp32 per (request, head).
#include "common.cuh"
#include "kernels.h"

namespace mb200 {
namespace {

constexpr int kMaxConvK = 8;

__device__ __forceinline__ float silu(float v) { return v / (1.f + __expf(-v)); }

// grid (ceil(C / 256), chunks, B); a CTA handles 256 channels of a run of tokens of one request
template <typename T>
__global__ void gdn_conv1d_silu_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ conv_state,
                                       const int* __restrict__ slots, const int* __restrict__ lens,
                                       const int* __restrict__ has_state, const int* __restrict__ q_start,
                                       T* __restrict__ out, int channels, int K, int chunk_tokens) {
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.z;
  const int n = lens[b];
  const int t0 = blockIdx.y * chunk_tokens;
  if (c >= channels || t0 >= n) return;
  const int t1 = min(n, t0 + chunk_tokens);
  const int64_t row0 = q_start[b];
  const T* st = conv_state + (static_cast<int64_t>(slots[b]) * channels + c) * (K - 1);
  const bool hist = has_state[b] != 0;
  float wv[kMaxConvK], win[kMaxConvK];
  for (int j = 0; j < K; ++j) wv[j] = to_f32(w[static_cast<int64_t>(c) * K + j]);
  // window = the K-1 inputs before token t0
  for (int j = 0; j < K - 1; ++j) {
    const int t = t0 - (K - 1) + j;
    win[j] = t >= 0 ? to_f32(x[(row0 + t) * channels + c]) : (hist ? to_f32(st[K - 1 + t]) : 0.f);
  }
  for (int t = t0; t < t1; ++t) {
    win[K - 1] = to_f32(x[(row0 + t) * channels + c]);
    float acc = 0.f;
    for (int j = 0; j < K; ++j) acc = fmaf(wv[j], win[j], acc);
    out[(row0 + t) * channels + c] = from_f32<T>(silu(acc));
    for (int j = 0; j < K - 1; ++j) win[j] = win[j + 1];
  }
}

// after the convolution: conv_state[slot, c, :] = last K-1 inputs (old history shifts in when n < K-1)
template <typename T>
__global__ void gdn_conv_state_update_kernel(const T* __restrict__ x, T* __restrict__ conv_state, const int* __restrict__ slots,
                                             const int* __restrict__ lens, const int* __restrict__ has_state,
                                             const int* __restrict__ q_start, int channels, int K) {
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  const int n = lens[b];
  if (c >= channels || n <= 0) return;
  const int64_t row0 = q_start[b];
  T* st = conv_state + (static_cast<int64_t>(slots[b]) * channels + c) * (K - 1);
  const bool hist = has_state[b] != 0;
  float nv[kMaxConvK];
  for (int j = 0; j < K - 1; ++j) {
    const int t = n - (K - 1) + j;  // token index relative to the first new token
    nv[j] = t >= 0 ? to_f32(x[(row0 + t) * channels + c]) : (hist ? to_f32(st[K - 1 + t]) : 0.f);
  }
  for (int j = 0; j < K - 1; ++j) st[j] = from_f32<T>(nv[j]);
}

// grid (H, B), 128 threads; thread j owns column j of the 128 x 128 state
template <typename T>
__global__ void __launch_bounds__(128) gdn_recurrent_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                                            const float* __restrict__ g, const float* __restrict__ beta,
                                                            float* __restrict__ state, const int* __restrict__ slots,
                                                            const int* __restrict__ lens, const int* __restrict__ has_state,
                                                            const int* __restrict__ q_start, T* __restrict__ out, int heads) {
  pdl_wait();
  constexpr int D = 128;
  __shared__ float sk[D], sq[D], red[8];
  const int h = blockIdx.x, b = blockIdx.y, j = threadIdx.x;
  const int n = lens[b];
  if (n <= 0) return;
  const int64_t row0 = q_start[b];
  float* S = state + ((static_cast<int64_t>(slots[b]) * heads + h) * D) * D;  // [Dk][Dv]
  float s[D];
  if (has_state[b] != 0) {
#pragma unroll
    for (int i = 0; i < D; ++i) s[i] = S[i * D + j];
  } else {
#pragma unroll
    for (int i = 0; i < D; ++i) s[i] = 0.f;
  }
  const float qscale = rsqrtf(static_cast<float>(D));
  for (int t = 0; t < n; ++t) {
    const int64_t base = ((row0 + t) * heads + h) * D;
    const float kj = to_f32(k[base + j]), qj = to_f32(q[base + j]);
    // l2 norms of k and q over the 128 features: warp sums, then four partials each in shared memory
    float kk = warp_sum(kj * kj), qq = warp_sum(qj * qj);
    __syncthreads();  // previous token's sk / sq / red are no longer read
    if ((j & 31) == 0) {
      red[j >> 5] = kk;
      red[4 + (j >> 5)] = qq;
    }
    __syncthreads();
    kk = red[0] + red[1] + red[2] + red[3];
    qq = red[4] + red[5] + red[6] + red[7];
    sk[j] = kj * rsqrtf(kk + 1e-6f);
    sq[j] = qj * rsqrtf(qq + 1e-6f) * qscale;
    __syncthreads();
    const float decay = __expf(g[(row0 + t) * heads + h]);
    const float bt = beta[(row0 + t) * heads + h];
    float mem = 0.f;
#pragma unroll
    for (int i = 0; i < D; ++i) {
      s[i] *= decay;
      mem = fmaf(s[i], sk[i], mem);
    }
    const float delta = (to_f32(v[base + j]) - mem) * bt;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < D; ++i) {
      s[i] = fmaf(sk[i], delta, s[i]);
      o = fmaf(s[i], sq[i], o);
    }
    out[base + j] = from_f32<T>(o);
  }
#pragma unroll
  for (int i = 0; i < D; ++i) S[i * D + j] = s[i];
}

// out = weight * round(rmsnorm(x)) * silu(gate); one warp per row, row width <= 256 (multiple of 8... any)
template <typename T>
__global__ void rmsnorm_gated_kernel(const T* __restrict__ x, const T* __restrict__ gate, const T* __restrict__ w,
                                     T* __restrict__ out, int rows, int width, float eps) {
  pdl_wait();
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const T* xr = x + static_cast<int64_t>(r) * width;
  float ss = 0.f;
  for (int c = lane; c < width; c += 32) {
    const float f = to_f32(xr[c]);
    ss += f * f;
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / static_cast<float>(width) + eps);
  for (int c = lane; c < width; c += 32) {
    const float nrm = to_f32(from_f32<T>(to_f32(xr[c]) * rstd));
    const float gt = to_f32(gate[static_cast<int64_t>(r) * width + c]);
    out[static_cast<int64_t>(r) * width + c] = from_f32<T>(to_f32(w[c]) * nrm * silu(gt));
  }
}

}  // namespace

int launch_gdn_conv1d_silu(const void* x, const void* w, void* conv_state, const int* slots, const int* lens,
                           const int* has_state, const int* q_start, void* out, int batch, int max_tokens, int channels, int K,
                           DType dt, cudaStream_t s) {
  if (batch <= 0 || max_tokens <= 0) return 0;
  if (K < 2 || K > kMaxConvK) return -1;
  const int chunk = 256;
  const dim3 grid((channels + 255) / 256, (max_tokens + chunk - 1) / chunk, batch), block(256);
  MB200_DISPATCH_HALF(dt, (launch_pdl(gdn_conv1d_silu_kernel<T>, grid, block, 0, s, static_cast<const T*>(x), static_cast<const T*>(w),
                                      static_cast<const T*>(conv_state), slots, lens, has_state, q_start, static_cast<T*>(out),
                                      channels, K, chunk)));
  const dim3 grid2((channels + 255) / 256, batch);
  MB200_DISPATCH_HALF(dt, (launch_pdl(gdn_conv_state_update_kernel<T>, grid2, block, 0, s, static_cast<const T*>(x),
                                      static_cast<T*>(conv_state), slots, lens, has_state, q_start, channels, K)));
  note_launch(2);
  return 0;
}

int launch_gdn_recurrent(const void* q, const void* k, const void* v, const float* g, const float* beta, float* state,
                         const int* slots, const int* lens, const int* has_state, const int* q_start, void* out, int batch,
                         int heads, int dk, int dv, DType dt, cudaStream_t s) {
  if (batch <= 0) return 0;
  if (dk != 128 || dv != 128) return -1;
  MB200_DISPATCH_HALF(dt, (launch_pdl(gdn_recurrent_kernel<T>, dim3(heads, batch), dim3(128), 0, s, static_cast<const T*>(q),
                                      static_cast<const T*>(k), static_cast<const T*>(v), g, beta, state, slots, lens, has_state,
                                      q_start, static_cast<T*>(out), heads)));
  note_launch();
  return 0;
}

void launch_rmsnorm_gated(const void* x, const void* gate, const void* w, void* out, int rows, int width, float eps, DType dt,
                          cudaStream_t s) {
  if (rows <= 0) return;
  const int warps = 8;
  MB200_DISPATCH_HALF(dt, (launch_pdl(rmsnorm_gated_kernel<T>, dim3((rows + warps - 1) / warps), dim3(warps * 32), 0, s,
                                      static_cast<const T*>(x), static_cast<const T*>(gate), static_cast<const T*>(w),
                                      static_cast<T*>(out), rows, width, eps)));
  note_launch();
}

}  // namespace mb200
