// Token sampling without a sort: temperature, top-k, top-p and min-p filtering followed by
// inverse-CDF sampling, one CTA per request row, plus the penalty kernel.
//
// With e_i = exp((logit_i - max) / T) (so the largest e is exactly 1) every filter keeps a prefix of
// the descending order, i.e. a set {e_i >= tau}:
//   top-k : tau_k = k-th largest e                       (radix select on counts)
//   top-p : tau_p = smallest e whose strictly-larger mass is below top_p * sum(e)   (radix select on mass)
//   min-p : tau_m = min_p
// Elements equal to the cut-off are all kept.  The kept set is {e_i >= max(tau_k, tau_p, tau_m)}; the
// sample is the first token id whose running kept mass (in id order) exceeds u * kept_mass.
// The radix select walks the 31 value bits of the non-negative floats in digits of 11, 11 and 9 bits.
// Rows with temperature <= 1e-6 are greedy (lowest id wins ties).
#include "common.cuh"
#include "kernels.h"

namespace mb200 {
namespace {

constexpr int kSampleThreads = 1024;
constexpr int kBins = 2048;

__device__ __forceinline__ float block_reduce_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : -INFINITY;
  return warp_max(r);
}
__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : 0.f;
  return warp_sum(r);
}

// Warp 0 only.  Walks `nbins` (multiple of 32) bins from the highest down and returns the bin in which the
// running total first reaches `need`; `before` = total of the bins above it.  Falls back to the lowest
// bin when the total never reaches `need`.
template <typename H>
__device__ int find_bin_desc(const H* hist, int nbins, H need, H& before) {
  const int lane = threadIdx.x & 31;
  const int per = nbins >> 5;
  const int hi = nbins - 1 - lane * per;
  H s = 0;
  for (int j = 0; j < per; ++j) s += hist[hi - j];
  H inc = s;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const H t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  const H exc = inc - s;
  const unsigned m = __ballot_sync(0xffffffffu, inc >= need);
  const int src = m ? (__ffs(m) - 1) : 31;
  int bin = hi - (per - 1);
  H bef = exc;
  if (lane == src) {
    H acc = exc;
    bool found = false;
    for (int j = 0; j < per; ++j) {
      const H h = hist[hi - j];
      if (!found && acc + h >= need) {
        bin = hi - j;
        bef = acc;
        found = true;
      }
      if (!found) acc += h;
    }
    if (!found) bef = acc - hist[bin];
  }
  bin = __shfl_sync(0xffffffffu, bin, src);
  before = __shfl_sync(0xffffffffu, bef, src);
  return bin;
}

template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const T* __restrict__ logits, int64_t stride, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ uniform, int64_t* __restrict__ out) {
  pdl_wait();
  __shared__ float red[32];
  __shared__ int redi[32];
  __shared__ unsigned hist_c[kBins];
  __shared__ float hist_m[kBins];
  __shared__ int s_bin;
  __shared__ float s_needf;
  __shared__ unsigned s_needc;
  __shared__ float scan[kSampleThreads / 32];
  __shared__ int s_owner;

  const int b = blockIdx.x;
  const T* row = logits + static_cast<int64_t>(b) * stride;
  const float temp = temperature[b];
  const int tid = threadIdx.x;

  // ---- max (and greedy argmax) ----
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = to_f32(row[i]);
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
  if (temp <= 1e-6f) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if ((tid & 31) == 0) {
      red[tid >> 5] = best;
      redi[tid >> 5] = bi;
    }
    __syncthreads();
    if (tid < 32) {
      best = red[tid];
      bi = redi[tid];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) {
          best = ov;
          bi = oi;
        }
      }
      if (tid == 0) out[b] = bi == 0x7fffffff ? 0 : bi;
    }
    return;
  }
  const float mx = block_reduce_max(best, red);
  const float inv_t = 1.f / temp;
  auto e_of = [&](int i) -> float { return __expf((to_f32(row[i]) - mx) * inv_t); };

  float part = 0.f;
  for (int i = tid; i < vocab; i += blockDim.x) part += e_of(i);
  const float total = block_reduce_sum(part, red);

  // ---- cut-offs ----
  uint32_t tau_bits = 0;
  const int k = top_k[b];
  const float tp = top_p[b];
  const int shifts[3] = {20, 9, 0};
  const int widths[3] = {11, 11, 9};
  if (k > 0 && k < vocab) {
    uint32_t prefix = 0, pmask = 0;
    unsigned need = static_cast<unsigned>(k);
    for (int lvl = 0; lvl < 3; ++lvl) {
      const int nb = 1 << widths[lvl];
      for (int i = tid; i < nb; i += blockDim.x) hist_c[i] = 0;
      __syncthreads();
      for (int i = tid; i < vocab; i += blockDim.x) {
        const uint32_t bits = __float_as_uint(e_of(i));
        if ((bits & pmask) == prefix) atomicAdd(&hist_c[(bits >> shifts[lvl]) & (nb - 1)], 1u);
      }
      __syncthreads();
      if (tid < 32) {
        unsigned before;
        const int bin = find_bin_desc<unsigned>(hist_c, nb, need, before);
        if (tid == 0) {
          s_bin = bin;
          s_needc = need - before;
        }
      }
      __syncthreads();
      prefix |= static_cast<uint32_t>(s_bin) << shifts[lvl];
      pmask |= static_cast<uint32_t>(nb - 1) << shifts[lvl];
      need = s_needc;
      __syncthreads();
    }
    tau_bits = prefix;
  }
  if (tp < 1.f) {
    uint32_t prefix = 0, pmask = 0;
    float need = fmaxf(tp * total, 1e-30f);  // > 0 so the crossing bin is never empty
    for (int lvl = 0; lvl < 3; ++lvl) {
      const int nb = 1 << widths[lvl];
      for (int i = tid; i < nb; i += blockDim.x) hist_m[i] = 0.f;
      __syncthreads();
      for (int i = tid; i < vocab; i += blockDim.x) {
        const float e = e_of(i);
        const uint32_t bits = __float_as_uint(e);
        if ((bits & pmask) == prefix) atomicAdd(&hist_m[(bits >> shifts[lvl]) & (nb - 1)], e);
      }
      __syncthreads();
      if (tid < 32) {
        float before;
        const int bin = find_bin_desc<float>(hist_m, nb, need, before);
        if (tid == 0) {
          s_bin = bin;
          s_needf = need - before;
        }
      }
      __syncthreads();
      prefix |= static_cast<uint32_t>(s_bin) << shifts[lvl];
      pmask |= static_cast<uint32_t>(nb - 1) << shifts[lvl];
      need = s_needf;
      __syncthreads();
    }
    tau_bits = max(tau_bits, prefix);
  }
  if (min_p != nullptr && min_p[b] > 0.f) tau_bits = max(tau_bits, __float_as_uint(fminf(min_p[b], 1.f)));
  const float tau = __uint_as_float(tau_bits);

  // ---- inverse CDF over the kept set in id order ----
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int i0 = min(vocab, tid * chunk), i1 = min(vocab, i0 + chunk);
  float mine = 0.f;
  for (int i = i0; i < i1; ++i) {
    const float e = e_of(i);
    if (e >= tau) mine += e;
  }
  // block exclusive scan
  float inc = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, inc, o);
    if ((tid & 31) >= o) inc += t;
  }
  if ((tid & 31) == 31) scan[tid >> 5] = inc;
  if (tid == 0) s_owner = -1;
  __syncthreads();
  if (tid < 32) {
    const float w = scan[tid];
    float winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, winc, o);
      if (tid >= o) winc += t;
    }
    scan[tid] = winc - w;  // exclusive offset of each warp
    if (tid == 31) red[0] = winc;
  }
  __syncthreads();
  const float excl = scan[tid >> 5] + inc - mine;
  const float kept_total = red[0];
  const float target = uniform[b] * kept_total;
  // the owner is the last thread with a non-empty chunk whose exclusive offset is <= target
  if (mine > 0.f && excl <= target) atomicMax(&s_owner, tid);
  __syncthreads();
  if (tid == s_owner) {
    float acc = excl;
    int pick = -1, last_kept = -1;
    for (int i = i0; i < i1; ++i) {
      const float e = e_of(i);
      if (e >= tau) {
        acc += e;
        last_kept = i;
        if (acc > target) {
          pick = i;
          break;
        }
      }
    }
    out[b] = pick >= 0 ? pick : last_kept;
  }
  if (s_owner < 0 && tid == 0) out[b] = 0;  // degenerate row (no finite logit)
}

// logits[b, v] -= freq[b] * count[b, v] + presence[b] * (count > 0); then the repetition penalty on
// tokens seen in the prompt or the output (divide positive logits, multiply negative ones).
__global__ void apply_penalties_kernel(float* __restrict__ logits, const int* __restrict__ counts,
                                       const uint8_t* __restrict__ prompt_mask, const float* __restrict__ freq,
                                       const float* __restrict__ presence, const float* __restrict__ repetition, int vocab) {
  pdl_wait();
  const int b = blockIdx.y;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= vocab) return;
  const int64_t idx = static_cast<int64_t>(b) * vocab + v;
  float l = logits[idx];
  const int c = counts[idx];
  l -= freq[b] * static_cast<float>(c) + (c > 0 ? presence[b] : 0.f);
  if (c > 0 || (prompt_mask != nullptr && prompt_mask[idx])) {
    const float rp = repetition[b];
    l = l > 0.f ? l / rp : l * rp;
  }
  logits[idx] = l;
}

}  // namespace

void launch_sample(const void* logits, int64_t stride, int rows, int vocab, const float* temperature, const int* top_k,
                   const float* top_p, const float* min_p, const float* uniform, int64_t* out, DType dt, cudaStream_t s) {
  if (rows == 0) return;
  if (dt == kF32) {
    launch_pdl(sample_kernel<float>, dim3(rows), dim3(kSampleThreads), 0, s, static_cast<const float*>(logits), stride,
               vocab, temperature, top_k, top_p, min_p, uniform, out);
  } else {
    MB200_DISPATCH_HALF(dt, (launch_pdl(sample_kernel<T>, dim3(rows), dim3(kSampleThreads), 0, s, static_cast<const T*>(logits),
                                        stride, vocab, temperature, top_k, top_p, min_p, uniform, out)));
  }
  note_launch();
}

void launch_apply_penalties(float* logits, const int* counts, const uint8_t* prompt_mask, const float* freq,
                            const float* presence, const float* repetition, int rows, int vocab, cudaStream_t s) {
  if (rows == 0) return;
  launch_pdl(apply_penalties_kernel, dim3((vocab + 255) / 256, rows), dim3(256), 0, s, logits, counts, prompt_mask, freq,
             presence, repetition, vocab);
  note_launch();
}

}  // namespace mb200
