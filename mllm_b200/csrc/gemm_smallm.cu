// out[m, n] = a[m, k] * b[n, k]^T for a handful of rows (m <= 8): the decode step of a small batch.
//
// With eight activation rows the product is a stream of the weight matrix through the SMs; the arithmetic
// is negligible and the cost of the tcgen05 path (tensor-memory allocation, a TMA ring to fill, a tile of
// 128 weight rows per CTA and therefore a split of k with partial sums exchanged between CTAs) is a fixed
// 6-8 us per launch, as much again as the streaming time of a 4096 x 4096 projection.  This kernel keeps
// nothing but registers between the load and the sum:
//   * a unit of work is 8 weight rows over the whole k range; a CTA (one per SM) owns a contiguous run of
//     units, its 16 warps take the 32-element k steps of a unit round-robin, so the warps of a CTA read 1 KB
//     of each of the 8 rows per round;
//   * a lane loads 16 bytes of one weight row and the 16 bytes of one activation row at the same k offset
//     and feeds them to two warp-level MMAs (m16n8k16: activations in the upper 8 rows of A, lower rows zero;
//     the 8 weight rows are B's columns).  The k positions inside an MMA are permuted the same way for both
//     operands, which a dot product does not notice, so no shuffling is needed to build fragments;
//   * weight loads run 16 steps ahead and cross unit boundaries.  They are cp.async copies into a slice of
//     shared memory that belongs to the lane alone: the lane later reads back exactly the 16 bytes it asked
//     for, so shared memory is only a deep queue behind the register file (128 KB in flight per SM; a
//     register ring of 8 steps reached 4.1 TB/s on a 1.2 GB matrix, the tcgen05 path's TMA ring 6.5) and
//     needs no barrier, just cp.async.wait_group.  Weights are requested before the stream-order wait when
//     they are model parameters (nothing in the stream writes them);
//   * the batch's 8 rows are copied to shared memory once per CTA (read through L1 they missed: the ring
//     leaves L1 too small, and every step then paid an L2 round trip), rows 64 bytes apart modulo 128 so
//     that a warp's read of 8 rows x 64 bytes has no bank conflict; hence k <= 4096.  (Walking a longer k in
//     pieces, with the activations of a piece staged at a time, was tried and was slower than the tcgen05
//     path: 32-43 us against 23 us for a 4096 x 12288 projection; so was a cluster of four CTAs sharing the k range
//     with one exchange of partial sums at the end: 37 clusters of four 200 KB CTAs do not fit one wave, 42.6 us.)
//   * at the end of a unit the warps' 8 x 8 partial sums meet in shared memory (double-buffered, one
//     __syncthreads per unit) and 64 threads add bias / residual or apply SwiGLU and store.
#include <algorithm>
#include <cstdint>

#include "common.cuh"
#include "kernels.h"

namespace mb200 {
namespace {

constexpr int kSmWarps = 16;         // warps per CTA, one CTA per SM
constexpr int kSmThreads = kSmWarps * 32;
constexpr int kSmDepth = 16;         // weight loads (k steps) in flight per lane
constexpr int kSmRingBytes = kSmWarps * kSmDepth * 512;   // 128 KB: 512 bytes per warp and step
constexpr int kSmMaxK = 4096;        // the 8 activation rows live in shared memory: 8 x (2 k + 64) bytes
constexpr int kSmRowPad = 64;        // bytes between activation rows beyond 2 k: two rows never share a bank half

struct SmallMParams {
  const uint8_t* a;      // activations
  const uint8_t* b;      // weights
  void* out;
  const void* bias;
  const void* residual;
  int m, n, k;
  int64_t lda_bytes, ldb_bytes, ldc, ld_res;
  int units;             // 8-row units (SwiGLU: 4 gate + 4 up rows, 4 outputs)
  int units_per_cta;
  int steps_per_warp;    // k / 32 / kSmWarps
  int swiglu;
  int b_static;
  int early_trigger;     // let the kernels behind this one start their set-up as soon as this one runs
  // fused prologue (norm_w != null): the rows fed to the product are rmsnorm(a + norm_res) * norm_w, with the sum
  // rounded to 16 bits first (it is the new residual stream, which CTA 0 also writes to norm_res_out)
  const void* norm_w;
  const uint8_t* norm_res;     // may be null: the rows of `a` are the residual stream already
  uint8_t* norm_res_out;       // may be null
  int64_t norm_res_ld_bytes, norm_res_out_ld_bytes;
  float norm_eps;
};

template <bool F16>
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  // rows 8..15 of A (registers a1, a3) are zero: only the batch's 8 rows carry data
  if constexpr (F16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
  }
}

template <bool F16>
__device__ __forceinline__ float half_to_f(uint16_t v) {
  if constexpr (F16) return __half2float(*reinterpret_cast<const __half*>(&v));
  return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&v));
}
template <bool F16>
__device__ __forceinline__ uint16_t f_to_half(float v) {
  if constexpr (F16) {
    const __half h = __float2half_rn(v);
    return *reinterpret_cast<const uint16_t*>(&h);
  }
  const __nv_bfloat16 h = __float2bfloat16_rn(v);
  return *reinterpret_cast<const uint16_t*>(&h);
}

template <bool F16>
__global__ void __launch_bounds__(kSmThreads, 1) gemm_smallm_kernel(const SmallMParams p) {
  __shared__ float partial[2][kSmWarps][64];
  extern __shared__ __align__(16) uint8_t smem_dyn[];
  uint8_t* ring_raw = smem_dyn;
  uint8_t* x_rows = smem_dyn + kSmRingBytes;     // 8 rows of 2 k + kSmRowPad bytes
  if (p.early_trigger) pdl_launch_dependents();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;   // weight row inside the unit, and activation row
  const int c = lane & 3;    // which 16 bytes of the 64-byte k step
  const int u0 = blockIdx.x * p.units_per_cta;
  const int u1 = min(p.units, u0 + p.units_per_cta);
  if (u0 >= u1) return;
  const int J = p.steps_per_warp;
  const int total = (u1 - u0) * J;   // k steps of this warp over the CTA's units
  const int x_pitch = 2 * p.k + kSmRowPad;

  // weight row of slot g of unit u (SwiGLU: slots 0-3 gate rows, 4-7 the matching up rows, 128 rows later)
  auto row_of = [&](int u) -> int64_t {
    if (!p.swiglu) return static_cast<int64_t>(u) * 8 + g;
    const int blk = u >> 5, q = u & 31;
    return static_cast<int64_t>(blk) * 256 + (g < 4 ? 0 : 128) + q * 4 + (g & 3);
  };
  const int64_t k_off0 = (static_cast<int64_t>(warp) * 32 + c * 8) * 2;   // bytes; step j adds j * kSmWarps * 64
  // this lane's 16 bytes of slot s of the ring
  const uint32_t ring = smem_u32(ring_raw) + (warp * kSmDepth * 32 + lane) * 16;
  // load cursor
  int lu = u0, lj = 0;
  const uint8_t* w_row = p.b + row_of(lu) * p.ldb_bytes + k_off0;
  auto load_w = [&](int slot) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring + slot * 512),
                 "l"(w_row + static_cast<int64_t>(lj) * (kSmWarps * 64))
                 : "memory");
  };
  auto commit = [&]() { asm volatile("cp.async.commit_group;" ::: "memory"); };
  auto advance = [&]() {
    if (++lj == J) {
      lj = 0;
      ++lu;
      if (lu < u1) w_row = p.b + row_of(lu) * p.ldb_bytes + k_off0;
    }
  };
  // prologue: the first kSmDepth steps.  Weights that are model parameters go out before the stream-order
  // wait; activations are written by the previous kernel.
  if (!p.b_static) pdl_wait();
#pragma unroll
  for (int s = 0; s < kSmDepth; ++s) {
    if (s < total) {
      load_w(s);
      advance();
    }
    commit();   // one group per step, empty past the end, so that "all but the newest 15" means step i
  }
  if (p.b_static) pdl_wait();
  // the batch's rows into shared memory (rows past m are zero); every warp reads all of them again and again
  const int vec_per_row = p.k >> 3;
  if (p.norm_w == nullptr) {
    for (int v = threadIdx.x; v < 8 * vec_per_row; v += kSmThreads) {
      const int r = v / vec_per_row, q = v - r * vec_per_row;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (r < p.m) val = __ldg(reinterpret_cast<const uint4*>(p.a + static_cast<int64_t>(r) * p.lda_bytes) + q);
      *reinterpret_cast<uint4*>(x_rows + r * x_pitch + q * 16) = val;
    }
    __syncthreads();
  } else {
    // Fused add + RMSNorm: every CTA normalises the same 8 rows for itself (a few tens of KB from L2, while
    // its weight copies are already in flight); CTA 0 also stores the new residual stream.
    float ss[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) ss[r] = 0.f;
    for (int q = threadIdx.x; q < vec_per_row; q += kSmThreads) {
      // all sixteen loads of this column of vectors first: one round trip to L2, not sixteen
      uint4 val[8], res[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        val[r] = make_uint4(0, 0, 0, 0);
        if (r < p.m) val[r] = __ldg(reinterpret_cast<const uint4*>(p.a + static_cast<int64_t>(r) * p.lda_bytes) + q);
      }
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        res[r] = make_uint4(0, 0, 0, 0);
        if (r < p.m && p.norm_res != nullptr)
          res[r] = __ldg(reinterpret_cast<const uint4*>(p.norm_res + static_cast<int64_t>(r) * p.norm_res_ld_bytes) + q);
      }
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < p.m) {
          uint16_t* e = reinterpret_cast<uint16_t*>(&val[r]);
          if (p.norm_res != nullptr) {
            const uint16_t* f = reinterpret_cast<const uint16_t*>(&res[r]);
#pragma unroll
            for (int i = 0; i < 8; ++i) e[i] = f_to_half<F16>(half_to_f<F16>(e[i]) + half_to_f<F16>(f[i]));
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float x = half_to_f<F16>(e[i]);
            ss[r] += x * x;
          }
          if (blockIdx.x == 0 && p.norm_res_out != nullptr)
            *(reinterpret_cast<uint4*>(p.norm_res_out + static_cast<int64_t>(r) * p.norm_res_out_ld_bytes) + q) = val[r];
        }
        *reinterpret_cast<uint4*>(x_rows + r * x_pitch + q * 16) = val[r];
      }
    }
    float* red = &partial[0][0][0];     // [warp][8] sums of squares, then [8] reciprocal root mean squares
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const float w = warp_sum(ss[r]);
      if (lane == 0) red[warp * 8 + r] = w;
    }
    __syncthreads();
    if (threadIdx.x < 8) {
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < kSmWarps; ++w) tot += red[w * 8 + threadIdx.x];
      red[kSmWarps * 8 + threadIdx.x] = rsqrtf(tot / static_cast<float>(p.k) + p.norm_eps);
    }
    __syncthreads();
    for (int q = threadIdx.x; q < vec_per_row; q += kSmThreads) {
      const uint4 wv = __ldg(reinterpret_cast<const uint4*>(p.norm_w) + q);
      const uint16_t* f = reinterpret_cast<const uint16_t*>(&wv);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < p.m) {
          const float rstd = red[kSmWarps * 8 + r];
          uint4 val = *reinterpret_cast<const uint4*>(x_rows + r * x_pitch + q * 16);
          uint16_t* e = reinterpret_cast<uint16_t*>(&val);
#pragma unroll
          for (int i = 0; i < 8; ++i) e[i] = f_to_half<F16>(half_to_f<F16>(e[i]) * rstd * half_to_f<F16>(f[i]));
          *reinterpret_cast<uint4*>(x_rows + r * x_pitch + q * 16) = val;
        }
      }
    }
    __syncthreads();
  }
  const uint32_t x_lane = smem_u32(x_rows) + g * x_pitch + static_cast<uint32_t>(k_off0);
  int xj = 0;

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  int cu = u0, cj = 0, buf = 0;
  for (int base = 0; base < total; base += kSmDepth) {
#pragma unroll
    for (int s = 0; s < kSmDepth; ++s) {
      const int i = base + s;
      if (i < total) {
        asm volatile("cp.async.wait_group %0;" ::"n"(kSmDepth - 1) : "memory");
        uint4 w;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                     : "r"(ring + s * 512)
                     : "memory");
        uint4 x;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(x.x), "=r"(x.y), "=r"(x.z), "=r"(x.w)
                     : "r"(x_lane + xj * (kSmWarps * 64))
                     : "memory");
        if (++xj == J) xj = 0;
        mma_16816<F16>(acc, x.x, x.y, w.x, w.y);
        mma_16816<F16>(acc, x.z, x.w, w.z, w.w);
        // refill the slot with the step kSmDepth ahead: after the MMAs, whose operands are the slot's old bytes
        if (i + kSmDepth < total) {
          load_w(s);
          advance();
        }
        commit();
        if (++cj == J) {
          // ---- end of a unit: all warps get here at the same step ----
          cj = 0;
          *reinterpret_cast<float2*>(&partial[buf][warp][lane * 2]) = make_float2(acc[0], acc[1]);
          acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
          __syncthreads();
          if (threadIdx.x < 64) {
            const int t = threadIdx.x;
            const int mrow = t >> 3, slot = t & 7;
            float v = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < kSmWarps; ++w8) v += partial[buf][w8][t];
            if (mrow < p.m) {
              if (p.swiglu) {
                if (slot < 4) {
                  float up = 0.f;
#pragma unroll
                  for (int w8 = 0; w8 < kSmWarps; ++w8) up += partial[buf][w8][t + 4];
                  const int blk = cu >> 5, q = cu & 31;
                  const int64_t col = static_cast<int64_t>(blk) * 128 + q * 4 + slot;
                  const float y = v / (1.f + __expf(-v)) * up;
                  static_cast<uint16_t*>(p.out)[mrow * p.ldc + col] = f_to_half<F16>(y);
                }
              } else {
                const int64_t col = static_cast<int64_t>(cu) * 8 + slot;
                if (p.bias != nullptr) v += half_to_f<F16>(static_cast<const uint16_t*>(p.bias)[col]);
                if (p.residual != nullptr)
                  v += half_to_f<F16>(static_cast<const uint16_t*>(p.residual)[mrow * p.ld_res + col]);
                static_cast<uint16_t*>(p.out)[mrow * p.ldc + col] = f_to_half<F16>(v);
              }
            }
          }
          ++cu;
          buf ^= 1;
        }
      }
    }
  }
}

}  // namespace

// Returns 0 when launched, 1 when the shape is not for this kernel (the caller goes on to the tcgen05 path).
int launch_gemm_smallm(const GemmArgs& a, cudaStream_t s) {
  static const int knob = [] {
    const char* e = std::getenv("MLLM_B200_GEMM_SMALLM");
    return e == nullptr ? 1 : std::atoi(e);
  }();
  if (!knob || a.m > 8 || a.is_int8 || a.gate_flags != nullptr || a.rs_tp > 0) return 1;
  if (a.k % (32 * kSmWarps) != 0 || a.k > kSmMaxK || a.n % 8 != 0) return 1;
  // matrices of hundreds of MB (the vocabulary head) stream at the full copy rate through the TMA ring of the
  // tcgen05 path, whose set-up cost no longer shows; this kernel is for the projections of a layer
  if (static_cast<int64_t>(a.n) * a.k * 2 > (int64_t(384) << 20)) return 1;
  if (a.swiglu && (a.n % 256 != 0 || a.bias != nullptr || a.residual != nullptr)) return 1;
  if ((a.lda * 2) % 16 != 0 || (a.ldb * 2) % 16 != 0) return 1;
  if (a.norm_weight != nullptr &&
      ((a.norm_residual_ld * 2) % 16 != 0 || (a.norm_residual_out_ld * 2) % 16 != 0 ||
       ((reinterpret_cast<uintptr_t>(a.norm_weight) | reinterpret_cast<uintptr_t>(a.norm_residual) |
         reinterpret_cast<uintptr_t>(a.norm_residual_out)) & 15) != 0 ||
       (a.norm_residual != nullptr && a.norm_residual == a.norm_residual_out)))
    return 1;
  SmallMParams p{};
  p.a = static_cast<const uint8_t*>(a.a);
  p.b = static_cast<const uint8_t*>(a.b);
  p.out = a.out;
  p.bias = a.bias;
  p.residual = a.residual;
  p.m = a.m;
  p.n = a.n;
  p.k = a.k;
  p.lda_bytes = a.lda * 2;
  p.ldb_bytes = a.ldb * 2;
  p.ldc = a.ldc;
  p.ld_res = a.ld_res;
  p.units = a.n / 8;
  p.steps_per_warp = a.k / (32 * kSmWarps);
  p.swiglu = a.swiglu;
  p.b_static = a.b_static;
  p.norm_w = a.norm_weight;
  p.norm_res = static_cast<const uint8_t*>(a.norm_residual);
  p.norm_res_out = static_cast<uint8_t*>(a.norm_residual_out);
  p.norm_res_ld_bytes = a.norm_residual_ld * 2;
  p.norm_res_out_ld_bytes = a.norm_residual_out_ld * 2;
  p.norm_eps = a.norm_eps;
  static const int trigger_knob = [] {
    // measured on the decode step of an 8B model: 5.22 ms per step with the trigger at the start, 4.95 ms without
    const char* e = std::getenv("MLLM_B200_GEMM_SMALLM_TRIGGER");
    return e == nullptr ? 0 : std::atoi(e);
  }();
  p.early_trigger = trigger_knob;
  // one CTA per SM, every CTA the same number of units (the stream is bound by memory, not by the number of SMs
  // that pull on it, as long as enough loads are in flight)
  const int slots = std::max(1, a.num_sms);
  p.units_per_cta = (p.units + slots - 1) / slots;
  const int grid = (p.units + p.units_per_cta - 1) / p.units_per_cta;
  const int smem = kSmRingBytes + 8 * (2 * a.k + kSmRowPad);
  cudaError_t err;
  if (a.dt == kF16) {
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(gemm_smallm_kernel<true>), kSmRingBytes + 8 * (2 * kSmMaxK + kSmRowPad)) != cudaSuccess) return -3;
    err = launch_pdl(gemm_smallm_kernel<true>, dim3(grid), dim3(kSmThreads), smem, s, p);
  } else {
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(gemm_smallm_kernel<false>), kSmRingBytes + 8 * (2 * kSmMaxK + kSmRowPad)) != cudaSuccess) return -3;
    err = launch_pdl(gemm_smallm_kernel<false>, dim3(grid), dim3(kSmThreads), smem, s, p);
  }
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}

}  // namespace mb200
