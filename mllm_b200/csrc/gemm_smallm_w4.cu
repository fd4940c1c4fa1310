// out[m, n] = x[m, k] * dequant(qweight[n, k])^T for a handful of rows (m <= 8), 4-bit weights with group scales.
//
// The decode step of a 4-bit checkpoint streams a quarter of the bytes of the 16-bit model, so it should be the
// faster one; through the tcgen05 kernel of gemm_w4a16.cu (nibbles expanded into a shared-memory operand, one
// handshake between producer, expansion warps and MMA thread per 64-wide k block) it was slower.  This is the
// register-streaming kernel of gemm_smallm.cu with the expansion done in registers between the load and the
// warp-level MMA:
//   * a unit is 8 weight rows over the whole k range; the warps of a CTA take the 128-element
//     k steps of a unit round-robin.  A lane owns 16 bytes of packed weights per step: 32 consecutive k of one row;
//   * those 16 bytes, the 4 bytes that hold the row's scale for the step's group and the 4 bytes that hold its
//     zero point travel as cp.async copies into a shared-memory slice owned by the lane alone, 6 steps ahead;
//   * per step a lane expands its four words with the exponent-bias trick (nibble | magic = 128 + q as a 16-bit
//     float, exact subtraction of 128 + zero, one multiply by the scale) and feeds each word, with the 16 bytes
//     of activations at the same k offset, to two m16n8k16 MMAs.  The words are taken in an order rotated by the
//     lane's position in its row, so that the eight lanes of a quarter warp read eight different 16-byte bank
//     groups of the activation rows;
//   * activations (8 rows) are staged once per CTA; partial sums meet in shared memory at the end of a unit as
//     in gemm_smallm.cu.  Because the packed stream needs a quarter of the copy queue, the activation rows may
//     take most of the shared memory: a second shape of CTA (16 warps, two steps in flight) serves k up to 12288.
#include <algorithm>
#include <cstdint>
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace mb200 {
namespace {

constexpr int kQSlot = 768;            // bytes per warp and step: 32 x 16 of weights, 32 x 4 scale words, 32 x 4 zero words
constexpr int kQRowPad = 64;
// Two shapes of CTA.  k <= 4096: 8 warps, 6 steps in flight, two CTAs of 107 KB per SM.  k <= 12288 (the MLP's
// second matrix): the activation rows alone take 197 KB, so one CTA of 16 warps with 2 steps in flight per lane.
template <int WARPS, int DEPTH, int MAXK, int BLOCKS>
struct QCfg {
  static constexpr int kWarps = WARPS, kThreads = WARPS * 32, kDepth = DEPTH, kMaxK = MAXK, kBlocks = BLOCKS;
  static constexpr int kRingBytes = WARPS * DEPTH * kQSlot;
  static constexpr int kSmemMax = kRingBytes + 8 * (2 * MAXK + kQRowPad);
};
using QSmall = QCfg<8, 6, 4096, 2>;
using QLong = QCfg<16, 2, 12288, 1>;

struct W4SmallParams {
  const uint8_t* x;
  const uint8_t* qweight;   // [n, k/8] words
  const uint8_t* scales;    // [n, k/group] 16-bit
  const uint8_t* zeros;     // [n, k/group] bytes or null (zero point 8)
  const void* bias;
  void* out;
  int m, n, k, group;
  int64_t ldx_bytes, ldq_bytes, ldc;
  int groups_per_row;
  int units, units_per_cta, steps_per_warp;
  int interleaved;
};

template <bool F16>
__device__ __forceinline__ void mma_16816_w4(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
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

// 16-bit float pair helpers on packed registers
template <bool F16>
__device__ __forceinline__ uint32_t sub_mul2(uint32_t v, uint32_t off2, uint32_t scale2) {
  if constexpr (F16) {
    __half2 a = *reinterpret_cast<const __half2*>(&v);
    a = __hmul2(__hsub2(a, *reinterpret_cast<const __half2*>(&off2)), *reinterpret_cast<const __half2*>(&scale2));
    return *reinterpret_cast<uint32_t*>(&a);
  } else {
    __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v);
    a = __hmul2(__hsub2(a, *reinterpret_cast<const __nv_bfloat162*>(&off2)),
                *reinterpret_cast<const __nv_bfloat162*>(&scale2));
    return *reinterpret_cast<uint32_t*>(&a);
  }
}
template <bool F16>
__device__ __forceinline__ uint32_t splat_f(float v) {
  if constexpr (F16) {
    __half2 r = __float2half2_rn(v);
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    __nv_bfloat162 r = __float2bfloat162_rn(v);
    return *reinterpret_cast<uint32_t*>(&r);
  }
}
template <bool F16>
__device__ __forceinline__ float half_bits_to_f(uint16_t v) {
  if constexpr (F16) return __half2float(*reinterpret_cast<const __half*>(&v));
  return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&v));
}
template <bool F16>
__device__ __forceinline__ uint16_t f_to_half_bits(float v) {
  if constexpr (F16) {
    const __half h = __float2half_rn(v);
    return *reinterpret_cast<const uint16_t*>(&h);
  }
  const __nv_bfloat16 h = __float2bfloat16_rn(v);
  return *reinterpret_cast<const uint16_t*>(&h);
}

template <bool F16, typename C>
__global__ void __launch_bounds__(C::kThreads, C::kBlocks) gemm_smallm_w4_kernel(const W4SmallParams p) {
  constexpr int kQWarps = C::kWarps, kQThreads = C::kThreads, kQDepth = C::kDepth, kQRingBytes = C::kRingBytes;
  constexpr uint32_t kMagic = F16 ? 0x64006400u : 0x43004300u;   // 1024 + q / 128 + q as a 16-bit float pair
  constexpr float kBase = F16 ? 1024.f : 128.f;
  __shared__ float partial[2][kQWarps][64];
  extern __shared__ __align__(16) uint8_t smem_dyn[];
  uint8_t* ring_raw = smem_dyn;
  uint8_t* x_rows = smem_dyn + kQRingBytes;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;   // weight row inside the unit, and activation row
  const int c = lane & 3;    // which 32 k of the step's 128
  const int u0 = blockIdx.x * p.units_per_cta;
  const int u1 = min(p.units, u0 + p.units_per_cta);
  if (u0 >= u1) return;
  const int J = p.steps_per_warp;
  const int total = (u1 - u0) * J;
  const int x_pitch = 2 * p.k + kQRowPad;

  // slot s of this warp's ring: the lanes' 16 bytes of weights, then their scale words, then their zero words
  const uint32_t ring = smem_u32(ring_raw) + warp * (kQDepth * kQSlot);
  int lu = u0, lj = 0;
  auto issue = [&](int slot) {
    const int64_t row = static_cast<int64_t>(lu) * 8 + g;
    const int kstep = warp + kQWarps * lj;                 // 128-element step of the row
    const int koff = kstep * 128 + c * 32;                 // first k of this lane
    const int grp = koff / p.group;
    const uint32_t dst = ring + slot * kQSlot;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + lane * 16), "l"(p.qweight + row * p.ldq_bytes + (koff >> 1))
                 : "memory");
    const uint8_t* sc = p.scales + (row * p.groups_per_row + grp) * 2;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 512 + lane * 4),
                 "l"(reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(sc) & ~uintptr_t(3)))
                 : "memory");
    if (p.zeros != nullptr) {
      const uint8_t* zp = p.zeros + row * p.groups_per_row + grp;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 640 + lane * 4),
                   "l"(reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(zp) & ~uintptr_t(3)))
                   : "memory");
    }
    if (++lj == J) {
      lj = 0;
      ++lu;
    }
  };
  auto commit = [&]() { asm volatile("cp.async.commit_group;" ::: "memory"); };
  // weights, scales and zero points are parameters: nothing in the stream writes them
#pragma unroll
  for (int s = 0; s < kQDepth; ++s) {
    if (s < total) issue(s);
    commit();
  }
  pdl_wait();
  {
    const int vec_per_row = p.k >> 3;
    for (int v = threadIdx.x; v < 8 * vec_per_row; v += kQThreads) {
      const int r = v / vec_per_row, q = v - r * vec_per_row;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (r < p.m) val = __ldg(reinterpret_cast<const uint4*>(p.x + static_cast<int64_t>(r) * p.ldx_bytes) + q);
      *reinterpret_cast<uint4*>(x_rows + r * x_pitch + q * 16) = val;
    }
  }
  __syncthreads();
  const uint32_t x_lane = smem_u32(x_rows) + g * x_pitch + c * 64;

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  int cu = u0, cj = 0, buf = 0;
  for (int base = 0; base < total; base += kQDepth) {
#pragma unroll
    for (int s = 0; s < kQDepth; ++s) {
      const int i = base + s;
      if (i < total) {
        asm volatile("cp.async.wait_group %0;" ::"n"(kQDepth - 1) : "memory");
        const uint32_t slot = ring + s * kQSlot;
        const int kstep = warp + kQWarps * cj;
        const int grp = (kstep * 128 + c * 32) / p.group;
        // scale and zero point of (row, group): the copies fetched the aligned words that hold them
        const int64_t row = static_cast<int64_t>(cu) * 8 + g;
        const uintptr_t sc_addr = reinterpret_cast<uintptr_t>(p.scales) + (row * p.groups_per_row + grp) * 2;
        uint32_t sw, zw = 0;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(sw) : "r"(slot + 512 + lane * 4) : "memory");
        const float scale = half_bits_to_f<F16>(static_cast<uint16_t>((sc_addr & 2) ? (sw >> 16) : (sw & 0xFFFFu)));
        float zero = 8.f;
        if (p.zeros != nullptr) {
          asm volatile("ld.shared.u32 %0, [%1];" : "=r"(zw) : "r"(slot + 640 + lane * 4) : "memory");
          const uintptr_t z_addr = reinterpret_cast<uintptr_t>(p.zeros) + row * p.groups_per_row + grp;
          zero = static_cast<float>((zw >> (8 * (z_addr & 3))) & 0xFFu);
        }
        const uint32_t off2 = splat_f<F16>(kBase + zero);
        const uint32_t scale2 = splat_f<F16>(scale);
        const uint32_t x_step = x_lane + kstep * 256;      // 128 k = 256 bytes of the row per step
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int jj = (t + c) & 3;                      // rotated: bank-conflict-free activation reads
          uint32_t w;
          asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(slot + lane * 16 + jj * 4) : "memory");
          uint4 x;
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(x.x), "=r"(x.y), "=r"(x.z), "=r"(x.w)
                       : "r"(x_step + jj * 16)
                       : "memory");
          uint32_t b0, b1, b2, b3;   // element pairs (0,1) (2,3) (4,5) (6,7) of the word
          if (p.interleaved) {
            b0 = sub_mul2<F16>((w & 0x000F000Fu) | kMagic, off2, scale2);
            b1 = sub_mul2<F16>(((w >> 4) & 0x000F000Fu) | kMagic, off2, scale2);
            b2 = sub_mul2<F16>(((w >> 8) & 0x000F000Fu) | kMagic, off2, scale2);
            b3 = sub_mul2<F16>(((w >> 12) & 0x000F000Fu) | kMagic, off2, scale2);
          } else {
            b0 = sub_mul2<F16>(((w & 0xFu) | ((w & 0xF0u) << 12)) | kMagic, off2, scale2);
            b1 = sub_mul2<F16>((((w >> 8) & 0xFu) | (((w >> 8) & 0xF0u) << 12)) | kMagic, off2, scale2);
            b2 = sub_mul2<F16>((((w >> 16) & 0xFu) | (((w >> 16) & 0xF0u) << 12)) | kMagic, off2, scale2);
            b3 = sub_mul2<F16>((((w >> 24) & 0xFu) | (((w >> 24) & 0xF0u) << 12)) | kMagic, off2, scale2);
          }
          mma_16816_w4<F16>(acc, x.x, x.y, b0, b1);
          mma_16816_w4<F16>(acc, x.z, x.w, b2, b3);
        }
        if (i + kQDepth < total) issue(s);   // after the loads above: the slot's old bytes are consumed
        commit();
        if (++cj == J) {
          cj = 0;
          *reinterpret_cast<float2*>(&partial[buf][warp][lane * 2]) = make_float2(acc[0], acc[1]);
          acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
          __syncthreads();
          if (threadIdx.x < 64) {
            const int tt = threadIdx.x;
            const int mrow = tt >> 3, slot_n = tt & 7;
            float v = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < kQWarps; ++w8) v += partial[buf][w8][tt];
            if (mrow < p.m) {
              const int64_t col = static_cast<int64_t>(cu) * 8 + slot_n;
              if (p.bias != nullptr) v += half_bits_to_f<F16>(static_cast<const uint16_t*>(p.bias)[col]);
              static_cast<uint16_t*>(p.out)[mrow * p.ldc + col] = f_to_half_bits<F16>(v);
            }
          }
          ++cu;
          buf ^= 1;
        }
      }
    }
  }
}

template <typename C>
int launch_w4_cfg(W4SmallParams p, const W4A16Args& a, cudaStream_t s) {
  p.steps_per_warp = a.k / (128 * C::kWarps);
  const int slots = std::max(1, a.num_sms > 0 ? a.num_sms : 148) * C::kBlocks;
  p.units_per_cta = (p.units + slots - 1) / slots;
  const int grid = (p.units + p.units_per_cta - 1) / p.units_per_cta;
  const int smem = C::kRingBytes + 8 * (2 * a.k + kQRowPad);
  cudaError_t err;
  if (a.dt == kF16) {
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(gemm_smallm_w4_kernel<true, C>), C::kSmemMax) != cudaSuccess) return -3;
    err = launch_pdl(gemm_smallm_w4_kernel<true, C>, dim3(grid), dim3(C::kThreads), smem, s, p);
  } else {
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(gemm_smallm_w4_kernel<false, C>), C::kSmemMax) != cudaSuccess) return -3;
    err = launch_pdl(gemm_smallm_w4_kernel<false, C>, dim3(grid), dim3(C::kThreads), smem, s, p);
  }
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}

}  // namespace

// Returns 0 when launched, 1 when the shape is not for this kernel (the caller goes on to the tcgen05 kernel).
int launch_w4a16_smallm(const W4A16Args& a, cudaStream_t s) {
  static const int knob = [] {
    const char* e = std::getenv("MLLM_B200_W4_SMALLM");
    return e == nullptr ? 1 : std::atoi(e);
  }();
  if (!knob || a.m > 8 || a.n % 8 != 0) return 1;
  const bool small_k = a.k <= QSmall::kMaxK && a.k % (128 * QSmall::kWarps) == 0;
  const bool long_k = a.k <= QLong::kMaxK && a.k % (128 * QLong::kWarps) == 0;
  if ((!small_k && !long_k) || a.group % 32 != 0 || a.k % a.group != 0) return 1;
  if ((a.ldx * 2) % 16 != 0 || ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.qweight)) & 15) != 0) return 1;
  if ((reinterpret_cast<uintptr_t>(a.scales) & 1) != 0) return 1;
  W4SmallParams p{};
  p.x = static_cast<const uint8_t*>(a.x);
  p.qweight = static_cast<const uint8_t*>(a.qweight);
  p.scales = static_cast<const uint8_t*>(a.scales);
  p.zeros = a.zeros;
  p.bias = a.bias;
  p.out = a.out;
  p.m = a.m;
  p.n = a.n;
  p.k = a.k;
  p.group = a.group;
  p.ldx_bytes = a.ldx * 2;
  p.ldq_bytes = static_cast<int64_t>(a.k) / 2;
  p.ldc = a.ldc;
  p.groups_per_row = a.k / a.group;
  p.units = a.n / 8;
  p.interleaved = a.interleaved;
  return small_k ? launch_w4_cfg<QSmall>(p, a, s) : launch_w4_cfg<QLong>(p, a, s);
}

}  // namespace mb200
