// W4A16 GEMM: out[m, n] = x[m, k] * dequant(qweight)[n, k]^T (+ bias) with 4-bit weights, group-wise
// scales (and optional zero points), on the tcgen05 tensor cores.
//
// qweight int32 [N, K/8] (nibble i of word j of a row = element 8j + i), scales [N, K/group] in the
// activation type, zeros uint8 [N, K/group] or null (symmetric: zero point 8).
//
// The packed weights are the 128-row MMA operand: TMA stages 128 bytes of nibbles per row (four
// 64-element K blocks) in shared memory, four "dequant" warps (thread = weight row) expand them with the exponent-bias trick (bf16 0x4300 | q is
// exactly 128 + q; fp16 0x6400 | q is 1024 + q), subtract the offset exactly, multiply by the group scale
// (one rounding, the same value as rounding the fp32 dequantised weight) and store the block in the
// 128-byte-swizzled K-major layout the MMA reads; activations arrive by TMA as the MMA N operand
// (16..256 tokens per tile), so decode-sized batches stream the 4-bit weights once at full MMA width and
// prefill-sized batches amortise the expansion over 256 tokens.  Accumulators live in tensor memory
// (two buffers); epilogue warps write out[token][row].  Small problems are split along K into fp32
// partials that a second kernel sums in split order (deterministic).
//
// Warp roles (512 threads): 0 TMA producer, 1 MMA issuer, 2 TMEM allocator, 4-11 dequant (two threads per
// weight row: each expands half of the row's 64-element k-block), 12-15 epilogue.
//
// Nibble order inside a 32-bit word.  "natural": nibble i = element 8j + i.  "interleaved" (what the loaders
// produce for this kernel): element 8j + 2p + h sits in nibble p + 4h, so that ((word >> 4p) & 0x000F000F) holds
// the ADJACENT elements 2p and 2p + 1 in the low bits of its two 16-bit halves: one shift and one logic
// operation per pair instead of five.
// Every barrier wait is bounded (kStatusPipelineTimeout on expiry).
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace mb200 {
namespace {

constexpr int kBM = 128;
constexpr int kRowBytes = 128;
constexpr int kUmmaKBytes = 32;
constexpr int kW4Threads = 512;

struct W4Params {
  const uint32_t* qweight;
  const void* scales;
  const uint8_t* zeros;
  const void* bias;
  void* out;
  float* workspace;
  int* status;
  int m, n, k, group;
  int k_blocks, kb_per_split, splits;
  int tiles_n, tiles_m;
  int64_t ldc;
  int out_f16;
  int interleaved;   // nibble order of qweight (see the head of this file)
  uint32_t idesc;
};

template <int BN>
struct W4Cfg {
  static constexpr int kWBytes = kBM * kRowBytes;  // 16 KB of expanded weights per stage
  static constexpr int kXBytes = BN * kRowBytes;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kRawStages = BN >= 128 ? 2 : 4;   // packed-weight ring: 128 rows x 128 B = four k-blocks each
  static constexpr int kRawBytes = kBM * kRowBytes;      // 16 KB
  static constexpr int kStagesRaw = (196608 - kRawStages * kRawBytes) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kTmemColsRaw = 2 * BN;
  static constexpr int kTmemCols =
      kTmemColsRaw <= 32 ? 32 : (kTmemColsRaw <= 64 ? 64 : (kTmemColsRaw <= 128 ? 128 : (kTmemColsRaw <= 256 ? 256 : 512)));
};

template <typename T>
struct W4Magic;
template <>
struct W4Magic<__nv_bfloat16> {
  static constexpr uint32_t kOr = 0x43004300u;  // 128 + q
  static constexpr float kBase = 128.f;
};
template <>
struct W4Magic<__half> {
  static constexpr uint32_t kOr = 0x64006400u;  // 1024 + q
  static constexpr float kBase = 1024.f;
};

// (word >> 8*i): two nibbles -> packed 16-bit pair {128 + e_lo, 128 + e_hi} - offset, times scale
template <typename T>
__device__ __forceinline__ uint32_t dequant_pair(uint32_t t, uint32_t off2, uint32_t scale2);
template <>
__device__ __forceinline__ uint32_t dequant_pair<__nv_bfloat16>(uint32_t t, uint32_t off2, uint32_t scale2) {
  const uint32_t p = ((t & 0xFu) | ((t & 0xF0u) << 12)) | W4Magic<__nv_bfloat16>::kOr;
  __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&p);
  v = __hsub2(v, *reinterpret_cast<const __nv_bfloat162*>(&off2));
  v = __hmul2(v, *reinterpret_cast<const __nv_bfloat162*>(&scale2));
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t dequant_pair<__half>(uint32_t t, uint32_t off2, uint32_t scale2) {
  const uint32_t p = ((t & 0xFu) | ((t & 0xF0u) << 12)) | W4Magic<__half>::kOr;
  __half2 v = *reinterpret_cast<const __half2*>(&p);
  v = __hsub2(v, *reinterpret_cast<const __half2*>(&off2));
  v = __hmul2(v, *reinterpret_cast<const __half2*>(&scale2));
  return *reinterpret_cast<uint32_t*>(&v);
}

// interleaved nibble order: t = word >> 4p holds elements 2p (bits 0-3) and 2p + 1 (bits 16-19)
template <typename T>
__device__ __forceinline__ uint32_t dequant_pair_il(uint32_t t, uint32_t off2, uint32_t scale2);
template <>
__device__ __forceinline__ uint32_t dequant_pair_il<__nv_bfloat16>(uint32_t t, uint32_t off2, uint32_t scale2) {
  const uint32_t p = (t & 0x000F000Fu) | W4Magic<__nv_bfloat16>::kOr;
  __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&p);
  v = __hsub2(v, *reinterpret_cast<const __nv_bfloat162*>(&off2));
  v = __hmul2(v, *reinterpret_cast<const __nv_bfloat162*>(&scale2));
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t dequant_pair_il<__half>(uint32_t t, uint32_t off2, uint32_t scale2) {
  const uint32_t p = (t & 0x000F000Fu) | W4Magic<__half>::kOr;
  __half2 v = *reinterpret_cast<const __half2*>(&p);
  v = __hsub2(v, *reinterpret_cast<const __half2*>(&off2));
  v = __hmul2(v, *reinterpret_cast<const __half2*>(&scale2));
  return *reinterpret_cast<uint32_t*>(&v);
}

template <typename T>
__device__ __forceinline__ uint32_t splat2(float v);
template <>
__device__ __forceinline__ uint32_t splat2<__nv_bfloat16>(float v) {
  __nv_bfloat162 r = __float2bfloat162_rn(v);
  return *reinterpret_cast<uint32_t*>(&r);
}
template <>
__device__ __forceinline__ uint32_t splat2<__half>(float v) {
  __half2 r = __float2half2_rn(v);
  return *reinterpret_cast<uint32_t*>(&r);
}

template <typename T, int BN>
__global__ void __launch_bounds__(kW4Threads, 1)
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const W4Params p) {
  using C = W4Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* raw_ring = smem + static_cast<size_t>(C::kStages) * C::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(raw_ring + C::kRawStages * C::kRawBytes);
  uint64_t* full_x = bars;
  uint64_t* full_w = bars + C::kStages;
  uint64_t* empty_bar = bars + 2 * C::kStages;
  uint64_t* acc_full = bars + 3 * C::kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* raw_full = acc_empty + 2;                 // [kRawStages] TMA bytes landed
  uint64_t* raw_empty = raw_full + C::kRawStages;     // [kRawStages] the four expansion warps have copied their rows out
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(raw_empty + C::kRawStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_x[s], 1);
      mbar_init(&full_w[s], 8);  // one arrival per expansion warp
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 128);
    }
    for (int s = 0; s < C::kRawStages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_w);
  }
  __syncthreads();
  if (warp == 2) {
    tmem_alloc(tmem_holder, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  pdl_wait();

  const int split = blockIdx.y;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
  const int total_tiles = p.tiles_n * p.tiles_m;
  auto fail = [&]() {
    *abort_flag = 1;
    if (p.status != nullptr) atomicExch(p.status, kStatusPipelineTimeout);
  };

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer: activations and packed weights ----------------
    int stage = 0, rstage = 0;
    uint32_t phase = 0, rphase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (((kb - kb0) & 3) == 0) {  // kb0 is a multiple of four: one 128-byte column block of nibbles
          if (*abort_flag || !mbar_wait_relaxed(&raw_empty[rstage], rphase ^ 1)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&raw_full[rstage], C::kRawBytes);
          tma_load_2d(raw_ring + rstage * C::kRawBytes, &tm_w, &raw_full[rstage], (kb >> 2) * kRowBytes, tn * kBM);
          if (++rstage == C::kRawStages) {
            rstage = 0;
            rphase ^= 1;
          }
        }
        if (*abort_flag || !mbar_wait_relaxed(&empty_bar[stage], phase ^ 1)) {
          ok = false;
          break;
        }
        uint8_t* sb = smem + static_cast<size_t>(stage) * C::kStageBytes;
        mbar_arrive_expect_tx(&full_x[stage], C::kXBytes);
        tma_load_2d(sb + C::kWBytes, &tm_x, &full_x[stage], kb * 64, tm * BN);
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (!ok) fail();
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer ----------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int idx = 0;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++idx) {
      const int acc = idx & 1;
      if (*abort_flag || !mbar_wait_relaxed(&acc_empty[acc], ((idx >> 1) & 1) ^ 1)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t d_base = tmem_base + acc * BN;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (*abort_flag || !mbar_wait_relaxed(&full_x[stage], phase, 40) || !mbar_wait_relaxed(&full_w[stage], phase, 40)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(smem + static_cast<size_t>(stage) * C::kStageBytes);
        const uint64_t a_base = umma_desc_k_sw128(sa);
        const uint64_t b_base = umma_desc_k_sw128(sa + C::kWBytes);
#pragma unroll
        for (int kk = 0; kk < kRowBytes / kUmmaKBytes; ++kk) {
          umma_f16(d_base, a_base + ((kk * kUmmaKBytes) >> 4), b_base + ((kk * kUmmaKBytes) >> 4), p.idesc,
                   (kb > kb0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[stage]);
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit(&acc_full[acc]);
    }
    if (!ok) fail();
  } else if (warp >= 4 && warp < 12) {
    // ---------------- weight expansion: two threads per weight row of the tile ----------------
    // The packed rows arrive by TMA, 128 bytes (four k-blocks) per row at a time, so DRAM sees whole
    // 128-byte lines; a thread copies its half of the row out of the (128-byte swizzled) staging tile,
    // releases it, and expands its 32 elements of one k-block per operand stage.
    const int r = (threadIdx.x - 128) & 127;
    const int hf = (threadIdx.x - 128) >> 7;   // which 16 bytes of a k-block's 32 packed bytes
    int stage = 0, rstage = 0;
    uint32_t phase = 0, rphase = 0;
    bool ok = true;
    const int groups_per_row = p.k / p.group;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const int tn = tile / p.tiles_m;
      const int64_t row = static_cast<int64_t>(tn) * kBM + r;
      const bool row_ok = row < p.n;
      for (int kbg = kb0; kbg < kb1 && ok; kbg += 4) {
        // scales / zero points of the (up to four) groups touched by this column block: requested first
        T sc[4];
        uint8_t zp[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int kb = min(kbg + u, kb1 - 1);
          const int64_t gi = (row_ok ? row : 0) * groups_per_row + (kb * 64) / p.group;
          sc[u] = static_cast<const T*>(p.scales)[gi];
          zp[u] = p.zeros != nullptr ? p.zeros[gi] : static_cast<uint8_t>(8);
        }
        if (*abort_flag || !mbar_wait(&raw_full[rstage], rphase)) {
          ok = false;
          break;
        }
        uint4 raw[4];   // this thread's 16 bytes of each of the four k-blocks
        {
          const uint8_t* src = raw_ring + rstage * C::kRawBytes + r * kRowBytes;
#pragma unroll
          for (int u = 0; u < 4; ++u) raw[u] = *reinterpret_cast<const uint4*>(src + (((2 * u + hf) ^ (r & 7)) << 4));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&raw_empty[rstage]);  // arrivals on one barrier serialise: one per warp
        if (++rstage == C::kRawStages) {
          rstage = 0;
          rphase ^= 1;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (kbg + u >= kb1) break;
          const uint32_t scale2 = splat2<T>(to_f32(sc[u]));
          const uint32_t off2 = splat2<T>(W4Magic<T>::kBase + static_cast<float>(zp[u]));
          if (*abort_flag || !mbar_wait(&empty_bar[stage], phase ^ 1)) {
            ok = false;
            break;
          }
          uint8_t* dst = smem + static_cast<size_t>(stage) * C::kStageBytes + r * kRowBytes;
          const uint32_t words[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            uint4 o4;
            if (row_ok) {
              const uint32_t w = words[jj];
              if (p.interleaved) {
                o4.x = dequant_pair_il<T>(w, off2, scale2);
                o4.y = dequant_pair_il<T>(w >> 4, off2, scale2);
                o4.z = dequant_pair_il<T>(w >> 8, off2, scale2);
                o4.w = dequant_pair_il<T>(w >> 12, off2, scale2);
              } else {
                o4.x = dequant_pair<T>(w, off2, scale2);
                o4.y = dequant_pair<T>(w >> 8, off2, scale2);
                o4.z = dequant_pair<T>(w >> 16, off2, scale2);
                o4.w = dequant_pair<T>(w >> 24, off2, scale2);
              }
            } else {
              o4 = make_uint4(0, 0, 0, 0);
            }
            *reinterpret_cast<uint4*>(dst + (((4 * hf + jj) ^ (r & 7)) << 4)) = o4;
          }
          fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
          __syncwarp();
          if (lane == 0) mbar_arrive(&full_w[stage]);
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
    if (!ok) fail();
  } else if (warp >= 12) {
    // ---------------- epilogue: thread = weight row (output column) ----------------
    const int ew = warp - 12;
    const int row_in_tile = ew * 32 + lane;
    bool ok = true;
    int idx = 0;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++idx) {
      const int tn = tile / p.tiles_m, tm = tile % p.tiles_m;
      const int acc = idx & 1;
      if (*abort_flag || !mbar_wait_relaxed(&acc_full[acc], (idx >> 1) & 1, 500)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t t_base = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * BN;
      const int64_t wrow = static_cast<int64_t>(tn) * kBM + row_in_tile;
      const int valid = min(BN, p.m - tm * BN);
      const float bias = (p.bias != nullptr && wrow < p.n && split == 0)
                             ? (p.out_f16 ? __half2float(static_cast<const __half*>(p.bias)[wrow])
                                          : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[wrow]))
                             : 0.f;
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        uint32_t v[16];
        tmem_ld_32x16(t_base + c, v);
        tmem_ld_wait();
        if (wrow >= p.n || c >= valid) continue;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c + j >= valid) break;
          const float x = __uint_as_float(v[j]) + bias;
          const int64_t tok = static_cast<int64_t>(tm) * BN + c + j;
          if (p.splits > 1) {
            p.workspace[(static_cast<int64_t>(split) * p.m + tok) * p.n + wrow] = x;
          } else if (p.out_f16) {
            static_cast<__half*>(p.out)[tok * p.ldc + wrow] = __float2half_rn(x);
          } else {
            static_cast<__nv_bfloat16*>(p.out)[tok * p.ldc + wrow] = __float2bfloat16_rn(x);
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&acc_empty[acc]);
    }
    if (!ok) fail();
  }

  pdl_launch_dependents();
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <typename T>
__global__ void w4a16_splitk_reduce_kernel(const float* __restrict__ ws, T* __restrict__ out, int m, int n, int64_t ldc,
                                           int splits) {
  pdl_wait();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<int64_t>(m) * n) return;
  float acc = 0.f;
  for (int s = 0; s < splits; ++s) acc += ws[static_cast<int64_t>(s) * m * n + i];
  out[(i / n) * ldc + (i % n)] = from_f32<T>(acc);
}

template <typename T, int BN>
int launch_w4_cfg(const CUtensorMap& tx, const CUtensorMap& tw, const W4Params& p, dim3 grid, cudaStream_t s) {
  using C = W4Cfg<BN>;
  auto kern = w4a16_gemm_kernel<T, BN>;
  const size_t smem = static_cast<size_t>(C::kStages) * C::kStageBytes + C::kRawStages * C::kRawBytes + 1024 + 512;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), static_cast<int>(smem)) != cudaSuccess) return -3;
  const cudaError_t err = launch_pdl(kern, grid, dim3(kW4Threads), smem, s, tx, tw, p);
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}

}  // namespace

size_t w4a16_workspace_bytes(int m, int n, int k, int num_sms) {
  (void)k;
  (void)num_sms;
  return m <= 256 ? static_cast<size_t>(16) * m * n * sizeof(float) : 0;
}

int launch_w4a16_gemm(const W4A16Args& a, cudaStream_t s) {
  if (a.m <= 0 || a.n <= 0) return 0;
  if (a.m <= 8) {   // a handful of rows: stream and expand in registers
    const int rc = launch_w4a16_smallm(a, s);
    if (rc <= 0) return rc;
  }
  if (a.k % 64 != 0 || a.group % 64 != 0 || a.k % a.group != 0 || a.ldx % 8 != 0 || (a.k / 2) % 16 != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.qweight)) & 15) return -1;
  int bn = 16;
  while (bn < a.m && bn < 256) bn <<= 1;
  W4Params p{};
  p.qweight = static_cast<const uint32_t*>(a.qweight);
  p.scales = a.scales;
  p.zeros = a.zeros;
  p.bias = a.bias;
  p.out = a.out;
  p.workspace = a.workspace;
  p.status = a.status;
  p.m = a.m;
  p.n = a.n;
  p.k = a.k;
  p.group = a.group;
  p.k_blocks = a.k / 64;
  p.tiles_n = (a.n + kBM - 1) / kBM;
  p.tiles_m = (a.m + bn - 1) / bn;
  p.ldc = a.ldc;
  p.out_f16 = a.dt == kF16 ? 1 : 0;
  p.interleaved = a.interleaved;
  const uint32_t fmt = a.dt == kF16 ? 0u : 1u;
  p.idesc = umma_idesc(kBM, bn, 1u, fmt, fmt);
  const int num_sms = a.num_sms > 0 ? a.num_sms : 148;
  const int tiles = p.tiles_n * p.tiles_m;
  int splits = 1;
  if (tiles < num_sms && a.workspace != nullptr) {
    splits = std::min({16, std::max(1, num_sms / tiles), std::max(1, p.k_blocks / 4)});
    while (splits > 1 && static_cast<size_t>(splits) * a.m * a.n * sizeof(float) > a.workspace_bytes) --splits;
  }
  p.kb_per_split = ((p.k_blocks + splits - 1) / splits + 3) / 4 * 4;  // whole 128-byte column blocks per split
  splits = (p.k_blocks + p.kb_per_split - 1) / p.kb_per_split;
  p.splits = splits;
  CUtensorMap tx, tw;
  if (!make_tma_operand_map(&tx, a.x, a.m, a.k, a.ldx, 2, a.dt == kF16 ? 1 : 0, bn)) return -2;
  // packed weights as bytes: [n, k/2], 128-byte x 128-row boxes
  if (!make_tma_operand_map(&tw, a.qweight, a.n, a.k / 2, a.k / 2, 1, 2, kBM)) return -2;
  const dim3 grid(std::min(tiles, num_sms), splits);
  int rc = -1;
#define MB200_W4_CASE(BNV)                                                             \
  case BNV:                                                                            \
    rc = a.dt == kF16 ? launch_w4_cfg<__half, BNV>(tx, tw, p, grid, s)                     \
                      : launch_w4_cfg<__nv_bfloat16, BNV>(tx, tw, p, grid, s);             \
    break;
  switch (bn) {
    MB200_W4_CASE(16)
    MB200_W4_CASE(32)
    MB200_W4_CASE(64)
    MB200_W4_CASE(128)
    MB200_W4_CASE(256)
  }
#undef MB200_W4_CASE
  if (rc != 0 || splits == 1) return rc;
  const int64_t total = static_cast<int64_t>(a.m) * a.n;
  const dim3 rgrid(static_cast<unsigned>((total + 255) / 256)), rblock(256);
  MB200_DISPATCH_HALF(a.dt, (launch_pdl(w4a16_splitk_reduce_kernel<T>, rgrid, rblock, 0, s, a.workspace,
                                        static_cast<T*>(a.out), a.m, a.n, a.ldc, splits)));
  note_launch();
  return 0;
}

}  // namespace mb200
