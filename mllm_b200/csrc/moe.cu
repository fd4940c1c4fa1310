// Mixture-of-experts kernels: router (softmax -> top-k -> renormalise), token alignment
// (counting sort of the (token, choice) pairs by expert, all on the device so a decode step can
// be captured in a CUDA graph), row gather, grouped expert GEMM on the tcgen05 tensor cores and
// the weighted combine.
//
// Grouped GEMM: for every local expert e, out[rows of e] = act[rows of e] * W[e]^T where the rows
// of e are a contiguous range of the expert-sorted activation matrix.  The weights are the
// 128-row MMA operand ("swap" tiling: weight rows = MMA M, tokens = MMA N), so an expert with a
// handful of tokens still issues full-width MMAs and the kernel streams every active expert's
// weights exactly once.  Work items (expert, token chunk) are written by the align kernel; CTAs
// are persistent and walk item x weight-row-tile pairs.  With SWIGLU the weights hold alternating
// 128-row gate / up blocks and the epilogue writes silu(gate) * up.
//
// Warp roles (256 threads): warp 0 TMA producer, warp 1 MMA issuer, warp 2 TMEM allocator,
// warps 4-7 epilogue.  Every barrier wait is bounded (kStatusPipelineTimeout on expiry).
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace mb200 {
namespace {

constexpr int kBM = 128;
constexpr int kRowBytes = 128;
constexpr int kUmmaKBytes = 32;
constexpr int kThreads = 256;
constexpr int kMaxExperts = 256;

// --------------------------------------------------------------------------------------------
// router: one warp per token
// --------------------------------------------------------------------------------------------
template <typename T>
__global__ void moe_router_topk_kernel(const T* __restrict__ logits, int64_t stride, float* __restrict__ w_out,
                                       int* __restrict__ id_out, int tokens, int experts, int top_k, int renorm) {
  pdl_wait();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const T* row = logits + static_cast<int64_t>(t) * stride;
  float v[kMaxExperts / 32];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxExperts / 32; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < experts ? to_f32(row[e]) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxExperts / 32; ++i) {
    v[i] = (lane + 32 * i) < experts ? __expf(v[i] - mx) : -1.f;  // probabilities are >= 0; -1 = absent
    if (v[i] > 0.f) sum += v[i];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  float chosen_w = 0.f;  // lane j keeps the j-th choice
  int chosen_e = 0;
  float ksum = 0.f;
  for (int j = 0; j < top_k; ++j) {
    float best = -2.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) {
      if (v[i] > best) {  // ascending i: the lowest index wins ties inside a lane
        best = v[i];
        bi = lane + 32 * i;
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
    if ((bi & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kMaxExperts / 32; ++i)
        if (i == (bi >> 5)) v[i] = -1.f;
    }
    const float pw = best * inv;
    ksum += pw;
    if (lane == j) {
      chosen_w = pw;
      chosen_e = bi;
    }
  }
  if (lane < top_k) {
    w_out[static_cast<int64_t>(t) * top_k + lane] = renorm ? chosen_w / ksum : chosen_w;
    id_out[static_cast<int64_t>(t) * top_k + lane] = chosen_e;
  }
}

// --------------------------------------------------------------------------------------------
// align: counting sort of the pairs by local expert + work list, one CTA
// --------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ topk_ids, int pairs, int top_k, int expert_offset, int experts, int bn,
                 int* __restrict__ sorted_pos, int* __restrict__ src_token, int* __restrict__ expert_offsets,
                 int2* __restrict__ work, int* __restrict__ n_work, int max_work) {
  pdl_wait();
  __shared__ int cnt[kMaxExperts], off[kMaxExperts + 1], wbase[kMaxExperts + 1], fill[kMaxExperts];
  for (int e = threadIdx.x; e < kMaxExperts; e += blockDim.x) {
    cnt[e] = 0;
    fill[e] = 0;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = topk_ids[i] - expert_offset;
    if (e >= 0 && e < experts) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, w = 0;
    for (int e = 0; e < experts; ++e) {
      off[e] = o;
      wbase[e] = w;
      o += cnt[e];
      w += (cnt[e] + bn - 1) / bn;
    }
    off[experts] = o;
    wbase[experts] = w;
    *n_work = min(w, max_work);
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) expert_offsets[e] = off[e];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int chunks = wbase[e + 1] - wbase[e];
    for (int c = 0; c < chunks; ++c)
      if (wbase[e] + c < max_work) work[wbase[e] + c] = make_int2(e, c);
  }
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = topk_ids[i] - expert_offset;
    if (e >= 0 && e < experts) {
      const int pos = off[e] + atomicAdd(&fill[e], 1);
      sorted_pos[i] = pos;
      src_token[pos] = i / top_k;
    } else {
      sorted_pos[i] = -1;
    }
  }
}

// xs[pos, :] = x[src_token[pos], :] for the local pairs (16-byte vectors)
__global__ void moe_gather_kernel(const uint4* __restrict__ x, int64_t x_stride_v, const int* __restrict__ src_token,
                                  const int* __restrict__ expert_offsets, int experts, uint4* __restrict__ xs,
                                  int row_vecs) {
  pdl_wait();
  const int pos = blockIdx.x;
  if (pos >= expert_offsets[experts]) return;
  const uint4* src = x + static_cast<int64_t>(src_token[pos]) * x_stride_v;
  uint4* dst = xs + static_cast<int64_t>(pos) * row_vecs;
  for (int i = threadIdx.x; i < row_vecs; i += blockDim.x) dst[i] = __ldg(src + i);
}

// out[t, :] = sum_j w[t, j] * y[sorted_pos[t*k + j], :]   (choices on other ranks contribute nothing)
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ sorted_pos,
                                   const float* __restrict__ topk_w, T* __restrict__ out, int hidden, int top_k) {
  pdl_wait();
  const int t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      const int pos = sorted_pos[t * top_k + j];
      if (pos < 0) continue;
      const float w = topk_w[t * top_k + j];
      const uint4 raw = *reinterpret_cast<const uint4*>(y + static_cast<int64_t>(pos) * hidden + c);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += w * to_f32(e[i]);
    }
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int i = 0; i < 8; ++i) oe[i] = from_f32<T>(acc[i]);
    *reinterpret_cast<uint4*>(out + static_cast<int64_t>(t) * hidden + c) = o;
  }
}

// --------------------------------------------------------------------------------------------
// grouped GEMM
// --------------------------------------------------------------------------------------------
struct GroupedParams {
  void* out;
  int64_t ldc;
  const int* expert_offsets;
  const int2* work;
  const int* n_work;
  int* status;
  int n;         // weight rows per expert
  int k_blocks;
  int tiles_r;   // weight-row tiles per expert
  int out_f16;
  uint32_t idesc;
};

template <int BN, bool SWIGLU>
struct GCfg {
  static constexpr int R = SWIGLU ? 2 : 1;
  static constexpr int kRowTileBytes = kBM * R * kRowBytes;
  static constexpr int kStageBytes = kRowTileBytes + BN * kRowBytes;
  static constexpr int kStagesRaw = 196608 / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kAccCols = R * BN;
  static constexpr int kTmemColsRaw = 2 * kAccCols;
  static constexpr int kTmemCols =
      kTmemColsRaw <= 32 ? 32 : (kTmemColsRaw <= 64 ? 64 : (kTmemColsRaw <= 128 ? 128 : (kTmemColsRaw <= 256 ? 256 : 512)));
  static_assert(kTmemColsRaw <= 512, "accumulators exceed tensor memory");
};

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }

template <int BN, bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
moe_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                        const GroupedParams p) {
  using C = GCfg<BN, SWIGLU>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(C::kStages) * C::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::kStages;
  uint64_t* acc_full = bars + 2 * C::kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 128);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
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

  const int total = *p.n_work * p.tiles_r;
  // item -> (expert, first sorted row of the chunk, valid rows in the chunk, weight-row tile)
  auto get_item = [&](int item, int& e, int& row0, int& valid, int& tile) {
    const int2 w = p.work[item / p.tiles_r];
    tile = item % p.tiles_r;
    e = w.x;
    const int o0 = p.expert_offsets[e], o1 = p.expert_offsets[e + 1];
    row0 = o0 + w.y * BN;
    valid = min(BN, o1 - row0);
  };

  if (warp == 0 && lane == 0) {
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < total; item += gridDim.x) {
      int e, row0, valid, tile;
      get_item(item, e, row0, valid, tile);
      const int wrow = e * p.n + tile * kBM * C::R;
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (*abort_flag || !mbar_wait(&empty_bar[stage], phase ^ 1)) {
          ok = false;
          break;
        }
        uint8_t* sb = smem + static_cast<size_t>(stage) * C::kStageBytes;
        mbar_arrive_expect_tx(&full_bar[stage], C::kStageBytes);
        tma_load_2d(sb, &tm_w, &full_bar[stage], kb * (kRowBytes / 2), wrow);
        tma_load_2d(sb + C::kRowTileBytes, &tm_x, &full_bar[stage], kb * (kRowBytes / 2), row0);
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (!ok) {
      *abort_flag = 1;
      if (p.status != nullptr) atomicExch(p.status, kStatusPipelineTimeout);
    }
  } else if (warp == 1 && lane == 0) {
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int idx = 0;
    for (int item = blockIdx.x; ok && item < total; item += gridDim.x, ++idx) {
      const int acc = idx & 1;
      const uint32_t acc_phase = (idx >> 1) & 1;
      if (*abort_flag || !mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t d_base = tmem_base + acc * C::kAccCols;
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (*abort_flag || !mbar_wait(&full_bar[stage], phase)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(smem + static_cast<size_t>(stage) * C::kStageBytes);
        const uint64_t a_base = umma_desc_k_sw128(sa);
        const uint64_t b_base = umma_desc_k_sw128(sa + C::kRowTileBytes);
#pragma unroll
        for (int r = 0; r < C::R; ++r) {
#pragma unroll
          for (int kk = 0; kk < kRowBytes / kUmmaKBytes; ++kk) {
            const uint64_t a_desc = a_base + ((r * (kBM * kRowBytes) + kk * kUmmaKBytes) >> 4);
            const uint64_t b_desc = b_base + ((kk * kUmmaKBytes) >> 4);
            umma_f16(d_base + r * BN, a_desc, b_desc, p.idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
        }
        umma_commit(&empty_bar[stage]);
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit(&acc_full[acc]);
    }
    if (!ok) {
      *abort_flag = 1;
      if (p.status != nullptr) atomicExch(p.status, kStatusPipelineTimeout);
    }
  } else if (warp >= 4) {
    const int ew = warp - 4;
    const int row_in_tile = ew * 32 + lane;
    bool ok = true;
    int idx = 0;
    for (int item = blockIdx.x; ok && item < total; item += gridDim.x, ++idx) {
      int e, row0, valid, tile;
      get_item(item, e, row0, valid, tile);
      const int acc = idx & 1;
      const uint32_t acc_phase = (idx >> 1) & 1;
      if (*abort_flag || !mbar_wait(&acc_full[acc], acc_phase)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t t_base = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * C::kAccCols;
      // this thread's weight row inside the expert and the output column it produces
      const int wrow = tile * kBM * C::R + row_in_tile;
      const int ocol = SWIGLU ? tile * kBM + row_in_tile : wrow;
      const bool row_ok = SWIGLU ? (wrow + kBM < p.n) : (wrow < p.n);
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        uint32_t v0[16], v1[16];
        tmem_ld_32x16(t_base + c, v0);
        if constexpr (SWIGLU) tmem_ld_32x16(t_base + BN + c, v1);
        tmem_ld_wait();
        if (!row_ok || c >= valid) continue;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c + j >= valid) break;
          float x = __uint_as_float(v0[j]);
          if constexpr (SWIGLU) x = silu_f(x) * __uint_as_float(v1[j]);
          const int64_t o = static_cast<int64_t>(row0 + c + j) * p.ldc + ocol;
          if (p.out_f16)
            static_cast<__half*>(p.out)[o] = __float2half_rn(x);
          else
            static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(x);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&acc_empty[acc]);
    }
    if (!ok) {
      *abort_flag = 1;
      if (p.status != nullptr) atomicExch(p.status, kStatusPipelineTimeout);
    }
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

template <int BN, bool SWIGLU>
int launch_grouped_cfg(const CUtensorMap& tw, const CUtensorMap& tx, const GroupedParams& p, int grid, cudaStream_t s) {
  using C = GCfg<BN, SWIGLU>;
  auto kern = moe_grouped_gemm_kernel<BN, SWIGLU>;
  const size_t smem = static_cast<size_t>(C::kStages) * C::kStageBytes + 1024 + 512;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), static_cast<int>(smem)) != cudaSuccess) return -3;
  const cudaError_t err = launch_pdl(kern, dim3(grid), dim3(kThreads), smem, s, tw, tx, p);
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}

}  // namespace

void launch_moe_router_topk(const void* logits, int64_t stride, float* w, int* ids, int tokens, int experts, int top_k,
                            int renorm, DType dt, cudaStream_t s) {
  if (tokens == 0) return;
  const int warps = 8;
  const dim3 grid((tokens + warps - 1) / warps), block(warps * 32);
  if (dt == kF32) {
    launch_pdl(moe_router_topk_kernel<float>, grid, block, 0, s, static_cast<const float*>(logits), stride, w, ids, tokens,
               experts, top_k, renorm);
  } else {
    MB200_DISPATCH_HALF(dt, (launch_pdl(moe_router_topk_kernel<T>, grid, block, 0, s, static_cast<const T*>(logits), stride,
                                        w, ids, tokens, experts, top_k, renorm)));
  }
  note_launch();
}

void launch_moe_align(const int* topk_ids, int pairs, int top_k, int expert_offset, int experts, int bn, int* sorted_pos,
                      int* src_token, int* expert_offsets, int* work, int* n_work, int max_work, cudaStream_t s) {
  launch_pdl(moe_align_kernel, dim3(1), dim3(1024), 0, s, topk_ids, pairs, top_k, expert_offset, experts, bn, sorted_pos,
             src_token, expert_offsets, reinterpret_cast<int2*>(work), n_work, max_work);
  note_launch();
}

void launch_moe_gather(const void* x, int64_t x_stride, const int* src_token, const int* expert_offsets, int experts,
                       void* xs, int pairs, int hidden, cudaStream_t s) {
  if (pairs == 0) return;
  launch_pdl(moe_gather_kernel, dim3(pairs), dim3(128), 0, s, static_cast<const uint4*>(x), x_stride / 8, src_token,
             expert_offsets, experts, static_cast<uint4*>(xs), hidden / 8);
  note_launch();
}

void launch_moe_combine(const void* y, const int* sorted_pos, const float* topk_w, void* out, int tokens, int hidden,
                        int top_k, DType dt, cudaStream_t s) {
  if (tokens == 0) return;
  MB200_DISPATCH_HALF(dt, (launch_pdl(moe_combine_kernel<T>, dim3(tokens), dim3(256), 0, s, static_cast<const T*>(y),
                                      sorted_pos, topk_w, static_cast<T*>(out), hidden, top_k)));
  note_launch();
}

int launch_moe_grouped_gemm(const MoeGemmArgs& a, cudaStream_t s) {
  if (a.rows_cap <= 0) return 0;
  if (a.k % 8 != 0 || a.ldc % 8 != 0 || a.n % 8 != 0) return -1;
  if (a.swiglu && a.n % 256 != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.w) | reinterpret_cast<uintptr_t>(a.out)) & 15) return -1;
  const int r = a.swiglu ? 2 : 1;
  GroupedParams p{};
  p.out = a.out;
  p.ldc = a.ldc;
  p.expert_offsets = a.expert_offsets;
  p.work = reinterpret_cast<const int2*>(a.work);
  p.n_work = a.n_work;
  p.status = a.status;
  p.n = a.n;
  p.k_blocks = (a.k + 63) / 64;
  p.tiles_r = (a.n + kBM * r - 1) / (kBM * r);
  p.out_f16 = a.dt == kF16 ? 1 : 0;
  const uint32_t ab_fmt = a.dt == kF16 ? 0u : 1u;
  p.idesc = umma_idesc(kBM, a.bn, 1u, ab_fmt, ab_fmt);
  CUtensorMap tw, tx;
  const int type = a.dt == kF16 ? 1 : 0;
  if (!make_tma_operand_map(&tw, a.w, static_cast<int64_t>(a.experts) * a.n, a.k, a.k, 2, type, kBM * r)) return -2;
  if (!make_tma_operand_map(&tx, a.x, a.rows_cap, a.k, a.ldx, 2, type, a.bn)) return -2;
  const int num_sms = a.num_sms > 0 ? a.num_sms : 148;
  const int64_t max_items = static_cast<int64_t>(a.max_work) * p.tiles_r;
  const int grid = static_cast<int>(std::min<int64_t>(num_sms, std::max<int64_t>(1, max_items)));
  switch (a.bn) {
#define MB200_MOE_CASE(BNV) \
  case BNV:                 \
    return a.swiglu ? launch_grouped_cfg<BNV, true>(tw, tx, p, grid, s) : launch_grouped_cfg<BNV, false>(tw, tx, p, grid, s);
    MB200_MOE_CASE(16)
    MB200_MOE_CASE(32)
    MB200_MOE_CASE(64)
    MB200_MOE_CASE(128)
#undef MB200_MOE_CASE
  }
  return -1;
}

}  // namespace mb200
