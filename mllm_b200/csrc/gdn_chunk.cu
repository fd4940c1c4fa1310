// Chunk-parallel prefill of the gated delta rule (the hybrid models' linear attention), 64 tokens at a time.
//
// The token recurrence  S *= exp(g_t);  S += k_t (x) ((v_t - S^T k_t) beta_t);  o_t = S^T q_t  is evaluated per
// chunk with matrix products.  With G_i the running sum of g inside the chunk and S0 the incoming state:
//
//   A[i, j] = beta_i exp(G_i - G_j) (k_i . k_j)   for j < i                  (strictly lower triangular)
//   (I + A) U = diag(beta) (V - exp(G) * (K S0))                            (forward substitution)
//   O     = exp(G) * (Q S0) + (M * (Q K^T)) U,   M[i, j] = exp(G_i - G_j) for j <= i
//   S_end = exp(G_C) S0 + K^T (exp(G_C - G) * U)
//
// Every exponent is of a non-positive number.  The columns of S (the value features) never mix, so a CTA owns one
// (request, head) and a block of BV value features: grid (128 / BV, heads, batch), 256 threads.  The products
// K K^T, Q K^T, K S0, Q S0, P U and K^T U' run on the tensor cores through warp-level MMA on tf32 operands with
// fp32 accumulation (tiles of 16 x 16 x 8 read from shared memory); the state stays in fp32 in shared memory for
// the whole sequence and is rounded to tf32 only as an MMA operand.  The substitution is the one sequential step;
// it runs 16 rows at a time (one thread per value feature inside a block, a tensor-core product to carry a solved
// block into the rows below): one thread walking all 64 rows kept the other warps at a barrier for a quarter of
// the kernel's issue slots.
// The 64 x 64 x BV tiles and the chunk-to-chunk dependency are too small and too serial for a tcgen05 pipeline
// (tensor-memory round trips between the six dependent products would dominate), hence the warp-level path.
#include <mma.h>

#include "common.cuh"
#include "kernels.h"

namespace mb200 {
namespace {

namespace wmma = nvcuda::wmma;

constexpr int kGC = 64;             // tokens per chunk
constexpr int kGD = 128;            // key / value head size
constexpr int kGLd = kGD + 4;       // row stride (floats) of the K and Q tiles
constexpr int kGLdC = kGC + 4;      // row stride of the chunk x chunk matrices
constexpr int kGThreads = 512;
constexpr int kGWarps = kGThreads / 32;

template <int BV>
struct GdnChunkCfg {
  static constexpr int kLdV = BV + 4;   // row stride of everything that is BV wide
  static constexpr int kFloats = 2 * kGC * kGLd + kGD * kLdV + 2 * kGC * kGLdC + 3 * kGC * kLdV + 6 * kGC;
  static constexpr int kSmem = kFloats * 4 + kGC * BV * 2 + 128;    // + the staged 16-bit V block of the next chunk
};

using FragA = wmma::fragment<wmma::matrix_a, 16, 16, 8, wmma::precision::tf32, wmma::row_major>;
using FragAT = wmma::fragment<wmma::matrix_a, 16, 16, 8, wmma::precision::tf32, wmma::col_major>;
using FragB = wmma::fragment<wmma::matrix_b, 16, 16, 8, wmma::precision::tf32, wmma::row_major>;
using FragBT = wmma::fragment<wmma::matrix_b, 16, 16, 8, wmma::precision::tf32, wmma::col_major>;
using FragC = wmma::fragment<wmma::accumulator, 16, 16, 8, float>;

// asynchronous global -> shared copies; with `valid` false nothing is read and the destination is zero-filled
__device__ __forceinline__ void stage16(void* dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void stage4(void* dst, const void* src, bool valid) {
  const int sz = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(sz) : "memory");
}

template <typename F>
__device__ __forceinline__ void to_tf32(F& f) {
#pragma unroll
  for (int i = 0; i < f.num_elements; ++i) f.x[i] = wmma::__float_to_tf32(f.x[i]);
}

template <typename T, int BV>
__global__ void __launch_bounds__(kGThreads, 1)
gdn_chunk_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const float* __restrict__ g,
                 const float* __restrict__ beta, float* __restrict__ state, const int* __restrict__ slots,
                 const int* __restrict__ lens, const int* __restrict__ has_state, const int* __restrict__ q_start,
                 T* __restrict__ out, int heads) {
  pdl_wait();
  using C = GdnChunkCfg<BV>;
  constexpr int kLdV = C::kLdV;
  constexpr int kVT = BV / 16;   // 16-wide tiles across the value block
  extern __shared__ uint8_t gdn_smem_raw[];
  float* sm = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(gdn_smem_raw) + 127) & ~uintptr_t(127));
  float* sK = sm;                        // [64][132] l2-normalised keys
  float* sQ = sK + kGC * kGLd;           // [64][132] l2-normalised, scaled queries
  float* sS = sQ + kGC * kGLd;           // [128][BV+4] state block
  float* sA = sS + kGD * kLdV;           // [64][68] K K^T, then A
  float* sP = sA + kGC * kGLdC;          // [64][68] Q K^T, then M * (Q K^T)
  float* sU = sP + kGC * kGLdC;          // [64][BV+4] V, then the right-hand side, then U
  float* sX = sU + kGC * kLdV;           // [64][BV+4] K S0, then exp(G_C - G) * U
  float* sY = sX + kGC * kLdV;           // [64][BV+4] Q S0, then O
  float* sG = sY + kGC * kLdV;           // [64] g, then its running sum G
  float* sB = sG + kGC;                  // [64] beta
  float* sE = sB + kGC;                  // [64] exp(G)
  float* sT = sE + kGC;                  // [64] exp(G_C - G)
  float* sGn = sT + kGC;                 // [64] staged g of the next chunk
  float* sBn = sGn + kGC;                // [64] staged beta of the next chunk
  T* sVn = reinterpret_cast<T*>(sBn + kGC);   // [64][BV] staged V block of the next chunk
  // The 16-bit K and Q rows of the next chunk are staged in the bytes of sQ, which nothing reads once Q K^T and
  // Q S0 of the current chunk are done: K rows at byte 0, Q rows at byte 16384, 256 bytes per row.
  T* sKn = reinterpret_cast<T*>(sQ);
  T* sQn = sKn + kGC * kGD;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int vb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n = lens[b];
  if (n <= 0) return;
  const int64_t row0 = q_start[b];
  float* S = state + ((static_cast<int64_t>(slots[b]) * heads + h) * kGD) * kGD + vb * BV;   // element (i, c) at S[i * 128 + c]
  const bool resume = has_state[b] != 0;
  for (int idx = tid; idx < kGD * BV; idx += kGThreads) {
    const int i = idx / BV, c = idx % BV;
    sS[i * kLdV + c] = resume ? S[i * kGD + c] : 0.f;
  }
  const float qscale = rsqrtf(static_cast<float>(kGD));

  // every copy of one chunk: 64 rows x 16 pieces of K and of Q, 64 x BV / 8 pieces of V, 64 scalars of g and beta
  auto stage_chunk = [&](int c0) {
    const int nv = min(kGC, n - c0);
    for (int idx = tid; idx < kGC * 16; idx += kGThreads) {
      const int r = idx >> 4, piece = idx & 15;
      const bool valid = r < nv;
      const int64_t at = ((row0 + c0 + (valid ? r : 0)) * heads + h) * kGD + piece * 8;
      stage16(sKn + r * kGD + piece * 8, k + at, valid);
      stage16(sQn + r * kGD + piece * 8, q + at, valid);
    }
    for (int idx = tid; idx < kGC * (BV / 8); idx += kGThreads) {
      const int r = idx / (BV / 8), piece = idx % (BV / 8);
      const bool valid = r < nv;
      stage16(sVn + r * BV + piece * 8, v + ((row0 + c0 + (valid ? r : 0)) * heads + h) * kGD + vb * BV + piece * 8, valid);
    }
    if (tid < kGC) {
      const bool valid = tid < nv;
      const int64_t at = (row0 + c0 + (valid ? tid : 0)) * heads + h;
      stage4(sGn + tid, g + at, valid);
      stage4(sBn + tid, beta + at, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  stage_chunk(0);

  for (int c0 = 0; c0 < n; c0 += kGC) {
    const int nv = min(kGC, n - c0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();      // the staged rows of this chunk are visible to every thread
    // ---- K and Q rows normalised (a warp per row; all rows are read before any is written: the staged rows
    // share their bytes with sQ), the V block widened, g and beta moved; rows past the end are zero ----
    {
      float kk[kGC / kGWarps][4], qq[kGC / kGWarps][4];
#pragma unroll
      for (int it = 0; it < kGC / kGWarps; ++it) {
        const int r = warp + it * kGWarps;
        const uint2 kr = *reinterpret_cast<const uint2*>(sKn + r * kGD + lane * 4);
        const uint2 qr = *reinterpret_cast<const uint2*>(sQn + r * kGD + lane * 4);
        const T* ke = reinterpret_cast<const T*>(&kr);
        const T* qe = reinterpret_cast<const T*>(&qr);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          kk[it][i] = to_f32(ke[i]);
          qq[it][i] = to_f32(qe[i]);
        }
      }
      for (int idx = tid; idx < kGC * BV; idx += kGThreads) {
        const int r = idx / BV, c = idx % BV;
        sU[r * kLdV + c] = to_f32(sVn[r * BV + c]);
      }
      if (tid < kGC) {
        sG[tid] = sGn[tid];
        sB[tid] = sBn[tid];
      }
      __syncthreads();    // every staged row has been read
#pragma unroll
      for (int it = 0; it < kGC / kGWarps; ++it) {
        const int r = warp + it * kGWarps;
        const float ks = warp_sum(kk[it][0] * kk[it][0] + kk[it][1] * kk[it][1] + kk[it][2] * kk[it][2] + kk[it][3] * kk[it][3]);
        const float qs = warp_sum(qq[it][0] * qq[it][0] + qq[it][1] * qq[it][1] + qq[it][2] * qq[it][2] + qq[it][3] * qq[it][3]);
        const float kn = rsqrtf(ks + 1e-6f), qn = rsqrtf(qs + 1e-6f) * qscale;
        *reinterpret_cast<float4*>(sK + r * kGLd + lane * 4) =
            make_float4(kk[it][0] * kn, kk[it][1] * kn, kk[it][2] * kn, kk[it][3] * kn);
        *reinterpret_cast<float4*>(sQ + r * kGLd + lane * 4) =
            make_float4(qq[it][0] * qn, qq[it][1] * qn, qq[it][2] * qn, qq[it][3] * qn);
      }
    }
    __syncthreads();

    // ---- running sum of g (warp 0: two entries per lane), exp(G), exp(G_C - G) ----
    if (warp == 0) {
      const float a = sG[2 * lane], ab = a + sG[2 * lane + 1];
      float incl = ab;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
      }
      const float before = incl - ab;
      const float g0 = before + a, g1 = before + ab;
      const float total = __shfl_sync(0xffffffffu, incl, 31);
      sG[2 * lane] = g0;
      sG[2 * lane + 1] = g1;
      sE[2 * lane] = expf(g0);
      sE[2 * lane + 1] = expf(g1);
      sT[2 * lane] = expf(total - g0);
      sT[2 * lane + 1] = expf(total - g1);
    }

    // ---- products that need no decay: K K^T -> sA, Q K^T -> sP (tiles on or below the diagonal), K S0 -> sX,
    // Q S0 -> sY; one list of tiles dealt round-robin to the warps ----
    for (int t = warp; t < 20 + 8 * kVT; t += kGWarps) {
      FragC acc;
      wmma::fill_fragment(acc, 0.f);
      if (t < 20) {       // the ten tiles on or below the diagonal of K K^T, then those of Q K^T
        const int which = t / 10, idx = t % 10;
        const int ti = idx >= 6 ? 3 : idx >= 3 ? 2 : idx >= 1 ? 1 : 0, tj = idx - ti * (ti + 1) / 2;
        const float* left = (which ? sQ : sK) + ti * 16 * kGLd;
        const float* right = sK + tj * 16 * kGLd;
#pragma unroll 4
        for (int k0 = 0; k0 < kGD; k0 += 8) {
          FragA fa;
          FragBT fb;
          wmma::load_matrix_sync(fa, left + k0, kGLd);
          wmma::load_matrix_sync(fb, right + k0, kGLd);     // B[k][j] = K[j][k]
          to_tf32(fa);
          to_tf32(fb);
          wmma::mma_sync(acc, fa, fb, acc);
        }
        wmma::store_matrix_sync((which ? sP : sA) + ti * 16 * kGLdC + tj * 16, acc, kGLdC, wmma::mem_row_major);
      } else {
        const int s2 = t - 20, which = s2 / (4 * kVT), rem = s2 % (4 * kVT), ti = rem / kVT, tc = rem % kVT;
        const float* left = (which ? sQ : sK) + ti * 16 * kGLd;
#pragma unroll 4
        for (int k0 = 0; k0 < kGD; k0 += 8) {
          FragA fa;
          FragB fb;
          wmma::load_matrix_sync(fa, left + k0, kGLd);
          wmma::load_matrix_sync(fb, sS + k0 * kLdV + tc * 16, kLdV);
          to_tf32(fa);
          to_tf32(fb);
          wmma::mma_sync(acc, fa, fb, acc);
        }
        wmma::store_matrix_sync((which ? sY : sX) + ti * 16 * kLdV + tc * 16, acc, kLdV, wmma::mem_row_major);
      }
    }
    __syncthreads();
    // sQ is free from here on: the next chunk's rows travel while this chunk is finished
    if (c0 + kGC < n) stage_chunk(c0 + kGC);

    // ---- decay masks, right-hand side ----
    for (int idx = tid; idx < kGC * kGC; idx += kGThreads) {
      const int i = idx >> 6, j = idx & 63;
      const float d = j <= i ? __expf(sG[i] - sG[j]) : 0.f;
      const float ka = sA[i * kGLdC + j], qa = sP[i * kGLdC + j];
      sA[i * kGLdC + j] = j < i ? sB[i] * d * ka : 0.f;
      sP[i * kGLdC + j] = j <= i ? d * qa : 0.f;
    }
    for (int idx = tid; idx < kGC * BV; idx += kGThreads) {
      const int i = idx / BV, c = idx % BV;
      const float e = sE[i];
      sU[i * kLdV + c] = sB[i] * (sU[i * kLdV + c] - e * sX[i * kLdV + c]);
      sY[i * kLdV + c] *= e;
    }
    __syncthreads();

    // ---- forward substitution (I + A) U = rhs, 16 rows at a time: the rows of a block are solved by one thread
    // per value feature (the block's unknowns in registers), then the block's contribution leaves the right-hand
    // sides of all rows below it as one small tensor-core product ----
    for (int blk = 0; blk < kGC / 16; ++blk) {
      if (tid < BV) {
        float u[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int row = blk * 16 + i;
          float a0 = sU[row * kLdV + tid], a1 = 0.f;
#pragma unroll
          for (int j4 = 0; j4 < (i + 3) / 4; ++j4) {
            const float4 ar = *reinterpret_cast<const float4*>(sA + row * kGLdC + blk * 16 + j4 * 4);   // zero at j >= i
            if (j4 * 4 + 0 < i) a0 = fmaf(-ar.x, u[j4 * 4 + 0], a0);
            if (j4 * 4 + 1 < i) a1 = fmaf(-ar.y, u[j4 * 4 + 1], a1);
            if (j4 * 4 + 2 < i) a0 = fmaf(-ar.z, u[j4 * 4 + 2], a0);
            if (j4 * 4 + 3 < i) a1 = fmaf(-ar.w, u[j4 * 4 + 3], a1);
          }
          u[i] = a0 + a1;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int row = blk * 16 + i;
          sU[row * kLdV + tid] = u[i];
          sX[row * kLdV + tid] = sT[row] * u[i];
        }
      }
      __syncthreads();
      if (blk + 1 < kGC / 16) {
        for (int t = warp; t < (kGC / 16 - 1 - blk) * kVT; t += kGWarps) {
          const int ti = blk + 1 + t / kVT, tc = t % kVT;
          float* tile = sU + ti * 16 * kLdV + tc * 16;
          FragC acc;
          wmma::load_matrix_sync(acc, tile, kLdV, wmma::mem_row_major);
#pragma unroll
          for (int k0 = 0; k0 < 16; k0 += 8) {
            FragA fa;
            FragB fb;
            wmma::load_matrix_sync(fa, sA + ti * 16 * kGLdC + blk * 16 + k0, kGLdC);
            wmma::load_matrix_sync(fb, sU + (blk * 16 + k0) * kLdV + tc * 16, kLdV);
#pragma unroll
            for (int i = 0; i < fa.num_elements; ++i) fa.x[i] = wmma::__float_to_tf32(-fa.x[i]);
            to_tf32(fb);
            wmma::mma_sync(acc, fa, fb, acc);
          }
          wmma::store_matrix_sync(tile, acc, kLdV, wmma::mem_row_major);
        }
        __syncthreads();
      }
    }

    // ---- O = exp(G) (Q S0) + P U  and  S = exp(G_C) S0 + K^T U' ----
    const float carry = sE[kGC - 1];
    for (int t = warp; t < (4 + 8) * kVT; t += kGWarps) {
      FragC acc;
      if (t < 4 * kVT) {
        const int ti = t / kVT, tc = t % kVT;
        float* tile = sY + ti * 16 * kLdV + tc * 16;
        wmma::load_matrix_sync(acc, tile, kLdV, wmma::mem_row_major);
        for (int k0 = 0; k0 < (ti + 1) * 16; k0 += 8) {      // P is zero to the right of the diagonal tile
          FragA fa;
          FragB fb;
          wmma::load_matrix_sync(fa, sP + ti * 16 * kGLdC + k0, kGLdC);
          wmma::load_matrix_sync(fb, sU + k0 * kLdV + tc * 16, kLdV);
          to_tf32(fa);
          to_tf32(fb);
          wmma::mma_sync(acc, fa, fb, acc);
        }
        wmma::store_matrix_sync(tile, acc, kLdV, wmma::mem_row_major);
      } else {
        const int s = t - 4 * kVT, tm = s / kVT, tc = s % kVT;
        float* tile = sS + tm * 16 * kLdV + tc * 16;
        wmma::load_matrix_sync(acc, tile, kLdV, wmma::mem_row_major);
#pragma unroll
        for (int i = 0; i < acc.num_elements; ++i) acc.x[i] *= carry;
#pragma unroll 4
        for (int k0 = 0; k0 < kGC; k0 += 8) {
          FragAT fa;
          FragB fb;
          wmma::load_matrix_sync(fa, sK + k0 * kGLd + tm * 16, kGLd);    // A[m][k] = K[k][m]
          wmma::load_matrix_sync(fb, sX + k0 * kLdV + tc * 16, kLdV);
          to_tf32(fa);
          to_tf32(fb);
          wmma::mma_sync(acc, fa, fb, acc);
        }
        wmma::store_matrix_sync(tile, acc, kLdV, wmma::mem_row_major);
      }
    }
    __syncthreads();

    // ---- outputs of the chunk ----
    for (int idx = tid; idx < nv * BV; idx += kGThreads) {
      const int i = idx / BV, c = idx % BV;
      out[((row0 + c0 + i) * heads + h) * kGD + vb * BV + c] = from_f32<T>(sY[i * kLdV + c]);
    }
    // the next iteration starts with a barrier, so sY is rewritten only after these reads
  }
  for (int idx = tid; idx < kGD * BV; idx += kGThreads) {
    const int i = idx / BV, c = idx % BV;
    S[i * kGD + c] = sS[i * kLdV + c];
  }
}

template <typename T, int BV>
int launch_chunk_cfg(const T* q, const T* k, const T* v, const float* g, const float* beta, float* state, const int* slots,
                     const int* lens, const int* has_state, const int* q_start, T* out, int batch, int heads, cudaStream_t s) {
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(gdn_chunk_kernel<T, BV>), GdnChunkCfg<BV>::kSmem) != cudaSuccess) return -3;
  const cudaError_t err = launch_pdl(gdn_chunk_kernel<T, BV>, dim3(kGD / BV, heads, batch), dim3(kGThreads), GdnChunkCfg<BV>::kSmem,
                                     s, q, k, v, g, beta, state, slots, lens, has_state, q_start, out, heads);
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}

}  // namespace

int launch_gdn_chunk(const void* q, const void* k, const void* v, const float* g, const float* beta, float* state,
                     const int* slots, const int* lens, const int* has_state, const int* q_start, void* out, int batch,
                     int heads, int dk, int dv, int num_sms, DType dt, cudaStream_t s) {
  if (batch <= 0) return 0;
  if (dk != kGD || dv != kGD) return -1;
  // narrower value blocks when the batch alone does not fill the GPU
  const bool narrow = batch * heads * 2 < num_sms;
  int rc = 0;
  MB200_DISPATCH_HALF(dt, (rc = narrow ? launch_chunk_cfg<T, 32>(static_cast<const T*>(q), static_cast<const T*>(k),
                                                                 static_cast<const T*>(v), g, beta, state, slots, lens, has_state,
                                                                 q_start, static_cast<T*>(out), batch, heads, s)
                                       : launch_chunk_cfg<T, 64>(static_cast<const T*>(q), static_cast<const T*>(k),
                                                                 static_cast<const T*>(v), g, beta, state, slots, lens, has_state,
                                                                 q_start, static_cast<T*>(out), batch, heads, s)));
  return rc;
}

}  // namespace mb200
