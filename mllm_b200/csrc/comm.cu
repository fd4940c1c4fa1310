// Tensor-parallel reduction fused with the residual add and RMSNorm, over NVLink peer memory.
//
// Every rank's row-parallel GEMM (o_proj / down_proj) leaves its partial sums in a buffer that all
// ranks have mapped (symmetric memory).  This kernel replaces "all-reduce, then add + RMSNorm":
// one CTA per token row signals the same-row CTA of every peer with a system-scope release
// increment, waits (bounded) until all peers have signalled, then pulls the row's partials from
// every rank with plain 16-byte peer loads, sums them in rank order in fp32 (so all ranks compute
// bit-identical results), adds the residual, writes the new residual and the normalised row.
// Flags are monotonically increasing counters and the expected value lives in device memory, so
// the kernel is CUDA-graph safe: nothing changes between replays.  No multimem, no TMA: plain
// ld/st/red on peer pointers only.
#include "common.cuh"
#include "kernels.h"

namespace mb200 {
namespace {

constexpr int kMaxTp = 8;

struct PeerPtrs {
  const void* data[kMaxTp];
  uint32_t* flags[kMaxTp];
};

__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ void unpack8v(const uint4& raw, float (&f)[8]) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = to_f(e[i]);
}
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half from_f<__half>(float v) {
  return __float2half_rn(v);
}
template <typename T>
__device__ __forceinline__ uint4 pack8v(const float (&f)[8]) {
  uint4 r;
  T* e = reinterpret_cast<T*>(&r);
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = from_f<T>(f[i]);
  return r;
}

constexpr int kVecPerThread = 4;

// grid = rows, block = hidden / 8 threads (<= 1024), hidden <= 8 * 1024 * kVecPerThread
template <typename T>
__global__ void tp_reduce_add_rmsnorm_kernel(PeerPtrs peers, uint32_t* __restrict__ local_seq, T* __restrict__ residual,
                                             const T* __restrict__ weight, T* __restrict__ out, int hidden, int tp,
                                             int rank, int64_t row_stride, float eps, int* status) {
  __shared__ float red[33];
  __shared__ int wait_ok;
  pdl_wait();
  const int row = blockIdx.x;
  if (threadIdx.x == 0) wait_ok = 1;
  __syncthreads();
  // 1) tell every rank (myself included) that my partial of this row is in place
  if (threadIdx.x < tp) red_add_release_sys(peers.flags[threadIdx.x] + row * kMaxTp + rank, 1u);
  // 2) wait for every rank's signal; the expected count advances by one per call
  const uint32_t expect = local_seq[row] + 1u;
  if (threadIdx.x < tp) {
    if (!wait_flag_ge(peers.flags[rank] + row * kMaxTp + threadIdx.x, expect, status)) {
      wait_ok = 0;
      if (status != nullptr) atomicExch(status, kStatusPeerTimeout);
    }
  }
  __syncthreads();
  if (!wait_ok) {  // leave the outputs untouched; the host raises on the status word
    if (threadIdx.x == 0) local_seq[row] = expect;
    return;
  }
  // 3) pull, sum in rank order, add the residual
  const int nvec = hidden >> 3;
  float cache[kVecPerThread][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kVecPerThread; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      // every rank's vector first, then the sum in rank order: the loads are independent and cross NVLink together
      // (issued one after the other, each behind the previous one's use, they cost one link round trip per rank)
      uint4 raw[kMaxTp];
#pragma unroll
      for (int r = 0; r < kMaxTp; ++r)
        if (r < tp) raw[r] = *(reinterpret_cast<const uint4*>(static_cast<const T*>(peers.data[r]) + row * row_stride) + v);
#pragma unroll
      for (int r = 0; r < kMaxTp; ++r) {
        if (r < tp) {
          float f[8];
          unpack8v<T>(raw[r], f);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += f[i];
        }
      }
      if (residual != nullptr) {
        uint4* rp = reinterpret_cast<uint4*>(residual + static_cast<int64_t>(row) * hidden) + v;
        float g[8];
        unpack8v<T>(*rp, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = to_f(from_f<T>(acc[i] + g[i]));
        *rp = pack8v<T>(acc);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = to_f(from_f<T>(acc[i]));
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        cache[it][i] = acc[i];
        ss += acc[i] * acc[i];
      }
    }
  }
  float rstd = 1.f;
  if (weight != nullptr) {
    ss = warp_sum(ss);
    if (lane_id() == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < ((blockDim.x + 31) >> 5) ? red[threadIdx.x] : 0.f;
      t = warp_sum(t);
      if (threadIdx.x == 0) red[32] = t;
    }
    __syncthreads();
    rstd = rsqrtf(red[32] / static_cast<float>(hidden) + eps);
  }
#pragma unroll
  for (int it = 0; it < kVecPerThread; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
      float o[8];
      if (weight != nullptr) {
        float g[8];
        unpack8v<T>(reinterpret_cast<const uint4*>(weight)[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = cache[it][i] * rstd * g[i];
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = cache[it][i];
      }
      reinterpret_cast<uint4*>(out + static_cast<int64_t>(row) * hidden)[v] = pack8v<T>(o);
    }
  }
  if (threadIdx.x == 0) local_seq[row] = expect;
}


// ---------------------------------------------------------------------------------------------
// prefill: reduce-scatter (from the inbox the peers' GEMM epilogues filled) + residual add + RMSNorm
// + all-gather by peer stores.  grid = own rows, block = hidden / 8 threads (<= 1024).
// ---------------------------------------------------------------------------------------------
struct GatherPtrs {
  void* hidden[kMaxTp];
  uint32_t* flags[kMaxTp];
};

constexpr int kRsRowsPerCta = 8;  // divides 128: a CTA's rows lie in one 128-row tile

template <typename T, int VPT>
__global__ void tp_rs_add_rmsnorm_ag_kernel(const T* __restrict__ inbox, int64_t inbox_rows_cap,
                                            const uint32_t* __restrict__ tile_flags, T* __restrict__ residual,
                                            const T* __restrict__ weight, GatherPtrs peers, int* __restrict__ ag_count,
                                            int rows, int hidden, int tp, int n_src, int rank, uint32_t epoch, float eps,
                                            int* status) {
  __shared__ float red[2][33];
  __shared__ int wait_ok;
  pdl_wait();
  const int row0 = blockIdx.x * kRsRowsPerCta;
  const int tile = row0 >> 7;
  if (threadIdx.x == 0) wait_ok = 1;
  __syncthreads();
  // n_src partial sums per row (tp for the reduce-scatter inbox; 1 when the rows arrive complete, e.g. from the
  // expert-parallel exchange, and tile_flags is then null)
  if (tile_flags != nullptr && threadIdx.x < n_src) {
    if (!wait_flag_ge(tile_flags + tile * kMaxTp + threadIdx.x, epoch, status)) {
      wait_ok = 0;
      if (status != nullptr) atomicExch(status, kStatusPeerTimeout);
    }
  }
  __syncthreads();
  if (!wait_ok) return;
  const int nvec = hidden >> 3;
  const int nwarps = (blockDim.x + 31) >> 5;
  // the norm weight is the same for every row of the CTA
  float gw[VPT][8];
#pragma unroll
  for (int it = 0; it < VPT; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) unpack8v<T>(reinterpret_cast<const uint4*>(weight)[v], gw[it]);
  }
#pragma unroll 1
  for (int rr = 0; rr < kRsRowsPerCta; ++rr) {
    const int row = row0 + rr;
    float cache[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < VPT; ++it) {
      const int v = threadIdx.x + it * blockDim.x;
      if (v < nvec) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
        for (int r = 0; r < n_src; ++r) {
          const uint4 raw =
              __ldcg(reinterpret_cast<const uint4*>(inbox + (static_cast<int64_t>(r) * inbox_rows_cap + row) * hidden) + v);
          float f[8];
          unpack8v<T>(raw, f);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += f[i];
        }
        uint4* rp = reinterpret_cast<uint4*>(residual + static_cast<int64_t>(row) * hidden) + v;
        float g[8];
        unpack8v<T>(*rp, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = to_f(from_f<T>(acc[i] + g[i]));
        *rp = pack8v<T>(acc);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          cache[it][i] = acc[i];
          ss += acc[i] * acc[i];
        }
      }
    }
    // block sum of squares; the two halves of `red` alternate so one barrier per row suffices
    float* rbuf = red[rr & 1];
    ss = warp_sum(ss);
    if (lane_id() == 0) rbuf[threadIdx.x >> 5] = ss;
    __syncthreads();
    float t = lane_id() < nwarps ? rbuf[lane_id()] : 0.f;
    t = warp_sum(t);
    const float rstd = rsqrtf(t / static_cast<float>(hidden) + eps);
    const int64_t grow = static_cast<int64_t>(rank) * rows + row;
#pragma unroll
    for (int it = 0; it < VPT; ++it) {
      const int v = threadIdx.x + it * blockDim.x;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = cache[it][i] * rstd * gw[it][i];
        const uint4 packed = pack8v<T>(o);
        for (int r = 0; r < tp; ++r) {
          const int dst = (rank + r) % tp;  // start with the local copy, spread the peers
          reinterpret_cast<uint4*>(static_cast<T*>(peers.hidden[dst]) + grow * hidden)[v] = packed;
        }
      }
    }
  }
  // publish: the barrier orders every thread's stores before thread 0's system-scope fence; the CTA
  // that completes a 128-row tile raises the tile's flag on every rank
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int old = atomicAdd(&ag_count[tile], kRsRowsPerCta);
    const int rows_in_tile = min(128, rows - tile * 128);
    if (old == rows_in_tile - kRsRowsPerCta) {
      ag_count[tile] = 0;
      __threadfence_system();
      const int gtile = static_cast<int>((static_cast<int64_t>(rank) * rows + row0) >> 7);
      for (int r = 0; r < tp; ++r) st_release_sys(peers.flags[r] + gtile, epoch);
    }
  }
}

__global__ void tp_wait_flags_kernel(const uint32_t* __restrict__ flags, int n, uint32_t epoch, int* status) {
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    if (!wait_flag_ge(flags + i, epoch, status)) {
      if (status != nullptr) atomicExch(status, kStatusPeerTimeout);
      return;
    }
  }
}

}  // namespace

int launch_tp_rs_add_rmsnorm_ag(const void* inbox, int64_t inbox_rows_cap, const uint32_t* tile_flags,
                                void* residual_shard, const void* weight, const uint64_t* peer_hidden,
                                const uint64_t* peer_gather_flags, int* ag_count, int rows, int hidden, int tp,
                                int n_src, int rank, uint32_t epoch, float eps, DType dt, int* status, cudaStream_t s) {
  if (rows == 0) return 0;
  if (tp < 1 || tp > kMaxTp || hidden % 8 != 0 || hidden > 8 * 1024 * kVecPerThread || rows % 128 != 0 ||
      residual_shard == nullptr || weight == nullptr)
    return -1;
  GatherPtrs gp{};
  for (int r = 0; r < tp; ++r) {
    gp.hidden[r] = reinterpret_cast<void*>(peer_hidden[r]);
    gp.flags[r] = reinterpret_cast<uint32_t*>(peer_gather_flags[r]);
  }
  int threads = ((hidden >> 3) + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  if (threads < 32) threads = 32;
  const int vpt = ((hidden >> 3) + threads - 1) / threads;
  cudaError_t err = cudaErrorInvalidValue;
  const dim3 grid(rows / kRsRowsPerCta), block(threads);
#define MB200_RS_LAUNCH(TT, V)                                                                                      \
  err = launch_pdl(tp_rs_add_rmsnorm_ag_kernel<TT, V>, grid, block, 0, s, static_cast<const TT*>(inbox), inbox_rows_cap, \
                   tile_flags, static_cast<TT*>(residual_shard), static_cast<const TT*>(weight), gp, ag_count, rows,   \
                   hidden, tp, n_src, rank, epoch, eps, status)
  if (dt == kBF16) {
    if (vpt == 1) MB200_RS_LAUNCH(__nv_bfloat16, 1);
    else if (vpt == 2) MB200_RS_LAUNCH(__nv_bfloat16, 2);
    else MB200_RS_LAUNCH(__nv_bfloat16, 4);
  } else {
    if (vpt == 1) MB200_RS_LAUNCH(__half, 1);
    else if (vpt == 2) MB200_RS_LAUNCH(__half, 2);
    else MB200_RS_LAUNCH(__half, 4);
  }
#undef MB200_RS_LAUNCH
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}

int launch_tp_wait_flags(const uint32_t* flags, int n, uint32_t epoch, int* status, cudaStream_t s) {
  if (n <= 0) return 0;
  const cudaError_t err = launch_pdl(tp_wait_flags_kernel, dim3(1), dim3(256), 0, s, flags, n, epoch, status);
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}

int launch_tp_reduce_add_rmsnorm(const uint64_t* peer_data, const uint64_t* peer_flags, uint32_t* local_seq,
                                 void* residual, const void* weight, void* out, int rows, int hidden, int tp, int rank,
                                 int64_t row_stride, float eps, DType dt, int* status, cudaStream_t s) {
  if (rows == 0) return 0;
  if (tp < 1 || tp > kMaxTp || hidden % 8 != 0 || hidden > 8 * 1024 * kVecPerThread) return -1;
  PeerPtrs pp{};
  for (int r = 0; r < tp; ++r) {
    pp.data[r] = reinterpret_cast<const void*>(peer_data[r]);
    pp.flags[r] = reinterpret_cast<uint32_t*>(peer_flags[r]);
  }
  int threads = ((hidden >> 3) + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  if (threads < 32) threads = 32;
  cudaError_t err;
  if (dt == kBF16) {
    err = launch_pdl(tp_reduce_add_rmsnorm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, s, pp, local_seq,
                     static_cast<__nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(weight),
                     static_cast<__nv_bfloat16*>(out), hidden, tp, rank, row_stride, eps, status);
  } else {
    err = launch_pdl(tp_reduce_add_rmsnorm_kernel<__half>, dim3(rows), dim3(threads), 0, s, pp, local_seq,
                     static_cast<__half*>(residual), static_cast<const __half*>(weight), static_cast<__half*>(out),
                     hidden, tp, rank, row_stride, eps, status);
  }
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}


}  // namespace mb200
