// Expert-parallel token exchange over NVLink peer memory: dispatch of routed token rows to the ranks that
// own their experts, and the return of the experts' outputs to the ranks that own the tokens.
//
// Layout of the job: the residual stream is sharded by rows over the ep ranks (rank r owns T/ep tokens), the
// experts are sharded by index (rank d owns experts [d * El, (d + 1) * El)).  Every rank routes its OWN
// tokens; a (token, choice) pair whose expert lives on rank d travels as one hidden-size row to d, is pushed
// through the grouped expert GEMMs there, and the result row travels back to be summed, with the router
// weights, into the token's output.  All traffic is plain peer stores issued by these kernels into buffers
// that every rank has mapped (symmetric memory); flags are monotonically increasing epochs, so nothing is
// reset between calls and the sequence can sit in a CUDA graph.  No multimem, no TMA.
//
//   ep_plan      one CTA: histogram of this rank's pairs per global expert -> pushed to every rank;
//                once all ranks' histograms are here, every rank knows the whole [rank][expert] matrix and
//                derives, without further messages, (a) where in each destination's receive slab its rows of
//                every expert start (rows are grouped by expert, then by source rank), (b) the row ranges of
//                its own experts and the work list of the grouped GEMM, (c) for every pair its destination
//                rank and row.  Rows beyond the slab's capacity raise kStatusBadIndex: nothing is dropped
//                silently.
//   ep_dispatch  one CTA per pair: copies the token's row into the destination's slab with 16-byte peer
//                stores and records (source rank, pair) beside it; the last CTA to finish fences and raises
//                this rank's flag on every destination.
//   ep_return    one CTA per slab row: sends the expert output row back to the pair's slot of the source
//                rank's return buffer; flags likewise.
// Waiting for flags is done by the callers with the generic flag-wait kernel (bounded).
#include "common.cuh"
#include "kernels.h"

namespace mb200 {
namespace {

constexpr int kMaxEp = 8;
constexpr int kMaxExpertsGlobal = 256;

struct EpPeers {
  int* cnt_all[kMaxEp];        // [ep][experts] histograms, one row per source rank
  uint32_t* cnt_flags[kMaxEp];  // [ep]
  void* recv_x[kMaxEp];        // [cap, hidden]
  int2* recv_meta[kMaxEp];     // [cap] (source rank, pair index)
  uint32_t* disp_flags[kMaxEp];
  void* ret_y[kMaxEp];         // [pairs_cap, hidden]
  uint32_t* ret_flags[kMaxEp];
};

__global__ void __launch_bounds__(1024)
ep_plan_kernel(const int* __restrict__ topk_ids, int pairs, EpPeers peers, int ep, int rank, int experts,
               int experts_local, int bn, int cap_rows, uint32_t epoch, int* __restrict__ pair_dst_rank,
               int* __restrict__ pair_dst_row, int* __restrict__ expert_offsets, int2* __restrict__ work,
               int* __restrict__ n_work, int max_work, int* __restrict__ recv_rows, int* status) {
  pdl_wait();
  __shared__ int cnt[kMaxExpertsGlobal], fill[kMaxExpertsGlobal], send_base[kMaxExpertsGlobal];
  __shared__ int total[kMaxExpertsGlobal], before_me[kMaxExpertsGlobal];
  __shared__ int off[kMaxExpertsGlobal + 1], wbase[kMaxExpertsGlobal + 1];
  __shared__ int wait_ok;
  const int tid = threadIdx.x;
  for (int e = tid; e < kMaxExpertsGlobal; e += blockDim.x) {
    cnt[e] = 0;
    fill[e] = 0;
  }
  if (tid == 0) wait_ok = 1;
  __syncthreads();
  for (int i = tid; i < pairs; i += blockDim.x) {
    const int e = topk_ids[i];
    if (e >= 0 && e < experts)
      atomicAdd(&cnt[e], 1);
    else if (status != nullptr)
      atomicExch(status, kStatusBadIndex);
  }
  __syncthreads();
  // 1) my histogram to every rank (myself included), then my flag
  for (int i = tid; i < ep * experts; i += blockDim.x) {
    const int r = i / experts, e = i - r * experts;
    peers.cnt_all[r][rank * experts + e] = cnt[e];
  }
  __threadfence_system();
  __syncthreads();
  if (tid < ep) st_release_sys(peers.cnt_flags[tid] + rank, epoch);
  // 2) everybody's histogram
  if (tid < ep) {
    if (!wait_flag_ge(peers.cnt_flags[rank] + tid, epoch, status)) {
      wait_ok = 0;
      if (status != nullptr) atomicExch(status, kStatusPeerTimeout);
    }
  }
  __syncthreads();
  if (!wait_ok) {
    if (tid == 0) {
      *n_work = 0;
      *recv_rows = 0;
    }
    for (int e = tid; e <= experts_local; e += blockDim.x) expert_offsets[e] = 0;
    for (int i = tid; i < pairs; i += blockDim.x) pair_dst_rank[i] = -1;
    return;
  }
  const int* all = peers.cnt_all[rank];
  for (int e = tid; e < experts; e += blockDim.x) {
    int t = 0, b = 0;
    for (int r = 0; r < ep; ++r) {
      const int c = __ldcg(all + r * experts + e);
      if (r < rank) b += c;
      t += c;
    }
    total[e] = t;
    before_me[e] = b;
  }
  __syncthreads();
  // 3) slab layout of every destination: its experts in order, each expert's rows by source rank
  if (tid < ep) {
    int o = 0;
    for (int e = tid * experts_local; e < (tid + 1) * experts_local; ++e) {
      send_base[e] = o + before_me[e];
      o += total[e];
    }
  }
  // 4) my own experts: row ranges and the grouped GEMM's work list
  if (tid == 0) {
    int o = 0, w = 0;
    for (int el = 0; el < experts_local; ++el) {
      const int c = total[rank * experts_local + el];
      off[el] = o;
      wbase[el] = w;
      o += c;
      w += (c + bn - 1) / bn;
    }
    off[experts_local] = o;
    wbase[experts_local] = w;
    *n_work = min(w, max_work);
    *recv_rows = min(o, cap_rows);
    if ((o > cap_rows || w > max_work) && status != nullptr) atomicExch(status, kStatusBadIndex);
  }
  __syncthreads();
  for (int el = tid; el <= experts_local; el += blockDim.x) expert_offsets[el] = min(off[el], cap_rows);
  for (int el = tid; el < experts_local; el += blockDim.x) {
    const int chunks = wbase[el + 1] - wbase[el];
    for (int c = 0; c < chunks; ++c)
      if (wbase[el] + c < max_work) work[wbase[el] + c] = make_int2(el, c);
  }
  // 5) destination of every pair
  for (int i = tid; i < pairs; i += blockDim.x) {
    const int e = topk_ids[i];
    if (e < 0 || e >= experts) {
      pair_dst_rank[i] = -1;
      continue;
    }
    const int row = send_base[e] + atomicAdd(&fill[e], 1);
    pair_dst_rank[i] = row < cap_rows ? e / experts_local : -1;   // a row past the slab is not sent (status set by its owner)
    pair_dst_row[i] = row;
  }
}

// x [tokens, hidden] -> destination slabs.  grid = pairs, block = 128.
__global__ void ep_dispatch_kernel(const uint4* __restrict__ x, int64_t x_stride_v, int top_k,
                                   const int* __restrict__ pair_dst_rank, const int* __restrict__ pair_dst_row,
                                   EpPeers peers, int ep, int rank, int row_vecs, uint32_t epoch,
                                   int* __restrict__ done_count) {
  pdl_wait();
  const int i = blockIdx.x;
  const int d = pair_dst_rank[i];
  if (d >= 0) {
    const int row = pair_dst_row[i];
    const uint4* src = x + static_cast<int64_t>(i / top_k) * x_stride_v;
    uint4* dst = static_cast<uint4*>(peers.recv_x[d]) + static_cast<int64_t>(row) * row_vecs;
    for (int v = threadIdx.x; v < row_vecs; v += blockDim.x) dst[v] = __ldg(src + v);
    if (threadIdx.x == 0) peers.recv_meta[d][row] = make_int2(rank, i);
  }
  // publish: the barrier orders every thread's stores before thread 0's system-scope fence; the CTA that
  // finishes last raises this rank's flag on every destination
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int old = atomicAdd(done_count, 1);
    if (old == static_cast<int>(gridDim.x) - 1) {
      *done_count = 0;   // self-reset for the next launch
      __threadfence_system();
      for (int r = 0; r < ep; ++r) st_release_sys(peers.disp_flags[r] + rank, epoch);
    }
  }
}

// ys [slab rows, hidden] -> the sources' return buffers.  grid = slab capacity, block = 128.
__global__ void ep_return_kernel(const uint4* __restrict__ ys, const int* __restrict__ recv_rows, EpPeers peers, int ep,
                                 int rank, int row_vecs, uint32_t epoch, int* __restrict__ done_count) {
  pdl_wait();
  const int row = blockIdx.x;
  if (row < *recv_rows) {
    const int2 meta = peers.recv_meta[rank][row];
    if (meta.x >= 0 && meta.x < ep) {
      const uint4* src = ys + static_cast<int64_t>(row) * row_vecs;
      uint4* dst = static_cast<uint4*>(peers.ret_y[meta.x]) + static_cast<int64_t>(meta.y) * row_vecs;
      for (int v = threadIdx.x; v < row_vecs; v += blockDim.x) dst[v] = src[v];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int old = atomicAdd(done_count, 1);
    if (old == static_cast<int>(gridDim.x) - 1) {
      *done_count = 0;
      __threadfence_system();
      for (int r = 0; r < ep; ++r) st_release_sys(peers.ret_flags[r] + rank, epoch);
    }
  }
}

EpPeers make_peers(const EpA2AArgs& a) {
  EpPeers p{};
  for (int r = 0; r < a.ep; ++r) {
    p.cnt_all[r] = reinterpret_cast<int*>(a.cnt_all[r]);
    p.cnt_flags[r] = reinterpret_cast<uint32_t*>(a.cnt_flags[r]);
    p.recv_x[r] = reinterpret_cast<void*>(a.recv_x[r]);
    p.recv_meta[r] = reinterpret_cast<int2*>(a.recv_meta[r]);
    p.disp_flags[r] = reinterpret_cast<uint32_t*>(a.disp_flags[r]);
    p.ret_y[r] = reinterpret_cast<void*>(a.ret_y[r]);
    p.ret_flags[r] = reinterpret_cast<uint32_t*>(a.ret_flags[r]);
  }
  return p;
}

bool args_ok(const EpA2AArgs& a) {
  return a.ep >= 1 && a.ep <= kMaxEp && a.rank >= 0 && a.rank < a.ep && a.experts >= 1 && a.experts <= kMaxExpertsGlobal &&
         a.experts % a.ep == 0 && a.hidden % 8 == 0;
}

}  // namespace

int launch_ep_plan(const EpA2AArgs& a, const int* topk_ids, int pairs, int bn, int* pair_dst_rank, int* pair_dst_row,
                   int* expert_offsets, int* work, int* n_work, int max_work, int* recv_rows, int* status,
                   cudaStream_t s) {
  if (!args_ok(a) || pairs < 0) return -1;
  const cudaError_t err =
      launch_pdl(ep_plan_kernel, dim3(1), dim3(1024), 0, s, topk_ids, pairs, make_peers(a), a.ep, a.rank, a.experts,
                 a.experts / a.ep, bn, a.cap_rows, a.epoch, pair_dst_rank, pair_dst_row, expert_offsets,
                 reinterpret_cast<int2*>(work), n_work, max_work, recv_rows, status);
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}

int launch_ep_dispatch(const EpA2AArgs& a, const void* x, int64_t x_stride, int pairs, int top_k, const int* pair_dst_rank,
                       const int* pair_dst_row, int* done_count, cudaStream_t s) {
  if (!args_ok(a) || x_stride % 8 != 0) return -1;
  if (pairs == 0) return 0;
  const cudaError_t err =
      launch_pdl(ep_dispatch_kernel, dim3(pairs), dim3(128), 0, s, static_cast<const uint4*>(x), x_stride / 8, top_k,
                 pair_dst_rank, pair_dst_row, make_peers(a), a.ep, a.rank, a.hidden / 8, a.epoch, done_count);
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}

int launch_ep_return(const EpA2AArgs& a, const void* ys, const int* recv_rows, int* done_count, cudaStream_t s) {
  if (!args_ok(a) || a.cap_rows <= 0) return -1;
  const cudaError_t err = launch_pdl(ep_return_kernel, dim3(a.cap_rows), dim3(128), 0, s, static_cast<const uint4*>(ys),
                                     recv_rows, make_peers(a), a.ep, a.rank, a.hidden / 8, a.epoch, done_count);
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}

}  // namespace mb200
