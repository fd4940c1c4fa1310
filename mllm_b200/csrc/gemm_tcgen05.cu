// out[m, n] = a[m, k] * b[n, k]^T (+ bias) (+ residual), or the SwiGLU of it, on the
// 5th-generation tensor cores: operands staged in shared memory by TMA (128-byte swizzle,
// no multicast), tcgen05.mma issued by one thread, fp32 / s32 accumulators in tensor
// memory, epilogue through tcgen05.ld.  bf16 / fp16 inputs use kind::f16, int8 inputs
// (W8A8 with per-row x per-column scales) use kind::i8; both share this file.
//
// Two tilings share one kernel body:
//   * "normal" (m > 256): 128 activation rows x BN weight rows per tile, persistent CTAs
//     walking a group-rasterised tile list, two accumulator buffers so the epilogue of
//     tile i overlaps the main loop of tile i+1.
//   * "swap" (m <= 256, decode): the weight matrix is the 128-row MMA operand and the
//     (padded) batch is the MMA N dimension, so tiny batches still use full-width MMAs and
//     the kernel is a pure weight stream.  Work is scheduled stream-K style: the
//     (tile, k-block) iteration space is cut into one equal contiguous range per CTA, so
//     every SM streams the same number of weight bytes in a single persistent wave; a tile
//     whose k range is shared by several CTAs is finished by the last one to arrive (ticket
//     counter), which sums the fp32 partials from the workspace in contributor order, so
//     the result does not depend on timing.
//
// Warp roles (256 threads): warp 0 = TMA producer, warp 1 = MMA issuer, warp 2 = TMEM
// allocator, warps 4-7 = epilogue (warp w reads TMEM lanes 32*(w%4)..).
// Every mbarrier wait is bounded; on expiry the kernel records kStatusPipelineTimeout in
// *status and all roles drain out, TMEM is freed, and the host raises.
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "common.cuh"
#include "kernels.h"

namespace mb200 {
namespace {

constexpr int kBM = 128;            // rows of the MMA "M" operand per instruction
constexpr int kRowBytes = 128;      // bytes of K per pipeline stage row (one swizzle span)
constexpr int kUmmaKBytes = 32;     // bytes of K consumed by one tcgen05.mma
constexpr int kThreads = 256;

struct KParams {
  void* out;
  const void* bias;
  const void* residual;
  const float* a_scale;
  const float* b_scale;
  float* workspace;
  int* counters;
  int* status;
  int m, n, k_blocks;
  int64_t ldc, ld_res;
  int tiles_r, tiles_c;  // tiles over the row-operand rows / column-operand rows
  int max_contrib;       // swap tiling: upper bound of CTAs sharing one tile (workspace stride)
  int whole_tiles;       // swap tiling: 1 = CTA ranges are rounded to tile boundaries (no sharing)
  int stages;            // ring depth in use (<= Cfg::kStages)
  int out_f16;           // 0: bf16 output, 1: fp16 output
  int is_int8;
  int row_static;        // swap tiling: the row operand (weights) is not written by earlier kernels of the stream
  int cluster_k;         // swap tiling: > 1 = the k range of a tile is split over the CTAs of a cluster of this size
  int early_trigger;     // swap tiling: let the kernels behind this one start their set-up as soon as this one runs
  uint32_t idesc;
  // ---- tensor-parallel fusion (normal tiling only) ----
  // all-gather -> GEMM: row tile t of the activations may be read once gate_flags[t] >= gate_epoch
  const uint32_t* gate_flags;
  uint32_t gate_epoch;
  // GEMM -> reduce-scatter: row tile t belongs to rank t / rs_tiles_per_rank; the tile is stored into
  // that rank's inbox (rs_out[owner], this rank's slot) and, once all column tiles of the row tile
  // have been stored, rs_flags[owner][local tile * 8 + rs_rank] is set to rs_epoch
  int rs_tp, rs_rank, rs_tiles_per_rank;
  // Row tiles are visited starting rs_shift tiles (of this kernel's row-tile size) further on, modulo the tile
  // count: rank r begins with the rows of owner r + 1 and ends with its own, so that at any moment the ranks
  // store into DIFFERENT owners' inboxes.  In the same order everywhere they would all push to owner 0 first
  // and share that one GPU's NVLink ingress while the others' links idle.
  int rs_shift;
  uint32_t rs_epoch;
  int64_t rs_ld;
  void* rs_out[8];
  uint32_t* rs_flags[8];
  int* rs_count;
};

constexpr int kStageRowBytes = 144;                      // 128 bytes of output + 16 bytes of padding
constexpr int kEpiStagingBytes = 4 * 32 * kStageRowBytes;  // four epilogue warps x 32 rows

// RT = 128-row MMA tiles of the row operand per stage (small-batch tiling only; SwiGLU needs 2: a
// gate block and its up block), KD = 128-byte K atoms per stage.  Larger stages mean fewer TMA boxes
// and barrier round trips per byte streamed.
template <int BN, bool SWAP, bool SWIGLU, int RT, int KD>
struct Cfg {
  static constexpr int R = SWAP ? RT : 1;
  static constexpr int kRowTileBytes = kBM * R * kRowBytes;   // 16 KB * R per K atom
  static constexpr int kColTileBytes = BN * kRowBytes;
  static constexpr int kAtomBytes = kRowTileBytes + kColTileBytes;
  static constexpr int kStageBytes = KD * kAtomBytes;
  // one or two CTAs per SM: the ring takes the shared memory that is left
  static constexpr int kStagesRaw = 200704 / kStageBytes;
  static constexpr int kStages = kStagesRaw > 12 ? 12 : kStagesRaw;
  static constexpr int kSub = SWIGLU ? 1 : R;                 // output rows finalised per epilogue thread
  static constexpr int kAccCols = R * BN;
  static constexpr int kAccBufs = (2 * kAccCols <= 512) ? 2 : 1;
  static constexpr int kTmemColsRaw = kAccBufs * kAccCols;
  static constexpr int kTmemCols =
      kTmemColsRaw <= 32 ? 32 : (kTmemColsRaw <= 64 ? 64 : (kTmemColsRaw <= 128 ? 128 : (kTmemColsRaw <= 256 ? 256 : 512)));
  static_assert(kStages >= 2, "stage too large for shared memory");
  static_assert(!SWIGLU || !SWAP || RT == 2, "SwiGLU small-batch tiles hold a gate block and an up block");
  static_assert(SWAP || (RT == 1 && KD == 1), "normal tiling uses single-atom stages");
  static_assert(kTmemColsRaw <= 512, "accumulators exceed tensor memory");
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "invalid MMA N");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `local` (an address in this CTA's shared memory) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_smem(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_cluster_v4f(uint32_t cluster_addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ void fence_acq_rel_cluster() { asm volatile("fence.acq_rel.cluster;" ::: "memory"); }

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }

__device__ __forceinline__ uint32_t pack_out2(float lo, float hi, int out_f16) {
  if (out_f16) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  return pack_bf16x2(lo, hi);
}
__device__ __forceinline__ float load_out1(const void* base, int64_t idx, int out_f16) {
  if (out_f16) return __half2float(static_cast<const __half*>(base)[idx]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
}
__device__ __forceinline__ void store_out1(void* base, int64_t idx, float v, int out_f16) {
  if (out_f16)
    static_cast<__half*>(base)[idx] = __float2half_rn(v);
  else
    static_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float acc_to_float(uint32_t raw, int is_int8) {
  return is_int8 ? static_cast<float>(static_cast<int32_t>(raw)) : __uint_as_float(raw);
}

template <int BN, bool SWAP, bool SWIGLU, int RT, int KD>
__global__ void __launch_bounds__(kThreads, SWAP ? 2 : 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_row, const __grid_constant__ CUtensorMap tm_col,
                    const KParams p) {
  using C = Cfg<BN, SWAP, SWIGLU, RT, KD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int n_stages = p.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(n_stages) * C::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + n_stages;
  uint64_t* acc_full = bars + 2 * n_stages;
  uint64_t* acc_empty = acc_full + 2;
  // reduce-scatter: number of (epilogue warp, tile) store batches issued so far.  A counter, not an mbarrier:
  // the publisher warp may fall several tiles behind the epilogue (its system-scope fence waits for peer
  // stores in flight), and a phase bit that is lapped twice reads as "not yet" for ever.
  uint32_t* rs_stored = reinterpret_cast<uint32_t*>(acc_empty + 2);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  int* ticket_slot = const_cast<int*>(abort_flag) + 1;
  uint8_t* epi_staging = reinterpret_cast<uint8_t*>(bars) + 512;  // normal tiling only
  // small-batch tiling with the k range split over a cluster: the leader's inbox for its partners' fp32
  // partial sums, [partner][row of the tile][BN], and the barrier the partners arrive on
  float* red_buf = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 512);
  uint64_t* red_bar = acc_empty + 6;   // first free 8-byte slot behind tmem_holder / abort_flag / ticket_slot

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 128);
    }
    *rs_stored = 0;
    *abort_flag = 0;
    if (SWAP && p.cluster_k > 1) mbar_init(red_bar, (p.cluster_k - 1) * 128);
    fence_barrier_init();
    tma_prefetch_desc(&tm_row);
    tma_prefetch_desc(&tm_col);
  }
  __syncthreads();
  if (warp == 2) {
    tmem_alloc(tmem_holder, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  if (SWAP && p.cluster_k > 1)
    cluster_sync_all();   // the leader's inbox barrier exists before any partner can reach it
  else
    __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  // set-up above touched no global memory; from here on inputs of earlier kernels are read.  In the
  // small-batch tiling the producer thread may first fill the ring with weight tiles, which no earlier
  // kernel of the stream writes, and waits for its predecessors only before it loads activations: the
  // weight stream then starts while the previous kernel is still draining.
  const bool early_weights = SWAP && p.row_static != 0;
  if (SWAP && p.early_trigger) pdl_launch_dependents();
  if (!(early_weights && threadIdx.x == 0)) pdl_wait();

  const int total_tiles = p.tiles_r * p.tiles_c;
  // swap tiling: this CTA's contiguous range of the (tile, k-block) iteration space
  const int64_t total_iters = static_cast<int64_t>(total_tiles) * p.k_blocks;
  const int64_t it_begin =
      !SWAP ? 0
            : (p.whole_tiles ? (static_cast<int64_t>(total_tiles) * blockIdx.x / gridDim.x) * p.k_blocks
                             : (total_iters * blockIdx.x) / gridDim.x);
  const int64_t it_end =
      !SWAP ? 0
            : (p.whole_tiles ? (static_cast<int64_t>(total_tiles) * (blockIdx.x + 1) / gridDim.x) * p.k_blocks
                             : (total_iters * (blockIdx.x + 1)) / gridDim.x);

  // idx-th piece of work of this CTA -> (row tile, column tile, k-block range); false when done
  auto get_work = [&](int idx, int& tr, int& tc, int& kb0, int& kb1) -> bool {
    if constexpr (SWAP) {
      if (p.cluster_k > 1) {
        // one tile per cluster, one slice of its k range per CTA of the cluster
        if (idx > 0) return false;
        const int r = static_cast<int>(blockIdx.x) % p.cluster_k;
        tr = static_cast<int>(blockIdx.x) / p.cluster_k;
        tc = 0;
        kb0 = p.k_blocks * r / p.cluster_k;
        kb1 = p.k_blocks * (r + 1) / p.cluster_k;
        return true;
      }
      int64_t it = it_begin;
      for (int i = 0;; ++i) {
        if (it >= it_end) return false;
        const int tile = static_cast<int>(it / p.k_blocks);
        const int k0 = static_cast<int>(it - static_cast<int64_t>(tile) * p.k_blocks);
        const int k1 = static_cast<int>(min(static_cast<int64_t>(p.k_blocks), k0 + (it_end - it)));
        if (i == idx) {
          tr = tile;
          tc = 0;
          kb0 = k0;
          kb1 = k1;
          return true;
        }
        it += k1 - k0;
      }
    } else {
      const int tile = blockIdx.x + idx * gridDim.x;
      if (tile >= total_tiles) return false;
      constexpr int kGroup = 16;  // row tiles per raster group: a wave shares ~16 A tiles x ~9 B tiles in L2
      const int per_group = kGroup * p.tiles_c;
      const int g = tile / per_group;
      const int first = g * kGroup;
      const int gsize = min(p.tiles_r - first, kGroup);
      const int in = tile - g * per_group;
      tr = first + in % gsize;
      if (p.rs_shift > 0) tr = (tr + p.rs_shift) % p.tiles_r;
      tc = in / gsize;
      kb0 = 0;
      kb1 = p.k_blocks;
      return true;
    }
  };
  // CTA that owns iteration x of the swap schedule: the largest c with floor(c * I / G) <= x
  auto cta_of = [&](int64_t x) -> int {
    return static_cast<int>(min(static_cast<int64_t>(gridDim.x) - 1, ((x + 1) * gridDim.x - 1) / total_iters));
  };

  if (warp == 0 && lane == 0) {
    // ------------------------------ TMA producer ------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int tr, tc, kb0, kb1;
    const int k_elems_per_block = p.is_int8 ? kRowBytes : kRowBytes / 2;
    int early = 0;  // iterations whose weight tiles were issued ahead of the dependency wait
    if constexpr (SWAP) {
      if (early_weights) {
        for (int idx = 0; early < n_stages && get_work(idx, tr, tc, kb0, kb1); ++idx) {
          for (int kb = kb0; kb < kb1 && early < n_stages; ++kb, ++early) {
            uint8_t* stage_base = smem + static_cast<size_t>(early) * C::kStageBytes;
            mbar_arrive_expect_tx(&full_bar[early], C::kStageBytes);
#pragma unroll
            for (int kd = 0; kd < KD; ++kd)
              tma_load_2d(stage_base + kd * C::kAtomBytes, &tm_row, &full_bar[early],
                          (kb * KD + kd) * k_elems_per_block, tr * kBM * C::R);
          }
        }
        pdl_wait();
      }
    }
    int seen = 0;   // iterations handled so far by the loop below
    for (int idx = 0; ok && get_work(idx, tr, tc, kb0, kb1); ++idx) {
      if constexpr (!SWAP) {
        if (p.gate_flags != nullptr) {
          // rows of this tile are written by peers (generic proxy); the TMA engine reads them
          if (!wait_flag_ge(p.gate_flags + tr, p.gate_epoch, p.status)) {
            ok = false;
            if (p.status != nullptr) atomicExch(p.status, kStatusPeerTimeout);
            break;
          }
          fence_proxy_async_all();
        }
      }
      for (int kb = kb0; kb < kb1; ++kb, ++seen) {
        uint8_t* stage_base = smem + static_cast<size_t>(stage) * C::kStageBytes;
        if (seen < early) {
          // first pass over the ring: the stage is free and its weight tiles are already on their way
#pragma unroll
          for (int kd = 0; kd < KD; ++kd)
            tma_load_2d(stage_base + kd * C::kAtomBytes + C::kRowTileBytes, &tm_col, &full_bar[stage],
                        (kb * KD + kd) * k_elems_per_block, tc * BN);
        } else {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full_bar[stage], C::kStageBytes);
#pragma unroll
          for (int kd = 0; kd < KD; ++kd) {
            uint8_t* row_tile = stage_base + kd * C::kAtomBytes;
            const int x = (kb * KD + kd) * k_elems_per_block;
            tma_load_2d(row_tile, &tm_row, &full_bar[stage], x, tr * kBM * C::R);
            tma_load_2d(row_tile + C::kRowTileBytes, &tm_col, &full_bar[stage], x, tc * BN);
          }
        }
        if (++stage == n_stages) {
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
    // ------------------------------ MMA issuer --------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int tr, tc, kb0, kb1;
    const uint64_t desc_stage0 = umma_desc_k_sw128(smem_u32(smem));
    const uint32_t idesc = p.idesc;
    for (int idx = 0; ok && get_work(idx, tr, tc, kb0, kb1); ++idx) {
      const int acc = idx % C::kAccBufs;
      const uint32_t acc_phase = (idx / C::kAccBufs) & 1;
      if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t d_base = tmem_base + acc * C::kAccCols;
      // The issuing thread is a serial chain of its own: it must get through a k-block in fewer cycles than
      // the tensor core needs for it, so the loop body is kept to the wait, the MMAs and the commit.  The
      // descriptor of a stage is the descriptor of stage 0 plus a multiple of 16 bytes in its low word.
      auto issue = [&](auto int8_tag) {
        constexpr bool kInt8 = decltype(int8_tag)::value;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t a_stage = desc_stage0 + static_cast<uint32_t>(stage) * (C::kStageBytes >> 4);
#pragma unroll
          for (int kd = 0; kd < KD; ++kd) {
#pragma unroll
            for (int r = 0; r < C::R; ++r) {
#pragma unroll
              for (int kk = 0; kk < kRowBytes / kUmmaKBytes; ++kk) {
                const uint64_t a_desc = a_stage + ((kd * C::kAtomBytes + r * (kBM * kRowBytes) + kk * kUmmaKBytes) >> 4);
                const uint64_t b_desc = a_stage + ((kd * C::kAtomBytes + C::kRowTileBytes + kk * kUmmaKBytes) >> 4);
                const uint32_t accum = (kd > 0 || kk > 0) ? 1u : (kb > kb0 ? 1u : 0u);
                if constexpr (kInt8)
                  umma_i8(d_base + r * BN, a_desc, b_desc, idesc, accum);
                else
                  umma_f16(d_base + r * BN, a_desc, b_desc, idesc, accum);
              }
            }
          }
          umma_commit(&empty_bar[stage]);  // stage reusable once these MMAs have read it
          if (++stage == n_stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      };
      if (p.is_int8)
        issue(std::true_type{});
      else
        issue(std::false_type{});
      if (ok) umma_commit(&acc_full[acc]);
    }
    if (!ok) {
      *abort_flag = 1;
      if (p.status != nullptr) atomicExch(p.status, kStatusPipelineTimeout);
    }
  } else if (warp == 3 && lane == 0 && !SWAP && p.rs_tp > 0) {
    // ------------------------------ reduce-scatter publisher ------------------
    // Waits until the four epilogue warps have issued a tile's stores (release increment / acquire load of
    // the shared counter orders them before this thread), makes them visible system-wide with one fence,
    // counts the tile in and, when the last column tile of a 128-row tile is done, raises the owner's flag.
    int tr, tc, kb0, kb1;
    for (int idx = 0; get_work(idx, tr, tc, kb0, kb1); ++idx) {
      const uint32_t want = 4u * static_cast<uint32_t>(idx + 1);
      bool seen = false;
      const uint64_t t0 = global_ns();
      for (uint32_t i = 0;; ++i) {
        if (ld_acquire_cta_smem(rs_stored) >= want) {
          seen = true;
          break;
        }
        __nanosleep(100);
        if ((i & 31u) == 31u && (*abort_flag || global_ns() - t0 > kPipelineWaitNs)) break;
      }
      if (!seen) {
        *abort_flag = 1;
        if (p.status != nullptr) atomicExch(p.status, kStatusPipelineTimeout);
        break;
      }
      __threadfence_system();
      const int owner = tr / p.rs_tiles_per_rank;
      const int local_tile = tr - owner * p.rs_tiles_per_rank;
      const int old = atomicAdd(&p.rs_count[tr], 1);
      if (old == p.tiles_c - 1) {
        p.rs_count[tr] = 0;  // self-reset for the next launch
        __threadfence_system();
        st_release_sys(p.rs_flags[owner] + local_tile * 8 + p.rs_rank, p.rs_epoch);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue -----------------------------------
    const int ew = warp - 4;             // TMEM lane quadrant
    const int row_in_tile = ew * 32 + lane;
    bool ok = true;
    int tr, tc, kb0, kb1;
    for (int idx = 0; ok && get_work(idx, tr, tc, kb0, kb1); ++idx) {
      const int acc = idx % C::kAccBufs;
      const uint32_t acc_phase = (idx / C::kAccBufs) & 1;
      if (*abort_flag || !mbar_wait(&acc_full[acc], acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t t_base = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * C::kAccCols;

      if constexpr (!SWAP) {
        constexpr int kOutCols = SWIGLU ? BN / 2 : BN;
        const int64_t col0 = static_cast<int64_t>(tc) * kOutCols;
        const int n_out = SWIGLU ? p.n / 2 : p.n;
        if (p.rs_tp > 0) {
          // Staged epilogue (reduce-scatter stores only): a thread owns one accumulator row; 64 output columns at a time are
          // rounded, parked in shared memory and written back so that eight lanes cover 128
          // contiguous bytes of one output row (full-line stores, local or to a peer's inbox).
          uint8_t* stage_buf = epi_staging + ew * (32 * kStageRowBytes);
          const int64_t tile_row0 = static_cast<int64_t>(tr) * kBM + ew * 32;
          const float sa = (p.is_int8 && tile_row0 + lane < p.m) ? p.a_scale[tile_row0 + lane] : 1.f;
          uint16_t* dst_base = static_cast<uint16_t*>(p.out);
          int64_t dst_ld = p.ldc;
          int64_t dst_row0 = tile_row0;
          int owner = 0, local_tile = 0;
          if (p.rs_tp > 0) {
            owner = tr / p.rs_tiles_per_rank;
            local_tile = tr - owner * p.rs_tiles_per_rank;
            dst_base = static_cast<uint16_t*>(p.rs_out[owner]);
            dst_ld = p.rs_ld;
            dst_row0 = static_cast<int64_t>(local_tile) * kBM + ew * 32;
          }
#pragma unroll 1
          for (int c = 0; c < kOutCols; c += 64) {
            uint32_t packed[32];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t r0[32], r1[32];
              tmem_ld_32x32(t_base + c + h * 32, r0);
              if constexpr (SWIGLU) tmem_ld_32x32(t_base + BN / 2 + c + h * 32, r1);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; j += 2) {
                float f[2];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                  const int cc = c + h * 32 + j + q;  // column inside the tile's output
                  float x = acc_to_float(r0[j + q], p.is_int8);
                  if constexpr (SWIGLU) {
                    float u = acc_to_float(r1[j + q], p.is_int8);
                    if (p.is_int8) {
                      x *= sa * p.b_scale[tc * BN + cc];
                      u *= sa * p.b_scale[tc * BN + BN / 2 + cc];
                    }
                    x = silu_f(x) * u;
                  } else {
                    const int64_t col = col0 + cc;
                    if (p.is_int8 && col < n_out) x *= sa * p.b_scale[col];
                    if (p.bias != nullptr && col < n_out) x += load_out1(p.bias, col, p.out_f16);
                  }
                  f[q] = x;
                }
                packed[h * 16 + j / 2] = pack_out2(f[0], f[1], p.out_f16);
              }
            }
            uint4* my_row = reinterpret_cast<uint4*>(stage_buf + lane * kStageRowBytes);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              my_row[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = i * 4 + (lane >> 3);
              const int piece = lane & 7;
              const int64_t col = col0 + c + piece * 8;
              if (tile_row0 + r < p.m && col < n_out) {
                const uint4 v = *reinterpret_cast<const uint4*>(stage_buf + r * kStageRowBytes + piece * 16);
                *reinterpret_cast<uint4*>(dst_base + (dst_row0 + r) * dst_ld + col) = v;
              }
            }
            __syncwarp();
          }
          // hand the tile to the publisher warp, which fences and signals off the epilogue's critical path
          __syncwarp();
          if (lane == 0) red_add_release_cta_smem(rs_stored, 1u);
        } else {
        // thread = one output row; columns in chunks of 32
        const int64_t row = static_cast<int64_t>(tr) * kBM + row_in_tile;
        const bool row_ok = row < p.m;
        const float sa = (p.is_int8 && row_ok) ? p.a_scale[row] : 1.f;
#pragma unroll 1
        for (int c = 0; c < kOutCols; c += 32) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(t_base + c, r0);
          if constexpr (SWIGLU) tmem_ld_32x32(t_base + BN / 2 + c, r1);
          tmem_ld_wait();
          if (!row_ok) continue;
#pragma unroll
          for (int v8 = 0; v8 < 4; ++v8) {
            const int64_t col = col0 + c + v8 * 8;
            if (col >= n_out) break;
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float x = acc_to_float(r0[v8 * 8 + j], p.is_int8);
              if constexpr (SWIGLU) {
                float u = acc_to_float(r1[v8 * 8 + j], p.is_int8);
                if (p.is_int8) {
                  x *= sa * p.b_scale[tc * BN + c + v8 * 8 + j];
                  u *= sa * p.b_scale[tc * BN + BN / 2 + c + v8 * 8 + j];
                }
                x = silu_f(x) * u;
              } else {
                if (p.is_int8) x *= sa * p.b_scale[col + j];
                if (p.bias != nullptr) x += load_out1(p.bias, col + j, p.out_f16);
              }
              f[j] = x;
            }
            if (!SWIGLU && p.residual != nullptr) {
              const uint4 rv = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.residual) +
                                                               row * p.ld_res + col);
              const uint32_t* ru = reinterpret_cast<const uint32_t*>(&rv);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float2 q;
                if (p.out_f16) {
                  q = __half22float2(*reinterpret_cast<const __half2*>(&ru[j]));
                } else {
                  q = unpack_bf16x2(ru[j]);
                }
                f[2 * j] += q.x;
                f[2 * j + 1] += q.y;
              }
            }
            uint4 o;
            o.x = pack_out2(f[0], f[1], p.out_f16);
            o.y = pack_out2(f[2], f[3], p.out_f16);
            o.z = pack_out2(f[4], f[5], p.out_f16);
            o.w = pack_out2(f[6], f[7], p.out_f16);
            *reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + row * p.ldc + col) = o;
          }
        }
        }
      } else {
        // thread = one weight row (output column); accumulator column j = activation row j
        const int64_t nrow0 = static_cast<int64_t>(tr) * kBM * C::R;  // first weight row of the tile
        const int m_cols = min(p.m, BN);
        const bool whole_tile = (kb0 == 0 && kb1 == p.k_blocks);
        const int crank = p.cluster_k > 1 ? static_cast<int>(blockIdx.x) % p.cluster_k : 0;
        if (p.cluster_k > 1 && crank != 0) {
          // partner of a cluster: the fp32 partial sums go straight into the leader's shared memory
          constexpr int kTileRows = kBM * C::R;
          const uint32_t inbox = mapa_smem(smem_u32(red_buf), 0) +
                                 static_cast<uint32_t>(crank - 1) * (kTileRows * BN * 4);
#pragma unroll 1
          for (int r = 0; r < C::R; ++r) {
            const uint32_t row_addr = inbox + static_cast<uint32_t>(r * kBM + row_in_tile) * (BN * 4);
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
              uint32_t v[16];
              tmem_ld_32x16(t_base + r * BN + c, v);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; j += 4)
                st_cluster_v4f(row_addr + (c + j) * 4, acc_to_float(v[j], p.is_int8), acc_to_float(v[j + 1], p.is_int8),
                               acc_to_float(v[j + 2], p.is_int8), acc_to_float(v[j + 3], p.is_int8));
            }
          }
          mbar_arrive_cluster(mapa_smem(smem_u32(red_bar), 0));   // release: orders the stores above
        } else if (!whole_tile && p.cluster_k <= 1) {
          // contributors of this tile are consecutive CTAs; this CTA's position among them
          const int first_cta = cta_of(static_cast<int64_t>(tr) * p.k_blocks);
          const int n_contrib = cta_of(static_cast<int64_t>(tr + 1) * p.k_blocks - 1) - first_cta + 1;
          const int split = static_cast<int>(blockIdx.x) - first_cta;
          constexpr int kTileRows = kBM * C::R;
          float* ws_tile = p.workspace + static_cast<int64_t>(tr) * p.max_contrib * kTileRows * BN;
          // 1) publish fp32 partials: ws_tile[contributor][row in tile][BN] (a thread's row is contiguous)
#pragma unroll 1
          for (int r = 0; r < C::R; ++r) {
            const int64_t wrow = nrow0 + r * kBM + row_in_tile;
            float* dst = ws_tile + (static_cast<int64_t>(split) * kTileRows + r * kBM + row_in_tile) * BN;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
              uint32_t v[16];
              tmem_ld_32x16(t_base + r * BN + c, v);
              tmem_ld_wait();
              if (wrow < p.n && c < m_cols) {
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                  *reinterpret_cast<float4*>(dst + c + j) =
                      make_float4(acc_to_float(v[j], p.is_int8), acc_to_float(v[j + 1], p.is_int8),
                                  acc_to_float(v[j + 2], p.is_int8), acc_to_float(v[j + 3], p.is_int8));
              }
            }
          }
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (row_in_tile == 0) {
            const int t = atomicAdd(&p.counters[tr], 1);
            *ticket_slot = t;
            if (t == n_contrib - 1) p.counters[tr] = 0;  // self-reset for the next launch
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const bool last = (*ticket_slot == n_contrib - 1);
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (last) {
            __threadfence();
            // sum of the contributions, in contributor order, for 16 batch columns of one weight
            // row; four contributions (16 independent 16-byte loads) are in flight at a time
            auto reduce16 = [&](int row_in_super_tile, int c0, float (&acc)[16]) {
#pragma unroll
              for (int i = 0; i < 16; ++i) acc[i] = 0.f;
              for (int s0 = 0; s0 < n_contrib; s0 += 4) {
                float4 v[4][4];
#pragma unroll
                for (int ss = 0; ss < 4; ++ss) {
                  const float* src = ws_tile + (static_cast<int64_t>(min(s0 + ss, n_contrib - 1)) * kTileRows + row_in_super_tile) * BN + c0;
#pragma unroll
                  for (int q4 = 0; q4 < 4; ++q4) v[ss][q4] = __ldcg(reinterpret_cast<const float4*>(src) + q4);
                }
#pragma unroll
                for (int ss = 0; ss < 4; ++ss) {
                  if (s0 + ss < n_contrib) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                      acc[4 * q4 + 0] += v[ss][q4].x;
                      acc[4 * q4 + 1] += v[ss][q4].y;
                      acc[4 * q4 + 2] += v[ss][q4].z;
                      acc[4 * q4 + 3] += v[ss][q4].w;
                    }
                  }
                }
              }
            };
#pragma unroll 1
            for (int sub = 0; sub < C::kSub; ++sub) {
              const int64_t wrow = nrow0 + sub * kBM + row_in_tile;
              if (wrow >= p.n) continue;
              for (int c0 = 0; c0 < m_cols; c0 += 16) {
                float x[16], u[16];
                reduce16(sub * kBM + row_in_tile, c0, x);
                if constexpr (SWIGLU) reduce16(kBM + row_in_tile, c0, u);
#pragma unroll
                for (int jj = 0; jj < 16; ++jj) {
                  const int j = c0 + jj;
                  if (j >= m_cols) break;
                  float xv = x[jj];
                  int64_t ocol;
                  if constexpr (SWIGLU) {
                    float uv = u[jj];
                    if (p.is_int8) {
                      xv *= p.a_scale[j] * p.b_scale[wrow];
                      uv *= p.a_scale[j] * p.b_scale[wrow + kBM];
                    }
                    xv = silu_f(xv) * uv;
                    ocol = static_cast<int64_t>(tr) * kBM + row_in_tile;
                  } else {
                    if (p.is_int8) xv *= p.a_scale[j] * p.b_scale[wrow];
                    if (p.bias != nullptr) xv += load_out1(p.bias, wrow, p.out_f16);
                    if (p.residual != nullptr) xv += load_out1(p.residual, j * p.ld_res + wrow, p.out_f16);
                    ocol = wrow;
                  }
                  store_out1(p.out, j * p.ldc + ocol, xv, p.out_f16);
                }
              }
            }
          }
        } else {
          constexpr int kTileRows = kBM * C::R;
          if (p.cluster_k > 1) {
            // leader of a cluster: wait for the partners' partial sums
            if (!mbar_wait(red_bar, 0, abort_flag)) {
              ok = false;
              break;
            }
            fence_acq_rel_cluster();
          }
#pragma unroll 1
          for (int sub = 0; sub < C::kSub; ++sub) {
          const int64_t wrow = nrow0 + sub * kBM + row_in_tile;
#pragma unroll 1
          for (int c = 0; c < BN; c += 16) {
            uint32_t v0[16], v1[16];
            tmem_ld_32x16(t_base + sub * BN + c, v0);
            if constexpr (SWIGLU) tmem_ld_32x16(t_base + BN + c, v1);
            tmem_ld_wait();
            if (wrow >= p.n) continue;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int mi = c + j;
              if (mi >= m_cols) break;
              float x = acc_to_float(v0[j], p.is_int8);
              float u_extra = 0.f;
              for (int s2 = 1; s2 < p.cluster_k; ++s2) {   // partners in rank order: the sum does not depend on timing
                const float* part = red_buf + static_cast<size_t>(s2 - 1) * kTileRows * BN;
                x += part[(sub * kBM + row_in_tile) * BN + mi];
                if constexpr (SWIGLU) u_extra += part[(kBM + row_in_tile) * BN + mi];
              }
              int64_t ocol;
              if constexpr (SWIGLU) {
                float u = acc_to_float(v1[j], p.is_int8) + u_extra;
                if (p.is_int8) {
                  x *= p.a_scale[mi] * p.b_scale[wrow];
                  u *= p.a_scale[mi] * p.b_scale[wrow + kBM];
                }
                x = silu_f(x) * u;
                ocol = static_cast<int64_t>(tr) * kBM + row_in_tile;
              } else {
                if (p.is_int8) x *= p.a_scale[mi] * p.b_scale[wrow];
                if (p.bias != nullptr) x += load_out1(p.bias, wrow, p.out_f16);
                if (p.residual != nullptr) x += load_out1(p.residual, mi * p.ld_res + wrow, p.out_f16);
                ocol = wrow;
              }
              store_out1(p.out, mi * p.ldc + ocol, x, p.out_f16);
            }
          }
          }
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

  pdl_launch_dependents();  // this CTA's work is done: the next kernel may start its set-up
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // give copies that may still be in flight time to land before the CTA's memory is reused
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}


// =========================================================================================
// Two-CTA tiling (large m): a cluster of two CTAs on neighbouring SMs computes one 256 x 256 output
// tile with tcgen05.mma.cta_group::2.  Each CTA stages 128 activation rows (its half of the tile's M)
// and 128 weight rows (its half of the tile's N) per 64-element k-block: 32 KB per CTA and k-block
// instead of the 48 KB a lone CTA needs for its 128 x 256 tile, i.e. a third less traffic from L2 into
// shared memory per FLOP, which is what bounds the one-CTA tiling.  The leader CTA (cluster rank 0)
// issues the MMAs for the pair; the hardware reads the A rows and the B half of each CTA from that CTA's
// shared memory and writes each CTA's 128 accumulator rows into that CTA's tensor memory.
//   * TMA loads of both CTAs signal the LEADER's full barrier (cp.async.bulk.tensor ... cta_group::2
//     with the barrier address mapped into the leader; no cluster multicast anywhere).
//   * tcgen05.commit (cta_group::2) arrives on the empty / accumulator-full barriers of BOTH CTAs
//     (two commits, one per CTA, each addressed through mapa).
//   * epilogue warps of both CTAs arrive on the leader's accumulator-empty barrier (remote arrive).
// Roles per CTA as in the one-CTA kernel: warp 0 TMA producer, warp 1 MMA issuer (leader only), warp 2
// tensor-memory allocator, warps 4-7 epilogue.  All waits are bounded; a CTA that gives up raises its own
// and its partner's abort flag.
// =========================================================================================
constexpr int kPairBN = 256;
constexpr int kPairStageBytes = 2 * kBM * kRowBytes;            // A half-tile + B half-tile: 32 KB
constexpr int kPairStages = 6;
constexpr int kPairSmem = kPairStages * kPairStageBytes + 1024 + 512 + kEpiStagingBytes;

// TMA load whose completion bytes are counted on a barrier that may live in the partner CTA
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_out, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_out)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// all pair MMAs issued so far by this thread arrive on the barrier at `bar_cluster_addr` when they finish
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}

template <bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_row, const __grid_constant__ CUtensorMap tm_col,
                 const KParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(kPairStages) * kPairStageBytes);
  uint64_t* full_bar = bars;                       // used in the leader: 1 arrival + bytes of both CTAs
  uint64_t* empty_bar = bars + kPairStages;        // per CTA: tcgen05.commit
  uint64_t* acc_full = bars + 2 * kPairStages;     // per CTA: tcgen05.commit
  uint64_t* acc_empty = acc_full + 2;              // used in the leader: 256 epilogue threads of the pair
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  uint32_t* rs_stored = tmem_holder + 2;   // reduce-scatter: (epilogue warp, tile) store batches issued so far
  uint8_t* epi_staging = reinterpret_cast<uint8_t*>(bars) + 512;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 256);
    }
    *abort_flag = 0;
    *rs_stored = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_row);
    tma_prefetch_desc(&tm_col);
  }
  __syncthreads();
  if (warp == 2) {
    tmem_alloc_pair(tmem_holder, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();   // both CTAs' barriers are initialised before either signals the other's
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  pdl_wait();

  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int total_tiles = p.tiles_r * p.tiles_c;   // tiles of 256 x 256
  auto get_tile = [&](int idx, int& tr, int& tc) -> bool {
    const int tile = pair + idx * num_pairs;
    if (tile >= total_tiles) return false;
    constexpr int kGroup = 8;  // 256-row tiles per raster group
    const int per_group = kGroup * p.tiles_c;
    const int g = tile / per_group;
    const int first = g * kGroup;
    const int gsize = min(p.tiles_r - first, kGroup);
    const int in = tile - g * per_group;
    tr = first + in % gsize;
    if (p.rs_shift > 0) tr = (tr + p.rs_shift) % p.tiles_r;
    tc = in / gsize;
    return true;
  };
  auto give_up = [&](int code) {
    *abort_flag = 1;
    st_cluster_u32(mapa_smem(smem_u32(const_cast<int*>(abort_flag)), rank ^ 1u), 1u);
    if (p.status != nullptr) atomicExch(p.status, code);
  };

  if (warp == 0 && lane == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    const int k_elems_per_block = p.is_int8 ? kRowBytes : kRowBytes / 2;
    const uint32_t full_leader0 = mapa_smem(smem_u32(&full_bar[0]), 0);   // barriers are 8 bytes apart
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int tr, tc;
    for (int idx = 0; ok && get_tile(idx, tr, tc); ++idx) {
      const int row0 = tr * 2 * kBM + static_cast<int>(rank) * kBM;       // this CTA's 128 activation rows
      const int col0 = tc * kPairBN + static_cast<int>(rank) * (kPairBN / 2);  // this CTA's 128 weight rows
      if (p.gate_flags != nullptr && row0 < p.m) {
        if (!wait_flag_ge(p.gate_flags + (row0 >> 7), p.gate_epoch, p.status)) {
          give_up(kStatusPeerTimeout);
          ok = false;
          break;
        }
        fence_proxy_async_all();
      }
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
          ok = false;
          break;
        }
        uint8_t* stage_base = smem + static_cast<size_t>(stage) * kPairStageBytes;
        const uint32_t full_leader = full_leader0 + static_cast<uint32_t>(stage) * 8u;
        if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * kPairStageBytes);
        const int x = kb * k_elems_per_block;
        tma_load_2d_pair(stage_base, &tm_row, full_leader, x, row0);
        tma_load_2d_pair(stage_base + kBM * kRowBytes, &tm_col, full_leader, x, col0);
        if (++stage == kPairStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (!ok) give_up(kStatusPipelineTimeout);
  } else if (warp == 1 && lane == 0 && leader) {
    // ------------------------------ MMA issuer (leader CTA) -------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int tr, tc;
    const uint64_t desc_stage0 = umma_desc_k_sw128(smem_u32(smem));
    const uint32_t idesc = p.idesc;
    const uint32_t empty0 = mapa_smem(smem_u32(&empty_bar[0]), 0), empty1 = mapa_smem(smem_u32(&empty_bar[0]), 1);
    for (int idx = 0; ok && get_tile(idx, tr, tc); ++idx) {
      const int acc = idx & 1;
      const uint32_t acc_phase = (idx >> 1) & 1;
      if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t d_base = tmem_base + acc * kPairBN;
      auto issue = [&](auto int8_tag) {
        constexpr bool kInt8 = decltype(int8_tag)::value;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t a_stage = desc_stage0 + static_cast<uint32_t>(stage) * (kPairStageBytes >> 4);
#pragma unroll
          for (int kk = 0; kk < kRowBytes / kUmmaKBytes; ++kk) {
            const uint64_t a_desc = a_stage + ((kk * kUmmaKBytes) >> 4);
            const uint64_t b_desc = a_stage + ((kBM * kRowBytes + kk * kUmmaKBytes) >> 4);
            const uint32_t accum = kk > 0 ? 1u : (kb > 0 ? 1u : 0u);
            if constexpr (kInt8)
              umma_i8_pair(d_base, a_desc, b_desc, idesc, accum);
            else
              umma_f16_pair(d_base, a_desc, b_desc, idesc, accum);
          }
          // the stage is reusable, in both CTAs, once these MMAs have read it
          umma_commit_pair(empty0 + static_cast<uint32_t>(stage) * 8u);
          umma_commit_pair(empty1 + static_cast<uint32_t>(stage) * 8u);
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      };
      if (p.is_int8)
        issue(std::true_type{});
      else
        issue(std::false_type{});
      if (ok) {
        umma_commit_pair(mapa_smem(smem_u32(&acc_full[acc]), 0));
        umma_commit_pair(mapa_smem(smem_u32(&acc_full[acc]), 1));
      }
    }
    if (!ok) give_up(kStatusPipelineTimeout);
  } else if (warp == 3 && lane == 0 && p.rs_tp > 0) {
    // ------------------------------ reduce-scatter publisher (both CTAs) ------------------
    // as in the one-CTA kernel: fence once per tile after the four epilogue warps have issued its stores,
    // count the tile in, and raise the owner's flag when the last column tile of a 128-row tile is done
    int tr, tc;
    for (int idx = 0; get_tile(idx, tr, tc); ++idx) {
      const uint32_t want = 4u * static_cast<uint32_t>(idx + 1);
      bool seen = false;
      const uint64_t t0 = global_ns();
      for (uint32_t i = 0;; ++i) {
        if (ld_acquire_cta_smem(rs_stored) >= want) {
          seen = true;
          break;
        }
        __nanosleep(100);
        if ((i & 31u) == 31u && (*abort_flag || global_ns() - t0 > kPipelineWaitNs)) break;
      }
      if (!seen) {
        give_up(kStatusPipelineTimeout);
        break;
      }
      __threadfence_system();
      const int tr128 = tr * 2 + static_cast<int>(rank);
      const int owner = tr128 / p.rs_tiles_per_rank;
      const int local_tile = tr128 - owner * p.rs_tiles_per_rank;
      const int old = atomicAdd(&p.rs_count[tr128], 1);
      if (old == p.tiles_c - 1) {
        p.rs_count[tr128] = 0;  // self-reset for the next launch
        __threadfence_system();
        st_release_sys(p.rs_flags[owner] + local_tile * 8 + p.rs_rank, p.rs_epoch);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue (both CTAs) ----------------------------------
    const int ew = warp - 4;
    const int row_in_tile = ew * 32 + lane;
    bool ok = true;
    int tr, tc;
    constexpr int kOutCols = SWIGLU ? kPairBN / 2 : kPairBN;
    const int n_out = SWIGLU ? p.n / 2 : p.n;
    for (int idx = 0; ok && get_tile(idx, tr, tc); ++idx) {
      const int acc = idx & 1;
      const uint32_t acc_phase = (idx >> 1) & 1;
      if (*abort_flag || !mbar_wait(&acc_full[acc], acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t t_base = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * kPairBN;
      const int64_t row = static_cast<int64_t>(tr) * 2 * kBM + static_cast<int64_t>(rank) * kBM + row_in_tile;
      const bool row_ok = row < p.m;
      const int64_t col0 = static_cast<int64_t>(tc) * kOutCols;
      const float sa = (p.is_int8 && row_ok) ? p.a_scale[row] : 1.f;
      if constexpr (!SWIGLU) {
        if (p.rs_tp > 0) {
          // reduce-scatter: 64 output columns at a time are rounded, parked in shared memory and written so that
          // eight lanes cover 128 contiguous bytes of one row of the owner's inbox (full-line peer stores)
          uint8_t* stage_buf = epi_staging + ew * (32 * kStageRowBytes);
          const int tr128 = tr * 2 + static_cast<int>(rank);
          const int owner = tr128 / p.rs_tiles_per_rank;
          const int local_tile = tr128 - owner * p.rs_tiles_per_rank;
          uint16_t* dst_base = static_cast<uint16_t*>(p.rs_out[owner]);
          const int64_t dst_row0 = static_cast<int64_t>(local_tile) * kBM + ew * 32;
          const int64_t tile_row0 = static_cast<int64_t>(tr128) * kBM + ew * 32;
#pragma unroll 1
          for (int c = 0; c < kOutCols; c += 64) {
            uint32_t packed[32];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t r0[32];
              tmem_ld_32x32(t_base + c + h * 32, r0);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; j += 2) {
                float f[2];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                  const int64_t col = col0 + c + h * 32 + j + q;
                  float x = acc_to_float(r0[j + q], p.is_int8);
                  if (p.is_int8 && col < n_out) x *= sa * p.b_scale[col];
                  if (p.bias != nullptr && col < n_out) x += load_out1(p.bias, col, p.out_f16);
                  f[q] = x;
                }
                packed[h * 16 + j / 2] = pack_out2(f[0], f[1], p.out_f16);
              }
            }
            uint4* my_row = reinterpret_cast<uint4*>(stage_buf + lane * kStageRowBytes);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              my_row[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = i * 4 + (lane >> 3);
              const int piece = lane & 7;
              const int64_t col = col0 + c + piece * 8;
              if (tile_row0 + r < p.m && col < n_out) {
                const uint4 v = *reinterpret_cast<const uint4*>(stage_buf + r * kStageRowBytes + piece * 16);
                *reinterpret_cast<uint4*>(dst_base + (dst_row0 + r) * p.rs_ld + col) = v;
              }
            }
            __syncwarp();
          }
          __syncwarp();
          if (lane == 0) red_add_release_cta_smem(rs_stored, 1u);
          tc_fence_before_sync();
          mbar_arrive_cluster(mapa_smem(smem_u32(&acc_empty[acc]), 0));
          continue;
        }
      }
#pragma unroll 1
      for (int c = 0; c < kOutCols; c += 32) {
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(t_base + c, r0);
        if constexpr (SWIGLU) tmem_ld_32x32(t_base + kPairBN / 2 + c, r1);
        tmem_ld_wait();
        if (!row_ok) continue;
#pragma unroll
        for (int v8 = 0; v8 < 4; ++v8) {
          const int64_t col = col0 + c + v8 * 8;
          if (col >= n_out) break;
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float x = acc_to_float(r0[v8 * 8 + j], p.is_int8);
            if constexpr (SWIGLU) {
              float u = acc_to_float(r1[v8 * 8 + j], p.is_int8);
              if (p.is_int8) {
                x *= sa * p.b_scale[tc * kPairBN + c + v8 * 8 + j];
                u *= sa * p.b_scale[tc * kPairBN + kPairBN / 2 + c + v8 * 8 + j];
              }
              x = silu_f(x) * u;
            } else {
              if (p.is_int8) x *= sa * p.b_scale[col + j];
              if (p.bias != nullptr) x += load_out1(p.bias, col + j, p.out_f16);
            }
            f[j] = x;
          }
          if (!SWIGLU && p.residual != nullptr) {
            const uint4 rv = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.residual) +
                                                             row * p.ld_res + col);
            const uint32_t* ru = reinterpret_cast<const uint32_t*>(&rv);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float2 q;
              if (p.out_f16) {
                q = __half22float2(*reinterpret_cast<const __half2*>(&ru[j]));
              } else {
                q = unpack_bf16x2(ru[j]);
              }
              f[2 * j] += q.x;
              f[2 * j + 1] += q.y;
            }
          }
          uint4 o;
          o.x = pack_out2(f[0], f[1], p.out_f16);
          o.y = pack_out2(f[2], f[3], p.out_f16);
          o.z = pack_out2(f[4], f[5], p.out_f16);
          o.w = pack_out2(f[6], f[7], p.out_f16);
          *reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + row * p.ldc + col) = o;
        }
      }
      tc_fence_before_sync();
      mbar_arrive_cluster(mapa_smem(smem_u32(&acc_empty[acc]), 0));
    }
    if (!ok) give_up(kStatusPipelineTimeout);
  }

  pdl_launch_dependents();
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // give copies that may still be in flight time to land before the CTAs' memory is reused
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  // neither CTA may leave while its partner can still read its shared memory or signal its barriers
  cluster_sync_all();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeFn>(sym);
    }
  });
  return fn;
}

int env_int(const char* name, int dflt) {
  const char* v = std::getenv(name);
  return (v != nullptr && *v != 0) ? std::atoi(v) : dflt;
}

CUtensorMapL2promotion l2_promotion() {
  static const int v = env_int("MLLM_B200_GEMM_L2_PROMO", 256);
  return v == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                : (v == 64 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                           : (v == 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
}

// 2-D row-major matrix [rows, k] (k contiguous, `ld` elements between rows); box = 128 bytes of k x box_rows.
bool make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int64_t ld, int elem_bytes,
                      CUtensorMapDataType type, int box_rows) {
  EncodeFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kRowBytes / elem_bytes), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, type, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, l2_promotion(),
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int BN, bool SWAP, bool SWIGLU, int RT = 1, int KD = 1>
int launch_cfg(const CUtensorMap& tr, const CUtensorMap& tc, KParams p, int grid, cudaStream_t s) {
  using C = Cfg<BN, SWAP, SWIGLU, RT, KD>;
  // tuning knob: MLLM_B200_GEMM_STAGES caps the ring depth of the small-batch tiling
  static const int stage_cap = env_int("MLLM_B200_GEMM_STAGES", 0);
  p.stages = C::kStages;
  if (SWAP && stage_cap >= 2 && stage_cap < p.stages) p.stages = stage_cap;
  auto kern = gemm_tcgen05_kernel<BN, SWAP, SWIGLU, RT, KD>;
  const size_t tail = 1024 + 512 + (SWAP ? 0 : kEpiStagingBytes);
  // cluster split of k: the leader's inbox for its partners' partial sums comes out of the ring's memory
  const size_t inbox = (SWAP && p.cluster_k > 1) ? static_cast<size_t>(p.cluster_k - 1) * kBM * C::R * BN * sizeof(float) : 0;
  while (p.stages > 2 && static_cast<size_t>(p.stages) * C::kStageBytes + tail + inbox > 232448) --p.stages;
  if (static_cast<size_t>(p.stages) * C::kStageBytes + tail + inbox > 232448) return -1;
  const size_t smem = static_cast<size_t>(p.stages) * C::kStageBytes + tail + inbox;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern),
                          static_cast<int>(std::max(smem, static_cast<size_t>(C::kStages) * C::kStageBytes + tail))) != cudaSuccess)
    return -3;
  cudaError_t err;
  if (SWAP && p.cluster_k > 1) {
    ensure_max_carveout(reinterpret_cast<const void*>(kern));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(p.cluster_k);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    err = cudaLaunchKernelEx(&cfg, kern, tr, tc, p);
  } else {
    err = launch_pdl(kern, dim3(grid), dim3(kThreads), smem, s, tr, tc, p);
  }
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}

template <bool SWIGLU>
int launch_pair_cfg(const CUtensorMap& tr, const CUtensorMap& tc, const KParams& p, int pairs, cudaStream_t s) {
  auto kern = gemm_pair_kernel<SWIGLU>;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), kPairSmem) != cudaSuccess) return -3;
  ensure_max_carveout(reinterpret_cast<const void*>(kern));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kPairSmem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const cudaError_t err = cudaLaunchKernelEx(&cfg, kern, tr, tc, p);
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}

}  // namespace

bool make_tma_operand_map(void* map, const void* base, int64_t rows, int64_t k, int64_t ld, int elem_bytes, int type,
                          int box_rows) {
  const CUtensorMapDataType t = type == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                          : (type == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  return make_operand_map(static_cast<CUtensorMap*>(map), base, rows, k, ld, elem_bytes, t, box_rows);
}

size_t gemm_workspace_bytes(int, int, int, int) { return size_t(64) << 20; }

int launch_gemm(const GemmArgs& a, cudaStream_t s) {
  if (a.m <= 0 || a.n <= 0) return 0;
  if (a.norm_weight != nullptr && a.m > 8) return -1;
  const int eb = a.is_int8 ? 1 : 2;
  const int k_per_block = kRowBytes / eb;
  if (a.k % (16 / eb) != 0 || a.lda % (16 / eb) != 0 || a.ldb % (16 / eb) != 0) return -1;
  if (a.n % 8 != 0 || a.ldc % 8 != 0) return -1;
  if (a.swiglu && (a.n % 256 != 0 || a.bias != nullptr || a.residual != nullptr)) return -1;
  if ((reinterpret_cast<uintptr_t>(a.a) | reinterpret_cast<uintptr_t>(a.b) | reinterpret_cast<uintptr_t>(a.out)) & 15)
    return -1;
  if (a.residual != nullptr && ((reinterpret_cast<uintptr_t>(a.residual) & 15) || a.ld_res % 8 != 0)) return -1;

  KParams p{};
  p.out = a.out;
  p.bias = a.bias;
  p.residual = a.residual;
  p.a_scale = a.a_scale;
  p.b_scale = a.b_scale;
  p.workspace = a.workspace;
  p.counters = a.counters;
  p.status = a.status;
  p.m = a.m;
  p.n = a.n;
  p.k_blocks = (a.k + k_per_block - 1) / k_per_block;
  p.ldc = a.ldc;
  p.ld_res = a.ld_res;
  p.out_f16 = (a.dt == kF16) ? 1 : 0;
  p.is_int8 = a.is_int8;
  p.row_static = a.b_static;
  {
    // The CTAs of a following small-batch GEMM fit beside ours when both keep their rings short: they are
    // then launched while this kernel still streams, fetch their first weight tiles, and take over the memory
    // pipe the moment our CTAs drain (tuning knobs; 0 / 0 = trigger at the end, ring as deep as memory allows).
    static const int early_knob = env_int("MLLM_B200_GEMM_EARLY_TRIGGER", 0);
    p.early_trigger = early_knob;
  }
  p.max_contrib = 1;

  const CUtensorMapDataType type =
      a.is_int8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                : (a.dt == kF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  const uint32_t ab_fmt = a.is_int8 ? 1u : (a.dt == kF16 ? 0u : 1u);
  const uint32_t c_fmt = a.is_int8 ? 2u : 1u;
  const int num_sms = a.num_sms > 0 ? a.num_sms : 148;
  CUtensorMap tm_row, tm_col;

  const bool tp_fused = a.gate_flags != nullptr || a.rs_tp > 0;
  if (tp_fused && (a.m <= 256 || a.residual != nullptr)) return -5;
  if (a.rs_tp > 0) {
    if (a.rs_tp > 8 || a.m % (kBM * a.rs_tp) != 0 || a.rs_count == nullptr || a.rs_ld % 8 != 0) return -5;
    p.rs_tp = a.rs_tp;
    p.rs_rank = a.rs_rank;
    p.rs_tiles_per_rank = a.m / kBM / a.rs_tp;
    p.rs_epoch = a.rs_epoch;
    p.rs_ld = a.rs_ld;
    p.rs_count = a.rs_count;
    for (int r = 0; r < a.rs_tp; ++r) {
      p.rs_out[r] = reinterpret_cast<void*>(a.rs_out[r]);
      p.rs_flags[r] = reinterpret_cast<uint32_t*>(a.rs_flags[r]);
      if (a.rs_out[r] & 15) return -5;
    }
  }
  p.gate_flags = a.gate_flags;
  p.gate_epoch = a.gate_epoch;
  if (a.m > 256) {
    // ---- two-CTA tiling: 256 x 256 tiles per pair of SMs, when there are enough of them to fill the GPU ----
    static const int pair_knob = env_int("MLLM_B200_GEMM_PAIR", 1);
    const int64_t tiles_pair = static_cast<int64_t>((a.m + 2 * kBM - 1) / (2 * kBM)) * ((a.n + kPairBN - 1) / kPairBN);
    const bool pair_rs_ok = a.rs_tp == 0 || (!a.swiglu && (a.m / kBM / a.rs_tp) % 2 == 0);
    const int rs_first_owner = a.rs_tp > 0 ? (a.rs_rank + 1) % a.rs_tp : 0;
    if (pair_knob && a.n % 256 == 0 && tiles_pair >= num_sms / 2 && pair_rs_ok) {
      if (a.rs_tp > 0) p.rs_shift = rs_first_owner * (p.rs_tiles_per_rank / 2);
      p.tiles_r = (a.m + 2 * kBM - 1) / (2 * kBM);
      p.tiles_c = (a.n + kPairBN - 1) / kPairBN;
      p.idesc = umma_idesc(2 * kBM, kPairBN, c_fmt, ab_fmt, ab_fmt);
      if (!make_operand_map(&tm_row, a.a, a.m, a.k, a.lda, eb, type, kBM)) return -2;
      if (!make_operand_map(&tm_col, a.b, a.n, a.k, a.ldb, eb, type, kPairBN / 2)) return -2;
      const int pairs = static_cast<int>(std::min<int64_t>(tiles_pair, num_sms / 2));
      return a.swiglu ? launch_pair_cfg<true>(tm_row, tm_col, p, pairs, s)
                      : launch_pair_cfg<false>(tm_row, tm_col, p, pairs, s);
    }
    // ---- normal tiling: activations are the 128-row operand ----
    int bn = 256;
    if (!a.swiglu) {
      const int64_t tiles256 = static_cast<int64_t>((a.m + kBM - 1) / kBM) * ((a.n + 255) / 256);
      if (tiles256 < num_sms || a.n % 256 != 0) bn = 128;
    }
    p.tiles_r = (a.m + kBM - 1) / kBM;
    p.tiles_c = (a.n + bn - 1) / bn;
    if (a.rs_tp > 0) p.rs_shift = rs_first_owner * p.rs_tiles_per_rank;
    p.idesc = umma_idesc(kBM, bn, c_fmt, ab_fmt, ab_fmt);
    if (!make_operand_map(&tm_row, a.a, a.m, a.k, a.lda, eb, type, kBM)) return -2;
    if (!make_operand_map(&tm_col, a.b, a.n, a.k, a.ldb, eb, type, bn)) return -2;
    const int grid = std::min(p.tiles_r * p.tiles_c, num_sms);
    if (a.swiglu) return launch_cfg<256, false, true>(tm_row, tm_col, p, grid, s);
    if (bn == 256) return launch_cfg<256, false, false>(tm_row, tm_col, p, grid, s);
    return launch_cfg<128, false, false>(tm_row, tm_col, p, grid, s);
  }

  // ---- a handful of rows: stream the weights through registers (gemm_smallm.cu) ----
  if (a.m <= 8) {
    const int rc = launch_gemm_smallm(a, s);
    if (rc <= 0) return rc;
  }
  if (a.norm_weight != nullptr) return -1;   // the fused norm prologue exists in that kernel only

  // ---- swap tiling: weights are the 128-row operand, the batch is MMA N ----
  int bn = 16;
  while (bn < a.m) bn <<= 1;
  // stage shape: two 128-row weight tiles and two K atoms per stage when the batch is small enough
  // for the stage to fit several times into shared memory (tuning knobs override)
  static const int rt_knob = env_int("MLLM_B200_GEMM_RT", 0);
  static const int kd_knob = env_int("MLLM_B200_GEMM_KD", 0);
  int rt = a.swiglu ? 2 : 1;
  int kd = (bn <= 64 && a.k >= 1024) ? 2 : 1;
  if (bn <= 64) {
    if (rt_knob == 1 && !a.swiglu) rt = 1;
    if (rt_knob == 2) rt = 2;
    if (kd_knob == 1 || kd_knob == 2) kd = kd_knob;
  }
  const int r = rt;
  const int k_per_stage = kd * k_per_block;
  p.k_blocks = (a.k + k_per_stage - 1) / k_per_stage;
  p.tiles_r = (a.n + kBM * r - 1) / (kBM * r);
  p.tiles_c = 1;
  p.idesc = umma_idesc(kBM, bn, c_fmt, ab_fmt, ab_fmt);
  if (!make_operand_map(&tm_row, a.b, a.n, a.k, a.ldb, eb, type, kBM * r)) return -2;
  if (!make_operand_map(&tm_col, a.a, a.m, a.k, a.lda, eb, type, bn)) return -2;
  // stream-K: one equal range of (tile, k-block) iterations per CTA, at least kMinBytes of weights each
  // so the fixed cost of a CTA stays small against its stream; fall back to whole tiles when there is
  // no room for the partial sums.
  const int64_t iters = static_cast<int64_t>(p.tiles_r) * p.k_blocks;
  const int64_t stage_weight_bytes = static_cast<int64_t>(kd) * kBM * r * kRowBytes;
  const int64_t min_iters = std::max<int64_t>(1, (128 * 1024) / stage_weight_bytes);
  static const int ctas_per_sm = std::max(1, env_int("MLLM_B200_GEMM_CTAS_PER_SM", 1));
  int grid = static_cast<int>(std::min<int64_t>(static_cast<int64_t>(num_sms) * ctas_per_sm,
                                                std::max<int64_t>(1, iters / min_iters)));
  const bool can_share = a.workspace != nullptr && a.counters != nullptr && p.tiles_r <= a.num_counters;
  auto contributors = [&](int g) {
    const int64_t per = std::max<int64_t>(1, iters / g);
    return static_cast<int>((p.k_blocks + per - 1) / per) + 1;
  };
  auto ws_need = [&](int g) {
    return static_cast<size_t>(p.tiles_r) * contributors(g) * kBM * r * bn * sizeof(float);
  };
  p.whole_tiles = 0;
  // Tiles fewer than SMs and a small batch: split the k range of every tile over a cluster of CTAs instead, and
  // sum the partial products through the leader's shared memory (no workspace round trip, no tickets).
  static const int cluster_knob = env_int("MLLM_B200_GEMM_CLUSTER_K", 1);
  p.cluster_k = 0;
  if (cluster_knob && !a.swiglu && bn == 16 && p.tiles_r * 2 <= num_sms) {
    // power-of-two cluster sizes only: clusters of 3 did not all fit one wave when measured (22.4 us against
    // 15.9 us for the 6144 x 4096 projection), 4-CTA clusters gained 1.4-1.9 us on 4096-row projections
    int split = std::min(8, num_sms / p.tiles_r);
    while (split & (split - 1)) --split;
    while (split > 1 && p.k_blocks < 4 * split) split >>= 1;
    if (split > 1 && p.tiles_r * split * 8 >= num_sms * 6) {   // at least three quarters of the SMs busy
      p.cluster_k = split;
      grid = p.tiles_r * split;
    }
  }
  if (p.cluster_k > 1) {
    // nothing shared through global memory
  } else if (!can_share || ws_need(grid) > a.workspace_bytes) {
    grid = std::min(grid, p.tiles_r);  // every CTA gets whole tiles: nothing is shared
    p.whole_tiles = 1;
  }
  p.max_contrib = contributors(grid);
#define MB200_SWAP_SMALL(BNV)                                                                       \
  case BNV:                                                                                         \
    if (a.swiglu)                                                                                   \
      return kd == 2 ? launch_cfg<BNV, true, true, 2, 2>(tm_row, tm_col, p, grid, s)                \
                     : launch_cfg<BNV, true, true, 2, 1>(tm_row, tm_col, p, grid, s);               \
    if (rt == 2)                                                                                    \
      return kd == 2 ? launch_cfg<BNV, true, false, 2, 2>(tm_row, tm_col, p, grid, s)               \
                     : launch_cfg<BNV, true, false, 2, 1>(tm_row, tm_col, p, grid, s);              \
    return kd == 2 ? launch_cfg<BNV, true, false, 1, 2>(tm_row, tm_col, p, grid, s)                 \
                   : launch_cfg<BNV, true, false, 1, 1>(tm_row, tm_col, p, grid, s);
#define MB200_SWAP_LARGE(BNV)                                                                       \
  case BNV:                                                                                         \
    return a.swiglu ? launch_cfg<BNV, true, true, 2, 1>(tm_row, tm_col, p, grid, s)                 \
                    : launch_cfg<BNV, true, false, 1, 1>(tm_row, tm_col, p, grid, s);
  switch (bn) {
    MB200_SWAP_SMALL(16)
    MB200_SWAP_SMALL(32)
    MB200_SWAP_SMALL(64)
    MB200_SWAP_LARGE(128)
    MB200_SWAP_LARGE(256)
  }
#undef MB200_SWAP_SMALL
#undef MB200_SWAP_LARGE
  return -1;
}

}  // namespace mb200
