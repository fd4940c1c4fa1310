// Attention over the slot-indexed KV pool on tcgen05 tensor cores.  The single-role kernel described first is
// instantiated for head sizes 64, 128 and 256 (one, two or four 64-feature halves per row; the figures below
// are those of 128); the warp-specialised prefill and decode kernels further down are for head size 128.
//
// One kernel serves prefill (ragged new tokens after an optional cached prefix, causal) and
// decode (one token per request, split over the KV length): a CTA owns one request, one KV
// head and a tile of 128 "rows", where a row is a (query token, query head of the GQA group)
// pair - the group's heads share every K/V tile that is loaded.  Per 64-token KV tile:
//   S = Q K^T      tcgen05.mma (M128 N64 K128), fp32 in tensor memory
//   softmax        one thread per row reads its S row with tcgen05.ld, online max/sum in the
//                  log2 domain, writes P (bf16) to shared memory in the MMA operand layout
//   O += P V       tcgen05.mma (M128 N128 K64), V used as an MN-major operand straight from
//                  the gathered [token, d] rows; O stays in tensor memory and is rescaled
//                  lazily (only when the running max grows by more than 2^8)
// K/V rows are gathered with cp.async through the request->slot table (any page size, no
// flat index list), double buffered, written directly in the 128-byte-swizzled operand
// layout.  Decode splits the KV range over CTAs; a small merge kernel combines the partial
// (O, log-sum-exp) pairs.  All mbarrier waits are bounded.
#include <algorithm>

#include <cstdlib>
#include <string>

#include "common.cuh"
#include "kernels.h"

namespace mb200 {
namespace {

constexpr int kD = 128;        // head dim of the specialised kernels (the single-role kernel also takes 64 and 256)
constexpr int kRows = 128;     // MMA M
constexpr int kKV = 64;        // KV tokens per tile
constexpr int kAttnThreads = 128;
constexpr int kHalfQ = kRows * 128;  // bytes of one 64-feature half of the Q tile
constexpr int kHalfKV = kKV * 128;   // bytes of one 64-feature half of a K or V tile
constexpr int kSmemP = kRows * 128;                // 16 KB
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;

struct AttnParams {
  const void* q;      // [T, Hq, D] with row stride q_stride (elements)
  const void* k_cache;
  const void* v_cache;
  void* out;          // [T, Hq, D] contiguous
  float* part_o;      // decode split: [B, Hq, splits, D]
  float* part_lse;    // decode split: [B, Hq, splits]
  const int* req_to_token;
  const int* req_pool_indices;
  const int* seq_lens;
  const int* prefix_lens;  // null in decode
  int non_causal;          // prefill only: every query row sees the whole sequence
  const int* q_start;      // null in decode
  int* status;
  int64_t q_stride;
  int64_t rtt_stride;
  int64_t num_slots;
  int64_t kv_tok_stride, kv_head_stride;  // elements: row of head h of slot s at s * tok + h * head
  // the caches seen as matrices of 128-wide rows: row of (slot, head) = slot * kv_row_mul + head * kv_row_add;
  // kv_runs = 1 when consecutive slots of one head are consecutive rows (head-major storage)
  int kv_row_mul, kv_row_add, kv_runs;
  int hq, hkv, group;
  int tokens_per_tile;     // query tokens per CTA tile = 128 / group (rounded down)
  int num_splits;          // decode only
  int is_decode;
  int out_f16;
  float scale_log2;        // softmax scale * log2(e)
  int window;              // sliding window: a query at position i sees keys i - window + 1 .. i (0 = everything)
  float logit_cap;         // soft cap: score = cap * tanh(score / cap) before the softmax (0 = off)
  float scale;             // softmax scale (used with the soft cap)
  float cap_pre, cap_post; // soft cap: score in the log2 domain = cap_post * tanh(raw * cap_pre)
  int kv_fmt;              // single-role kernel only: 1 / 2 = the caches hold unscaled e4m3 / e5m2 bytes
  uint32_t idesc_s, idesc_o;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
// hardware tanh (one special-function instruction, relative error about 2^-11): enough for a soft cap whose
// result is rounded to 16 bits two instructions later
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// offset of 16-byte chunk `chunk` (0..15 over 128 features) of row `row` inside a tile made of
// two 64-feature halves of `half_bytes` each, rows of 128 bytes, 128-byte swizzle
__device__ __forceinline__ uint32_t swz_off(int row, int chunk, int half_bytes) {
  return (chunk >> 3) * half_bytes + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

// NH = number of 64-feature halves of a head: head sizes 64, 128 and 256
template <int NH>
struct FwdCfg {
  static constexpr int kD = 64 * NH;                   // head dim
  static constexpr int kChunks = 8 * NH;               // 16-byte chunks per row
  static constexpr int kTokPerPass = kAttnThreads / kChunks;   // KV tokens one pass of the CTA's threads covers
  static constexpr int kPasses = kKV / kTokPerPass;
  static constexpr int kSmemQ = NH * kHalfQ;
  static constexpr int kSmemKVBuf = NH * kHalfKV;      // per tensor per buffer
  static constexpr int kSmem = kSmemQ + 4 * kSmemKVBuf + kSmemP + 1024 + 64;
  static constexpr int kTmemCols = NH == 1 ? 128 : (NH == 2 ? 256 : 512);   // 64 (S) + kD (O), a power of two
  static constexpr int kCtasPerSm = NH == 4 ? 1 : 2;
};

// KV8: the caches hold 8-bit floats; a tile is then read with plain loads, widened to the activation dtype in
// registers and stored into the same swizzled operand layout (the tensor core sees 16-bit operands either way)
template <int NH, bool KV8>
__global__ void __launch_bounds__(kAttnThreads, FwdCfg<NH>::kCtasPerSm) attn_fwd_kernel(const AttnParams p) {
  using C = FwdCfg<NH>;
  constexpr int kD = C::kD;
  constexpr int kSmemQ = C::kSmemQ;
  constexpr int kSmemKVBuf = C::kSmemKVBuf;
  pdl_wait();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kSmemQ;                 // 2 buffers
  uint8_t* sV = sK + 2 * kSmemKVBuf;         // 2 buffers
  uint8_t* sP = sV + 2 * kSmemKVBuf;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kSmemP);
  uint64_t* bar_s = bars;
  uint64_t* bar_o = bars + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int b = blockIdx.z;
  const int hk = blockIdx.y;
  const int req = p.req_pool_indices[b];
  const int seq_len = p.seq_lens[b];

  // ---- work range of this CTA ------------------------------------------------------------
  int q0, q_len, prefix, kv_begin, kv_end, q_row0;
  if (p.is_decode) {
    q0 = 0;
    q_len = 1;
    prefix = seq_len - 1;
    q_row0 = b;
    const int lo = p.window > 0 ? max(0, seq_len - p.window) / kKV * kKV : 0;   // first tile the window touches
    const int tiles = (seq_len - lo + kKV - 1) / kKV;
    const int per = (tiles + p.num_splits - 1) / p.num_splits;
    kv_begin = lo + blockIdx.x * per * kKV;
    kv_end = min(seq_len, kv_begin + per * kKV);
  } else {
    prefix = p.prefix_lens[b];
    q_len = seq_len - prefix;
    q0 = blockIdx.x * p.tokens_per_tile;
    q_row0 = p.q_start[b];
    // with a window the tile's first query row bounds the keys from below
    kv_begin = (p.window > 0 && !p.non_causal) ? max(0, prefix + q0 - p.window + 1) / kKV * kKV : 0;
    kv_end = p.non_causal ? seq_len
                          : min(seq_len, prefix + min(q_len, q0 + p.tokens_per_tile));  // causal upper bound of the tile
    if (q0 >= q_len) return;
  }
  const int g = p.group;
  const int split = blockIdx.x;
  if (p.is_decode && kv_begin >= kv_end) {
    // empty split: publish a neutral partial
    for (int i = tid; i < g * kD; i += kAttnThreads) {
      const int head = hk * g + i / kD;
      p.part_o[((static_cast<int64_t>(b) * p.hq + head) * p.num_splits + split) * kD + (i % kD)] = 0.f;
    }
    if (tid < g) p.part_lse[(static_cast<int64_t>(b) * p.hq + hk * g + tid) * p.num_splits + split] = -INFINITY;
    return;
  }
  const int n_tiles = (kv_end - kv_begin + kKV - 1) / kKV;

  if (tid == 0) {
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (warp == 0) {
    tmem_alloc(tmem_holder, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_s = tmem_base;         // 64 columns
  const uint32_t tmem_o = tmem_base + 64;    // kD columns
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;

  // ---- this thread's row ------------------------------------------------------------------
  const int row = tid;
  const int row_tok = row / g;              // token inside the tile
  const int row_head = hk * g + row % g;
  const bool row_valid = (row_tok < p.tokens_per_tile) && (q0 + row_tok < q_len);
  const int kv_limit = (p.non_causal && !p.is_decode) ? seq_len - 1
                                                      : (row_valid ? (prefix + q0 + row_tok) : prefix + q0);  // last visible key (inclusive)

  const uint16_t* qbase = static_cast<const uint16_t*>(p.q);
  const uint16_t* kbase = static_cast<const uint16_t*>(p.k_cache);
  const uint16_t* vbase = static_cast<const uint16_t*>(p.v_cache);
  const int* rtt = p.req_to_token + static_cast<int64_t>(req) * p.rtt_stride;

  // ---- Q tile: 128 rows x (2 kD) B, kChunks chunks per row ----------------------------------
  {
    const uint32_t sq = smem_u32(sQ);
    for (int c = tid; c < kRows * C::kChunks; c += kAttnThreads) {
      const int r = c / C::kChunks, ch = c % C::kChunks;
      const int tok = r / g;
      const bool ok = (tok < p.tokens_per_tile) && (q0 + tok < q_len);
      const int head = hk * g + r % g;
      const uint16_t* src = qbase + static_cast<int64_t>(q_row0 + q0 + (ok ? tok : 0)) * p.q_stride +
                            static_cast<int64_t>(head) * kD + ch * 8;
      cp_async16(sq + swz_off(r, ch, kHalfQ), src, ok);
    }
  }

  // gather of one KV tile: 64 tokens x kChunks chunks for K and V; thread handles token
  // tid / kChunks + kTokPerPass * i
  int slots_next[C::kPasses];
  auto fetch_slots = [&](int tile) {
    const int t0 = kv_begin + tile * kKV;
#pragma unroll
    for (int i = 0; i < C::kPasses; ++i) {
      const int t = t0 + tid / C::kChunks + C::kTokPerPass * i;
      slots_next[i] = (tile < n_tiles && t < kv_end) ? __ldg(rtt + t) : -1;
    }
    bool bad = false;
#pragma unroll
    for (int i = 0; i < C::kPasses; ++i) {
      if (slots_next[i] < -1 || slots_next[i] >= p.num_slots) {
        bad = true;
        slots_next[i] = -1;
      }
    }
    if (bad && p.status != nullptr) atomicExch(p.status, kStatusBadIndex);
  };
  auto gather = [&](int buf) {
    const uint32_t sk = smem_u32(sK + buf * kSmemKVBuf);
    const uint32_t sv = smem_u32(sV + buf * kSmemKVBuf);
    const int ch = tid % C::kChunks;
    if constexpr (KV8) {
      // all loads of the tile first (they are independent), then widen and store
      const uint8_t* k8 = static_cast<const uint8_t*>(p.k_cache);
      const uint8_t* v8 = static_cast<const uint8_t*>(p.v_cache);
      uint2 kr[C::kPasses], vr[C::kPasses];
#pragma unroll
      for (int i = 0; i < C::kPasses; ++i) {
        const int s = slots_next[i];
        kr[i] = vr[i] = make_uint2(0u, 0u);
        if (s >= 0) {
          const int64_t off = static_cast<int64_t>(s) * p.kv_tok_stride + hk * p.kv_head_stride + ch * 8;
          kr[i] = __ldg(reinterpret_cast<const uint2*>(k8 + off));
          vr[i] = __ldg(reinterpret_cast<const uint2*>(v8 + off));
        }
      }
      auto widen = [&](uint32_t two) -> uint32_t {   // two fp8 bytes -> two 16-bit values of the activation dtype
        const float2 f = unpack_fp8x2(two, p.kv_fmt);
        if (p.out_f16) {
          __half2 h = __floats2half2_rn(f.x, f.y);
          return *reinterpret_cast<uint32_t*>(&h);
        }
        return pack_bf16x2(f.x, f.y);
      };
#pragma unroll
      for (int i = 0; i < C::kPasses; ++i) {
        const int r = tid / C::kChunks + C::kTokPerPass * i;
        const uint32_t so = swz_off(r, ch, kHalfKV);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sk + so), "r"(widen(kr[i].x)), "r"(widen(kr[i].x >> 16)),
                     "r"(widen(kr[i].y)), "r"(widen(kr[i].y >> 16))
                     : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sv + so), "r"(widen(vr[i].x)), "r"(widen(vr[i].x >> 16)),
                     "r"(widen(vr[i].y)), "r"(widen(vr[i].y >> 16))
                     : "memory");
      }
    } else {
#pragma unroll
      for (int i = 0; i < C::kPasses; ++i) {
        const int r = tid / C::kChunks + C::kTokPerPass * i;
        const int s = slots_next[i];
        const bool ok = s >= 0;
        const int64_t off = static_cast<int64_t>(ok ? s : 0) * p.kv_tok_stride + hk * p.kv_head_stride + ch * 8;
        const uint32_t so = swz_off(r, ch, kHalfKV);
        cp_async16(sk + so, kbase + off, ok);
        cp_async16(sv + so, vbase + off, ok);
      }
    }
  };

  fetch_slots(0);
  gather(0);
  cp_async_commit();  // group: Q + tile 0
  fetch_slots(1);

  float m_used = -INFINITY;  // max in use for the exponent (log2 domain)
  float l_sum = 0.f;
  bool ok_all = true;

  for (int j = 0; j < n_tiles; ++j) {
    const int buf = j & 1;
    cp_async_wait<0>();
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();  // tile j (and Q) visible to the tensor core

    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t qa = smem_u32(sQ);
      const uint32_t ka = smem_u32(sK + buf * kSmemKVBuf);
#pragma unroll
      for (int kk = 0; kk < 4 * NH; ++kk) {
        const uint64_t a_desc = umma_desc_k_sw128(qa + (kk >> 2) * kHalfQ + (kk & 3) * 32);
        const uint64_t b_desc = umma_desc_k_sw128(ka + (kk >> 2) * kHalfKV + (kk & 3) * 32);
        umma_f16(tmem_s, a_desc, b_desc, p.idesc_s, kk > 0 ? 1u : 0u);
      }
      umma_commit(bar_s);
    }
    // previous P*V must be finished before P, O and the other KV buffer are touched
    if (j > 0) {
      if (!mbar_wait(bar_o, (j - 1) & 1)) ok_all = false;
      tc_fence_after_sync();
    }
    if (j + 1 < n_tiles) {
      gather(buf ^ 1);
      cp_async_commit();
      fetch_slots(j + 2);
    }
    if (!mbar_wait(bar_s, j & 1)) ok_all = false;
    tc_fence_after_sync();

    // ---- softmax on this thread's row --------------------------------------------------
    uint32_t sraw[2][32];
    tmem_ld_32x32(tmem_s + lane_base, sraw[0]);
    tmem_ld_32x32(tmem_s + lane_base + 32, sraw[1]);
    tmem_ld_wait();
    const int col0 = kv_begin + j * kKV;
    const int visible = min(kv_limit, kv_end - 1) - col0;  // columns 0..visible are allowed
    const int first_vis = (p.window > 0 && !(p.non_causal && !p.is_decode)) ? kv_limit - p.window + 1 - col0 : -(1 << 30);
    float sc[64];
    float m_tile = -INFINITY;
    if (p.logit_cap > 0.f) {   // uniform branch, kept outside the loop: the tanh must not be paid by plain scores
#pragma unroll
      for (int c = 0; c < 64; ++c)
        sc[c] = p.cap_post * tanhf(__uint_as_float(sraw[c >> 5][c & 31]) * p.cap_pre);
    } else {
#pragma unroll
      for (int c = 0; c < 64; ++c) sc[c] = __uint_as_float(sraw[c >> 5][c & 31]) * p.scale_log2;
    }
#pragma unroll
    for (int c = 0; c < 64; ++c) {
      const float v = (c <= visible && c >= first_vis) ? sc[c] : -INFINITY;
      sc[c] = v;
      m_tile = fmaxf(m_tile, v);
    }
    float factor = 1.f;
    bool need = false;
    if (m_used == -INFINITY) {
      // no visible key so far (first tile, or tiles in front of this row's window): the accumulator row is
      // still all zero, so the first finite maximum is adopted without a rescale
      m_used = m_tile;
    } else if (m_tile > m_used + kRescaleThreshold) {
      factor = exp2f(m_used - m_tile);
      m_used = m_tile;
      need = true;
    }
    if (__any_sync(0xffffffffu, need)) {
      // rescale this warp's 32 rows of O in tensor memory
      l_sum *= factor;
#pragma unroll 1
      for (int c = 0; c < kD; c += 32) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_o + lane_base + c, o);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
        tmem_st_32x32(tmem_o + lane_base + c, o);
      }
      tmem_st_wait();
    }
    float psum = 0.f;
    const float m_exp = (m_used == -INFINITY) ? 0.f : m_used;   // a row without a visible key yet: all p = 0
    {
      const uint32_t sp = smem_u32(sP);
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float p0 = fast_exp2(sc[ch * 8 + 2 * i] - m_exp);
          const float p1 = fast_exp2(sc[ch * 8 + 2 * i + 1] - m_exp);
          // sum what the tensor core will actually see (bf16-rounded probabilities)
          const uint32_t pk = p.out_f16 ? 0u : pack_bf16x2(p0, p1);
          if (p.out_f16) {
            __half2 h = __floats2half2_rn(p0, p1);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
            float2 f = __half22float2(h);
            psum += f.x + f.y;
          } else {
            w[i] = pk;
            float2 f = unpack_bf16x2(pk);
            psum += f.x + f.y;
          }
        }
        const uint32_t dst = sp + row * 128 + ((ch ^ (row & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                     : "memory");
      }
    }
    l_sum += psum;

    tc_fence_before_sync();
    fence_proxy_async_smem();
    __syncthreads();  // P written by all rows, O rescaled

    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t pa = smem_u32(sP);
      const uint32_t va = smem_u32(sV + buf * kSmemKVBuf);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint64_t a_desc = umma_desc_k_sw128(pa + kk * 32);
        const uint64_t b_desc = umma_desc_mn_sw128(va + kk * 2048, kHalfKV, 1024);
        umma_f16(tmem_o, a_desc, b_desc, p.idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
      }
      umma_commit(bar_o);
    }
  }

  if (!mbar_wait(bar_o, (n_tiles - 1) & 1)) ok_all = false;
  tc_fence_after_sync();
  if (!ok_all && p.status != nullptr) atomicExch(p.status, kStatusPipelineTimeout);

  // ---- epilogue -----------------------------------------------------------------------------
  const float inv_l = l_sum > 0.f ? 1.f / l_sum : 0.f;
  if (p.is_decode && p.num_splits > 1) {
    float* po = p.part_o + ((static_cast<int64_t>(b) * p.hq + row_head) * p.num_splits + split) * kD;
#pragma unroll 1
    for (int c = 0; c < kD; c += 32) {
      uint32_t o[32];
      tmem_ld_32x32(tmem_o + lane_base + c, o);
      tmem_ld_wait();
      if (row_valid && ok_all) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float4 v = make_float4(__uint_as_float(o[i]) * inv_l, __uint_as_float(o[i + 1]) * inv_l,
                                 __uint_as_float(o[i + 2]) * inv_l, __uint_as_float(o[i + 3]) * inv_l);
          *reinterpret_cast<float4*>(po + c + i) = v;
        }
      }
    }
    if (row_valid)
      p.part_lse[(static_cast<int64_t>(b) * p.hq + row_head) * p.num_splits + split] =
          l_sum > 0.f ? (m_used + log2f(l_sum)) : -INFINITY;
  } else {
    uint16_t* orow = static_cast<uint16_t*>(p.out) +
                     (static_cast<int64_t>(q_row0 + q0 + (row_valid ? row_tok : 0)) * p.hq + row_head) * kD;
#pragma unroll 1
    for (int c = 0; c < kD; c += 32) {
      uint32_t o[32];
      tmem_ld_32x32(tmem_o + lane_base + c, o);
      tmem_ld_wait();
      if (row_valid && ok_all) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 v;
          uint32_t* vv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
          for (int k2 = 0; k2 < 4; ++k2) {
            const float a = __uint_as_float(o[i + 2 * k2]) * inv_l;
            const float bb = __uint_as_float(o[i + 2 * k2 + 1]) * inv_l;
            if (p.out_f16) {
              __half2 h = __floats2half2_rn(a, bb);
              vv[k2] = *reinterpret_cast<uint32_t*>(&h);
            } else {
              vv[k2] = pack_bf16x2(a, bb);
            }
          }
          *reinterpret_cast<uint4*>(orow + c + i) = v;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}


template <int N>
__device__ __forceinline__ float m_used_at(const float (&m)[N], int idx) {
  float v = 0.f;
#pragma unroll
  for (int c = 0; c < N; ++c) v = (c == idx) ? m[c] : v;
  return v;
}

// ---------------------------------------------------------------------------------------------
// Decode-specialised kernel: one query token per request, so the roles of the MMA dimensions are
// swapped - the 128 KV tokens of a tile are the MMA M dimension and the (padded) query heads of
// the GQA group are the N dimension:
//   S^T[tok, q] = K[tok, d] Q^T          (A = K tile, K-major; B = Q, K-major)
//   O^T[d, q]  += V^T[d, tok] P^T[tok, q] (A = V tile as gathered, used MN-major; B = P^T, K-major)
// A softmax thread owns one token (only the per-head maximum crosses threads, once per tile; the
// row sums stay per-thread until the end) and one feature d of the output, so the final store is
// coalesced.  The CTA is warp-specialised and coupled by mbarriers only:
//   warps 0-3  softmax: tcgen05.ld S^T, running max, exponentials, P^T to shared memory
//   warp  4    producer: reads the request's slot table and moves K and V rows with the TMA engine into
//              two three-deep rings, in the 128-byte-swizzled operand layout.  Groups of 16 tokens whose
//              slots are consecutive (paged allocation, or a prompt that was given one run of slots) are
//              plain 2 KB boxes when the pool is stored head-major; other groups are gathered row by row
//              (cp.async.bulk.tensor ... tile::gather4: four pool rows, given by index, per copy).
//   warp  5    one thread issues the MMAs: S^T of tile t is queued before P*V of tile t-1, so the
//              tensor-core and barrier latency of S^T hides behind the softmax of the tile before
// ---------------------------------------------------------------------------------------------
constexpr int kDT = 128;                       // tokens per decode tile
constexpr int kDecHalf = kDT * 128;            // bytes of one 64-feature half of a K or V tile
constexpr int kDecTileBytes = 2 * kDecHalf;    // 32 KB per tensor
constexpr int kDecBufs = 3;
constexpr int kDecThreads = 192;

template <int NQ>
struct DecCfg {
  static constexpr int kQBytes = 2 * NQ * 128;   // Q^T operand: two halves of NQ rows x 128 B
  static constexpr int kPBytes = 2 * NQ * 128;   // P^T operand: two halves (64 tokens each)
  static constexpr int kSmem = kDecBufs * 2 * kDecTileBytes + kQBytes + kPBytes + 1024 + 256 + 9 * NQ * 4;
};

// Four rows of a 2-D tensor (row indices r[0..3], 64 16-bit columns starting at column x: one 128-byte
// swizzle span per row) to four consecutive 128-byte rows of shared memory.  The tensor map's box is
// {64, 1}; the copy signals 512 bytes on `bar`.  x * 2 bytes must be a multiple of 16.
__device__ __forceinline__ void tma_gather4(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x,
                                            const int (&r)[4]) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3])
      : "memory");
}

template <int NQ>
__global__ void __launch_bounds__(kDecThreads, 1)
attn_decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const __grid_constant__ CUtensorMap tm_k_run, const __grid_constant__ CUtensorMap tm_v_run,
                   const AttnParams p) {
  using C = DecCfg<NQ>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;                                   // kDecBufs tiles
  uint8_t* sV = sK + kDecBufs * kDecTileBytes;          // kDecBufs tiles
  uint8_t* sQ = sV + kDecBufs * kDecTileBytes;
  uint8_t* sP = sQ + C::kQBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + C::kPBytes);
  uint64_t* k_full = bars;            // [3] TMA transaction bytes
  uint64_t* k_empty = bars + 3;       // [3] tcgen05.commit
  uint64_t* v_full = bars + 6;        // [3]
  uint64_t* v_empty = bars + 9;       // [3]
  uint64_t* s_full = bars + 12;       // [2] tcgen05.commit
  uint64_t* s_empty = bars + 14;      // [2] 128 softmax threads
  uint64_t* p_full = bars + 16;       // 128 softmax threads
  uint64_t* p_empty = bars + 17;      // tcgen05.commit (P*V of the tile finished)
  uint64_t* q_full = bars + 18;       // producer warp: Q^T operand written
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 19);
  int* fail_flag = reinterpret_cast<int*>(tmem_holder + 1);
  float* red = reinterpret_cast<float*>(bars + 20);     // [2][4 warps][NQ] tile maxima, double buffered
  float* red2 = red + 8 * NQ;                           // [NQ] totals

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int b = blockIdx.z;
  const int hk = blockIdx.y;
  const int split = blockIdx.x;
  const int g = p.group;

  if (tid == 0) {
    for (int i = 0; i < 3; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 128);
    }
    mbar_init(p_full, 128);
    mbar_init(p_empty, 1);
    mbar_init(q_full, 1);
    *fail_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_k_run);
    tma_prefetch_desc(&tm_v_run);
  }
  // rows of P^T beyond the group are never written again: clear them once
  for (int i = tid; i < C::kPBytes / 16; i += kDecThreads) reinterpret_cast<uint4*>(sP)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  __syncthreads();
  if (warp == 5) {
    tmem_alloc(tmem_holder, 128);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_s = tmem_base;            // two buffers of NQ columns
  const uint32_t tmem_o = tmem_base + 2 * NQ;   // NQ columns
  // everything above touched no global memory; sequence lengths, slot table, Q and the KV pool are
  // written by earlier kernels of the stream
  pdl_wait();

  const int req = p.req_pool_indices[b];
  const int seq_len = p.seq_lens[b];
  const int kv_lo = p.window > 0 ? max(0, seq_len - p.window) : 0;   // first key the (single) query sees
  const int lo_tile = kv_lo / kDT * kDT;
  const int tiles = (seq_len - lo_tile + kDT - 1) / kDT;
  const int per = (tiles + p.num_splits - 1) / p.num_splits;
  const int kv_begin = lo_tile + split * per * kDT;
  const int kv_end = min(seq_len, kv_begin + per * kDT);
  const int n_tiles = kv_begin < kv_end ? (kv_end - kv_begin + kDT - 1) / kDT : 0;

  if (n_tiles == 0) {
    // nothing to attend to: a neutral partial for the merge, or an all-zero output row
    if (p.num_splits > 1) {
      for (int i = tid; i < g * kD; i += kDecThreads) {
        const int head = hk * g + i / kD;
        p.part_o[((static_cast<int64_t>(b) * p.hq + head) * p.num_splits + split) * kD + (i % kD)] = 0.f;
      }
      if (tid < g) p.part_lse[(static_cast<int64_t>(b) * p.hq + hk * g + tid) * p.num_splits + split] = -INFINITY;
    } else {
      for (int i = tid; i < g * kD; i += kDecThreads)
        static_cast<uint16_t*>(p.out)[(static_cast<int64_t>(b) * p.hq + hk * g) * kD + i] = 0;
    }
  } else if (warp == 4) {
    // =============================== producer warp ===============================
    const int* rtt = p.req_to_token + static_cast<int64_t>(req) * p.rtt_stride;
    bool ok_all = true, bad = false;
    // A lane owns four consecutive tokens of the tile; the four lanes of a quad own a group of 16.  When the
    // 16 slots of a group are consecutive and the storage is head-major, the group's K and V rows are four
    // plain 2 KB boxes (K low / high feature half, V low / high) and each lane of the quad issues one of them;
    // otherwise every lane gathers its own four rows, four at a time by index.
    const int grp = lane >> 2, sub = lane & 3;
    auto load_slots = [&](int tile, int (&sl4)[4]) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int tk = min(kv_begin + tile * kDT + grp * 16 + sub * 4 + j, kv_end - 1);
        sl4[j] = tile < n_tiles ? __ldg(rtt + tk) : 0;
      }
    };
    int cur[4], nxt[4];
    load_slots(0, cur);
    for (int t = 0; t < n_tiles && ok_all; ++t) {
      const int sl = t % kDecBufs;
      const uint32_t ph = (t / kDecBufs) & 1;
      load_slots(t + 1, nxt);   // used one tile from now
      bool run = p.kv_runs != 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (cur[j] < 0 || cur[j] >= p.num_slots) {
          bad = true;
          cur[j] = 0;
        }
      }
      const int first = __shfl_sync(0xffffffffu, cur[0], lane & ~3);   // slot of the group's first token
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int tk = kv_begin + t * kDT + grp * 16 + sub * 4 + j;
        // tokens past the end repeat the last slot and are masked: they do not break a run
        run = run && (tk >= kv_end || cur[j] == first + sub * 4 + j);
      }
      const uint32_t votes = __ballot_sync(0xffffffffu, run);
      run = ((votes >> (lane & ~3)) & 0xFu) == 0xFu && first + 16 <= p.num_slots;
      if (!mbar_wait(&k_empty[sl], ph ^ 1, fail_flag)) ok_all = false;
      if (!mbar_wait(&v_empty[sl], ph ^ 1, fail_flag)) ok_all = false;
      if (!__all_sync(0xffffffffu, ok_all)) {
        ok_all = false;
        break;
      }
      if (lane == 0) {
        mbar_arrive_expect_tx(&k_full[sl], kDecTileBytes);
        mbar_arrive_expect_tx(&v_full[sl], kDecTileBytes);
      }
      __syncwarp();
      uint8_t* tile_k = sK + sl * kDecTileBytes;
      uint8_t* tile_v = sV + sl * kDecTileBytes;
      if (run) {
        const int row0 = first * p.kv_row_mul + hk * p.kv_row_add;
        const int half = sub & 1;
        uint8_t* dst = (sub < 2 ? tile_k : tile_v) + half * kDecHalf + grp * 16 * 128;
        tma_load_2d(dst, sub < 2 ? &tm_k_run : &tm_v_run, sub < 2 ? &k_full[sl] : &v_full[sl], half * 64, row0);
      } else {
        int rows[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) rows[j] = cur[j] * p.kv_row_mul + hk * p.kv_row_add;
        const int off = (grp * 16 + sub * 4) * 128;
        tma_gather4(tile_k + off, &tm_k, &k_full[sl], 0, rows);
        tma_gather4(tile_k + kDecHalf + off, &tm_k, &k_full[sl], 64, rows);
        tma_gather4(tile_v + off, &tm_v, &v_full[sl], 0, rows);
        tma_gather4(tile_v + kDecHalf + off, &tm_v, &v_full[sl], 64, rows);
      }
      if (t == 0) {   // the first K and V tiles are on their way: stage the Q^T operand meanwhile
      {  // Q^T operand: NQ rows (query heads, zero beyond the group) x 16 chunks of 16 bytes
        const uint16_t* qbase = static_cast<const uint16_t*>(p.q);
        for (int c = lane; c < NQ * 16; c += 32) {
          const int r = c >> 4, qc = c & 15;
          uint4 v = make_uint4(0, 0, 0, 0);
          if (r < g)
            v = *reinterpret_cast<const uint4*>(qbase + static_cast<int64_t>(b) * p.q_stride +
                                                static_cast<int64_t>(hk * g + r) * kD + qc * 8);
          *reinterpret_cast<uint4*>(sQ + swz_off(r, qc, NQ * 128)) = v;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(q_full);
      }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) cur[j] = nxt[j];
    }
    if (bad && p.status != nullptr) atomicExch(p.status, kStatusBadIndex);
    if (!ok_all) *fail_flag = 1;
  } else if (warp == 5) {
    // =============================== MMA issuer ===============================
    if (lane == 0) {
      bool ok_all = mbar_wait(q_full, 0, fail_flag);
      auto issue_pv = [&](int u) {
        const int sl = u % kDecBufs;
        if (!mbar_wait(&v_full[sl], (u / kDecBufs) & 1, fail_flag)) ok_all = false;
        if (!mbar_wait(p_full, u & 1, fail_flag)) ok_all = false;
        if (!ok_all) return;
        tc_fence_after_sync();
        const uint32_t va = smem_u32(sV + sl * kDecTileBytes);
        const uint32_t pa = smem_u32(sP);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a_desc = umma_desc_mn_sw128(va + kk * 2048, kDecHalf, 1024);
          const uint64_t b_desc = umma_desc_k_sw128(pa + (kk >> 2) * (NQ * 128) + (kk & 3) * 32);
          umma_f16(tmem_o, a_desc, b_desc, p.idesc_o, (u > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[sl]);
        umma_commit(p_empty);
      };
      for (int t = 0; t < n_tiles && ok_all; ++t) {
        const int sl = t % kDecBufs;
        if (!mbar_wait(&k_full[sl], (t / kDecBufs) & 1, fail_flag)) ok_all = false;
        if (!mbar_wait(&s_empty[t & 1], ((t >> 1) & 1) ^ 1, fail_flag)) ok_all = false;
        if (!ok_all) break;
        tc_fence_after_sync();
        const uint32_t ka = smem_u32(sK + sl * kDecTileBytes);
        const uint32_t qa = smem_u32(sQ);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a_desc = umma_desc_k_sw128(ka + (kk >> 2) * kDecHalf + (kk & 3) * 32);
          const uint64_t b_desc = umma_desc_k_sw128(qa + (kk >> 2) * (NQ * 128) + (kk & 3) * 32);
          umma_f16(tmem_s + (t & 1) * NQ, a_desc, b_desc, p.idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[sl]);
        umma_commit(&s_full[t & 1]);
        if (t > 0) issue_pv(t - 1);
      }
      if (ok_all) issue_pv(n_tiles - 1);
      if (!ok_all) *fail_flag = 1;
    }
  } else {
    // =============================== softmax warps ===============================
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    float m_used[NQ];
    float l_part[NQ];
#pragma unroll
    for (int c = 0; c < NQ; ++c) {
      m_used[c] = 0.f;
      l_part[c] = 0.f;
    }
    bool ok_all = true;
    for (int t = 0; t < n_tiles; ++t) {
      if (!mbar_wait(&s_full[t & 1], (t >> 1) & 1, fail_flag)) {
        ok_all = false;
        break;
      }
      tc_fence_after_sync();
      float sc[NQ];
      {
        uint32_t raw[16];
#pragma unroll
        for (int c0 = 0; c0 < NQ; c0 += 16) {
          tmem_ld_32x16(tmem_s + (t & 1) * NQ + lane_base + c0, raw);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) sc[c0 + i] = __uint_as_float(raw[i]);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&s_empty[t & 1]);  // the S^T buffer may be overwritten by tile t+2
      const int tok_pos = kv_begin + t * kDT + tid;
      const bool tok_ok = tok_pos < kv_end && tok_pos >= kv_lo;
      float* redt = red + (t & 1) * 4 * NQ;
      if (p.logit_cap > 0.f) {   // uniform branch outside the loop: plain scores pay one multiply
#pragma unroll
        for (int c = 0; c < NQ; ++c) sc[c] = p.cap_post * tanhf(sc[c] * p.cap_pre);
      } else {
#pragma unroll
        for (int c = 0; c < NQ; ++c) sc[c] *= p.scale_log2;
      }
#pragma unroll
      for (int c = 0; c < NQ; ++c) {
        if (c < g) {
          sc[c] = tok_ok ? sc[c] : -INFINITY;
          const float wm = warp_max(sc[c]);
          if (lane == 0) redt[warp * NQ + c] = wm;
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      bool need = false;
      float factor[NQ];
#pragma unroll
      for (int c = 0; c < NQ; ++c) {
        factor[c] = 1.f;
        if (c < g) {
          const float mt = fmaxf(fmaxf(redt[c], redt[NQ + c]), fmaxf(redt[2 * NQ + c], redt[3 * NQ + c]));
          if (t == 0) {
            m_used[c] = mt;  // the first tile of a non-empty range always holds a visible token
          } else if (mt > m_used[c] + kRescaleThreshold) {
            factor[c] = fast_exp2(m_used[c] - mt);
            m_used[c] = mt;
            l_part[c] *= factor[c];
            need = true;
          }
        }
      }
      // P*V of the previous tile must be finished before P^T and O^T are touched again
      if (t > 0) {
        if (!mbar_wait(p_empty, (t - 1) & 1, fail_flag)) {
          ok_all = false;
          break;
        }
        tc_fence_after_sync();
      }
      if (need) {  // uniform over the four warps: every thread sees the same maxima
        uint32_t o[16];
#pragma unroll
        for (int c0 = 0; c0 < NQ; c0 += 16) {
          tmem_ld_32x16(tmem_o + lane_base + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor[c0 + i]);
          tmem_st_32x16(tmem_o + lane_base + c0, o);
        }
        tmem_st_wait();
      }
      // P^T operand: row = query head, 128 tokens in two 64-token halves; this thread writes column tid
      {
        uint8_t* pbase = sP + (tid >> 6) * (NQ * 128);
        const int tk = tid & 63;
#pragma unroll
        for (int c = 0; c < NQ; ++c) {
          if (c < g) {
            const float pv = fast_exp2(sc[c] - m_used[c]);
            uint16_t bits;
            float back;
            if (p.out_f16) {
              const __half ph = __float2half_rn(pv);
              bits = *reinterpret_cast<const uint16_t*>(&ph);
              back = __half2float(ph);
            } else {
              const __nv_bfloat16 pb = __float2bfloat16_rn(pv);
              bits = *reinterpret_cast<const uint16_t*>(&pb);
              back = __bfloat162float(pb);
            }
            l_part[c] += back;
            *reinterpret_cast<uint16_t*>(pbase + c * 128 + (((tk >> 3) ^ (c & 7)) << 4) + (tk & 7) * 2) = bits;
          }
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(p_full);
    }
    if (ok_all && !mbar_wait(p_empty, (n_tiles - 1) & 1, fail_flag)) ok_all = false;
    tc_fence_after_sync();
    if (!ok_all) *fail_flag = 1;

    // ---- totals of the row sums over the 128 token-threads ----
    float* redt = red;
#pragma unroll
    for (int c = 0; c < NQ; ++c) {
      if (c < g) {
        const float ws = warp_sum(l_part[c]);
        if (lane == 0) redt[warp * NQ + c] = ws;
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (tid < g) red2[tid] = redt[tid] + redt[NQ + tid] + redt[2 * NQ + tid] + redt[3 * NQ + tid];
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const bool good = ok_all && (*fail_flag == 0);

    // ---- output: this thread owns feature d = tid of every head of the group ----
    uint32_t o[16];
#pragma unroll
    for (int c0 = 0; c0 < NQ; c0 += 16) {
      tmem_ld_32x16(tmem_o + lane_base + c0, o);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int c = c0 + i;
        if (c < g && good) {
          const float l = red2[c];
          const float v = l > 0.f ? __uint_as_float(o[i]) / l : 0.f;
          const int head = hk * g + c;
          if (p.num_splits > 1) {
            p.part_o[((static_cast<int64_t>(b) * p.hq + head) * p.num_splits + split) * kD + tid] = v;
          } else {
            const int64_t oi = (static_cast<int64_t>(b) * p.hq + head) * kD + tid;
            if (p.out_f16)
              static_cast<__half*>(p.out)[oi] = __float2half_rn(v);
            else
              static_cast<__nv_bfloat16*>(p.out)[oi] = __float2bfloat16_rn(v);
          }
        }
      }
    }
    if (p.num_splits > 1 && tid < g) {
      const float l = red2[tid];
      p.part_lse[(static_cast<int64_t>(b) * p.hq + hk * g + tid) * p.num_splits + split] =
          l > 0.f ? (m_used_at(m_used, tid) + log2f(l)) : -INFINITY;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*fail_flag) {
    if (tid == 0 && p.status != nullptr) atomicExch(p.status, kStatusPipelineTimeout);
    // copies of the producer may still be in flight: give them time to land before the CTA's memory is reused
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 128);
  }
}

// ---------------------------------------------------------------------------------------------
// Prefill kernel, warp-specialised.  A CTA owns one request, one KV head and TWO tiles of 128 rows (a row is a
// (query token, query head of the GQA group) pair, as above), so every K/V tile that reaches shared memory
// serves both; KV tiles hold 128 tokens.  The CTA's roles meet only at mbarriers:
//   warps 0-3  softmax of row tile A      warps 4-7  softmax of row tile B
//   warp  8    producer: the decode kernel's TMA path (2 KB boxes over runs of 16 consecutive slots, else
//              gather4 by row index) into a two-slot K ring and a single V slot
//   warp  9    one thread issues the MMAs.  Tensor memory holds S_A, S_B (128 columns each) and O_A, O_B.
// A softmax thread pulls its whole S row (128 scores) into registers with four tcgen05.ld and releases the S
// buffer at once, so the scores of tile t+1 are computed while the exponentials of tile t are; P*V of tile t
// runs under the softmax of tile t+1.  K is fetched two tiles ahead, V one.  The running maximum and the row
// sum are kept in several independent chains (a single chain of 128 dependent operations would cost more than
// the exponentials).  Tiles that need no causal / window mask and no soft cap take one FMA and one exponential
// per score.
// ---------------------------------------------------------------------------------------------
constexpr int kPfThreads = 320;
constexpr int kPfTile = 128;                    // KV tokens per tile
constexpr int kPfHalf = 128 * 128;              // 16 KB: 128 rows of one 128-byte swizzle span
constexpr int kPfTileBytes = 2 * kPfHalf;       // 32 KB: a Q tile, a K or V tile, or one group's P tile
constexpr int kPfSmem = (2 + 2 + 3) * kPfTileBytes + 1024 + 256;

__global__ void __launch_bounds__(kPfThreads, 1)
attn_prefill_ws_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                       const __grid_constant__ CUtensorMap tm_k_run, const __grid_constant__ CUtensorMap tm_v_run,
                       const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                             // two row tiles
  uint8_t* sP = sQ + 2 * kPfTileBytes;            // two row tiles of probabilities
  uint8_t* sK = sP + 2 * kPfTileBytes;            // two K tiles
  uint8_t* sV = sK + 2 * kPfTileBytes;            // one V tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kPfTileBytes);
  uint64_t* k_full = bars;             // [2] TMA transaction bytes
  uint64_t* k_empty = bars + 2;        // [2] tcgen05.commit
  uint64_t* v_full = bars + 4;         // TMA transaction bytes
  uint64_t* v_empty = bars + 5;        // tcgen05.commit
  uint64_t* s_full = bars + 6;         // [2] tcgen05.commit: scores of a group are in tensor memory
  uint64_t* s_free = bars + 8;         // [2] 128 threads: the group holds its scores in registers
  uint64_t* p_full = bars + 10;        // [2] 128 threads: the group has written P (and rescaled O)
  uint64_t* o_done = bars + 12;        // [2] tcgen05.commit: the group's P*V has finished
  uint64_t* q_full = bars + 14;        // 256 threads: both Q tiles are in shared memory
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 15);
  int* fail_flag = reinterpret_cast<int*>(tmem_holder + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int b = blockIdx.z;
  const int hk = blockIdx.y;
  const int g = p.group;
  const int tpt = p.tokens_per_tile;             // query tokens per row tile
  pdl_wait();

  const int req = p.req_pool_indices[b];
  const int seq_len = p.seq_lens[b];
  const int prefix = p.prefix_lens[b];
  const int q_len = seq_len - prefix;
  const int q0 = (static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x)) * 2 * tpt;   // long rows first
  if (q0 >= q_len) return;
  const int q_row0 = p.q_start[b];
  const int kv_begin = (p.window > 0 && !p.non_causal) ? max(0, prefix + q0 - p.window + 1) / kPfTile * kPfTile : 0;
  const int kv_end = p.non_causal ? seq_len : min(seq_len, prefix + min(q_len, q0 + 2 * tpt));
  const int n_tiles = (kv_end - kv_begin + kPfTile - 1) / kPfTile;   // >= 1: the tile's first row sees itself

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 128);
      mbar_init(&p_full[i], 128);
      mbar_init(&o_done[i], 1);
    }
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(q_full, 256);
    *fail_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_k_run);
    tma_prefetch_desc(&tm_v_run);
  }
  __syncthreads();
  if (warp == 9) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 8) {
    // =============================== producer warp ===============================
    // Order of the copies: K0, K1, V0, K2, V1, K3, V2, ...  (K two tiles ahead of the tile being multiplied, V one)
    const int* rtt = p.req_to_token + static_cast<int64_t>(req) * p.rtt_stride;
    bool ok_all = true, bad = false;
    // lane = four consecutive tokens; a quad = 16 tokens, one 2 KB box per 64-feature half when their slots
    // are consecutive
    const int grp = lane >> 2, sub = lane & 3;
    auto load_tile = [&](int t, bool is_v) {
      int cur[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int tk = min(kv_begin + t * kPfTile + grp * 16 + sub * 4 + j, kv_end - 1);
        cur[j] = __ldg(rtt + tk);
        if (cur[j] < 0 || cur[j] >= p.num_slots) {
          bad = true;
          cur[j] = 0;
        }
      }
      bool run = p.kv_runs != 0;
      const int first = __shfl_sync(0xffffffffu, cur[0], lane & ~3);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int tk = kv_begin + t * kPfTile + grp * 16 + sub * 4 + j;
        run = run && (tk >= kv_end || cur[j] == first + sub * 4 + j);   // tokens past the end are masked
      }
      const uint32_t votes = __ballot_sync(0xffffffffu, run);
      run = ((votes >> (lane & ~3)) & 0xFu) == 0xFu && first + 16 <= p.num_slots;
      uint64_t* full = is_v ? v_full : &k_full[t & 1];
      uint64_t* empty = is_v ? v_empty : &k_empty[t & 1];
      const uint32_t ph = is_v ? (t & 1) : ((t >> 1) & 1);
      if (!mbar_wait(empty, ph ^ 1, fail_flag)) ok_all = false;
      if (!__all_sync(0xffffffffu, ok_all)) {
        ok_all = false;
        return;
      }
      if (lane == 0) mbar_arrive_expect_tx(full, kPfTileBytes);
      __syncwarp();
      uint8_t* tile = is_v ? sV : sK + (t & 1) * kPfTileBytes;
      if (run) {
        const int row0 = first * p.kv_row_mul + hk * p.kv_row_add;
        if (sub < 2)
          tma_load_2d(tile + sub * kPfHalf + grp * 16 * 128, is_v ? &tm_v_run : &tm_k_run, full, sub * 64, row0);
      } else {
        int rows[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) rows[j] = cur[j] * p.kv_row_mul + hk * p.kv_row_add;
        const int off = (grp * 16 + sub * 4) * 128;
        tma_gather4(tile + off, is_v ? &tm_v : &tm_k, full, 0, rows);
        tma_gather4(tile + kPfHalf + off, is_v ? &tm_v : &tm_k, full, 64, rows);
      }
    };
    load_tile(0, false);
    if (ok_all && n_tiles > 1) load_tile(1, false);
    for (int t = 0; t < n_tiles && ok_all; ++t) {
      load_tile(t, true);
      if (ok_all && t + 2 < n_tiles) load_tile(t + 2, false);
    }
    if (bad && p.status != nullptr) atomicExch(p.status, kStatusBadIndex);
    if (!ok_all) *fail_flag = 1;
  } else if (warp == 9) {
    // =============================== MMA issuer ===============================
    if (lane == 0) {
      bool ok_all = mbar_wait(q_full, 0, fail_flag);
      auto wait_on = [&](uint64_t* bar, uint32_t parity) {
        if (ok_all && !mbar_wait(bar, parity, fail_flag)) ok_all = false;
        if (ok_all) tc_fence_after_sync();
      };
      auto issue_s = [&](int grp_i, int t) {        // S = Q K^T of group grp_i and KV tile t
        const uint32_t qa = smem_u32(sQ + grp_i * kPfTileBytes);
        const uint32_t ka = smem_u32(sK + (t & 1) * kPfTileBytes);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a_desc = umma_desc_k_sw128(qa + (kk >> 2) * kPfHalf + (kk & 3) * 32);
          const uint64_t b_desc = umma_desc_k_sw128(ka + (kk >> 2) * kPfHalf + (kk & 3) * 32);
          umma_f16(tmem_base + grp_i * 128, a_desc, b_desc, p.idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[grp_i]);
      };
      auto issue_pv = [&](int grp_i, int t) {       // O += P V
        const uint32_t pa = smem_u32(sP + grp_i * kPfTileBytes);
        const uint32_t va = smem_u32(sV);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a_desc = umma_desc_k_sw128(pa + (kk >> 2) * kPfHalf + (kk & 3) * 32);
          const uint64_t b_desc = umma_desc_mn_sw128(va + kk * 2048, kPfHalf, 1024);
          umma_f16(tmem_base + 256 + grp_i * 128, a_desc, b_desc, p.idesc_o, (t > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&o_done[grp_i]);
      };
      wait_on(&k_full[0], 0);
      if (ok_all) {
        issue_s(0, 0);
        issue_s(1, 0);
        umma_commit(&k_empty[0]);
      }
      for (int t = 0; t < n_tiles && ok_all; ++t) {
        if (t + 1 < n_tiles) {
          // scores of the next tile, as soon as the groups hold the current ones in registers
          wait_on(&k_full[(t + 1) & 1], ((t + 1) >> 1) & 1);
          wait_on(&s_free[0], t & 1);
          if (ok_all) issue_s(0, t + 1);
          wait_on(&s_free[1], t & 1);
          if (ok_all) {
            issue_s(1, t + 1);
            umma_commit(&k_empty[(t + 1) & 1]);
          }
        }
        wait_on(v_full, t & 1);
        wait_on(&p_full[0], t & 1);
        if (ok_all) issue_pv(0, t);
        wait_on(&p_full[1], t & 1);
        if (ok_all) {
          issue_pv(1, t);
          umma_commit(v_empty);
        }
      }
      if (!ok_all) *fail_flag = 1;
    }
  } else {
    // =============================== softmax groups ===============================
    const int grp_i = warp >> 2;                    // 0 = row tile A, 1 = row tile B
    const int row = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem_base + grp_i * 128 + lane_base;
    const uint32_t tmem_o = tmem_base + 256 + grp_i * 128 + lane_base;
    const int tile_q0 = q0 + grp_i * tpt;           // first query token of this group's row tile
    const int row_tok = row / g;
    const int row_head = hk * g + row % g;
    const bool row_valid = (row_tok < tpt) && (tile_q0 + row_tok < q_len);
    const int kv_limit = p.non_causal ? seq_len - 1 : (row_valid ? prefix + tile_q0 + row_tok : prefix + q0);

    // ---- Q tile of this group: 128 rows x 256 B ----
    {
      const uint16_t* qbase = static_cast<const uint16_t*>(p.q);
      const uint32_t sq = smem_u32(sQ + grp_i * kPfTileBytes);
      for (int c = row; c < kRows * 16; c += 128) {
        const int r = c >> 4, ch = c & 15;
        const int tok = r / g;
        const bool ok = (tok < tpt) && (tile_q0 + tok < q_len);
        const int head = hk * g + r % g;
        const uint16_t* src = qbase + static_cast<int64_t>(q_row0 + (ok ? tile_q0 + tok : 0)) * p.q_stride +
                              static_cast<int64_t>(head) * kD + ch * 8;
        cp_async16(sq + swz_off(r, ch, kPfHalf), src, ok);
      }
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async_smem();
      mbar_arrive(q_full);
    }

    float m_used = -INFINITY;   // running maximum in use for the exponent (log2 domain)
    float l_sum = 0.f;
    bool ok_all = true;
    const uint32_t sp = smem_u32(sP + grp_i * kPfTileBytes) + row * 128;
    const bool plain_scores = p.logit_cap <= 0.f;

    for (int t = 0; t < n_tiles; ++t) {
      if (!mbar_wait(&s_full[grp_i], t & 1, fail_flag)) {
        ok_all = false;
        break;
      }
      tc_fence_after_sync();
      uint32_t raw[kPfTile];
#pragma unroll
      for (int c0 = 0; c0 < kPfTile; c0 += 32)
        tmem_ld_32x32(tmem_s + c0, *reinterpret_cast<uint32_t(*)[32]>(&raw[c0]));
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(&s_free[grp_i]);   // the scores of the next tile may overwrite the buffer

      const int col0 = kv_begin + t * kPfTile;
      const int visible = min(kv_limit, kv_end - 1) - col0;      // columns 0..visible are allowed
      const int first_vis = (p.window > 0 && !p.non_causal) ? kv_limit - p.window + 1 - col0 : -(1 << 30);
      const bool fast = __all_sync(0xffffffffu, plain_scores && visible >= kPfTile - 1 && first_vis <= 0);
      float mul = p.scale_log2;
      if (!fast) {
        // masked / capped tile: turn the raw products into final scores in place
        if (plain_scores) {
#pragma unroll
          for (int c = 0; c < kPfTile; ++c) raw[c] = __float_as_uint(__uint_as_float(raw[c]) * p.scale_log2);
        } else {
#pragma unroll   // full: a partly unrolled loop would index raw[] dynamically and push it out of the registers
          for (int c = 0; c < kPfTile; ++c)
            raw[c] = __float_as_uint(p.cap_post * tanh_approx(__uint_as_float(raw[c]) * p.cap_pre));
        }
#pragma unroll
        for (int c = 0; c < kPfTile; ++c)
          raw[c] = (c <= visible && c >= first_vis) ? raw[c] : __float_as_uint(-INFINITY);
        mul = 1.f;
      }
      float mx[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx[i] = __uint_as_float(raw[i]);
#pragma unroll
      for (int c = 8; c < kPfTile; c += 8) {
#pragma unroll
        for (int i = 0; i < 8; ++i) mx[i] = fmaxf(mx[i], __uint_as_float(raw[c + i]));
      }
      const float m_tile = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])),
                                 fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7]))) * mul;   // mul > 0
      float factor = 1.f;
      bool need = false;
      if (m_used == -INFINITY) {
        m_used = m_tile;   // no visible key so far: the accumulator row is all zero, adopt without a rescale
      } else if (m_tile > m_used + kRescaleThreshold) {
        factor = exp2f(m_used - m_tile);
        m_used = m_tile;
        need = true;
      }
      const float m_exp = (m_used == -INFINITY) ? 0.f : m_used;
      // The group's previous P*V must have finished before P is overwritten and O is rescaled.  It was queued a
      // whole softmax ago, so this wait is short; taking it here lets the exponentials go to shared memory as
      // they are computed instead of waiting in 64 registers.
      if (t > 0) {
        if (!mbar_wait(&o_done[grp_i], (t - 1) & 1, fail_flag)) {
          ok_all = false;
          break;
        }
        tc_fence_after_sync();
      }
      if (__any_sync(0xffffffffu, need)) {
        l_sum *= factor;
#pragma unroll 1
        for (int c = 0; c < kD; c += 32) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_o + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
          tmem_st_32x32(tmem_o + c, o);
        }
        tmem_st_wait();
      }
      // exponentials -> P in the operand layout: two 64-token halves of 128-byte rows, 16-byte chunks swizzled
      // by the row
      float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int q16 = 0; q16 < 16; ++q16) {
        uint32_t w4[4];
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const int i = q16 * 4 + k4;
          const float p0 = fast_exp2(fmaf(__uint_as_float(raw[2 * i]), mul, -m_exp));
          const float p1 = fast_exp2(fmaf(__uint_as_float(raw[2 * i + 1]), mul, -m_exp));
          ps[k4] += p0 + p1;
          if (p.out_f16) {
            __half2 h = __floats2half2_rn(p0, p1);
            w4[k4] = *reinterpret_cast<uint32_t*>(&h);
          } else {
            w4[k4] = pack_bf16x2(p0, p1);
          }
        }
        const uint32_t dst = sp + (q16 >> 3) * kPfHalf + (((q16 & 7) ^ (row & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w4[0]), "r"(w4[1]), "r"(w4[2]), "r"(w4[3])
                     : "memory");
      }
      l_sum += (ps[0] + ps[1]) + (ps[2] + ps[3]);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&p_full[grp_i]);
    }
    if (ok_all && !mbar_wait(&o_done[grp_i], (n_tiles - 1) & 1, fail_flag)) ok_all = false;
    tc_fence_after_sync();
    if (!ok_all) *fail_flag = 1;

    // ---- epilogue: normalise, park the group's 128 rows x 256 B in its P buffer (free now), then store them
    // row by row: 16 lanes cover one output row, and the g rows of a token are adjacent in memory ----
    const float inv_l = l_sum > 0.f ? 1.f / l_sum : 0.f;
#pragma unroll 1
    for (int c = 0; c < kD; c += 32) {
      uint32_t o[32];
      tmem_ld_32x32(tmem_o + c, o);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint32_t vv[4];
#pragma unroll
        for (int k2 = 0; k2 < 4; ++k2) {
          const float a = __uint_as_float(o[i + 2 * k2]) * inv_l;
          const float bb = __uint_as_float(o[i + 2 * k2 + 1]) * inv_l;
          if (p.out_f16) {
            __half2 h = __floats2half2_rn(a, bb);
            vv[k2] = *reinterpret_cast<uint32_t*>(&h);
          } else {
            vv[k2] = pack_bf16x2(a, bb);
          }
        }
        const int chunk = (c + i) >> 3;   // 16-byte chunk of the 256-byte row
        const uint32_t dst = smem_u32(sP + grp_i * kPfTileBytes) + row * 256 + ((chunk ^ (row & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(vv[0]), "r"(vv[1]), "r"(vv[2]), "r"(vv[3])
                     : "memory");
      }
    }
    if (grp_i == 0)
      asm volatile("bar.sync 1, 128;" ::: "memory");
    else
      asm volatile("bar.sync 2, 128;" ::: "memory");
    if (ok_all) {
      const int w4 = warp & 3;
      const int chunk = lane & 15;
#pragma unroll 4
      for (int it = 0; it < 16; ++it) {
        const int r = it * 8 + w4 * 2 + (lane >> 4);
        const int tok = r / g;
        if (tok < tpt && tile_q0 + tok < q_len) {
          const uint4 v = *reinterpret_cast<const uint4*>(sP + grp_i * kPfTileBytes + r * 256 + ((chunk ^ (r & 7)) << 4));
          uint16_t* dst = static_cast<uint16_t*>(p.out) +
                          (static_cast<int64_t>(q_row0 + tile_q0 + tok) * p.hq + hk * g + r % g) * kD + chunk * 8;
          *reinterpret_cast<uint4*>(dst) = v;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*fail_flag) {
    if (tid == 0 && p.status != nullptr) atomicExch(p.status, kStatusPipelineTimeout);
    // copies of the producer may still be in flight: give them time to land before the CTA's memory is reused
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// combine decode partials: out[b, h, :] = sum_s w_s * O_s with w_s = 2^(lse_s - max) / sum
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                  void* __restrict__ out, int hq, int splits, int out_f16) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y, h = blockIdx.x, d = threadIdx.x;
  const int hd = blockDim.x;                       // one thread per feature of the head
  const int64_t base = (static_cast<int64_t>(b) * hq + h) * splits;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_lse[base + s]);
  float den = 0.f, acc = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float l = part_lse[base + s];
    const float w = (l == -INFINITY) ? 0.f : exp2f(l - m);
    den += w;
    acc += w * part_o[(base + s) * hd + d];
  }
  const float v = den > 0.f ? acc / den : 0.f;
  const int64_t o = (static_cast<int64_t>(b) * hq + h) * hd + d;
  if (out_f16)
    static_cast<__half*>(out)[o] = __float2half_rn(v);
  else
    static_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(v);
}

template <int NH, bool KV8>
int launch_fwd_one(const AttnParams& p, dim3 grid, cudaStream_t s) {
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(attn_fwd_kernel<NH, KV8>), FwdCfg<NH>::kSmem) != cudaSuccess) return -3;
  const cudaError_t err = launch_pdl(attn_fwd_kernel<NH, KV8>, grid, dim3(kAttnThreads), FwdCfg<NH>::kSmem, s, p);
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}
template <int NH>
int launch_fwd_cfg(const AttnParams& p, dim3 grid, cudaStream_t s) {
  return p.kv_fmt != 0 ? launch_fwd_one<NH, true>(p, grid, s) : launch_fwd_one<NH, false>(p, grid, s);
}

}  // namespace

int decode_num_splits(int batch, int hkv, int max_seq_len, int num_sms) {
  const int ctas = std::max(1, batch * hkv);
  // one resident CTA per SM: fill a single wave, never start a second one for a remainder
  const int tiles = std::max(1, (max_seq_len + kDT - 1) / kDT);
  int splits = num_sms / ctas;
  splits = std::min(splits, std::max(1, tiles / 2));
  return std::max(1, std::min(splits, 64));
}

// Prefill through the warp-specialised kernel; returns 1 when this launch is not for it (storage that is neither
// head-major nor slot-major, or MLLM_B200_ATTN_PREFILL=legacy) and the single-role kernel should run instead.
int launch_prefill_ws(AttnParams p, const AttnArgs& a, cudaStream_t s) {
  const char* knob = std::getenv("MLLM_B200_ATTN_PREFILL");   // read per call: tests switch it
  const bool legacy = knob != nullptr && std::string(knob) == "legacy";
  if (legacy || p.kv_row_mul == 0) return 1;
  const int64_t rows = a.num_slots * static_cast<int64_t>(a.hkv);
  if (rows >= (int64_t(1) << 31)) return 1;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(attn_prefill_ws_kernel), kPfSmem) != cudaSuccess) return -3;
  CUtensorMap tm_k, tm_v, tm_k_run, tm_v_run;
  const int type = a.dt == kF16 ? 1 : 0;
  if (!make_tma_operand_map(&tm_k, a.k_cache, rows, kD, kD, 2, type, 1)) return -2;
  if (!make_tma_operand_map(&tm_v, a.v_cache, rows, kD, kD, 2, type, 1)) return -2;
  if (!make_tma_operand_map(&tm_k_run, a.k_cache, rows, kD, kD, 2, type, 16)) return -2;
  if (!make_tma_operand_map(&tm_v_run, a.v_cache, rows, kD, kD, 2, type, 16)) return -2;
  const uint32_t fmt = a.dt == kF16 ? 0u : 1u;
  p.idesc_s = umma_idesc(kRows, kPfTile, 1, fmt, fmt, 0, 0);
  p.idesc_o = umma_idesc(kRows, kD, 1, fmt, fmt, 0, 1);
  const int q_tiles = (a.max_q_len + 2 * p.tokens_per_tile - 1) / (2 * p.tokens_per_tile);
  if (q_tiles <= 0) return 0;
  const cudaError_t err = launch_pdl(attn_prefill_ws_kernel, dim3(q_tiles, a.hkv, a.batch), dim3(kPfThreads), kPfSmem, s,
                                     tm_k, tm_v, tm_k_run, tm_v_run, p);
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}

template <int NQ>
int launch_decode_cfg(const AttnParams& p, const AttnArgs& a, dim3 grid, cudaStream_t s) {
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(attn_decode_kernel<NQ>), DecCfg<NQ>::kSmem) != cudaSuccess)
    return -3;
  // the K and V pools as 2-D tensors [slots * kv heads, 128] with one 64-column row per box: the form
  // the gather copies take
  CUtensorMap tm_k, tm_v, tm_k_run, tm_v_run;
  const int type = a.dt == kF16 ? 1 : 0;
  const int64_t rows = a.num_slots * static_cast<int64_t>(a.hkv);
  if (rows >= (int64_t(1) << 31)) return -1;
  if (!make_tma_operand_map(&tm_k, a.k_cache, rows, kD, kD, 2, type, 1)) return -2;
  if (!make_tma_operand_map(&tm_v, a.v_cache, rows, kD, kD, 2, type, 1)) return -2;
  if (!make_tma_operand_map(&tm_k_run, a.k_cache, rows, kD, kD, 2, type, 16)) return -2;
  if (!make_tma_operand_map(&tm_v_run, a.v_cache, rows, kD, kD, 2, type, 16)) return -2;
  const cudaError_t err = launch_pdl(attn_decode_kernel<NQ>, grid, dim3(kDecThreads), DecCfg<NQ>::kSmem, s, tm_k, tm_v,
                                     tm_k_run, tm_v_run, p);
  note_launch();
  return err == cudaSuccess ? 0 : -4;
}

int launch_attention(const AttnArgs& a, cudaStream_t s) {
  // head size 128 has the specialised prefill and decode kernels; 64 and 256 run on the single-role kernel
  const int hd = a.head_dim;
  if ((hd != 64 && hd != 128 && hd != 256) || a.hq % a.hkv != 0) return -1;
  // the specialised kernels move K and V with the TMA engine as they are stored: a cache of the activation dtype
  const bool specialised = hd == kD && a.kv_fmt == 0;
  const int g = a.hq / a.hkv;
  if (g > kRows) return -1;
  AttnParams p{};
  p.q = a.q;
  p.k_cache = a.k_cache;
  p.v_cache = a.v_cache;
  p.out = a.out;
  p.part_o = a.part_o;
  p.part_lse = a.part_lse;
  p.req_to_token = a.req_to_token;
  p.req_pool_indices = a.req_pool_indices;
  p.seq_lens = a.seq_lens;
  p.prefix_lens = a.prefix_lens;
  p.non_causal = a.non_causal;
  p.q_start = a.q_start;
  p.status = a.status;
  p.q_stride = a.q_stride;
  p.rtt_stride = a.rtt_stride;
  p.num_slots = a.num_slots;
  p.kv_tok_stride = a.kv_tok_stride;
  p.kv_head_stride = a.kv_head_stride;
  if (a.kv_tok_stride == static_cast<int64_t>(a.hkv) * hd && a.kv_head_stride == hd) {
    p.kv_row_mul = a.hkv;        // slot-major: rows of one slot are adjacent
    p.kv_row_add = 1;
    p.kv_runs = a.hkv == 1 ? 1 : 0;
  } else if (a.kv_tok_stride == hd && a.kv_head_stride == a.num_slots * hd) {
    p.kv_row_mul = 1;            // head-major: consecutive slots of a head are consecutive rows
    p.kv_row_add = static_cast<int>(a.num_slots);
    p.kv_runs = 1;
  } else if (a.is_decode && specialised && g <= 32) {
    return -1;                   // the decode kernel reads the caches through 2-D tensor maps
  }
  p.hq = a.hq;
  p.hkv = a.hkv;
  p.group = g;
  p.tokens_per_tile = a.is_decode ? 1 : kRows / g;
  p.num_splits = a.is_decode ? a.num_splits : 1;
  p.is_decode = a.is_decode;
  p.out_f16 = a.dt == kF16 ? 1 : 0;
  p.scale_log2 = a.scale * kLog2e;
  p.scale = a.scale;
  p.window = a.window > 0 ? a.window : 0;
  p.logit_cap = a.logit_cap > 0.f ? a.logit_cap : 0.f;
  p.cap_pre = p.logit_cap > 0.f ? a.scale / p.logit_cap : 0.f;
  p.cap_post = p.logit_cap * kLog2e;
  p.kv_fmt = a.kv_fmt;
  const uint32_t fmt = a.dt == kF16 ? 0u : 1u;
  p.idesc_s = umma_idesc(kRows, kKV, 1, fmt, fmt, 0, 0);
  p.idesc_o = umma_idesc(kRows, hd, 1, fmt, fmt, 0, 1);
  if (a.batch <= 0) return 0;
  dim3 grid;
  if (specialised && a.is_decode && g <= 32) {
    const int nq = g <= 16 ? 16 : 32;
    p.idesc_s = umma_idesc(kRows, nq, 1, fmt, fmt, 0, 0);
    p.idesc_o = umma_idesc(kRows, nq, 1, fmt, fmt, 1, 0);
    grid = dim3(p.num_splits, a.hkv, a.batch);
    const int rc = nq == 16 ? launch_decode_cfg<16>(p, a, grid, s) : launch_decode_cfg<32>(p, a, grid, s);
    if (rc != 0) return rc;
    if (p.num_splits > 1) {
      launch_pdl(attn_merge_kernel, dim3(a.hq, a.batch), dim3(kD), 0, s, a.part_o, a.part_lse, a.out, a.hq, p.num_splits, p.out_f16);
      note_launch();
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  if (specialised && !a.is_decode) {
    const int rc = launch_prefill_ws(p, a, s);
    if (rc <= 0) return rc;
  }
  if (a.is_decode) {
    grid = dim3(p.num_splits, a.hkv, a.batch);
  } else {
    const int q_tiles = (a.max_q_len + p.tokens_per_tile - 1) / p.tokens_per_tile;
    if (q_tiles <= 0) return 0;
    grid = dim3(q_tiles, a.hkv, a.batch);
  }
  const int rc = hd == 64 ? launch_fwd_cfg<1>(p, grid, s) : hd == 128 ? launch_fwd_cfg<2>(p, grid, s) : launch_fwd_cfg<4>(p, grid, s);
  if (rc != 0) return rc;
  if (a.is_decode && p.num_splits > 1) {
    launch_pdl(attn_merge_kernel, dim3(a.hq, a.batch), dim3(hd), 0, s, a.part_o, a.part_lse, a.out, a.hq, p.num_splits, p.out_f16);
    note_launch();
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace mb200
