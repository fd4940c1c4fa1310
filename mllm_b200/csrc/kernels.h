// Host-callable launchers of the sm_100a kernels (plain C++ signatures: raw
// device pointers + a stream, no framework types). The PyTorch binding in
// bindings.cpp validates tensors and forwards here; other hosts can link the
// same symbols.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mb200 {

enum DType : int { kBF16 = 0, kF16 = 1, kF32 = 2 };

// Number of kernel launches issued through these launchers since load.
uint64_t launch_count();
void note_launch(int n = 1);

// ----- element-wise / normalisation --------------------------------------------------
void launch_rmsnorm(const void* x, const void* w, void* out, int rows, int hidden, int64_t x_stride,
                    int64_t out_stride, float eps, DType dt, cudaStream_t s);
void launch_fused_add_rmsnorm(void* x, void* residual, const void* w, int rows, int hidden, float eps, DType dt,
                              cudaStream_t s);
void launch_layernorm(const void* x, const void* w, const void* b, void* out, int rows, int hidden, float eps,
                      DType dt, cudaStream_t s);
// act: 0 = silu(gate)*up, 1 = gelu_tanh(gate)*up ; x is [rows, 2*inter] = [gate | up]
void launch_act_and_mul(const void* x, void* out, int rows, int inter, int act, DType dt, cudaStream_t s);
void launch_gelu_tanh(const void* x, void* out, int64_t n, DType dt, cudaStream_t s);
void launch_embedding(const int64_t* ids, const void* table, void* out, int tokens, int hidden, int vocab,
                      DType dt, int* status, cudaStream_t s);

// Per-head RMSNorm of q and k (weights may be null), NeoX rotary embedding and the
// write of K (normed, rotated) and V into the slot-indexed cache; q and k are updated
// in place inside the fused qkv activation. head_dim is 128.  kv_fmt 1 / 2: the caches hold unscaled e4m3 / e5m2
// bytes and K and V are rounded to that format on the way in.
// positions: [pos_rows, tokens] int64 with pos_rows 1 (plain RoPE) or 3 (M-RoPE: t,h,w);
// axis_map[head_dim/2] selects the position row per frequency (null -> row 0).
// The caches are addressed by strides (in elements): the row of head h of slot s starts at
// s * kv_tok_stride + h * kv_head_stride, which covers both the slot-major [slots, heads, D] and the head-major
// [heads, slots, D] layout.
void launch_qk_norm_rope_kv_write(void* qkv, const void* q_w, const void* k_w, const int64_t* positions,
                                  int pos_rows, const int8_t* axis_map, const float* inv_freq,
                                  const int64_t* cache_loc, void* k_cache, void* v_cache, int64_t kv_tok_stride,
                                  int64_t kv_head_stride, int tokens,
                                  int num_q_heads, int num_kv_heads, int head_dim, int64_t qkv_stride,
                                  int64_t num_slots, float eps, DType dt, int kv_fmt, int* status, cudaStream_t s);
void launch_kv_write(const void* k, const void* v, const int64_t* loc, void* k_cache, void* v_cache,
                     int64_t kv_tok_stride, int64_t kv_head_stride, int head_elems, int tokens,
                     int row_elems, int64_t k_stride, int64_t v_stride, int64_t num_slots, DType dt, int kv_fmt, int* status,
                     cudaStream_t s);

// Bookkeeping of one decode step of a static batch (see decode_prepare_kernel): one launch instead of a dozen
// small framework kernels.
void launch_decode_prepare(const int64_t* last_ids, const int32_t* req_rows, const int64_t* own, int64_t own_stride,
                           int used, int32_t* seq_lens, int32_t* req_to_token, int64_t rtt_stride,
                           int64_t* g_input_ids, int32_t* g_req_rows, int32_t* g_seq_lens, int64_t* g_out_loc,
                           int64_t* g_positions, int batch, cudaStream_t s);

// ----- quantisation -------------------------------------------------------------------
void launch_per_token_quant_int8(const void* x, int8_t* q, float* scale, int rows, int k, DType dt,
                                 cudaStream_t s);

// ----- sampling -------------------------------------------------------------------------
void launch_argmax(const void* logits, int64_t* out, int rows, int vocab, int64_t stride, DType dt,
                   cudaStream_t s);
// two-stage variant for few rows x wide vocabulary; part_val / part_idx hold rows * 32 entries
int launch_argmax_split(const void* logits, int64_t* out, float* part_val, int* part_idx, int rows, int vocab,
                        int64_t stride, DType dt, cudaStream_t s);

// one token per row: temperature (<= 1e-6: greedy), top-k (<= 0: off), top-p, min-p (may be null),
// inverse-CDF draw with uniform[row] in [0, 1)
void launch_sample(const void* logits, int64_t stride, int rows, int vocab, const float* temperature, const int* top_k,
                   const float* top_p, const float* min_p, const float* uniform, int64_t* out, DType dt, cudaStream_t s);
void launch_apply_penalties(float* logits, const int* counts, const uint8_t* prompt_mask, const float* freq,
                            const float* presence, const float* repetition, int rows, int vocab, cudaStream_t s);

// ----- GEMM (tcgen05 + TMEM + TMA) ---------------------------------------------------
struct GemmArgs {
  const void* a;         // [m, k] row-major activations
  const void* b;         // [n, k] row-major weights (out = a * b^T)
  void* out;             // [m, n_out] row-major
  const void* bias;      // [n] or null
  const void* residual;  // [m, n] or null (added before rounding)
  const float* a_scale;  // int8 only: per-row scale [m]
  const float* b_scale;  // int8 only: per-column scale [n]
  int m, n, k;
  int64_t lda, ldb, ldc, ld_res;
  int swiglu;            // 1: b rows alternate 128 gate / 128 up rows; out is [m, n/2]
  DType dt;              // element type of a, b (kBF16 / kF16) ; out has the same type
  int is_int8;           // 1: a, b are int8, out type given by dt
  float* workspace;      // split-K partial sums (small-m path), may be null when not needed
  size_t workspace_bytes;
  int* counters;         // split-K tile tickets, zero-initialised, self-resetting
  int num_counters;
  int* status;           // device int, set non-zero when a bounded wait ran out
  int num_sms;
  int b_static;          // 1: b (the weights) is not written by kernels that precede this launch in its stream
  // ---- fused add + RMSNorm prologue, batches of up to 8 rows only (norm_weight null = off) ----
  // the product is taken of rmsnorm(a + norm_residual) * norm_weight; the 16-bit sum a + norm_residual (the new
  // residual stream) is written to norm_residual_out, which must not alias norm_residual (other CTAs still read it)
  const void* norm_weight;        // [k]
  const void* norm_residual;      // [m, k] or null
  void* norm_residual_out;        // [m, k] or null
  int64_t norm_residual_ld, norm_residual_out_ld;   // elements
  float norm_eps;
  // ---- tensor-parallel fusion, large-m tiling only (all zero = off) ----
  // all-gather -> GEMM: 128-row tile t of `a` is read only once gate_flags[t] >= gate_epoch
  const uint32_t* gate_flags;
  uint32_t gate_epoch;
  // GEMM -> reduce-scatter: m must be a multiple of 128 * rs_tp; 128-row tile t goes to rank
  // t / (m / 128 / rs_tp): stored at rs_out[owner] + local_row * rs_ld (this rank's slot of the owner's
  // inbox), and rs_flags[owner][local_tile * 8 + rs_rank] is set to rs_epoch when the row tile is complete.
  // rs_count: local int[m / 128], zero-initialised, self-resetting.  `out` is ignored.
  int rs_tp, rs_rank;
  uint32_t rs_epoch;
  int64_t rs_ld;
  uint64_t rs_out[8];
  uint64_t rs_flags[8];
  int* rs_count;
};
// Returns 0 on success, a negative code when the shape is unsupported (caller falls back / raises).
int launch_gemm(const GemmArgs& args, cudaStream_t s);
size_t gemm_workspace_bytes(int m, int n, int k, int num_sms);
// m <= 8, 16-bit operands: the weight matrix streamed through registers and warp-level MMAs (no tensor memory, no
// shared-memory ring, no split of k between CTAs).  Returns 0 when launched, 1 when the shape is not for it.
int launch_gemm_smallm(const GemmArgs& args, cudaStream_t s);

// ----- W4A16 GEMM (4-bit weights expanded in shared memory, tcgen05) ----------------------------
struct W4A16Args {
  const void* x;        // [m, k] activations (bf16 / fp16), row stride ldx
  const void* qweight;  // int32 [n, k/8]; nibble i of word j = element 8j + i, or (interleaved = 1) element
                        // 8j + 2p + h in nibble p + 4h
  const void* scales;   // [n, k/group] in the activation type
  const uint8_t* zeros; // [n, k/group] or null (zero point 8)
  const void* bias;     // [n] or null
  void* out;            // [m, n] row stride ldc
  float* workspace;     // split-K partials (may be null: no split)
  size_t workspace_bytes;
  int* status;
  int m, n, k, group;
  int64_t ldx, ldc;
  DType dt;
  int num_sms;
  int interleaved;
};
int launch_w4a16_gemm(const W4A16Args& args, cudaStream_t s);
// m <= 8, k <= 4096: packed weights streamed and expanded in registers (gemm_smallm_w4.cu).  0 launched, 1 not for it.
int launch_w4a16_smallm(const W4A16Args& args, cudaStream_t s);

// 128-byte-swizzled 2-D tensor map over a row-major [rows, k] matrix (box = 128 bytes of k x box_rows);
// map points at a CUtensorMap.  type: 0 bf16, 1 fp16, 2 uint8.
bool make_tma_operand_map(void* map, const void* base, int64_t rows, int64_t k, int64_t ld, int elem_bytes, int type,
                          int box_rows);

// ----- expert-parallel token exchange (ep_a2a.cu) -------------------------------------------
// Addresses of every rank's copy of the shared buffers (index = rank), this rank's id and the call's epoch.
struct EpA2AArgs {
  int ep, rank, experts, hidden, cap_rows;
  uint32_t epoch;
  uint64_t cnt_all[8];     // int32 [ep][experts]
  uint64_t cnt_flags[8];   // uint32 [ep]
  uint64_t recv_x[8];      // 16-bit [cap_rows][hidden]
  uint64_t recv_meta[8];   // int32 [cap_rows][2]
  uint64_t disp_flags[8];  // uint32 [ep]
  uint64_t ret_y[8];       // 16-bit [pairs capacity][hidden]
  uint64_t ret_flags[8];   // uint32 [ep]
};
int launch_ep_plan(const EpA2AArgs& a, const int* topk_ids, int pairs, int bn, int* pair_dst_rank, int* pair_dst_row,
                   int* expert_offsets, int* work, int* n_work, int max_work, int* recv_rows, int* status,
                   cudaStream_t s);
int launch_ep_dispatch(const EpA2AArgs& a, const void* x, int64_t x_stride, int pairs, int top_k, const int* pair_dst_rank,
                       const int* pair_dst_row, int* done_count, cudaStream_t s);
int launch_ep_return(const EpA2AArgs& a, const void* ys, const int* recv_rows, int* done_count, cudaStream_t s);

// ----- mixture of experts ----------------------------------------------------------------
// router: fp32 softmax over `experts` (<= 256) logits -> top_k (<= 32, sorted, lowest index wins ties)
void launch_moe_router_topk(const void* logits, int64_t stride, float* w, int* ids, int tokens, int experts, int top_k,
                            int renorm, DType dt, cudaStream_t s);
// counting sort of the (token, choice) pairs by local expert.  sorted_pos[pair] = row in the sorted
// matrix or -1 (expert on another rank); src_token[row] = token; expert_offsets[experts + 1];
// work[i] = (expert, chunk of bn rows), *n_work items.
void launch_moe_align(const int* topk_ids, int pairs, int top_k, int expert_offset, int experts, int bn, int* sorted_pos,
                      int* src_token, int* expert_offsets, int* work, int* n_work, int max_work, cudaStream_t s);
void launch_moe_gather(const void* x, int64_t x_stride, const int* src_token, const int* expert_offsets, int experts,
                       void* xs, int pairs, int hidden, cudaStream_t s);
void launch_moe_combine(const void* y, const int* sorted_pos, const float* topk_w, void* out, int tokens, int hidden,
                        int top_k, DType dt, cudaStream_t s);
struct MoeGemmArgs {
  const void* x;    // [rows_cap, k] expert-sorted activations
  const void* w;    // [experts, n, k]
  void* out;        // [rows_cap, n_out]
  const int* expert_offsets;
  const int* work;
  const int* n_work;
  int* status;
  int64_t ldx, ldc;
  int rows_cap, experts, n, k, bn, max_work, swiglu, num_sms;
  DType dt;
};
int launch_moe_grouped_gemm(const MoeGemmArgs& args, cudaStream_t s);

// ----- attention over the slot-indexed KV pool (tcgen05, head_dim 128) -----------------
struct AttnArgs {
  const void* q;            // [T, Hq, 128], token stride q_stride elements
  const void* k_cache;      // row of head h of slot s at s * kv_tok_stride + h * kv_head_stride (elements)
  const void* v_cache;
  int64_t kv_tok_stride;    // slot-major [slots, Hkv, 128]: Hkv * 128 and 128; head-major [Hkv, slots, 128]:
  int64_t kv_head_stride;   // 128 and slots * 128 (consecutive slots of a head are then contiguous)
  void* out;                // [T, Hq, 128] contiguous
  float* part_o;            // decode with num_splits > 1: [B, Hq, splits, 128]
  float* part_lse;          // decode with num_splits > 1: [B, Hq, splits]
  const int* req_to_token;  // [reqs, rtt_stride]
  const int* req_pool_indices;  // [B]
  const int* seq_lens;          // [B]
  const int* prefix_lens;       // [B], prefill only
  const int* q_start;           // [B], prefill only: first query row of each request
  int* status;
  int64_t q_stride, rtt_stride, num_slots;
  int batch, hq, hkv, head_dim;
  int max_q_len;            // prefill: longest run of new tokens in the batch
  int num_splits;           // decode
  int is_decode;
  int non_causal;           // prefill only: bidirectional attention inside each sequence
  float scale;
  int window;               // > 0: a query at position i sees keys i - window + 1 .. i only (causal attention)
  float logit_cap;          // > 0: scores pass through cap * tanh(score / cap) before the softmax
  DType dt;
  int kv_fmt;               // 0: the caches hold dt; 1 / 2: unscaled e4m3 / e5m2 bytes (strides then count bytes)
};
int launch_attention(const AttnArgs& args, cudaStream_t s);
int decode_num_splits(int batch, int hkv, int max_seq_len, int num_sms);

// ----- gated delta net (hybrid models) -----------------------------------------------------------
// Ragged sequences: request b owns rows q_start[b] .. q_start[b] + lens[b] of the token-major inputs and
// row slots[b] of the state tensors; has_state[b] != 0 resumes from the stored state.
int launch_gdn_conv1d_silu(const void* x, const void* w, void* conv_state, const int* slots, const int* lens,
                           const int* has_state, const int* q_start, void* out, int batch, int max_tokens, int channels, int K,
                           DType dt, cudaStream_t s);
int launch_gdn_recurrent(const void* q, const void* k, const void* v, const float* g, const float* beta, float* state,
                         const int* slots, const int* lens, const int* has_state, const int* q_start, void* out, int batch,
                         int heads, int dk, int dv, DType dt, cudaStream_t s);
// The same rule evaluated 64 tokens at a time with tensor-core products (prefill); same arguments and state layout.
int launch_gdn_chunk(const void* q, const void* k, const void* v, const float* g, const float* beta, float* state,
                     const int* slots, const int* lens, const int* has_state, const int* q_start, void* out, int batch,
                     int heads, int dk, int dv, int num_sms, DType dt, cudaStream_t s);
void launch_rmsnorm_gated(const void* x, const void* gate, const void* w, void* out, int rows, int width, float eps, DType dt,
                          cudaStream_t s);

// ----- vision tower helpers ------------------------------------------------------------------
// qkv [T, 3, H, D] (D <= 128, D % 8 == 0) -> q, k, v [T, H, 128] zero-padded; q and k get the 2-D rotary
// embedding: out[i] = x[i] c[i] - x[i + D/2] s[i], out[i + D/2] = x[i + D/2] c[i] + x[i] s[i], cos/sin fp32 [T, D/2].
void launch_vision_rope_split_pad(const void* qkv, const float* cos, const float* sin, void* q, void* k, void* v,
                                  int tokens, int heads, int head_dim, int out_dim, DType dt, cudaStream_t s);
// x[t, :] += sum_i w[i, t] * table[idx[i, t], :]  (i < 4: bilinear corners); idx int64 [4, T], w fp32 [4, T]
void launch_vision_pos_embed_add(void* x, const void* table, const int64_t* idx, const float* w, int tokens, int hidden,
                                 DType dt, cudaStream_t s);
void launch_gelu_erf(const void* x, void* out, int64_t n, DType dt, cudaStream_t s);

// ----- tensor-parallel reduction + residual add + RMSNorm over peer memory ----------------
// peer_data / peer_flags: host arrays of `tp` device addresses (every rank's partial-sum buffer
// and flag block, mapped into this process).  flags: uint32 [max_rows][8] per rank, zero-initialised;
// local_seq: uint32 [max_rows] on this device, zero-initialised.  weight may be null (plain sum).
int launch_tp_reduce_add_rmsnorm(const uint64_t* peer_data, const uint64_t* peer_flags, uint32_t* local_seq,
                                 void* residual, const void* weight, void* out, int rows, int hidden, int tp, int rank,
                                 int64_t row_stride, float eps, DType dt, int* status, cudaStream_t s);


// ----- tensor-parallel prefill: reduce-scatter + residual add + RMSNorm + all-gather -------
// This rank owns `rows` consecutive token rows (global rows rank * rows ...).  inbox: local
// [tp][inbox_rows_cap][hidden] partial sums written by every rank's GEMM epilogue; tile_flags: local
// uint32 [tiles][8], slot (tile, src) holds the epoch of src's last completed delivery of that 128-row
// tile.  For each own row: sum the tp partials in rank order, add the residual shard (in place; when
// residual is null the sum itself is the new residual... the caller passes the shard), normalise, and
// store the row into every rank's gathered buffer (peer_hidden[r] + global_row * hidden).  When a
// 128-row tile is complete, gather_flags[global tile] on every rank is set to `epoch`.
// ag_count: local int[tiles], zero-initialised, self-resetting.  rows must be a multiple of 128.
// n_src = partial sums per row in the inbox: tp for the reduce-scatter inbox; 1 with tile_flags == nullptr when
// the rows of this rank are already complete (output of the expert-parallel exchange).
int launch_tp_rs_add_rmsnorm_ag(const void* inbox, int64_t inbox_rows_cap, const uint32_t* tile_flags,
                                void* residual_shard, const void* weight, const uint64_t* peer_hidden,
                                const uint64_t* peer_gather_flags, int* ag_count, int rows, int hidden, int tp,
                                int n_src, int rank, uint32_t epoch, float eps, DType dt, int* status, cudaStream_t s);
// Bounded wait until flags[i] >= epoch for all i < n (makes peers' deliveries visible to later kernels).
int launch_tp_wait_flags(const uint32_t* flags, int n, uint32_t epoch, int* status, cudaStream_t s);

}  // namespace mb200
