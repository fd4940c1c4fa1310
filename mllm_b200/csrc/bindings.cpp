// PyTorch binding of the sm_100a kernels: checks tensors, picks the current CUDA
// stream and forwards raw pointers to the launchers declared in kernels.h.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <mutex>
#include <unordered_map>

#include "kernels.h"

namespace {

using torch::Tensor;

mb200::DType dtype_of(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kBFloat16: return mb200::kBF16;
    case at::kHalf: return mb200::kF16;
    case at::kFloat: return mb200::kF32;
    default: TORCH_CHECK(false, "mllm_b200: unsupported dtype ", t.scalar_type());
  }
}

void check_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), "mllm_b200: ", name, " must be a CUDA tensor");
}
void check_half(const Tensor& t, const char* name) {
  check_cuda(t, name);
  TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kHalf, "mllm_b200: ", name,
              " must be bf16 or fp16");
}

struct DeviceState {
  Tensor status;     // int32[1]
  Tensor workspace;  // float, split-K partials
  Tensor counters;   // int32 tickets
  int num_sms = 0;
};

DeviceState& device_state(int device) {
  static std::mutex mu;
  static std::unordered_map<int, DeviceState> states;
  std::lock_guard<std::mutex> lock(mu);
  auto it = states.find(device);
  if (it == states.end()) {
    DeviceState st;
    auto opts_i = torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, device);
    st.status = torch::zeros({4}, opts_i);
    st.counters = torch::zeros({4096}, opts_i);
    st.workspace = torch::empty({static_cast<int64_t>(mb200::gemm_workspace_bytes(0, 0, 0, 0) / 4)},
                                torch::TensorOptions().dtype(torch::kFloat32).device(torch::kCUDA, device));
    st.num_sms = at::cuda::getDeviceProperties(device)->multiProcessorCount;
    it = states.emplace(device, std::move(st)).first;
  }
  return it->second;
}

cudaStream_t stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

// --------------------------------------------------------------------------------------
void rmsnorm(const Tensor& x, const Tensor& w, Tensor& out, double eps) {
  check_half(x, "x");
  TORCH_CHECK(x.dim() == 2 && out.dim() == 2 && x.stride(1) == 1 && out.stride(1) == 1, "rmsnorm: 2-D row-major");
  const int hidden = x.size(1);
  TORCH_CHECK(hidden % 8 == 0 && hidden <= 32768 && w.numel() == hidden && w.is_contiguous(), "rmsnorm: hidden");
  TORCH_CHECK(x.stride(0) % 8 == 0 && out.stride(0) % 8 == 0, "rmsnorm: row strides must be multiples of 8");
  c10::cuda::CUDAGuard g(x.device());
  mb200::launch_rmsnorm(x.data_ptr(), w.data_ptr(), out.data_ptr(), x.size(0), hidden, x.stride(0), out.stride(0),
                        static_cast<float>(eps), dtype_of(x), stream_of(x));
}

void fused_add_rmsnorm(Tensor& x, Tensor& residual, const Tensor& w, double eps) {
  check_half(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && residual.is_contiguous() && residual.sizes() == x.sizes(),
              "fused_add_rmsnorm: contiguous 2-D tensors of equal shape");
  const int hidden = x.size(1);
  TORCH_CHECK(hidden % 8 == 0 && hidden <= 32768 && w.numel() == hidden, "fused_add_rmsnorm: hidden");
  c10::cuda::CUDAGuard g(x.device());
  mb200::launch_fused_add_rmsnorm(x.data_ptr(), residual.data_ptr(), w.data_ptr(), x.size(0), hidden,
                                  static_cast<float>(eps), dtype_of(x), stream_of(x));
}

void layernorm(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& b, Tensor& out, double eps) {
  check_half(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && out.is_contiguous(), "layernorm: contiguous 2-D");
  const int hidden = x.size(1);
  TORCH_CHECK(hidden % 8 == 0 && hidden <= 32768, "layernorm: hidden");
  c10::cuda::CUDAGuard g(x.device());
  mb200::launch_layernorm(x.data_ptr(), w.data_ptr(), b.has_value() ? b->data_ptr() : nullptr, out.data_ptr(),
                          x.size(0), hidden, static_cast<float>(eps), dtype_of(x), stream_of(x));
}

void act_and_mul(const Tensor& x, Tensor& out, int64_t act) {
  check_half(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && out.is_contiguous(), "act_and_mul: contiguous 2-D");
  const int inter = x.size(1) / 2;
  TORCH_CHECK(inter % 8 == 0 && out.size(1) == inter, "act_and_mul: width");
  c10::cuda::CUDAGuard g(x.device());
  mb200::launch_act_and_mul(x.data_ptr(), out.data_ptr(), x.size(0), inter, static_cast<int>(act), dtype_of(x),
                            stream_of(x));
}

void gelu_tanh(const Tensor& x, Tensor& out) {
  check_half(x, "x");
  TORCH_CHECK(x.is_contiguous() && out.is_contiguous() && x.numel() % 8 == 0, "gelu_tanh: contiguous, numel % 8");
  c10::cuda::CUDAGuard g(x.device());
  mb200::launch_gelu_tanh(x.data_ptr(), out.data_ptr(), x.numel(), dtype_of(x), stream_of(x));
}

void embedding(const Tensor& ids, const Tensor& table, Tensor& out) {
  check_half(table, "table");
  TORCH_CHECK(ids.scalar_type() == at::kLong && ids.is_contiguous() && table.is_contiguous() && out.is_contiguous(),
              "embedding: int64 ids, contiguous tensors");
  TORCH_CHECK(table.size(1) % 8 == 0, "embedding: hidden % 8");
  c10::cuda::CUDAGuard g(table.device());
  auto& st = device_state(table.get_device());
  mb200::launch_embedding(ids.data_ptr<int64_t>(), table.data_ptr(), out.data_ptr(), ids.numel(), table.size(1),
                          table.size(0), dtype_of(table), st.status.data_ptr<int>(), stream_of(table));
}

// K and V caches: [slots, kv heads, head_dim] views with unit stride along head_dim, equal strides for K and V
// and rows aligned to 8 elements; slot-major and head-major storage both qualify.  The element type is the
// activation dtype (returns 0) or an unscaled 8-bit float (returns 1 for e4m3, 2 for e5m2).
static int check_kv_cache(const Tensor& k_cache, const Tensor& v_cache, at::ScalarType dt, int64_t hkv, int64_t head_dim) {
  const auto ct = k_cache.scalar_type();
  const int fmt = ct == dt ? 0 : ct == at::kFloat8_e4m3fn ? 1 : ct == at::kFloat8_e5m2 ? 2 : -1;
  TORCH_CHECK(k_cache.dim() == 3 && v_cache.dim() == 3 && k_cache.sizes() == v_cache.sizes() &&
                  k_cache.strides() == v_cache.strides() && k_cache.stride(2) == 1 && k_cache.size(1) == hkv &&
                  k_cache.size(2) == head_dim && k_cache.stride(0) % 8 == 0 && k_cache.stride(1) % 8 == 0 &&
                  fmt >= 0 && v_cache.scalar_type() == ct && k_cache.is_cuda() && v_cache.is_cuda(),
              "kv cache: [slots, kv_heads, head_dim] views of the activation dtype, float8_e4m3fn or float8_e5m2, "
              "with unit inner stride");
  return fmt;
}

void qk_norm_rope_kv_write(Tensor& qkv, const c10::optional<Tensor>& q_w, const c10::optional<Tensor>& k_w,
                           const Tensor& positions, const c10::optional<Tensor>& axis_map, const Tensor& inv_freq,
                           const Tensor& cache_loc, Tensor& k_cache, Tensor& v_cache, int64_t hq, int64_t hkv,
                           int64_t head_dim, double eps) {
  check_half(qkv, "qkv");
  TORCH_CHECK(head_dim == 128, "qk_norm_rope_kv_write: head_dim must be 128");
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) == (hq + 2 * hkv) * head_dim, "qkv shape");
  TORCH_CHECK(qkv.stride(0) % 4 == 0, "qkv row stride");
  TORCH_CHECK(positions.scalar_type() == at::kLong && positions.is_contiguous(), "positions int64 contiguous");
  TORCH_CHECK(cache_loc.scalar_type() == at::kLong && cache_loc.is_contiguous(), "cache_loc int64 contiguous");
  TORCH_CHECK(inv_freq.scalar_type() == at::kFloat && inv_freq.numel() == head_dim / 2, "inv_freq fp32 [D/2]");
  const int kv_fmt = check_kv_cache(k_cache, v_cache, qkv.scalar_type(), hkv, head_dim);
  const int tokens = qkv.size(0);
  const int pos_rows = positions.dim() == 2 ? positions.size(0) : 1;
  TORCH_CHECK(positions.numel() == static_cast<int64_t>(pos_rows) * tokens, "positions size");
  TORCH_CHECK(cache_loc.numel() == tokens, "cache_loc size");
  c10::cuda::CUDAGuard g(qkv.device());
  auto& st = device_state(qkv.get_device());
  mb200::launch_qk_norm_rope_kv_write(
      qkv.data_ptr(), q_w.has_value() ? q_w->data_ptr() : nullptr, k_w.has_value() ? k_w->data_ptr() : nullptr,
      positions.data_ptr<int64_t>(), pos_rows, axis_map.has_value() ? axis_map->data_ptr<int8_t>() : nullptr,
      inv_freq.data_ptr<float>(), cache_loc.data_ptr<int64_t>(), k_cache.data_ptr(), v_cache.data_ptr(),
      k_cache.stride(0), k_cache.stride(1), tokens, hq,
      hkv, head_dim, qkv.stride(0), k_cache.size(0), static_cast<float>(eps), dtype_of(qkv), kv_fmt,
      st.status.data_ptr<int>(), stream_of(qkv));
}

void kv_write(const Tensor& k, const Tensor& v, const Tensor& loc, Tensor& k_cache, Tensor& v_cache) {
  check_half(k, "k");
  TORCH_CHECK(loc.scalar_type() == at::kLong && loc.is_contiguous(), "loc int64 contiguous");
  const int tokens = loc.numel();
  const int kv_fmt = check_kv_cache(k_cache, v_cache, k.scalar_type(), k_cache.size(1), k_cache.size(2));
  const int64_t row = k_cache.size(1) * k_cache.size(2);
  TORCH_CHECK(k_cache.size(2) % 8 == 0 && k.numel() == tokens * row && v.numel() == tokens * row, "kv_write: row size");
  auto k2 = k.reshape({tokens, row});
  auto v2 = v.reshape({tokens, row});
  TORCH_CHECK(k2.stride(1) == 1 && v2.stride(1) == 1 && k2.stride(0) % 8 == 0 && v2.stride(0) % 8 == 0, "kv strides");
  c10::cuda::CUDAGuard g(k.device());
  auto& st = device_state(k.get_device());
  mb200::launch_kv_write(k2.data_ptr(), v2.data_ptr(), loc.data_ptr<int64_t>(), k_cache.data_ptr(),
                         v_cache.data_ptr(), k_cache.stride(0), k_cache.stride(1), k_cache.size(2), tokens, row,
                         k2.stride(0), v2.stride(0), k_cache.size(0), dtype_of(k), kv_fmt,
                         st.status.data_ptr<int>(), stream_of(k));
}

void decode_prepare(const Tensor& last_ids, const Tensor& req_rows, const Tensor& own, int64_t used, Tensor& seq_lens,
                    Tensor& req_to_token, Tensor& g_input_ids, Tensor& g_req_rows, Tensor& g_seq_lens, Tensor& g_out_loc,
                    Tensor& g_positions) {
  check_cuda(last_ids, "last_ids");
  const int64_t bs = last_ids.numel();
  TORCH_CHECK(last_ids.scalar_type() == at::kLong && last_ids.is_contiguous(), "last_ids int64 contiguous");
  TORCH_CHECK(req_rows.scalar_type() == at::kInt && req_rows.numel() == bs && req_rows.is_contiguous(), "req_rows int32 [bs]");
  TORCH_CHECK(own.scalar_type() == at::kLong && own.dim() == 2 && own.size(0) == bs && own.stride(1) == 1 && used >= 0 &&
                  used < own.size(1),
              "own int64 [bs, cap] and 0 <= used < cap");
  TORCH_CHECK(seq_lens.scalar_type() == at::kInt && seq_lens.numel() == bs && seq_lens.is_contiguous(), "seq_lens int32 [bs]");
  TORCH_CHECK(req_to_token.scalar_type() == at::kInt && req_to_token.dim() == 2 && req_to_token.stride(1) == 1, "req_to_token");
  TORCH_CHECK(g_input_ids.scalar_type() == at::kLong && g_out_loc.scalar_type() == at::kLong &&
                  g_positions.scalar_type() == at::kLong && g_req_rows.scalar_type() == at::kInt &&
                  g_seq_lens.scalar_type() == at::kInt,
              "graph input buffers: int64 ids / slots / positions, int32 rows / lengths");
  TORCH_CHECK(g_input_ids.numel() >= bs && g_req_rows.numel() >= bs && g_seq_lens.numel() >= bs && g_out_loc.numel() >= bs &&
                  g_positions.numel() >= bs && g_input_ids.is_contiguous() && g_req_rows.is_contiguous() &&
                  g_seq_lens.is_contiguous() && g_out_loc.is_contiguous() && g_positions.is_contiguous(),
              "graph input buffers too small");
  c10::cuda::CUDAGuard g(last_ids.device());
  mb200::launch_decode_prepare(last_ids.data_ptr<int64_t>(), req_rows.data_ptr<int32_t>(), own.data_ptr<int64_t>(),
                               own.stride(0), static_cast<int>(used), seq_lens.data_ptr<int32_t>(),
                               req_to_token.data_ptr<int32_t>(), req_to_token.stride(0), g_input_ids.data_ptr<int64_t>(),
                               g_req_rows.data_ptr<int32_t>(), g_seq_lens.data_ptr<int32_t>(), g_out_loc.data_ptr<int64_t>(),
                               g_positions.data_ptr<int64_t>(), static_cast<int>(bs), stream_of(last_ids));
}

std::vector<Tensor> per_token_quant_int8(const Tensor& x) {
  check_half(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && x.size(1) % 16 == 0 && x.size(1) <= 32768, "quant: [M,K], K%16");
  c10::cuda::CUDAGuard g(x.device());
  auto q = torch::empty_like(x, x.options().dtype(torch::kInt8));
  auto scale = torch::empty({x.size(0), 1}, x.options().dtype(torch::kFloat32));
  mb200::launch_per_token_quant_int8(x.data_ptr(), q.data_ptr<int8_t>(), scale.data_ptr<float>(), x.size(0),
                                     x.size(1), dtype_of(x), stream_of(x));
  return {q, scale};
}

void argmax(const Tensor& logits, Tensor& out) {
  check_cuda(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && out.scalar_type() == at::kLong && out.is_contiguous(),
              "argmax: [B,V] logits, int64 out");
  c10::cuda::CUDAGuard g(logits.device());
  const int64_t rows = logits.size(0), vocab = logits.size(1);
  if (rows <= 64 && vocab >= 32768) {
    // few rows of a wide vocabulary: spread every row over 32 CTAs (scratch from the caching allocator)
    auto pv = torch::empty({rows * 32}, torch::TensorOptions().dtype(torch::kFloat32).device(logits.device()));
    auto pi = torch::empty({rows * 32}, torch::TensorOptions().dtype(torch::kInt32).device(logits.device()));
    mb200::launch_argmax_split(logits.data_ptr(), out.data_ptr<int64_t>(), pv.data_ptr<float>(), pi.data_ptr<int>(), rows,
                               vocab, logits.stride(0), dtype_of(logits), stream_of(logits));
    return;
  }
  mb200::launch_argmax(logits.data_ptr(), out.data_ptr<int64_t>(), rows, vocab, logits.stride(0), dtype_of(logits),
                       stream_of(logits));
}

void sample(const Tensor& logits, const Tensor& temperature, const Tensor& top_k, const Tensor& top_p,
            const c10::optional<Tensor>& min_p, const Tensor& uniform, Tensor& out) {
  check_cuda(logits, "logits");
  const int64_t rows = logits.size(0);
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && out.scalar_type() == at::kLong && out.is_contiguous() &&
                  out.numel() == rows,
              "sample: [B,V] logits, int64 out [B]");
  TORCH_CHECK(temperature.scalar_type() == at::kFloat && top_p.scalar_type() == at::kFloat &&
                  uniform.scalar_type() == at::kFloat && top_k.scalar_type() == at::kInt && temperature.numel() == rows &&
                  top_p.numel() == rows && top_k.numel() == rows && uniform.numel() == rows && temperature.is_cuda() &&
                  top_k.is_cuda() && top_p.is_cuda() && uniform.is_cuda(),
              "sample: per-row parameter vectors on the device");
  if (min_p.has_value())
    TORCH_CHECK(min_p->scalar_type() == at::kFloat && min_p->numel() == rows && min_p->is_cuda(), "sample: min_p");
  c10::cuda::CUDAGuard g(logits.device());
  mb200::launch_sample(logits.data_ptr(), logits.stride(0), rows, logits.size(1), temperature.data_ptr<float>(),
                       top_k.data_ptr<int>(), top_p.data_ptr<float>(), min_p.has_value() ? min_p->data_ptr<float>() : nullptr,
                       uniform.data_ptr<float>(), out.data_ptr<int64_t>(), dtype_of(logits), stream_of(logits));
}

void apply_penalties(Tensor& logits, const Tensor& counts, const c10::optional<Tensor>& prompt_mask, const Tensor& freq,
                     const Tensor& presence, const Tensor& repetition) {
  check_cuda(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.is_contiguous() && logits.scalar_type() == at::kFloat && counts.is_contiguous() &&
                  counts.scalar_type() == at::kInt && counts.sizes() == logits.sizes() && counts.is_cuda(),
              "apply_penalties: fp32 logits and int32 counts [B,V]");
  if (prompt_mask.has_value())
    TORCH_CHECK(prompt_mask->scalar_type() == at::kByte && prompt_mask->is_contiguous() &&
                    prompt_mask->sizes() == logits.sizes() && prompt_mask->is_cuda(),
                "apply_penalties: uint8 prompt mask [B,V]");
  const int64_t rows = logits.size(0);
  for (const Tensor* t : {&freq, &presence, &repetition})
    TORCH_CHECK(t->scalar_type() == at::kFloat && t->numel() == rows && t->is_cuda() && t->is_contiguous(),
                "apply_penalties: fp32 [B] penalties");
  c10::cuda::CUDAGuard g(logits.device());
  mb200::launch_apply_penalties(logits.data_ptr<float>(), counts.data_ptr<int>(),
                                prompt_mask.has_value() ? prompt_mask->data_ptr<uint8_t>() : nullptr,
                                freq.data_ptr<float>(), presence.data_ptr<float>(), repetition.data_ptr<float>(), rows,
                                logits.size(1), stream_of(logits));
}

int64_t w4a16_gemm(const Tensor& x, const Tensor& qweight, const Tensor& scales, const c10::optional<Tensor>& zeros,
                   int64_t group, const c10::optional<Tensor>& bias, Tensor& out, bool interleaved) {
  check_half(x, "x");
  check_cuda(qweight, "qweight");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && qweight.dim() == 2 && qweight.is_contiguous() &&
                  qweight.scalar_type() == at::kInt && qweight.size(1) * 8 == x.size(1),
              "w4a16_gemm: x [M, K], qweight int32 [N, K/8]");
  const int64_t N = qweight.size(0), K = x.size(1);
  TORCH_CHECK(scales.is_cuda() && scales.is_contiguous() && scales.scalar_type() == x.scalar_type() && scales.dim() == 2 &&
                  scales.size(0) == N && scales.size(1) * group == K,
              "w4a16_gemm: scales [N, K/group] of x's dtype");
  if (zeros.has_value())
    TORCH_CHECK(zeros->is_cuda() && zeros->is_contiguous() && zeros->scalar_type() == at::kByte &&
                    zeros->sizes() == scales.sizes(),
                "w4a16_gemm: uint8 zeros [N, K/group]");
  if (bias.has_value())
    TORCH_CHECK(bias->is_cuda() && bias->is_contiguous() && bias->scalar_type() == x.scalar_type() && bias->numel() == N,
                "w4a16_gemm: bias [N]");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == x.size(0) && out.size(1) == N && out.stride(1) == 1 &&
                  out.scalar_type() == x.scalar_type(),
              "w4a16_gemm: out [M, N]");
  c10::cuda::CUDAGuard g(x.device());
  auto& st = device_state(x.get_device());
  mb200::W4A16Args a{};
  a.x = x.data_ptr();
  a.qweight = qweight.data_ptr();
  a.scales = scales.data_ptr();
  a.zeros = zeros.has_value() ? zeros->data_ptr<uint8_t>() : nullptr;
  a.bias = bias.has_value() ? bias->data_ptr() : nullptr;
  a.out = out.data_ptr();
  a.workspace = st.workspace.data_ptr<float>();
  a.workspace_bytes = st.workspace.numel() * sizeof(float);
  a.status = st.status.data_ptr<int>();
  a.m = x.size(0);
  a.n = N;
  a.k = K;
  a.group = group;
  a.ldx = x.stride(0);
  a.ldc = out.stride(0);
  a.dt = dtype_of(x);
  a.num_sms = st.num_sms;
  a.interleaved = interleaved ? 1 : 0;
  return mb200::launch_w4a16_gemm(a, stream_of(x));
}

// ---- gated delta net ----
void rmsnorm_gated(const Tensor& x, const Tensor& gate, const Tensor& w, Tensor& out, double eps) {
  check_half(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && gate.is_contiguous() && gate.sizes() == x.sizes() && out.is_contiguous() &&
                  out.sizes() == x.sizes() && w.numel() == x.size(1) && w.scalar_type() == x.scalar_type() &&
                  gate.scalar_type() == x.scalar_type() && out.scalar_type() == x.scalar_type(),
              "rmsnorm_gated: x, gate, out [R, W] and weight [W] of one 16-bit type");
  c10::cuda::CUDAGuard g(x.device());
  mb200::launch_rmsnorm_gated(x.data_ptr(), gate.data_ptr(), w.data_ptr(), out.data_ptr(), x.size(0), x.size(1),
                              static_cast<float>(eps), dtype_of(x), stream_of(x));
}

static void check_ragged(const Tensor& slots, const Tensor& lens, const Tensor& has, const Tensor& q_start) {
  for (const Tensor* t : {&slots, &lens, &has, &q_start})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->is_contiguous() && t->numel() == slots.numel(),
                "ragged metadata: int32 device vectors of one length");
}

void gdn_conv1d_silu(const Tensor& x, const Tensor& w, Tensor& conv_state, const Tensor& slots, const Tensor& lens,
                     const Tensor& has, const Tensor& q_start, Tensor& out) {
  check_half(x, "x");
  check_ragged(slots, lens, has, q_start);
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && out.is_contiguous() && out.sizes() == x.sizes() && w.dim() == 2 &&
                  w.is_contiguous() && w.size(0) == x.size(1) && conv_state.dim() == 3 && conv_state.is_contiguous() &&
                  conv_state.size(1) == x.size(1) && conv_state.size(2) == w.size(1) - 1 &&
                  w.scalar_type() == x.scalar_type() && conv_state.scalar_type() == x.scalar_type(),
              "gdn_conv1d_silu: x [T, C], w [C, K], conv_state [slots, C, K-1]");
  c10::cuda::CUDAGuard g(x.device());
  const int rc = mb200::launch_gdn_conv1d_silu(x.data_ptr(), w.data_ptr(), conv_state.data_ptr(), slots.data_ptr<int>(),
                                               lens.data_ptr<int>(), has.data_ptr<int>(), q_start.data_ptr<int>(),
                                               out.data_ptr(), slots.numel(), x.size(0), x.size(1), w.size(1), dtype_of(x),
                                               stream_of(x));
  TORCH_CHECK(rc == 0, "gdn_conv1d_silu: unsupported kernel width");
}

void gdn_recurrent(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& g, const Tensor& beta, Tensor& state,
                   const Tensor& slots, const Tensor& lens, const Tensor& has, const Tensor& q_start, Tensor& out) {
  check_half(q, "q");
  check_ragged(slots, lens, has, q_start);
  TORCH_CHECK(q.dim() == 3 && q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && k.sizes() == q.sizes() &&
                  v.size(0) == q.size(0) && v.size(1) == q.size(1) && out.is_contiguous() && out.sizes() == v.sizes() &&
                  g.scalar_type() == at::kFloat && beta.scalar_type() == at::kFloat && g.is_contiguous() && beta.is_contiguous() &&
                  g.numel() == q.size(0) * q.size(1) && beta.numel() == g.numel() && state.scalar_type() == at::kFloat &&
                  state.is_contiguous() && state.dim() == 4 && state.size(1) == q.size(1) && state.size(2) == q.size(2) &&
                  state.size(3) == v.size(2),
              "gdn_recurrent: q, k [T, H, Dk], v [T, H, Dv], g / beta fp32 [T, H], state fp32 [slots, H, Dk, Dv]");
  c10::cuda::CUDAGuard gd(q.device());
  const int rc = mb200::launch_gdn_recurrent(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr<float>(), beta.data_ptr<float>(),
                                             state.data_ptr<float>(), slots.data_ptr<int>(), lens.data_ptr<int>(),
                                             has.data_ptr<int>(), q_start.data_ptr<int>(), out.data_ptr(), slots.numel(),
                                             q.size(1), q.size(2), v.size(2), dtype_of(q), stream_of(q));
  TORCH_CHECK(rc == 0, "gdn_recurrent: head dims must be 128");
}

void gdn_chunk(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& g, const Tensor& beta, Tensor& state,
               const Tensor& slots, const Tensor& lens, const Tensor& has, const Tensor& q_start, Tensor& out) {
  check_half(q, "q");
  check_ragged(slots, lens, has, q_start);
  TORCH_CHECK(q.dim() == 3 && q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && k.sizes() == q.sizes() &&
                  v.size(0) == q.size(0) && v.size(1) == q.size(1) && out.is_contiguous() && out.sizes() == v.sizes() &&
                  k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type() && out.scalar_type() == q.scalar_type() &&
                  g.scalar_type() == at::kFloat && beta.scalar_type() == at::kFloat && g.is_contiguous() && beta.is_contiguous() &&
                  g.numel() == q.size(0) * q.size(1) && beta.numel() == g.numel() && state.scalar_type() == at::kFloat &&
                  state.is_contiguous() && state.dim() == 4 && state.size(1) == q.size(1) && state.size(2) == q.size(2) &&
                  state.size(3) == v.size(2),
              "gdn_chunk: q, k [T, H, Dk], v [T, H, Dv], g / beta fp32 [T, H], state fp32 [slots, H, Dk, Dv]");
  c10::cuda::CUDAGuard gd(q.device());
  auto& st = device_state(q.get_device());
  const int rc = mb200::launch_gdn_chunk(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr<float>(), beta.data_ptr<float>(),
                                         state.data_ptr<float>(), slots.data_ptr<int>(), lens.data_ptr<int>(),
                                         has.data_ptr<int>(), q_start.data_ptr<int>(), out.data_ptr(), slots.numel(),
                                         q.size(1), q.size(2), v.size(2), st.num_sms, dtype_of(q), stream_of(q));
  TORCH_CHECK(rc == 0, "gdn_chunk: head dims must be 128 (code ", rc, ")");
}

// ---- vision tower ----
void vision_rope_split_pad(const Tensor& qkv, const Tensor& cos, const Tensor& sin, Tensor& q, Tensor& k, Tensor& v) {
  check_half(qkv, "qkv");
  TORCH_CHECK(qkv.dim() == 4 && qkv.size(1) == 3 && qkv.is_contiguous() && qkv.size(3) <= 128 && qkv.size(3) % 2 == 0,
              "vision_rope_split_pad: qkv [T, 3, H, D <= 128]");
  const int64_t T = qkv.size(0), H = qkv.size(2), D = qkv.size(3);
  TORCH_CHECK(cos.is_cuda() && cos.scalar_type() == at::kFloat && cos.is_contiguous() && cos.size(0) == T &&
                  cos.size(1) == D / 2 && sin.sizes() == cos.sizes() && sin.scalar_type() == at::kFloat && sin.is_contiguous(),
              "vision_rope_split_pad: fp32 cos / sin [T, D/2]");
  const int64_t W = q.dim() == 3 ? q.size(2) : 0;
  for (Tensor* t : {&q, &k, &v})
    TORCH_CHECK(t->is_contiguous() && t->dim() == 3 && t->size(0) == T && t->size(1) == H && t->size(2) == W && W >= D &&
                    W <= 128 && t->scalar_type() == qkv.scalar_type(),
                "vision_rope_split_pad: outputs [T, H, W] with D <= W <= 128");
  c10::cuda::CUDAGuard g(qkv.device());
  mb200::launch_vision_rope_split_pad(qkv.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), q.data_ptr(),
                                      k.data_ptr(), v.data_ptr(), T, H, D, W, dtype_of(qkv), stream_of(qkv));
}

void vision_pos_embed_add(Tensor& x, const Tensor& table, const Tensor& idx, const Tensor& w) {
  check_half(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && table.is_contiguous() && table.size(1) == x.size(1) &&
                  table.scalar_type() == x.scalar_type() && idx.scalar_type() == at::kLong && idx.is_contiguous() &&
                  idx.size(0) == 4 && idx.size(1) == x.size(0) && w.scalar_type() == at::kFloat && w.is_contiguous() &&
                  w.sizes() == idx.sizes() && idx.is_cuda() && w.is_cuda(),
              "vision_pos_embed_add: x [T, E], table [P, E], idx int64 [4, T], w fp32 [4, T]");
  c10::cuda::CUDAGuard g(x.device());
  mb200::launch_vision_pos_embed_add(x.data_ptr(), table.data_ptr(), idx.data_ptr<int64_t>(), w.data_ptr<float>(),
                                     x.size(0), x.size(1), dtype_of(x), stream_of(x));
}

void gelu_erf(const Tensor& x, Tensor& out) {
  check_half(x, "x");
  TORCH_CHECK(x.is_contiguous() && out.is_contiguous() && out.numel() == x.numel() && out.scalar_type() == x.scalar_type(),
              "gelu_erf: contiguous tensors of one shape");
  c10::cuda::CUDAGuard g(x.device());
  mb200::launch_gelu_erf(x.data_ptr(), out.data_ptr(), x.numel(), dtype_of(x), stream_of(x));
}

// ---- mixture of experts ----
void moe_router_topk(const Tensor& logits, Tensor& w, Tensor& ids, bool renorm) {
  check_cuda(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && logits.size(1) <= 256, "moe_router_topk: [T,E<=256] logits");
  TORCH_CHECK(w.scalar_type() == at::kFloat && ids.scalar_type() == at::kInt && w.is_contiguous() && ids.is_contiguous() &&
                  w.dim() == 2 && w.size(0) == logits.size(0) && w.size(1) <= 32 && ids.sizes() == w.sizes(),
              "moe_router_topk: fp32 weights / int32 ids [T,k<=32]");
  c10::cuda::CUDAGuard g(logits.device());
  mb200::launch_moe_router_topk(logits.data_ptr(), logits.stride(0), w.data_ptr<float>(), ids.data_ptr<int>(),
                                logits.size(0), logits.size(1), w.size(1), renorm ? 1 : 0, dtype_of(logits),
                                stream_of(logits));
}

void moe_align(const Tensor& topk_ids, int64_t expert_offset, int64_t experts, int64_t bn, Tensor& sorted_pos,
               Tensor& src_token, Tensor& expert_offsets, Tensor& work, Tensor& n_work) {
  check_cuda(topk_ids, "topk_ids");
  TORCH_CHECK(topk_ids.scalar_type() == at::kInt && topk_ids.is_contiguous() && topk_ids.dim() == 2, "moe_align: int32 [T,k] ids");
  TORCH_CHECK(experts >= 1 && experts <= 256, "moe_align: 1..256 local experts");
  const int64_t pairs = topk_ids.numel();
  for (const Tensor* t : {&sorted_pos, &src_token, &expert_offsets, &work, &n_work})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->is_contiguous(), "moe_align: int32 outputs");
  TORCH_CHECK(sorted_pos.numel() >= pairs && src_token.numel() >= pairs && expert_offsets.numel() >= experts + 1 &&
                  work.dim() == 2 && work.size(1) == 2 && n_work.numel() >= 1,
              "moe_align: output sizes");
  c10::cuda::CUDAGuard g(topk_ids.device());
  mb200::launch_moe_align(topk_ids.data_ptr<int>(), pairs, topk_ids.size(1), expert_offset, experts, bn,
                          sorted_pos.data_ptr<int>(), src_token.data_ptr<int>(), expert_offsets.data_ptr<int>(),
                          work.data_ptr<int>(), n_work.data_ptr<int>(), work.size(0), stream_of(topk_ids));
}

void moe_gather(const Tensor& x, const Tensor& src_token, const Tensor& expert_offsets, Tensor& xs) {
  check_cuda(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.size(1) % 8 == 0 && x.stride(0) % 8 == 0 && xs.is_contiguous() &&
                  xs.size(1) == x.size(1) && x.element_size() == 2 && xs.scalar_type() == x.scalar_type(),
              "moe_gather: 16-bit rows, hidden % 8 == 0");
  c10::cuda::CUDAGuard g(x.device());
  mb200::launch_moe_gather(x.data_ptr(), x.stride(0), src_token.data_ptr<int>(), expert_offsets.data_ptr<int>(),
                           expert_offsets.numel() - 1, xs.data_ptr(), xs.size(0), x.size(1), stream_of(x));
}

void moe_combine(const Tensor& y, const Tensor& sorted_pos, const Tensor& topk_w, Tensor& out) {
  check_cuda(y, "y");
  TORCH_CHECK(y.is_contiguous() && out.is_contiguous() && y.size(1) == out.size(1) && y.size(1) % 8 == 0 &&
                  topk_w.scalar_type() == at::kFloat && topk_w.is_contiguous() && topk_w.size(0) == out.size(0) &&
                  sorted_pos.numel() >= topk_w.numel() && y.scalar_type() == out.scalar_type() && y.element_size() == 2,
              "moe_combine: shapes");
  c10::cuda::CUDAGuard g(y.device());
  mb200::launch_moe_combine(y.data_ptr(), sorted_pos.data_ptr<int>(), topk_w.data_ptr<float>(), out.data_ptr(),
                            out.size(0), out.size(1), topk_w.size(1), dtype_of(y), stream_of(y));
}

// out[rows of e] = x[rows of e] @ w[e]^T (SwiGLU-fused when swiglu) over the expert-sorted rows
int64_t moe_grouped_gemm(const Tensor& x, const Tensor& w, Tensor& out, const Tensor& expert_offsets, const Tensor& work,
                      const Tensor& n_work, int64_t bn, bool swiglu) {
  check_cuda(x, "x");
  check_cuda(w, "w");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 3 && out.dim() == 2 && x.stride(1) == 1 && w.is_contiguous() && out.stride(1) == 1 &&
                  x.size(1) == w.size(2) && x.scalar_type() == w.scalar_type() && out.scalar_type() == x.scalar_type() &&
                  x.element_size() == 2,
              "moe_grouped_gemm: x [R,K], w [E,N,K], 16-bit");
  TORCH_CHECK(out.size(0) == x.size(0) && out.size(1) == (swiglu ? w.size(1) / 2 : w.size(1)), "moe_grouped_gemm: out shape");
  TORCH_CHECK(expert_offsets.numel() == w.size(0) + 1, "moe_grouped_gemm: offsets");
  c10::cuda::CUDAGuard g(x.device());
  DeviceState& st = device_state(x.get_device());
  mb200::MoeGemmArgs a{};
  a.x = x.data_ptr();
  a.w = w.data_ptr();
  a.out = out.data_ptr();
  a.expert_offsets = expert_offsets.data_ptr<int>();
  a.work = work.data_ptr<int>();
  a.n_work = n_work.data_ptr<int>();
  a.status = st.status.data_ptr<int>();
  a.ldx = x.stride(0);
  a.ldc = out.stride(0);
  a.rows_cap = x.size(0);
  a.experts = w.size(0);
  a.n = w.size(1);
  a.k = w.size(2);
  a.bn = bn;
  a.max_work = work.size(0);
  a.swiglu = swiglu ? 1 : 0;
  a.num_sms = st.num_sms;
  a.dt = dtype_of(x);
  return mb200::launch_moe_grouped_gemm(a, stream_of(x));
}

// out = a @ b^T (+bias) (+residual) | swiglu.  a [M,K], b [N,K].
struct TpFusion {
  const uint32_t* gate_flags = nullptr;
  uint32_t gate_epoch = 0;
  int rs_tp = 0, rs_rank = 0;
  uint32_t rs_epoch = 0;
  int64_t rs_ld = 0;
  uint64_t rs_out[8] = {0}, rs_flags[8] = {0};
  int* rs_count = nullptr;
};

// fused add + RMSNorm in front of a small-batch product (see GemmArgs)
struct NormFusion {
  const Tensor* weight = nullptr;
  const Tensor* residual = nullptr;      // may stay null
  Tensor* residual_out = nullptr;        // may stay null
  double eps = 1e-6;
};

int64_t gemm_impl(const Tensor& a, const Tensor& b, Tensor& out, const c10::optional<Tensor>& bias,
                  const c10::optional<Tensor>& residual, bool swiglu, const c10::optional<Tensor>& a_scale,
                  const c10::optional<Tensor>& b_scale, const TpFusion* tp, bool b_static = false,
                  const NormFusion* norm = nullptr) {
  check_cuda(a, "a");
  check_cuda(b, "b");
  const bool is_int8 = a.scalar_type() == at::kChar;
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 &&
                  out.stride(1) == 1,
              "gemm: 2-D row-major operands");
  TORCH_CHECK(a.size(1) == b.size(1) && a.scalar_type() == b.scalar_type(), "gemm: K / dtype mismatch");
  TORCH_CHECK(out.size(0) == a.size(0) && out.size(1) == (swiglu ? b.size(0) / 2 : b.size(0)), "gemm: out shape");
  if (is_int8) {
    TORCH_CHECK(a_scale.has_value() && b_scale.has_value(), "gemm: int8 needs scales");
    TORCH_CHECK(a_scale->scalar_type() == at::kFloat && b_scale->scalar_type() == at::kFloat &&
                    a_scale->numel() == a.size(0) && b_scale->numel() == b.size(0) && a_scale->is_contiguous() &&
                    b_scale->is_contiguous(),
                "gemm: scale shapes");
  } else {
    check_half(a, "a");
    TORCH_CHECK(out.scalar_type() == a.scalar_type(), "gemm: out dtype");
  }
  check_half(out, "out");
  c10::cuda::CUDAGuard g(a.device());
  auto& st = device_state(a.get_device());
  mb200::GemmArgs args{};
  args.a = a.data_ptr();
  args.b = b.data_ptr();
  args.out = out.data_ptr();
  args.bias = bias.has_value() ? bias->data_ptr() : nullptr;
  args.residual = residual.has_value() ? residual->data_ptr() : nullptr;
  if (bias.has_value())
    TORCH_CHECK(bias->scalar_type() == out.scalar_type() && bias->numel() == b.size(0) && bias->is_contiguous(), "bias");
  if (residual.has_value())
    TORCH_CHECK(residual->scalar_type() == out.scalar_type() && residual->sizes() == out.sizes() &&
                    residual->stride(1) == 1,
                "residual");
  args.a_scale = is_int8 ? a_scale->data_ptr<float>() : nullptr;
  args.b_scale = is_int8 ? b_scale->data_ptr<float>() : nullptr;
  args.m = a.size(0);
  args.n = b.size(0);
  args.k = a.size(1);
  args.lda = a.stride(0);
  args.ldb = b.stride(0);
  args.ldc = out.stride(0);
  args.ld_res = residual.has_value() ? residual->stride(0) : 0;
  args.swiglu = swiglu ? 1 : 0;
  args.dt = dtype_of(out);
  args.is_int8 = is_int8 ? 1 : 0;
  args.workspace = st.workspace.data_ptr<float>();
  args.workspace_bytes = st.workspace.numel() * sizeof(float);
  args.counters = st.counters.data_ptr<int>();
  args.num_counters = st.counters.numel();
  args.status = st.status.data_ptr<int>();
  args.num_sms = st.num_sms;
  args.b_static = b_static ? 1 : 0;
  if (tp != nullptr) {
    args.gate_flags = tp->gate_flags;
    args.gate_epoch = tp->gate_epoch;
    args.rs_tp = tp->rs_tp;
    args.rs_rank = tp->rs_rank;
    args.rs_epoch = tp->rs_epoch;
    args.rs_ld = tp->rs_ld;
    args.rs_count = tp->rs_count;
    for (int r = 0; r < 8; ++r) {
      args.rs_out[r] = tp->rs_out[r];
      args.rs_flags[r] = tp->rs_flags[r];
    }
  }
  if (norm != nullptr) {
    const Tensor& w = *norm->weight;
    TORCH_CHECK(w.is_cuda() && w.dim() == 1 && w.is_contiguous() && w.numel() == a.size(1) && w.scalar_type() == a.scalar_type(),
                "gemm: norm weight [k] of the activations' dtype");
    args.norm_weight = w.data_ptr();
    args.norm_eps = static_cast<float>(norm->eps);
    for (const Tensor* t : {norm->residual, static_cast<const Tensor*>(norm->residual_out)}) {
      if (t == nullptr) continue;
      TORCH_CHECK(t->is_cuda() && t->dim() == 2 && t->stride(1) == 1 && t->sizes() == a.sizes() &&
                      t->scalar_type() == a.scalar_type(),
                  "gemm: residual tensors of the fused norm must match the activations");
    }
    if (norm->residual != nullptr) {
      args.norm_residual = norm->residual->data_ptr();
      args.norm_residual_ld = norm->residual->stride(0);
    }
    if (norm->residual_out != nullptr) {
      args.norm_residual_out = norm->residual_out->data_ptr();
      args.norm_residual_out_ld = norm->residual_out->stride(0);
    }
  }
  // 0 on success; a negative code (unsupported shape / launch failure) is raised by the Python caller
  return mb200::launch_gemm(args, stream_of(a));
}

// b_static: b holds model weights, which no kernel of the stream writes; the small-batch tiling may then
// start streaming them before the kernels in front of this launch have finished.
int64_t gemm(const Tensor& a, const Tensor& b, Tensor& out, const c10::optional<Tensor>& bias,
             const c10::optional<Tensor>& residual, bool swiglu, const c10::optional<Tensor>& a_scale,
             const c10::optional<Tensor>& b_scale, bool b_static) {
  return gemm_impl(a, b, out, bias, residual, swiglu, a_scale, b_scale, nullptr, b_static);
}

// out = (rmsnorm(a + residual) * norm_weight) b^T [+ bias | SwiGLU] for up to 8 rows, with a + residual (rounded to
// the activations' type) written to residual_out.  Returns 0 when launched; a negative code when the shape is not
// served by the fused kernel (the caller then runs the norm and the product separately).
int64_t gemm_norm(const Tensor& a, const Tensor& b, Tensor& out, const c10::optional<Tensor>& bias, bool swiglu,
                  const Tensor& norm_weight, const c10::optional<Tensor>& residual, c10::optional<Tensor> residual_out,
                  double eps, bool b_static) {
  NormFusion nf;
  nf.weight = &norm_weight;
  nf.eps = eps;
  if (residual.has_value()) nf.residual = &*residual;
  if (residual_out.has_value()) nf.residual_out = &*residual_out;
  return gemm_impl(a, b, out, bias, c10::nullopt, swiglu, c10::nullopt, c10::nullopt, nullptr, b_static, &nf);
}

// Tensor-parallel prefill GEMM.  gate_flags (uint32 as int32 tensor, one per 128-row tile of a) delays
// the load of a row tile until its flag reaches gate_epoch.  With rs_out_ptrs (one address per rank: this
// rank's slot in that rank's inbox) the output tiles are stored into the owners' inboxes instead of
// `out` (which only supplies shape and dtype) and rs_flag_ptrs[owner][local tile * 8 + rank] is set to
// rs_epoch per completed row tile.
int64_t gemm_tp(const Tensor& a, const Tensor& b, Tensor& out, bool swiglu, const c10::optional<Tensor>& gate_flags,
                int64_t gate_epoch, std::vector<int64_t> rs_out_ptrs, std::vector<int64_t> rs_flag_ptrs,
                const c10::optional<Tensor>& rs_count, int64_t rs_rank, int64_t rs_epoch, int64_t rs_ld) {
  TpFusion tp;
  if (gate_flags.has_value()) {
    TORCH_CHECK(gate_flags->is_cuda() && gate_flags->scalar_type() == at::kInt && gate_flags->is_contiguous() &&
                    gate_flags->numel() * 128 >= a.size(0),
                "gemm_tp: gate flags");
    tp.gate_flags = reinterpret_cast<const uint32_t*>(gate_flags->data_ptr<int>());
    tp.gate_epoch = static_cast<uint32_t>(gate_epoch);
  }
  if (!rs_out_ptrs.empty()) {
    TORCH_CHECK(rs_out_ptrs.size() == rs_flag_ptrs.size() && rs_out_ptrs.size() <= 8 && rs_count.has_value() &&
                    rs_count->is_cuda() && rs_count->scalar_type() == at::kInt && rs_count->numel() * 128 >= a.size(0),
                "gemm_tp: reduce-scatter arguments");
    tp.rs_tp = static_cast<int>(rs_out_ptrs.size());
    tp.rs_rank = static_cast<int>(rs_rank);
    tp.rs_epoch = static_cast<uint32_t>(rs_epoch);
    tp.rs_ld = rs_ld;
    tp.rs_count = rs_count->data_ptr<int>();
    for (size_t r = 0; r < rs_out_ptrs.size(); ++r) {
      tp.rs_out[r] = static_cast<uint64_t>(rs_out_ptrs[r]);
      tp.rs_flags[r] = static_cast<uint64_t>(rs_flag_ptrs[r]);
    }
  }
  return gemm_impl(a, b, out, c10::nullopt, c10::nullopt, swiglu, c10::nullopt, c10::nullopt, &tp);
}

int64_t tp_rs_add_rmsnorm_ag(const Tensor& inbox, const Tensor& tile_flags, Tensor& residual_shard, const Tensor& weight,
                             std::vector<int64_t> peer_hidden, std::vector<int64_t> peer_gather_flags, Tensor& ag_count,
                             int64_t rank, int64_t epoch, double eps) {
  check_half(residual_shard, "residual_shard");
  TORCH_CHECK(inbox.dim() == 3 && inbox.is_contiguous() && residual_shard.dim() == 2 && residual_shard.is_contiguous() &&
                  inbox.size(2) == residual_shard.size(1) && inbox.size(1) >= residual_shard.size(0) &&
                  inbox.scalar_type() == residual_shard.scalar_type() && weight.scalar_type() == residual_shard.scalar_type(),
              "tp_rs_add_rmsnorm_ag: inbox [tp, rows_cap, hidden], residual shard [rows, hidden]");
  // inbox [tp, ...]: one partial sum per rank, tile_flags tell when they are in; inbox [1, ...] with an empty
  // tile_flags tensor: the rows are already complete (e.g. the output of the expert-parallel exchange)
  const bool complete_rows = inbox.size(0) == 1 && tile_flags.numel() == 0;
  TORCH_CHECK(peer_hidden.size() == peer_gather_flags.size() && peer_hidden.size() <= 8 &&
                  (complete_rows || static_cast<int64_t>(peer_hidden.size()) == inbox.size(0)),
              "tp_rs_add_rmsnorm_ag: peer lists");
  TORCH_CHECK(tile_flags.scalar_type() == at::kInt && ag_count.scalar_type() == at::kInt &&
                  ag_count.numel() * 128 >= residual_shard.size(0) &&
                  (complete_rows || tile_flags.numel() * 16 >= residual_shard.size(0)),
              "tp_rs_add_rmsnorm_ag: flag blocks");
  c10::cuda::CUDAGuard g(residual_shard.device());
  auto& st = device_state(residual_shard.get_device());
  std::vector<uint64_t> h(peer_hidden.begin(), peer_hidden.end()), f(peer_gather_flags.begin(), peer_gather_flags.end());
  return mb200::launch_tp_rs_add_rmsnorm_ag(
      inbox.data_ptr(), inbox.size(1),
      complete_rows ? nullptr : reinterpret_cast<const uint32_t*>(tile_flags.data_ptr<int>()),
      residual_shard.data_ptr(), weight.data_ptr(), h.data(), f.data(), ag_count.data_ptr<int>(), residual_shard.size(0),
      residual_shard.size(1), static_cast<int>(h.size()), static_cast<int>(inbox.size(0)), static_cast<int>(rank),
      static_cast<uint32_t>(epoch),
      static_cast<float>(eps), dtype_of(residual_shard), st.status.data_ptr<int>(), stream_of(residual_shard));
}

// ---- expert-parallel token exchange: every list holds one address per rank (index = rank) ----
static mb200::EpA2AArgs ep_args(const std::vector<std::vector<int64_t>>& ptrs, int64_t rank, int64_t experts, int64_t hidden,
                                int64_t cap_rows, int64_t epoch) {
  TORCH_CHECK(ptrs.size() == 7, "ep: seven address lists (cnt_all, cnt_flags, recv_x, recv_meta, disp_flags, ret_y, ret_flags)");
  const size_t ep = ptrs[0].size();
  TORCH_CHECK(ep >= 1 && ep <= 8, "ep: 1..8 ranks");
  mb200::EpA2AArgs a{};
  a.ep = static_cast<int>(ep);
  a.rank = static_cast<int>(rank);
  a.experts = static_cast<int>(experts);
  a.hidden = static_cast<int>(hidden);
  a.cap_rows = static_cast<int>(cap_rows);
  a.epoch = static_cast<uint32_t>(epoch);
  uint64_t* dst[7] = {a.cnt_all, a.cnt_flags, a.recv_x, a.recv_meta, a.disp_flags, a.ret_y, a.ret_flags};
  for (int k = 0; k < 7; ++k) {
    TORCH_CHECK(ptrs[k].size() == ep, "ep: address lists of equal length");
    for (size_t r = 0; r < ep; ++r) dst[k][r] = static_cast<uint64_t>(ptrs[k][r]);
  }
  return a;
}

int64_t ep_plan(const Tensor& topk_ids, std::vector<std::vector<int64_t>> ptrs, int64_t rank, int64_t experts, int64_t hidden,
                int64_t cap_rows, int64_t epoch, int64_t bn, Tensor& pair_dst_rank, Tensor& pair_dst_row,
                Tensor& expert_offsets, Tensor& work, Tensor& n_work, Tensor& recv_rows) {
  check_cuda(topk_ids, "topk_ids");
  TORCH_CHECK(topk_ids.scalar_type() == at::kInt && topk_ids.is_contiguous() && topk_ids.dim() == 2, "ep_plan: int32 [T,k] ids");
  const int pairs = topk_ids.numel();
  for (const Tensor* t : {&pair_dst_rank, &pair_dst_row, &expert_offsets, &work, &n_work, &recv_rows})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->is_contiguous(), "ep_plan: int32 outputs");
  const auto a = ep_args(ptrs, rank, experts, hidden, cap_rows, epoch);
  TORCH_CHECK(pair_dst_rank.numel() >= pairs && pair_dst_row.numel() >= pairs &&
                  expert_offsets.numel() >= experts / a.ep + 1 && work.dim() == 2 && work.size(1) == 2,
              "ep_plan: output sizes");
  c10::cuda::CUDAGuard g(topk_ids.device());
  auto& st = device_state(topk_ids.get_device());
  return mb200::launch_ep_plan(a, topk_ids.data_ptr<int>(), pairs, static_cast<int>(bn), pair_dst_rank.data_ptr<int>(),
                               pair_dst_row.data_ptr<int>(), expert_offsets.data_ptr<int>(), work.data_ptr<int>(),
                               n_work.data_ptr<int>(), static_cast<int>(work.size(0)), recv_rows.data_ptr<int>(),
                               st.status.data_ptr<int>(), stream_of(topk_ids));
}

int64_t ep_dispatch(const Tensor& x, int64_t top_k, const Tensor& pair_dst_rank, const Tensor& pair_dst_row,
                    std::vector<std::vector<int64_t>> ptrs, int64_t rank, int64_t experts, int64_t cap_rows, int64_t epoch,
                    Tensor& done_count) {
  check_half(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.size(1) % 8 == 0 && x.stride(0) % 8 == 0, "ep_dispatch: x [T, hidden]");
  const int pairs = x.size(0) * top_k;
  TORCH_CHECK(pair_dst_rank.numel() >= pairs && pair_dst_row.numel() >= pairs && done_count.scalar_type() == at::kInt,
              "ep_dispatch: plan tensors");
  const auto a = ep_args(ptrs, rank, experts, x.size(1), cap_rows, epoch);
  c10::cuda::CUDAGuard g(x.device());
  return mb200::launch_ep_dispatch(a, x.data_ptr(), x.stride(0), pairs, static_cast<int>(top_k), pair_dst_rank.data_ptr<int>(),
                                   pair_dst_row.data_ptr<int>(), done_count.data_ptr<int>(), stream_of(x));
}

int64_t ep_return(const Tensor& ys, const Tensor& recv_rows, std::vector<std::vector<int64_t>> ptrs, int64_t rank,
                  int64_t experts, int64_t epoch, Tensor& done_count) {
  check_half(ys, "ys");
  TORCH_CHECK(ys.dim() == 2 && ys.is_contiguous() && ys.size(1) % 8 == 0, "ep_return: ys [slab rows, hidden]");
  const auto a = ep_args(ptrs, rank, experts, ys.size(1), ys.size(0), epoch);
  c10::cuda::CUDAGuard g(ys.device());
  return mb200::launch_ep_return(a, ys.data_ptr(), recv_rows.data_ptr<int>(), done_count.data_ptr<int>(), stream_of(ys));
}

int64_t tp_wait_flags(const Tensor& flags, int64_t n, int64_t epoch) {
  TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == at::kInt && flags.numel() >= n, "tp_wait_flags: int32 flags");
  c10::cuda::CUDAGuard g(flags.device());
  auto& st = device_state(flags.get_device());
  return mb200::launch_tp_wait_flags(reinterpret_cast<const uint32_t*>(flags.data_ptr<int>()), static_cast<int>(n),
                                     static_cast<uint32_t>(epoch), st.status.data_ptr<int>(), stream_of(flags));
}

void attention_prefill(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& req_to_token,
                       const Tensor& req_pool_indices, const Tensor& seq_lens, const Tensor& prefix_lens,
                       const Tensor& q_start, double scale, Tensor& out, int64_t max_q_len, bool causal, int64_t window,
                       double logit_cap) {
  check_half(q, "q");
  TORCH_CHECK(q.dim() == 3, "q must be [T,Hq,D]");
  const int64_t hd = q.size(2);
  TORCH_CHECK((hd == 64 || hd == 128 || hd == 256) && q.stride(2) == 1 && q.stride(1) == hd, "q must be [T,Hq,D], D 64, 128 or 256");
  TORCH_CHECK(out.is_contiguous() && out.sizes() == q.sizes() && out.scalar_type() == q.scalar_type(), "out");
  const int kv_fmt = check_kv_cache(k_cache, v_cache, q.scalar_type(), k_cache.size(1), hd);
  for (const Tensor* t : {&req_to_token, &req_pool_indices, &seq_lens, &prefix_lens, &q_start})
    TORCH_CHECK(t->scalar_type() == at::kInt && t->is_cuda(), "index tensors must be int32 CUDA tensors");
  TORCH_CHECK(req_to_token.dim() == 2 && req_to_token.stride(1) == 1, "req_to_token layout");
  c10::cuda::CUDAGuard g(q.device());
  auto& st = device_state(q.get_device());
  mb200::AttnArgs a{};
  a.q = q.data_ptr();
  a.k_cache = k_cache.data_ptr();
  a.v_cache = v_cache.data_ptr();
  a.kv_tok_stride = k_cache.stride(0);
  a.kv_head_stride = k_cache.stride(1);
  a.out = out.data_ptr();
  a.req_to_token = req_to_token.data_ptr<int>();
  a.req_pool_indices = req_pool_indices.data_ptr<int>();
  a.seq_lens = seq_lens.data_ptr<int>();
  a.prefix_lens = prefix_lens.data_ptr<int>();
  a.q_start = q_start.data_ptr<int>();
  a.status = st.status.data_ptr<int>();
  a.q_stride = q.stride(0);
  a.rtt_stride = req_to_token.stride(0);
  a.num_slots = k_cache.size(0);
  a.batch = req_pool_indices.numel();
  a.hq = q.size(1);
  a.hkv = k_cache.size(1);
  a.head_dim = static_cast<int>(hd);
  a.kv_fmt = kv_fmt;
  a.max_q_len = max_q_len > 0 ? max_q_len : q.size(0);
  a.num_splits = 1;
  a.is_decode = 0;
  a.non_causal = causal ? 0 : 1;
  a.scale = static_cast<float>(scale);
  a.window = static_cast<int>(window);
  a.logit_cap = static_cast<float>(logit_cap);
  a.dt = dtype_of(q);
  const int rc = mb200::launch_attention(a, stream_of(q));
  TORCH_CHECK(rc == 0, "mllm_b200 attention_prefill: unsupported configuration (code ", rc, ")");
}

void attention_decode(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& req_to_token,
                      const Tensor& req_pool_indices, const Tensor& seq_lens, double scale, Tensor& out,
                      int64_t max_seq_len, int64_t window, double logit_cap) {
  check_half(q, "q");
  TORCH_CHECK(q.dim() == 3, "q must be [B,Hq,D]");
  const int64_t hd = q.size(2);
  TORCH_CHECK((hd == 64 || hd == 128 || hd == 256) && q.stride(2) == 1 && q.stride(1) == hd, "q must be [B,Hq,D], D 64, 128 or 256");
  TORCH_CHECK(out.is_contiguous() && out.sizes() == q.sizes() && out.scalar_type() == q.scalar_type(), "out");
  const int kv_fmt = check_kv_cache(k_cache, v_cache, q.scalar_type(), k_cache.size(1), hd);
  for (const Tensor* t : {&req_to_token, &req_pool_indices, &seq_lens})
    TORCH_CHECK(t->scalar_type() == at::kInt && t->is_cuda(), "index tensors must be int32 CUDA tensors");
  c10::cuda::CUDAGuard g(q.device());
  auto& st = device_state(q.get_device());
  mb200::AttnArgs a{};
  a.batch = req_pool_indices.numel();
  TORCH_CHECK(q.size(0) == a.batch, "decode: one query row per request");
  a.hq = q.size(1);
  a.hkv = k_cache.size(1);
  a.num_splits = mb200::decode_num_splits(a.batch, a.hkv, max_seq_len > 0 ? max_seq_len : req_to_token.size(1),
                                           st.num_sms);
  Tensor part_o, part_lse;
  if (a.num_splits > 1) {
    part_o = torch::empty({a.batch, a.hq, a.num_splits, hd}, q.options().dtype(torch::kFloat32));
    part_lse = torch::empty({a.batch, a.hq, a.num_splits}, q.options().dtype(torch::kFloat32));
    a.part_o = part_o.data_ptr<float>();
    a.part_lse = part_lse.data_ptr<float>();
  }
  a.q = q.data_ptr();
  a.k_cache = k_cache.data_ptr();
  a.v_cache = v_cache.data_ptr();
  a.kv_tok_stride = k_cache.stride(0);
  a.kv_head_stride = k_cache.stride(1);
  a.out = out.data_ptr();
  a.req_to_token = req_to_token.data_ptr<int>();
  a.req_pool_indices = req_pool_indices.data_ptr<int>();
  a.seq_lens = seq_lens.data_ptr<int>();
  a.status = st.status.data_ptr<int>();
  a.q_stride = q.stride(0);
  a.rtt_stride = req_to_token.stride(0);
  a.num_slots = k_cache.size(0);
  a.head_dim = static_cast<int>(hd);
  a.kv_fmt = kv_fmt;
  a.is_decode = 1;
  a.scale = static_cast<float>(scale);
  a.window = static_cast<int>(window);
  a.logit_cap = static_cast<float>(logit_cap);
  a.dt = dtype_of(q);
  const int rc = mb200::launch_attention(a, stream_of(q));
  TORCH_CHECK(rc == 0, "mllm_b200 attention_decode: unsupported configuration (code ", rc, ")");
}

// partial sums of every rank (peer pointers) -> residual += sum ; out = rmsnorm(residual) * weight
void tp_reduce_add_rmsnorm(std::vector<int64_t> peer_data, std::vector<int64_t> peer_flags, Tensor& local_seq,
                           const c10::optional<Tensor>& residual, const c10::optional<Tensor>& weight, Tensor& out,
                           int64_t rank, int64_t row_stride, double eps) {
  check_half(out, "out");
  TORCH_CHECK(out.dim() == 2 && out.is_contiguous(), "out must be [rows, hidden] contiguous");
  TORCH_CHECK(peer_data.size() == peer_flags.size() && !peer_data.empty() && peer_data.size() <= 8, "peer lists");
  TORCH_CHECK(local_seq.scalar_type() == at::kInt && local_seq.numel() >= out.size(0), "local_seq int32 [>= rows]");
  if (residual.has_value()) TORCH_CHECK(residual->is_contiguous() && residual->sizes() == out.sizes(), "residual");
  c10::cuda::CUDAGuard g(out.device());
  auto& st = device_state(out.get_device());
  std::vector<uint64_t> d(peer_data.begin(), peer_data.end()), f(peer_flags.begin(), peer_flags.end());
  const int rc = mb200::launch_tp_reduce_add_rmsnorm(
      d.data(), f.data(), reinterpret_cast<uint32_t*>(local_seq.data_ptr<int>()),
      residual.has_value() ? residual->data_ptr() : nullptr, weight.has_value() ? weight->data_ptr() : nullptr,
      out.data_ptr(), out.size(0), out.size(1), static_cast<int>(d.size()), static_cast<int>(rank), row_stride,
      static_cast<float>(eps), dtype_of(out), st.status.data_ptr<int>(), stream_of(out));
  TORCH_CHECK(rc == 0, "mllm_b200 tp_reduce_add_rmsnorm: unsupported configuration (code ", rc, ")");
}

// Reads (and clears) the device status word; non-zero means a kernel gave up on a bounded wait
// or met an out-of-range index. Synchronises the device.
int64_t read_status(int64_t device) {
  auto& st = device_state(static_cast<int>(device));
  auto host = st.status.cpu();
  const int v = host.data_ptr<int>()[0];
  if (v != 0) st.status.zero_();
  return v;
}

int64_t launch_count() { return static_cast<int64_t>(mb200::launch_count()); }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("rmsnorm", &rmsnorm);
  m.def("fused_add_rmsnorm", &fused_add_rmsnorm);
  m.def("layernorm", &layernorm);
  m.def("act_and_mul", &act_and_mul);
  m.def("gelu_tanh", &gelu_tanh);
  m.def("embedding", &embedding);
  m.def("qk_norm_rope_kv_write", &qk_norm_rope_kv_write);
  m.def("kv_write", &kv_write);
  m.def("per_token_quant_int8", &per_token_quant_int8);
  m.def("argmax", &argmax);
  m.def("sample", &sample);
  m.def("apply_penalties", &apply_penalties);
  m.def("decode_prepare", &decode_prepare);
  m.def("ep_plan", &ep_plan);
  m.def("ep_dispatch", &ep_dispatch);
  m.def("ep_return", &ep_return);
  m.def("gemm", &gemm);
  m.def("gemm_norm", &gemm_norm);
  m.def("gemm_tp", &gemm_tp);
  m.def("w4a16_gemm", &w4a16_gemm);
  m.def("tp_rs_add_rmsnorm_ag", &tp_rs_add_rmsnorm_ag);
  m.def("tp_wait_flags", &tp_wait_flags);
  m.def("rmsnorm_gated", &rmsnorm_gated);
  m.def("gdn_conv1d_silu", &gdn_conv1d_silu);
  m.def("gdn_recurrent", &gdn_recurrent);
  m.def("gdn_chunk", &gdn_chunk);
  m.def("vision_rope_split_pad", &vision_rope_split_pad);
  m.def("vision_pos_embed_add", &vision_pos_embed_add);
  m.def("gelu_erf", &gelu_erf);
  m.def("moe_router_topk", &moe_router_topk);
  m.def("moe_align", &moe_align);
  m.def("moe_gather", &moe_gather);
  m.def("moe_combine", &moe_combine);
  m.def("moe_grouped_gemm", &moe_grouped_gemm);
  m.def("attention_prefill", &attention_prefill);
  m.def("attention_decode", &attention_decode);
  m.def("tp_reduce_add_rmsnorm", &tp_reduce_add_rmsnorm);
  m.def("read_status", &read_status);
  m.def("launch_count", &launch_count);
}
