// Stand-alone fp32 CPU implementation of the Qwen3 decoder (batch 1): the oracle and timed CPU baseline
// for the "Qwen3-0.6B-shaped, prefill 128 tokens, greedy-decode 32" configuration.  It shares no code
// with the GPU path or with PyTorch: weights come from a `.mllm` file, the math is plain loops
// (RMSNorm with fused residual order, per-head q/k RMSNorm, NeoX rotary embedding, causal GQA attention
// over a growing KV cache, SwiGLU MLP, tied or untied LM head, greedy argmax), parallelised over output
// rows with std::thread.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace mb200host {

struct OracleConfig {
  int vocab = 0, hidden = 0, inter = 0, layers = 0, heads = 0, kv_heads = 0, head_dim = 0;
  float eps = 1e-6f, theta = 1e6f;
  bool tie = true;
};

struct OracleResult {
  std::vector<int64_t> tokens;       // generated ids
  std::vector<float> prefill_logits; // logits after the prompt
  std::vector<float> last_logits;    // logits that produced the last generated token
  double prefill_seconds = 0, decode_seconds = 0;
};

OracleResult qwen3_cpu_generate(const std::string& mllm_path, const OracleConfig& cfg, const std::vector<int64_t>& prompt,
                                int new_tokens, int threads);

}  // namespace mb200host
