#include "host/cpu_oracle.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <functional>
#include <stdexcept>
#include <thread>
#include <unordered_map>

#include "host/mllm_file.h"

namespace mb200host {
namespace {

float bf16_to_f32(uint16_t v) {
  uint32_t b = static_cast<uint32_t>(v) << 16;
  float f;
  std::memcpy(&f, &b, 4);
  return f;
}

float f16_to_f32(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FF, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      exp = 113;
      while ((man & 0x400) == 0) {
        man <<= 1;
        --exp;
      }
      bits = sign | (exp << 23) | ((man & 0x3FF) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

// weights as fp32 views (fp32 tensors are used in place from the mapping; 16-bit ones are expanded once)
class Weights {
 public:
  explicit Weights(const std::string& path) : file_(path) {}
  const float* get(const std::string& name, size_t expect) {
    auto it = cache_.find(name);
    if (it != cache_.end()) return it->second;
    const MllmParam* p = file_.find(name);
    if (p == nullptr) throw std::runtime_error("cpu oracle: missing tensor " + name);
    const uint8_t* raw = file_.data(*p);
    const float* out = nullptr;
    if (p->dtype == kFloat32) {
      if (p->size != expect * 4) throw std::runtime_error("cpu oracle: wrong size for " + name);
      out = reinterpret_cast<const float*>(raw);
    } else if (p->dtype == kBFloat16 || p->dtype == kFloat16) {
      if (p->size != expect * 2) throw std::runtime_error("cpu oracle: wrong size for " + name);
      owned_.emplace_back(expect);
      const uint16_t* src = reinterpret_cast<const uint16_t*>(raw);
      for (size_t i = 0; i < expect; ++i) owned_.back()[i] = p->dtype == kBFloat16 ? bf16_to_f32(src[i]) : f16_to_f32(src[i]);
      out = owned_.back().data();
    } else {
      throw std::runtime_error("cpu oracle: unsupported dtype for " + name);
    }
    cache_[name] = out;
    return out;
  }

 private:
  MllmFile file_;
  std::unordered_map<std::string, const float*> cache_;
  std::vector<std::vector<float>> owned_;
};

void parallel_rows(int n, int threads, const std::function<void(int, int)>& fn) {
  threads = std::max(1, std::min(threads, n));
  if (threads == 1) {
    fn(0, n);
    return;
  }
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t) pool.emplace_back(fn, n * t / threads, n * (t + 1) / threads);
  for (auto& th : pool) th.join();
}

// y[T, N] = x[T, K] * w[N, K]^T
void matmul(const float* x, const float* w, float* y, int T, int N, int K, int threads) {
  parallel_rows(N, threads, [&](int n0, int n1) {
    for (int n = n0; n < n1; ++n) {
      const float* wr = w + static_cast<size_t>(n) * K;
      for (int t = 0; t < T; ++t) {
        const float* xr = x + static_cast<size_t>(t) * K;
        float a0 = 0, a1 = 0, a2 = 0, a3 = 0;
        int k = 0;
        for (; k + 4 <= K; k += 4) {
          a0 += xr[k] * wr[k];
          a1 += xr[k + 1] * wr[k + 1];
          a2 += xr[k + 2] * wr[k + 2];
          a3 += xr[k + 3] * wr[k + 3];
        }
        for (; k < K; ++k) a0 += xr[k] * wr[k];
        y[static_cast<size_t>(t) * N + n] = (a0 + a1) + (a2 + a3);
      }
    }
  });
}

void rmsnorm(const float* x, const float* w, float* y, int rows, int width, float eps) {
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + static_cast<size_t>(r) * width;
    double ss = 0;
    for (int i = 0; i < width; ++i) ss += static_cast<double>(xr[i]) * xr[i];
    const float rstd = 1.0f / std::sqrt(static_cast<float>(ss / width) + eps);
    for (int i = 0; i < width; ++i) y[static_cast<size_t>(r) * width + i] = xr[i] * rstd * w[i];
  }
}

}  // namespace

OracleResult qwen3_cpu_generate(const std::string& path, const OracleConfig& c, const std::vector<int64_t>& prompt,
                                int new_tokens, int threads) {
  if (prompt.empty() || new_tokens < 1) throw std::invalid_argument("cpu oracle: empty prompt or no tokens to generate");
  if (threads <= 0) threads = static_cast<int>(std::thread::hardware_concurrency());
  Weights W(path);
  const int H = c.hidden, D = c.head_dim, Hq = c.heads, Hkv = c.kv_heads, I = c.inter, V = c.vocab;
  const int qd = Hq * D, kd = Hkv * D, group = Hq / Hkv;
  const int max_len = static_cast<int>(prompt.size()) + new_tokens;
  const float* embed = W.get("model.embed_tokens.weight", static_cast<size_t>(V) * H);
  const float* head = c.tie ? embed : W.get("lm_head.weight", static_cast<size_t>(V) * H);
  const float* final_norm = W.get("model.norm.weight", H);
  std::vector<std::vector<float>> kc(c.layers, std::vector<float>(static_cast<size_t>(max_len) * kd));
  std::vector<std::vector<float>> vc(c.layers, std::vector<float>(static_cast<size_t>(max_len) * kd));
  std::vector<float> inv_freq(D / 2);
  for (int i = 0; i < D / 2; ++i) inv_freq[i] = 1.0f / std::pow(c.theta, static_cast<float>(2 * i) / D);

  OracleResult res;
  int cur = 0;  // tokens already in the cache
  auto forward = [&](const std::vector<int64_t>& ids, std::vector<float>* logits_out) {
    const int T = static_cast<int>(ids.size());
    std::vector<float> x(static_cast<size_t>(T) * H), nrm(x.size()), q(static_cast<size_t>(T) * qd), k(static_cast<size_t>(T) * kd),
        v(k.size()), att(q.size()), proj(x.size()), gate(static_cast<size_t>(T) * I), up(gate.size());
    for (int t = 0; t < T; ++t) {
      if (ids[t] < 0 || ids[t] >= V) throw std::out_of_range("cpu oracle: token id out of range");
      std::memcpy(&x[static_cast<size_t>(t) * H], embed + static_cast<size_t>(ids[t]) * H, sizeof(float) * H);
    }
    for (int l = 0; l < c.layers; ++l) {
      const std::string p = "model.layers." + std::to_string(l) + ".";
      rmsnorm(x.data(), W.get(p + "input_layernorm.weight", H), nrm.data(), T, H, c.eps);
      matmul(nrm.data(), W.get(p + "self_attn.q_proj.weight", static_cast<size_t>(qd) * H), q.data(), T, qd, H, threads);
      matmul(nrm.data(), W.get(p + "self_attn.k_proj.weight", static_cast<size_t>(kd) * H), k.data(), T, kd, H, threads);
      matmul(nrm.data(), W.get(p + "self_attn.v_proj.weight", static_cast<size_t>(kd) * H), v.data(), T, kd, H, threads);
      const float* qn = W.get(p + "self_attn.q_norm.weight", D);
      const float* kn = W.get(p + "self_attn.k_norm.weight", D);
      rmsnorm(q.data(), qn, q.data(), T * Hq, D, c.eps);   // per-head norm: rows of width D
      rmsnorm(k.data(), kn, k.data(), T * Hkv, D, c.eps);
      for (int t = 0; t < T; ++t) {                       // rotary embedding, pairs (i, i + D/2)
        const float pos = static_cast<float>(cur + t);
        for (int hh = 0; hh < Hq + Hkv; ++hh) {
          float* r = hh < Hq ? &q[(static_cast<size_t>(t) * Hq + hh) * D] : &k[(static_cast<size_t>(t) * Hkv + (hh - Hq)) * D];
          for (int i = 0; i < D / 2; ++i) {
            const float ang = pos * inv_freq[i], cs = std::cos(ang), sn = std::sin(ang);
            const float a = r[i], b = r[i + D / 2];
            r[i] = a * cs - b * sn;
            r[i + D / 2] = b * cs + a * sn;
          }
        }
        std::memcpy(&kc[l][static_cast<size_t>(cur + t) * kd], &k[static_cast<size_t>(t) * kd], sizeof(float) * kd);
        std::memcpy(&vc[l][static_cast<size_t>(cur + t) * kd], &v[static_cast<size_t>(t) * kd], sizeof(float) * kd);
      }
      const float scale = 1.0f / std::sqrt(static_cast<float>(D));
      parallel_rows(T * Hq, threads, [&](int r0, int r1) {
        std::vector<float> sc(max_len);
        for (int r = r0; r < r1; ++r) {
          const int t = r / Hq, hq = r % Hq, hk = hq / group;
          const int n = cur + t + 1;  // causal: keys 0 .. cur + t
          const float* qr = &q[(static_cast<size_t>(t) * Hq + hq) * D];
          float mx = -INFINITY;
          for (int j = 0; j < n; ++j) {
            const float* kr = &kc[l][static_cast<size_t>(j) * kd + static_cast<size_t>(hk) * D];
            float s = 0;
            for (int d = 0; d < D; ++d) s += qr[d] * kr[d];
            sc[j] = s * scale;
            mx = std::max(mx, sc[j]);
          }
          float den = 0;
          for (int j = 0; j < n; ++j) {
            sc[j] = std::exp(sc[j] - mx);
            den += sc[j];
          }
          float* o = &att[(static_cast<size_t>(t) * Hq + hq) * D];
          std::fill(o, o + D, 0.f);
          for (int j = 0; j < n; ++j) {
            const float pw = sc[j] / den;
            const float* vr = &vc[l][static_cast<size_t>(j) * kd + static_cast<size_t>(hk) * D];
            for (int d = 0; d < D; ++d) o[d] += pw * vr[d];
          }
        }
      });
      matmul(att.data(), W.get(p + "self_attn.o_proj.weight", static_cast<size_t>(H) * qd), proj.data(), T, H, qd, threads);
      for (size_t i = 0; i < x.size(); ++i) x[i] += proj[i];
      rmsnorm(x.data(), W.get(p + "post_attention_layernorm.weight", H), nrm.data(), T, H, c.eps);
      matmul(nrm.data(), W.get(p + "mlp.gate_proj.weight", static_cast<size_t>(I) * H), gate.data(), T, I, H, threads);
      matmul(nrm.data(), W.get(p + "mlp.up_proj.weight", static_cast<size_t>(I) * H), up.data(), T, I, H, threads);
      for (size_t i = 0; i < gate.size(); ++i) gate[i] = gate[i] / (1.0f + std::exp(-gate[i])) * up[i];
      matmul(gate.data(), W.get(p + "mlp.down_proj.weight", static_cast<size_t>(H) * I), proj.data(), T, H, I, threads);
      for (size_t i = 0; i < x.size(); ++i) x[i] += proj[i];
    }
    cur += T;
    std::vector<float> last(H);
    rmsnorm(&x[static_cast<size_t>(T - 1) * H], final_norm, last.data(), 1, H, c.eps);
    logits_out->assign(V, 0.f);
    matmul(last.data(), head, logits_out->data(), 1, V, H, threads);
  };
  auto argmax = [](const std::vector<float>& v) {
    return static_cast<int64_t>(std::max_element(v.begin(), v.end()) - v.begin());
  };

  using clk = std::chrono::steady_clock;
  std::vector<float> logits;
  auto t0 = clk::now();
  forward(prompt, &logits);
  res.prefill_seconds = std::chrono::duration<double>(clk::now() - t0).count();
  res.prefill_logits = logits;
  t0 = clk::now();
  for (int i = 0; i < new_tokens; ++i) {
    const int64_t tok = argmax(logits);
    res.tokens.push_back(tok);
    res.last_logits = logits;
    if (i + 1 < new_tokens) forward({tok}, &logits);
  }
  res.decode_seconds = std::chrono::duration<double>(clk::now() - t0).count();
  return res;
}

}  // namespace mb200host
