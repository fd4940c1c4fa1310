// Allocation-free decode attention: see no_alloc.h for who needs it and for the contract.
//
// The split-KV decode kernel writes one partial (output row, log-sum-exp) per request, head
// and split and a second kernel merges them.  The allocating op gets that buffer from the
// framework's allocator; here it lives in a file-scope __device__ array.  In host code the
// array's name is only a stand-in for the symbol - it is not a device address - so the
// address is resolved once per device with cudaGetSymbolAddress and that pointer is what the
// kernel receives.
#include <cstdio>
#include <mutex>

#include "kernels.h"
#include "no_alloc.h"

namespace {

constexpr size_t kScratchFloats = MLLM_B200_NOALLOC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_noalloc_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
struct PerDevice {
  std::once_flag once;
  float* scratch = nullptr;
  int num_sms = 0;
  cudaError_t err = cudaSuccess;
};
PerDevice g_dev[kMaxDevices];

thread_local char g_last_error[256] = "";

int fail(int code, const char* fmt, long long a = 0, long long b = 0) {
  std::snprintf(g_last_error, sizeof(g_last_error), fmt, a, b);
  return code;
}

// Runs once per device with that device current: resolve the scratch address, read the SM count.
PerDevice* setup_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  PerDevice* pd = &g_dev[dev];
  std::call_once(pd->once, [pd, dev] {
    void* ptr = nullptr;
    pd->err = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (pd->err == cudaSuccess) {
      pd->scratch = static_cast<float*>(ptr);
      pd->err = cudaDeviceGetAttribute(&pd->num_sms, cudaDevAttrMultiProcessorCount, dev);
    }
  });
  return pd;
}

}  // namespace

extern "C" const char* mllm_b200_noalloc_last_error(void) { return g_last_error; }

extern "C" int mllm_b200_attention_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                                  const int32_t* req_to_token, const int32_t* req_pool_indices,
                                                  const int32_t* seq_lens, void* out, int batch, int hq, int hkv,
                                                  int head_dim, int64_t q_stride, int64_t rtt_stride,
                                                  int64_t num_slots, int max_seq_len, float scale, int is_fp16,
                                                  cudaStream_t stream) {
  g_last_error[0] = '\0';
  if (q == nullptr || k_cache == nullptr || v_cache == nullptr || req_to_token == nullptr ||
      req_pool_indices == nullptr || seq_lens == nullptr || out == nullptr)
    return fail(MLLM_B200_NOALLOC_BAD_ARGUMENT, "null pointer argument");
  if (head_dim != 128) return fail(MLLM_B200_NOALLOC_BAD_ARGUMENT, "head_dim must be 128, got %lld", head_dim);
  if (batch < 0 || hq <= 0 || hkv <= 0 || hq % hkv != 0 || hq / hkv > 128 || max_seq_len <= 0)
    return fail(MLLM_B200_NOALLOC_BAD_ARGUMENT, "bad shape: hq=%lld hkv=%lld", hq, hkv);
  if (batch == 0) return MLLM_B200_NOALLOC_OK;

  PerDevice* pd = setup_current_device();
  if (pd == nullptr) return fail(MLLM_B200_NOALLOC_CUDA_ERROR, "no current CUDA device");
  if (pd->err != cudaSuccess)
    return fail(MLLM_B200_NOALLOC_CUDA_ERROR, "set-up failed: cudaGetSymbolAddress / attribute query, error %lld",
                static_cast<long long>(pd->err));

  const int splits = mb200::decode_num_splits(batch, hkv, max_seq_len, pd->num_sms);
  // per (request, head, split): 128 output floats + 1 log-sum-exp
  const size_t need = static_cast<size_t>(batch) * hq * splits * (128 + 1);
  if (splits > 1 && need > kScratchFloats)
    return fail(MLLM_B200_NOALLOC_TOO_LARGE,
                "decode needs %lld scratch floats but the built-in array holds %lld; lower batch or max_seq_len",
                static_cast<long long>(need), static_cast<long long>(kScratchFloats));

  mb200::AttnArgs a{};
  a.q = q;
  a.k_cache = k_cache;
  a.v_cache = v_cache;
  a.kv_tok_stride = static_cast<int64_t>(hkv) * head_dim;   // the documented slot-major layout
  a.kv_head_stride = head_dim;
  a.out = out;
  a.part_o = splits > 1 ? pd->scratch : nullptr;
  a.part_lse = splits > 1 ? pd->scratch + static_cast<size_t>(batch) * hq * splits * 128 : nullptr;
  a.req_to_token = req_to_token;
  a.req_pool_indices = req_pool_indices;
  a.seq_lens = seq_lens;
  a.prefix_lens = nullptr;
  a.q_start = nullptr;
  a.status = nullptr;
  a.q_stride = q_stride;
  a.rtt_stride = rtt_stride;
  a.num_slots = num_slots;
  a.batch = batch;
  a.hq = hq;
  a.hkv = hkv;
  a.head_dim = head_dim;
  a.max_q_len = 1;
  a.num_splits = splits;
  a.is_decode = 1;
  a.scale = scale;
  a.dt = is_fp16 ? mb200::kF16 : mb200::kBF16;
  const int rc = mb200::launch_attention(a, stream);
  if (rc != 0) return fail(MLLM_B200_NOALLOC_CUDA_ERROR, "kernel launch failed (code %lld)", rc);
  return MLLM_B200_NOALLOC_OK;
}
