// Decode attention for hosts that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference implementation; it exists for
// embedders of this library whose device memory is fully planned before the library is
// loaded: a runtime that hands every byte to its own arena at start-up, a real-time loop
// that must not enter the allocator (cudaMalloc may synchronise the whole device and its
// latency is unbounded), or a plug-in running under a memory quota that forbids further
// allocations.  Such callers own the inputs and outputs already; what they cannot supply is
// the temporary buffer the split-KV decode kernel needs for its per-split partial results.
// Here that buffer is a fixed array inside the library image.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch array in bytes (8 MiB). Every GPU that loads the library
// holds one copy of it until the process exits.
#define MLLM_B200_NOALLOC_SCRATCH_BYTES (8u << 20)

// Return codes.
#define MLLM_B200_NOALLOC_OK 0
#define MLLM_B200_NOALLOC_BAD_ARGUMENT 1     // null pointer, head_dim != 128, hq % hkv != 0 ...
#define MLLM_B200_NOALLOC_TOO_LARGE 2        // batch * hq * splits * 129 floats exceed the scratch array
#define MLLM_B200_NOALLOC_CUDA_ERROR 3       // a CUDA runtime call failed (set-up or launch)

// One query token per request over the slot-indexed KV pool; same mathematics and the same
// kernel as the allocating decode-attention op of this library.
//
//   q                [batch, hq, 128]   bf16 (is_fp16 = 0) or fp16 (is_fp16 = 1); q_stride =
//                                       elements between consecutive requests
//   k_cache, v_cache [num_slots, hkv, 128], same element type
//   req_to_token     [*, rtt_stride] int32: row r lists the KV slots of request r in order
//   req_pool_indices [batch] int32: the row of each request;  seq_lens [batch] int32
//   out              [batch, hq, 128] contiguous, same element type as q
//   max_seq_len      upper bound of seq_lens (sizes the split of the KV range; the bound, not
//                    the live lengths, so the launch shape is fixed for a given bound)
//
// Nothing is allocated: no cudaMalloc / cudaFree, no allocating library routine.  The first
// call on each device resolves the device address of the scratch array (one
// cudaGetSymbolAddress with that device current) and raises the kernel's shared-memory
// limit; make that first call before any stream capture begins.  All calls on a device share
// the one scratch array, which keeps the previous call's contents: every element that a call
// reads it has written first, so nothing needs clearing, but two calls whose kernels overlap
// on the GPU (different streams, no dependency between them) race on it - serialise them.
// A request larger than the array is refused with MLLM_B200_NOALLOC_TOO_LARGE;
// mllm_b200_noalloc_last_error() then says by how much.
int mllm_b200_attention_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                       const int32_t* req_to_token, const int32_t* req_pool_indices,
                                       const int32_t* seq_lens, void* out, int batch, int hq, int hkv,
                                       int head_dim, int64_t q_stride, int64_t rtt_stride, int64_t num_slots,
                                       int max_seq_len, float scale, int is_fp16, cudaStream_t stream);

// Human-readable reason of the calling thread's last non-zero return code.
const char* mllm_b200_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
