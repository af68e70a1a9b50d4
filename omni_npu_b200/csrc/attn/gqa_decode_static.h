// Split-KV paged decode attention through an entry point that allocates nothing.
//
// This entry point has no counterpart in the reference project; it exists for
// callers of this library's C ABI that cannot obtain device memory at call time.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest scratch footprint the built-in buffer can serve (bytes).  The buffer
// is part of the library image: every GPU that loads the library holds this
// much device memory until the process exits.
#define B200_GQA_DECODE_STATIC_SCRATCH_BYTES (8u << 20)

// Same computation and argument meaning as b200_gqa_decode(), but the split-KV
// partial results live in a fixed device buffer inside the library instead of
// caller-provided scratch.  See gqa_decode_static.cu for the contract.
// Returns 0 on success, a negative code otherwise (b200_gqa_decode_static_strerror).
// num_cache_blocks: blocks held by k_cache / v_cache (bounds the kernel's view of the cache).
int b200_gqa_decode_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                           const int* block_tables, const int* seq_lens, int num_seqs, int q_len,
                           int max_blocks, int block_size, int num_cache_blocks, int num_q_heads,
                           int num_kv_heads, int head_dim, long long q_stride, long long out_stride,
                           float scale, int window, int splits, cudaStream_t stream);

// Status word of the calls made on the current device so far: 0 when every CTA ran to the end,
// otherwise the code a CTA recorded when one of its bounded waits ran out (its output rows are
// then not valid).  Copies one int from the device, so it waits for the device; call it after
// synchronising the stream.  clear != 0 resets a non-zero word.  Negative: the call itself failed.
int b200_gqa_decode_static_status(int clear);

// Bytes of the built-in buffer a call with these sizes would use.
size_t b200_gqa_decode_static_required_bytes(int num_seqs, int num_kv_heads, int head_dim, int splits);

const char* b200_gqa_decode_static_strerror(int code);

#ifdef __cplusplus
}
#endif
