// Argument block shared by the paged GQA attention kernels (prefill and decode variants).
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace b200 {

static constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
  const __nv_bfloat16* q;     // [T, Hq, DQK]
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  __nv_bfloat16* out;         // [T, Hq, DV]
  float* lse;                 // [T, Hq] or null (natural log)
  const int* block_tables;    // [B, max_blocks]
  const int* cu_q;            // [B+1] query start offsets (prefill) / null
  const int* seq_lens;        // [B] total kv length including this step's tokens
  int max_blocks;
  int block_size;
  int Hq, Hk;
  long long q_stride;         // elements between tokens in q
  long long out_stride;       // elements between tokens in out
  float scale_log2;           // softmax scale * log2(e)
  int causal;
  int window;                 // sliding window (keys older than pos - window + 1 masked), 0 = off
  int sink;                   // leading keys [0, sink) stay visible whatever the window (0 = none)
  // decode only
  int q_len;                  // tokens per sequence in this step (>=1)
  int splits;
  float* o_part;              // [B, splits, 16, DV] fp32
  float* lse_part;            // [B, splits, 16]   (per kv head: index includes head)
  int* status;                // error word for bounded waits (may be null)
  int num_cache_blocks;       // blocks in the cache tensors (bounds the TMA view)
  int* work_counter;          // persistent decode: [ticket, finished CTAs], zero at rest; null = strided items
  int persistent;             // decode: 1 = persistent-CTA kernel when the problem allows it
};

}  // namespace b200
