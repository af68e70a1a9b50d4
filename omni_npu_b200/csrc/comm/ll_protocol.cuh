// Device-side pieces of the push ("LL") all-reduce protocol, shared by the stand-alone
// all-reduce kernel and by GEMM kernels that push their output tiles to peer GPUs.
//
// Every rank PUSHES 16-byte vectors into a slot of every peer's receive buffer; the payload
// itself tells the receiver when it has arrived: slots are pre-filled with a sentinel bit
// pattern (the bf16 pair -0.0/-0.0 in every 32-bit word, which senders never emit: they turn
// such a word into +0.0/+0.0), and the receiver polls its OWN memory until the four words of
// a vector differ from the sentinel.  Receive buffer of a rank:
// [3 slots][world source ranks][slot_vecs vectors]; call e uses slot e % 3 and re-arms slot
// (e + 2) % 3 at its end.  `epoch` points at four device words: the epoch and the number of
// vectors per source that the last call in each slot wrote.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

static constexpr int kMaxRanks = 8;
static constexpr uint32_t kMaxFlagPolls = 1u << 24;   // ~ a second of polling

union Pack8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

__device__ __forceinline__ void add8(float (&acc)[8], const uint4& v) {
  Pack8 p;
  p.u = v;
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] += __bfloat162float(p.h[i]);
}

__device__ __forceinline__ uint4 pack8(const float (&acc)[8]) {
  Pack8 p;
#pragma unroll
  for (int i = 0; i < 8; ++i) p.h[i] = __float2bfloat16(acc[i]);
  return p.u;
}

static constexpr uint32_t kLLSentinel = 0x80008000u;

struct LLGroup {
  uint4* recv[kMaxRanks];     // peer-mapped receive buffers (own at index rank)
  uint32_t* epoch;            // this rank's [epoch, vectors written in slot 0, 1, 2] (device memory)
  int world;
  int rank;
  long long slot_vecs;        // capacity of one (slot, source) region in 16-byte vectors
};

__device__ __forceinline__ uint4 ll_sanitize(uint4 v) {
  if (v.x == kLLSentinel) v.x = 0u;
  if (v.y == kLLSentinel) v.y = 0u;
  if (v.z == kLLSentinel) v.z = 0u;
  if (v.w == kLLSentinel) v.w = 0u;
  return v;
}

__device__ __forceinline__ void ll_store(uint4* p, const uint4& v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

__device__ __forceinline__ uint4 ll_load(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Poll until the vector has arrived (bounded).  Returns false on expiry.
__device__ __forceinline__ bool ll_wait(const uint4* p, uint4& v) {
  for (uint32_t i = 0; i < kMaxFlagPolls; ++i) {
    v = ll_load(p);
    if (v.x != kLLSentinel && v.y != kLLSentinel && v.z != kLLSentinel && v.w != kLLSentinel) return true;
  }
  return false;
}

}  // namespace b200
