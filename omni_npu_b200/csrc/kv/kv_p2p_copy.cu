// GPU-to-GPU KV-cache block copy for prefill/decode disaggregation.
//
// The decode instance maps the prefill instance's KV-cache tensors (CUDA IPC) and
// pulls the blocks of a request with ONE launch that covers every layer tensor:
// CTA (pair p, tensor l) copies block src_block[p] of remote tensor l into block
// dst_block[p] of local tensor l with 16-byte loads over NVLink (plain ld/st; the
// destination is always this GPU's own memory).
//
// Replaces llm_datadist's pull_blocks (omni_npu/connector/llmdatadist_manager_v1.py:303-349).

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

struct KvCopyTensor {
  const char* src;      // remote tensor base
  char* dst;            // local tensor base
  long long block_bytes;
};

__global__ void __launch_bounds__(256)
kv_p2p_copy_kernel(const KvCopyTensor* __restrict__ tensors, const int* __restrict__ src_blocks,
                   const int* __restrict__ dst_blocks, int num_pairs) {
  const int pair = blockIdx.x;
  const KvCopyTensor t = tensors[blockIdx.y];
  const long long nvec = t.block_bytes >> 4;
  const uint4* src = reinterpret_cast<const uint4*>(t.src + static_cast<long long>(src_blocks[pair]) * t.block_bytes);
  uint4* dst = reinterpret_cast<uint4*>(t.dst + static_cast<long long>(dst_blocks[pair]) * t.block_bytes);
  // several chunks of a block may be assigned to different CTAs along z
  const long long per = (nvec + gridDim.z - 1) / gridDim.z;
  const long long b = per * blockIdx.z, e = min(nvec, b + per);
  long long i = b + threadIdx.x;
  for (; i + 3LL * blockDim.x < e; i += 4LL * blockDim.x) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldcv(src + i + u * blockDim.x);
#pragma unroll
    for (int u = 0; u < 4; ++u) dst[i + u * blockDim.x] = v[u];
  }
  for (; i < e; i += blockDim.x) dst[i] = __ldcv(src + i);
}

}  // namespace b200

// tensors: device array of num_tensors descriptors; src_blocks / dst_blocks: device int arrays.
extern "C" int b200_kv_p2p_copy(const void* tensors, int num_tensors, const int* src_blocks,
                                const int* dst_blocks, int num_pairs, long long max_block_bytes,
                                cudaStream_t stream) {
  if (num_pairs <= 0 || num_tensors <= 0) return 0;
  if (num_tensors > 65535) return -1;
  int z = static_cast<int>((max_block_bytes + (64 << 10) - 1) / (64 << 10));   // ~64 KiB per CTA
  if (z < 1) z = 1;
  if (z > 16) z = 16;
  dim3 grid(num_pairs, num_tensors, z);
  b200::kv_p2p_copy_kernel<<<grid, 256, 0, stream>>>(static_cast<const b200::KvCopyTensor*>(tensors),
                                                     src_blocks, dst_blocks, num_pairs);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
