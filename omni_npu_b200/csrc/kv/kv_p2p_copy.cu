// GPU-to-GPU KV-cache block copy for prefill/decode disaggregation.
//
// The decode instance maps the prefill instance's KV-cache tensors (CUDA IPC) and
// pulls the blocks of a request with ONE launch that covers every layer tensor:
// block src_block[p] of remote tensor l goes into block dst_block[p] of local tensor l
// with 16-byte loads over NVLink (plain ld/st; the destination is always this GPU's
// own memory).
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

// Work items are (block pair, tensor, 32 KiB chunk), flattened; a fixed grid of CTAs strides over
// them.  Every thread keeps eight 16-byte loads in flight (32 KiB per CTA): a pull over NVLink is
// latency bound (a few microseconds per round trip), so bytes in flight, not CTA count, set the
// bandwidth.
static constexpr int kKvChunkBytes = 32 << 10;

__global__ void __launch_bounds__(256)
kv_p2p_copy_kernel(const KvCopyTensor* __restrict__ tensors, const int* __restrict__ src_blocks,
                   const int* __restrict__ dst_blocks, int num_pairs, int num_tensors, int chunks_per_block) {
  const long long total = static_cast<long long>(num_pairs) * num_tensors * chunks_per_block;
  for (long long item = blockIdx.x; item < total; item += gridDim.x) {
    const int chunk = static_cast<int>(item % chunks_per_block);
    const int ti = static_cast<int>((item / chunks_per_block) % num_tensors);
    const int pair = static_cast<int>(item / (static_cast<long long>(chunks_per_block) * num_tensors));
    const KvCopyTensor t = tensors[ti];
    const long long b = static_cast<long long>(chunk) * kKvChunkBytes;
    if (b >= t.block_bytes) continue;
    const long long nvec = (min(t.block_bytes, b + kKvChunkBytes) - b) >> 4;
    const uint4* src = reinterpret_cast<const uint4*>(t.src + static_cast<long long>(src_blocks[pair]) * t.block_bytes + b);
    uint4* dst = reinterpret_cast<uint4*>(t.dst + static_cast<long long>(dst_blocks[pair]) * t.block_bytes + b);
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const long long i = threadIdx.x + u * 256LL;
      if (i < nvec) v[u] = __ldcv(src + i);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const long long i = threadIdx.x + u * 256LL;
      if (i < nvec) dst[i] = v[u];
    }
  }
}

}  // namespace b200

// tensors: device array of num_tensors descriptors; src_blocks / dst_blocks: device int arrays.
// Block sizes are multiples of 16 bytes.
extern "C" int b200_kv_p2p_copy(const void* tensors, int num_tensors, const int* src_blocks,
                                const int* dst_blocks, int num_pairs, long long max_block_bytes,
                                cudaStream_t stream) {
  if (num_pairs <= 0 || num_tensors <= 0) return 0;
  if (num_tensors > 65535 || max_block_bytes <= 0) return -1;
  const int chunks = static_cast<int>((max_block_bytes + b200::kKvChunkBytes - 1) / b200::kKvChunkBytes);
  const long long total = static_cast<long long>(num_pairs) * num_tensors * chunks;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  const long long cap = 8LL * sms;                       // 8 CTAs of 256 threads per SM
  const int grid = static_cast<int>(total < cap ? total : cap);
  b200::kv_p2p_copy_kernel<<<grid, 256, 0, stream>>>(static_cast<const b200::KvCopyTensor*>(tensors),
                                                     src_blocks, dst_blocks, num_pairs, num_tensors, chunks);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Reads (and thereby clears) the runtime's last-error state.  A runtime call made outside torch
// that fails, e.g. pinning a mapping that cannot be pinned, leaves its code there, and the next
// unrelated call that checks for errors would report it.
extern "C" int b200_cuda_take_last_error() { return static_cast<int>(cudaGetLastError()); }
