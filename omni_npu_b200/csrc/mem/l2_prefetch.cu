// L2 prefetch hints: ask the memory system to bring a byte range (the next layer's
// weights, a KV block) into L2 while other kernels run.  One thread issues one
// `cp.async.bulk.prefetch.L2` per 32 KiB chunk; the instruction does not wait for the
// data, so the kernel retires in a few microseconds and the fills proceed in the
// background.  Launch it on a side stream so it overlaps the compute stream.
//
// Counterpart of the `npu_prefetch` hints issued by omni_npu/v1/layers/prefetch.py:9-77.

#include <cuda_runtime.h>

#include <cstdint>

namespace b200 {

static constexpr unsigned kPrefetchChunk = 32768;

__global__ void l2_prefetch_kernel(const char* __restrict__ base, unsigned long long bytes) {
  const unsigned long long idx = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const unsigned long long off = idx * kPrefetchChunk;
  if (off >= bytes) return;
  unsigned long long left = bytes - off;
  unsigned size = left < kPrefetchChunk ? static_cast<unsigned>(left) : kPrefetchChunk;
  size &= ~15u;   // the bulk prefetch takes a multiple of 16 bytes
  if (size == 0) return;
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + off), "r"(size) : "memory");
}

}  // namespace b200

// ptr must be 16-byte aligned; at most `max_bytes` of the range are requested.
extern "C" int b200_l2_prefetch(const void* ptr, unsigned long long bytes, unsigned long long max_bytes,
                                cudaStream_t stream) {
  if (ptr == nullptr || bytes == 0) return 0;
  if (reinterpret_cast<uintptr_t>(ptr) & 15u) return -1;
  if (max_bytes > 0 && bytes > max_bytes) bytes = max_bytes;
  const unsigned long long chunks = (bytes + b200::kPrefetchChunk - 1) / b200::kPrefetchChunk;
  const int threads = 128;
  const unsigned blocks = static_cast<unsigned>((chunks + threads - 1) / threads);
  b200::l2_prefetch_kernel<<<blocks, threads, 0, stream>>>(static_cast<const char*>(ptr), bytes);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
