// b200_gqa_decode_static: paged GQA decode attention with split-KV whose scratch
// memory is a fixed device array compiled into this library.
//
// Who needs this.  The regular entry point, b200_gqa_decode(), wants the caller
// to hand in fp32 scratch for the per-split partial outputs.  Inside this
// framework that scratch comes from torch's caching allocator.  Two kinds of
// callers have no such source:
//   * programs that use the library through its C symbols from a runtime that
//     is not PyTorch (a C++ serving process, another language's FFI): they have
//     no caching allocator to borrow from, and a raw cudaMalloc/cudaFree in the
//     decode loop synchronises the whole device and stalls every other stream;
//   * processes whose device memory is already spoken for: the engine sizes the
//     KV cache to fill what is left of HBM after profiling, so a late request
//     for a few more MiB can fail outright.
// For them the scratch lives here, in a file-scope __device__ array of
// B200_GQA_DECODE_STATIC_SCRATCH_BYTES (8 MiB).  That is enough for, e.g.,
// 16 sequences x 8 KV heads x 4 splits at head size 128 (4.1 MiB).  Larger
// problems are refused with kErrTooLarge; use b200_gqa_decode() with your own
// scratch for those.
//
// Contract.
//   * No cudaMalloc, cudaFree or allocating library routine is called, on any call.
//   * The first call on each device resolves the device address of the array
//     (cudaGetSymbolAddress, with that device current) and caches it.  That
//     first call per device does set-up work beyond a kernel launch, so make it
//     early: before the serving loop and before any stream capture begins.
//   * All calls on a device share the one array, and it keeps whatever the
//     previous call left in it.  Nothing in it has to start at zero: every entry
//     the merge step reads is written by the split kernel of the same call.
//     Because the array is shared, two calls whose kernels overlap on the GPU
//     (different streams, no ordering between them) race on it; order them.
//   * The current device at call time must be the one that owns the pointers.
//   * Bounded waits.  The kernel's waits on its own TMA copies have an iteration
//     limit; a CTA that gives up records a code in a status word and leaves its
//     output rows unwritten.  The status word is a second file-scope __device__
//     variable (no allocation); read it with b200_gqa_decode_static_status()
//     after the stream has been synchronised.  0 means every CTA finished.
//   * num_cache_blocks is the number of blocks in k_cache / v_cache.  The TMA
//     view of the cache is sized from it, so a block-table entry beyond the
//     cache reads zeros instead of memory that belongs to something else.
//   * Host threads: the per-device address cache is filled under std::call_once,
//     so first calls from several threads are safe.  The cached addresses do not
//     survive cudaDeviceReset(); a process that resets a device must not call
//     this entry point on it afterwards.

#include "gqa_decode_static.h"

#include <stdint.h>

#include <mutex>

extern "C" size_t b200_gqa_decode_scratch_bytes(int B, int Hk, int D, int splits);
extern "C" int b200_gqa_decode(const void* q, const void* k_cache, const void* v_cache, void* out,
                               float* lse, const int* block_tables, const int* seq_lens, int B,
                               int q_len, int max_blocks, int block_size, int Hq, int Hk, int D,
                               long long q_stride, long long out_stride, float scale, int window,
                               int splits, void* scratch, int num_cache_blocks, int* status,
                               cudaStream_t stream);

namespace {

// In host code this name is only a handle for the runtime; it is NOT a device
// address and must never be passed to a kernel.  The address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_decode_scratch[B200_GQA_DECODE_STATIC_SCRATCH_BYTES];

// Set by a CTA whose bounded wait ran out (same codes as the status word of b200_gqa_decode).
static __device__ int g_decode_status;

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {nullptr};
int* g_status_addr[kMaxDevices] = {nullptr};
int g_setup_rc[kMaxDevices] = {0};
std::once_flag g_once[kMaxDevices];

enum : int {
  kErrTooLarge = -100,
  kErrNoDevice = -101,
  kErrSymbol = -102,
  kErrBadSplits = -103,
  kErrBadCache = -104,
};

// Device addresses of the scratch array and the status word on the current device,
// resolved once per device (with that device current) and zeroing the status word.
int addrs_for_current_device(void** scratch, int** status) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return kErrNoDevice;
  std::call_once(g_once[dev], [dev] {
    void* p = nullptr;
    void* st = nullptr;
    if (cudaGetSymbolAddress(&p, g_decode_scratch) != cudaSuccess || p == nullptr ||
        cudaGetSymbolAddress(&st, g_decode_status) != cudaSuccess || st == nullptr ||
        cudaMemset(st, 0, sizeof(int)) != cudaSuccess) {
      (void)cudaGetLastError();
      g_setup_rc[dev] = kErrSymbol;
      return;
    }
    g_scratch_addr[dev] = p;
    g_status_addr[dev] = static_cast<int*>(st);
  });
  if (g_setup_rc[dev] != 0) return g_setup_rc[dev];
  *scratch = g_scratch_addr[dev];
  *status = g_status_addr[dev];
  return 0;
}

}  // namespace

extern "C" size_t b200_gqa_decode_static_required_bytes(int num_seqs, int num_kv_heads, int head_dim,
                                                        int splits) {
  return b200_gqa_decode_scratch_bytes(num_seqs, num_kv_heads, head_dim, splits);
}

extern "C" const char* b200_gqa_decode_static_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case kErrTooLarge:
      return "problem needs more than the built-in 8 MiB scratch buffer; call b200_gqa_decode with "
             "caller-provided scratch instead";
    case kErrNoDevice: return "no current CUDA device (or device ordinal >= 64)";
    case kErrSymbol: return "cudaGetSymbolAddress failed for the built-in scratch buffer";
    case kErrBadSplits: return "splits must be >= 1";
    case kErrBadCache: return "num_cache_blocks must be >= 1";
    default: return "error reported by the decode attention launcher (see b200_gqa_decode)";
  }
}

extern "C" int b200_gqa_decode_static(const void* q, const void* k_cache, const void* v_cache,
                                      void* out, const int* block_tables, const int* seq_lens,
                                      int num_seqs, int q_len, int max_blocks, int block_size,
                                      int num_cache_blocks, int num_q_heads, int num_kv_heads,
                                      int head_dim, long long q_stride, long long out_stride,
                                      float scale, int window, int splits, cudaStream_t stream) {
  if (splits < 1) return kErrBadSplits;
  if (num_cache_blocks < 1) return kErrBadCache;
  const size_t need = b200_gqa_decode_scratch_bytes(num_seqs, num_kv_heads, head_dim, splits);
  if (need > static_cast<size_t>(B200_GQA_DECODE_STATIC_SCRATCH_BYTES)) return kErrTooLarge;
  void* scratch = nullptr;
  int* status = nullptr;
  const int rc = addrs_for_current_device(&scratch, &status);
  if (rc != 0) return rc;
  return b200_gqa_decode(q, k_cache, v_cache, out, nullptr, block_tables, seq_lens, num_seqs, q_len,
                         max_blocks, block_size, num_q_heads, num_kv_heads, head_dim, q_stride,
                         out_stride, scale, window, splits, splits > 1 ? scratch : nullptr,
                         num_cache_blocks, status, stream);
}

extern "C" int b200_gqa_decode_static_status(int clear) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return kErrNoDevice;
  if (g_status_addr[dev] == nullptr) return 0;      // no call has been made on this device yet
  int v = 0;
  if (cudaMemcpy(&v, g_status_addr[dev], sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
    (void)cudaGetLastError();
    return kErrSymbol;
  }
  if (clear && v != 0) (void)cudaMemset(g_status_addr[dev], 0, sizeof(int));
  return v;
}
