// All-reduce through the NVSwitch: multimem.ld_reduce / multimem.st on a multicast address.
//
// The buffer is symmetric memory that is also bound to an NVLink multicast object.  A load
// with reduction from the multicast address returns the SUM over every rank's copy, computed
// inside the switch (one pass over the link per rank, whatever the world size); a store to it
// lands in every rank's copy.  These are plain load / store class instructions on this rank's
// own mapping of the multicast object: no TMA, no cluster multicast.
//
// Layout of every rank's buffer (identical on all ranks):
//   [flags: 2 x kMaxChunks x kMaxRanks uint32][pad to 64 KiB][half 0: in | out][half 1: in | out]
// Calls alternate between the two halves; flags carry the call's epoch (monotonic), so nothing
// is reset between calls and CUDA-graph replays need no host update.
//
// Two variants, both one kernel, CTA c of every rank owning chunk c:
//   one shot (small messages): copy own rows into `in`, tell every peer (flag c), wait for all
//     peers' flag c, multimem.ld_reduce the chunk, then optionally residual += sum and RMSNorm,
//     write the local result.  Every rank reduces every chunk (world x the switch traffic of the
//     two-shot form, one barrier only).
//   two shot (large messages): copy, flag, wait; rank r reduces slice r of every chunk with
//     multimem.ld_reduce and broadcasts it with multimem.st into `out` of all ranks; flag again,
//     wait; copy `out` to the local result (with the optional residual / RMSNorm tail).
// Why two halves are enough: a rank passes the wait of call e + 1 only after every peer has
// signalled in call e + 1, i.e. after every peer has finished reading call e; so half e % 2 is
// free again when call e + 2 writes it.
//
// Every wait is bounded; on expiry the CTA records a status code and returns.
// Replaces HCCL's all-reduce behind omni_npu/distributed/communicator.py:52-55 and the
// add + RMSNorm that follows it (omni_npu/layers/npu_rms_norm.py:21-28).

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ll_protocol.cuh"
#include "../common/ptx.cuh"

namespace b200 {

static constexpr int kNvlsMaxChunks = 256;
static constexpr size_t kNvlsFlagBytes = 64 << 10;
static constexpr int kNvlsThreads = 512;
static constexpr int kStatusNvlsTimeout = 31;

struct NvlsParams {
  uint8_t* mc_base;              // multicast mapping of the whole buffer
  uint8_t* peer_base[kMaxRanks]; // unicast mappings (own at index rank)
  int world, rank;
  size_t half_bytes;             // bytes of one half (in + out regions)
  const __nv_bfloat16* x;        // [rows, h] input (local)
  __nv_bfloat16* out;            // [rows, h] result (local)
  __nv_bfloat16* residual;       // [rows, h] or null: residual += sum, in place
  const __nv_bfloat16* norm_w;   // [h] or null: out = RMSNorm(residual) * w
  float eps;
  int rows, h;                   // h % 8 == 0
  int rows_per_chunk;
  uint32_t* epoch;               // device word: calls so far
  uint32_t* done;                // device word: CTAs finished (zero at rest)
  int* status;
};

__device__ __forceinline__ void st_flag(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_flag(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Sum over all ranks of eight bf16 at a multicast address, accumulated in fp32 by the switch.
__device__ __forceinline__ uint4 mc_ld_reduce(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void mc_st(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// Tell every rank that this CTA's chunk reached `phase` of call `epoch`, then wait (bounded) until
// every rank said the same.  Flags: [phase][chunk][source rank].
__device__ __forceinline__ bool chunk_barrier(const NvlsParams& p, int phase, int chunk, uint32_t epoch) {
  __threadfence_system();
  __syncthreads();
  const size_t slot = (static_cast<size_t>(phase) * kNvlsMaxChunks + chunk) * kMaxRanks;
  if (threadIdx.x < p.world)
    st_flag(reinterpret_cast<uint32_t*>(p.peer_base[threadIdx.x]) + slot + p.rank, epoch);
  bool ok = true;
  if (threadIdx.x < p.world) {
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.peer_base[p.rank]) + slot + threadIdx.x;
    ok = false;
    for (uint32_t i = 0; i < kMaxFlagPolls; ++i) {
      // flags only grow; a later call's value also means "arrived"
      if (static_cast<int32_t>(ld_flag(mine) - epoch) >= 0) {
        ok = true;
        break;
      }
    }
  }
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  if (!ok && threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, kStatusNvlsTimeout);
  return ok;
}

// residual += v (when given), then v = RMSNorm(row) * w over the row held by the CTA in `srow`
// (fp32, h values); writes the bf16 result.  One CTA per row range, called row by row.
__device__ __forceinline__ void finish_row(const NvlsParams& p, int row, float* srow, float* sred) {
  const int h = p.h;
  __nv_bfloat16* res = p.residual ? p.residual + static_cast<size_t>(row) * h : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x * 8; c < h; c += kNvlsThreads * 8) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = srow[c + i];
    if (res) {
      Pack8 r;
      r.u = *reinterpret_cast<const uint4*>(res + c);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += __bfloat162float(r.h[i]);
      // the residual stream keeps the bf16-rounded sum, and the norm sees the same values
      const uint4 packed = pack8(v);
      *reinterpret_cast<uint4*>(res + c) = packed;
      r.u = packed;
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __bfloat162float(r.h[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      srow[c + i] = v[i];
      ss += v[i] * v[i];
    }
  }
  __nv_bfloat16* dst = p.out + static_cast<size_t>(row) * h;
  if (p.norm_w == nullptr) {
    __syncthreads();
    for (int c = threadIdx.x * 8; c < h; c += kNvlsThreads * 8) {
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = srow[c + i];
      *reinterpret_cast<uint4*>(dst + c) = pack8(v);
    }
    __syncthreads();
    return;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) sred[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < kNvlsThreads / 32; ++i) tot += sred[i];
  const float inv = rsqrtf(tot / h + p.eps);
  for (int c = threadIdx.x * 8; c < h; c += kNvlsThreads * 8) {
    Pack8 w;
    w.u = *reinterpret_cast<const uint4*>(p.norm_w + c);
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = srow[c + i] * inv * __bfloat162float(w.h[i]);
    *reinterpret_cast<uint4*>(dst + c) = pack8(v);
  }
  __syncthreads();
}

template <bool TWO_SHOT>
__global__ void __launch_bounds__(kNvlsThreads) nvls_all_reduce_kernel(const NvlsParams p) {
  extern __shared__ float s_row[];                   // h floats + 16 partial sums
  float* s_red = s_row + p.h;
  const int chunk = blockIdx.x;
  const uint32_t epoch = *p.epoch + 1;
  const int h = p.h;
  const int row0 = chunk * p.rows_per_chunk;
  const int nrows = min(p.rows_per_chunk, p.rows - row0);
  const size_t half_off = kNvlsFlagBytes + static_cast<size_t>(epoch & 1) * p.half_bytes;
  const size_t in_off = half_off;
  const size_t out_off = half_off + p.half_bytes / 2;
  const size_t chunk_elems = static_cast<size_t>(nrows) * h;
  const size_t chunk_off = static_cast<size_t>(row0) * h * 2;   // bytes from the start of the region
  const bool tail = p.residual != nullptr || p.norm_w != nullptr;
  bool ok = true;

  // 1. own rows of this chunk into the symmetric input region
  {
    const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(row0) * h);
    uint4* dst = reinterpret_cast<uint4*>(p.peer_base[p.rank] + in_off + chunk_off);
    for (size_t i = threadIdx.x; i < chunk_elems / 8; i += kNvlsThreads) dst[i] = src[i];
  }
  ok = chunk_barrier(p, 0, chunk, epoch);

  if (ok) {
    if (!TWO_SHOT) {
      // 2. every rank reduces the whole chunk in the switch
      for (int r = 0; r < nrows; ++r) {
        const uint8_t* mc_row = p.mc_base + in_off + chunk_off + static_cast<size_t>(r) * h * 2;
        if (tail) {
          for (int c = threadIdx.x * 8; c < h; c += kNvlsThreads * 8) {
            Pack8 v;
            v.u = mc_ld_reduce(mc_row + static_cast<size_t>(c) * 2);
#pragma unroll
            for (int i = 0; i < 8; ++i) s_row[c + i] = __bfloat162float(v.h[i]);
          }
          __syncthreads();
          finish_row(p, row0 + r, s_row, s_red);
        } else {
          uint4* dst = reinterpret_cast<uint4*>(p.out + static_cast<size_t>(row0 + r) * h);
          for (int c = threadIdx.x * 8; c < h; c += kNvlsThreads * 8)
            dst[c / 8] = mc_ld_reduce(mc_row + static_cast<size_t>(c) * 2);
        }
      }
    } else {
      // 2. this rank reduces its slice of the chunk and broadcasts it into every rank's output region
      const size_t vecs = chunk_elems / 8;
      const size_t per = (vecs + p.world - 1) / p.world;
      const size_t v0 = per * p.rank, v1 = min(vecs, v0 + per);
      for (size_t i = v0 + threadIdx.x; i < v1; i += kNvlsThreads) {
        const uint4 v = mc_ld_reduce(p.mc_base + in_off + chunk_off + i * 16);
        mc_st(p.mc_base + out_off + chunk_off + i * 16, v);
      }
      ok = chunk_barrier(p, 1, chunk, epoch);
      if (ok) {
        // 3. the complete chunk is in the local output region
        const uint8_t* loc = p.peer_base[p.rank] + out_off + chunk_off;
        for (int r = 0; r < nrows; ++r) {
          const uint4* src = reinterpret_cast<const uint4*>(loc + static_cast<size_t>(r) * h * 2);
          if (tail) {
            for (int c = threadIdx.x * 8; c < h; c += kNvlsThreads * 8) {
              Pack8 v;
              v.u = src[c / 8];
#pragma unroll
              for (int i = 0; i < 8; ++i) s_row[c + i] = __bfloat162float(v.h[i]);
            }
            __syncthreads();
            finish_row(p, row0 + r, s_row, s_red);
          } else {
            uint4* dst = reinterpret_cast<uint4*>(p.out + static_cast<size_t>(row0 + r) * h);
            for (int c = threadIdx.x * 8; c < h; c += kNvlsThreads * 8) dst[c / 8] = src[c / 8];
          }
        }
      }
    }
  }
  // the last CTA to finish advances the epoch (also after a timeout: the ranks stay in step)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.done, 1u) == gridDim.x - 1) {
      *p.done = 0u;
      *p.epoch = epoch;
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_nvls_flag_bytes() { return kNvlsFlagBytes; }
extern "C" int b200_nvls_max_chunks() { return kNvlsMaxChunks; }

// x, out [rows, h] bf16 (h % 8 == 0, h <= 16384); residual / norm_w optional.  mode 1 = one shot,
// 2 = two shot.  `half_bytes`: bytes of one half of the data area (input region + output region).
// epoch / done: device words owned by the caller (epoch counts calls, done is zero at rest).
extern "C" int b200_nvls_all_reduce(void* mc_base, void* const* peer_base, int world, int rank, size_t half_bytes,
                                    const void* x, void* out, void* residual, const void* norm_w, float eps,
                                    int rows, int h, int mode, void* epoch, void* done, int* status,
                                    cudaStream_t stream) {
  if (world < 2 || world > kMaxRanks || rows <= 0) return -1;
  if ((h & 7) != 0 || h > 16384) return -2;
  const size_t bytes = static_cast<size_t>(rows) * h * 2;
  if (bytes > half_bytes / 2) return -3;
  NvlsParams p{};
  p.mc_base = static_cast<uint8_t*>(mc_base);
  for (int r = 0; r < world; ++r) p.peer_base[r] = static_cast<uint8_t*>(peer_base[r]);
  p.world = world;
  p.rank = rank;
  p.half_bytes = half_bytes;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.residual = static_cast<__nv_bfloat16*>(residual);
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  p.eps = eps;
  p.rows = rows;
  p.h = h;
  p.epoch = static_cast<uint32_t*>(epoch);
  p.done = static_cast<uint32_t*>(done);
  p.status = status;
  // chunks of whole rows, about one per SM, at most kNvlsMaxChunks
  int sms = 148;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int chunks = rows < sms ? rows : sms;
  if (chunks > kNvlsMaxChunks) chunks = kNvlsMaxChunks;
  p.rows_per_chunk = (rows + chunks - 1) / chunks;
  chunks = (rows + p.rows_per_chunk - 1) / p.rows_per_chunk;
  const size_t smem = (static_cast<size_t>(h) + 32) * sizeof(float);
  if (mode == 2)
    nvls_all_reduce_kernel<true><<<chunks, kNvlsThreads, smem, stream>>>(p);
  else
    nvls_all_reduce_kernel<false><<<chunks, kNvlsThreads, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
