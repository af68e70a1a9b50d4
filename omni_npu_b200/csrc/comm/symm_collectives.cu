// Collectives over peer-mapped ("symmetric") device memory: every rank of a group
// owns one data buffer and one signal pad, all ranks have all of them mapped
// (CUDA IPC), and the kernels below move data with plain loads / stores over
// NVLink + NVSwitch.  One process per GPU; every rank launches the same kernel.
//
//  * all_reduce, one shot   (small messages): stage own data, flag barrier,
//        every rank reads all ranks' data and sums in rank order.
//  * all_reduce, two shot   (large messages): stage, barrier, each rank reduces
//        its slice from all peers (reduce-scatter), barrier, each rank gathers
//        the reduced slices from all peers (all-gather).
//  * both optionally fuse  "+ residual, RMSNorm"  into the final pass, which is
//        what follows the o_proj / down_proj all-reduce in a decoder layer.
//  * all_gather / reduce_scatter for the sequence-parallel residual stream.
//
// Synchronisation: a monotonically increasing epoch kept in device memory (so
// CUDA-graph replays need no host update) and per-(rank, block) flags in every
// rank's signal pad.  Data buffers are split in two halves used alternately
// (epoch parity): the barrier that opens call n+1 proves every rank has left
// call n, so half (n & 1) is free again when call n+2 stages into it.
// Every flag wait is bounded; on expiry the kernel records a status code and
// returns without touching peer memory again.
//
// Replaces HCCL all_reduce / all_gather / reduce_scatter call sites of the
// reference (omni_npu/distributed/communicator.py:52-83) on the latency-bound
// paths; NCCL remains the transport for everything else.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "ll_protocol.cuh"

namespace b200 {

static constexpr int kMaxCommBlocks = 144;

struct SymmGroup {
  void* data[kMaxRanks];        // peer-mapped data buffers (this rank's own at index rank)
  uint32_t* signal[kMaxRanks];  // peer-mapped signal pads: [kMaxRanks][kMaxCommBlocks] flags, then epoch
  int world;
  int rank;
  size_t half_bytes;            // bytes of one half of a data buffer
};

// Layout of a signal pad (uint32 words):
//   [0, kMaxRanks*kMaxCommBlocks)        flags[src_rank][block]
//   [kMaxRanks*kMaxCommBlocks]           epoch counter (local use only)
//   [kAgFlagWord, kAgFlagWord + kMaxRanks)  "rank r has staged its block" flags of the fused all-gather GEMM
static constexpr int kEpochWord = kMaxRanks * kMaxCommBlocks;
static constexpr int kAgFlagWord = kEpochWord + 4;
//   [kRsFlagWord, kRsFlagWord + kMaxRanks)  "rank r has pushed all its partial rows" flags of the fused GEMM + reduce-scatter
static constexpr int kRsFlagWord = kAgFlagWord + kMaxRanks;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Barrier between block `blockIdx.x` of every rank.  Thread t < world signals
// peer t and waits for peer t.  Returns false if a peer did not show up in time.
__device__ __forceinline__ bool block_barrier(const SymmGroup& g, uint32_t epoch, int* status) {
  __syncthreads();
  bool ok = true;
  if (threadIdx.x < g.world) {
    __threadfence_system();
    const int peer = threadIdx.x;
    st_release_sys(g.signal[peer] + g.rank * kMaxCommBlocks + blockIdx.x, epoch);
    const uint32_t* mine = g.signal[g.rank] + peer * kMaxCommBlocks + blockIdx.x;
    uint32_t i = 0;
    // flags only grow; a peer that is already one call ahead has a larger value
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if (++i > kMaxFlagPolls) {
        ok = false;
        break;
      }
    }
    if (!ok && status) atomicCAS(status, 0, 5);
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// Each call advances the epoch by `steps` barriers.  The value is read by every
// block before block 0 bumps it at the very end of the kernel.
__device__ __forceinline__ uint32_t read_epoch(const SymmGroup& g) {
  return *reinterpret_cast<volatile uint32_t*>(g.signal[g.rank] + kEpochWord);
}

// ---------------------------------------------------------------- one shot
// in/out: [n_vec] vectors of 8 bf16.  Rows are `row_vecs` vectors long when the
// fused norm is requested (residual / norm_w non-null): out = RMSNorm(residual +=
// sum) * norm_w, with the updated residual written back.
__global__ void __launch_bounds__(512)
allreduce_oneshot_kernel(SymmGroup g, const uint4* __restrict__ in, uint4* __restrict__ out,
                         long long n_vec, uint4* __restrict__ residual,
                         const uint4* __restrict__ norm_w, int row_vecs, float eps,
                         uint32_t* done_counter, int* status) {
  const uint32_t epoch0 = read_epoch(g);
  const uint32_t epoch = epoch0 + 1;
  const int half = epoch & 1;
  uint4* stage = reinterpret_cast<uint4*>(static_cast<char*>(g.data[g.rank]) + half * g.half_bytes);
  const bool fused = norm_w != nullptr;
  // Work split: contiguous chunk per block (whole rows when fused).
  long long begin, end;
  if (fused) {
    const long long rows = n_vec / row_vecs;
    const long long per = (rows + gridDim.x - 1) / gridDim.x;
    begin = min(rows, per * blockIdx.x) * row_vecs;
    end = min(rows, per * (blockIdx.x + 1)) * row_vecs;
  } else {
    const long long per = (n_vec + gridDim.x - 1) / gridDim.x;
    begin = min(n_vec, per * blockIdx.x);
    end = min(n_vec, per * (blockIdx.x + 1));
  }
  for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) stage[i] = in[i];
  const bool ok = block_barrier(g, epoch, status);
  if (ok) {
    const uint4* src[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      src[r] = r < g.world ? reinterpret_cast<const uint4*>(static_cast<const char*>(g.data[r]) +
                                                            half * g.half_bytes)
                           : nullptr;
    if (!fused) {
      for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < g.world) add8(acc, __ldcv(src[r] + i));
        out[i] = pack8(acc);
      }
    } else {
      __shared__ float red[32];
      // one row at a time per block; a thread owns up to 4 vectors of the row
      for (long long row0 = begin; row0 < end; row0 += row_vecs) {
        float vals[4][8];
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int v = threadIdx.x + k * blockDim.x;
          if (v < row_vecs) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
              if (r < g.world) add8(acc, __ldcv(src[r] + row0 + v));
            // the reduced value is rounded to bf16 before the residual add, exactly
            // as an unfused all-reduce followed by add+norm would do
            Pack8 y;
            y.u = pack8(acc);
            Pack8 rs;
            rs.u = residual[row0 + v];
            Pack8 nr;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              nr.h[j] = __float2bfloat16(__bfloat162float(y.h[j]) + __bfloat162float(rs.h[j]));
              vals[k][j] = __bfloat162float(nr.h[j]);
              ss += vals[k][j] * vals[k][j];
            }
            residual[row0 + v] = nr.u;
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < (blockDim.x >> 5); ++w) tot += red[w];
        __syncthreads();
        const float inv = rsqrtf(tot / static_cast<float>(row_vecs * 8) + eps);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int v = threadIdx.x + k * blockDim.x;
          if (v < row_vecs) {
            Pack8 w8, o8;
            w8.u = norm_w[v];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              o8.h[j] = __float2bfloat16(vals[k][j] * inv * __bfloat162float(w8.h[j]));
            out[row0 + v] = o8.u;
          }
        }
      }
    }
  }
  // The last block to finish advances the epoch for the next call.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done_counter, 1u) == gridDim.x - 1) {
      *done_counter = 0;
      *reinterpret_cast<volatile uint32_t*>(g.signal[g.rank] + kEpochWord) = epoch;
    }
  }
}

// ---------------------------------------------------------------- two shot
// Stage -> barrier -> reduce my slice (into my "reduced" area) -> barrier ->
// gather all slices.  The slice of rank r covers vectors [r*slice, (r+1)*slice).
// Every pass splits each slice across the blocks in the same way, so block b only
// ever consumes data produced by block b of a peer and the per-block barrier is
// all the ordering that is needed.
__device__ __forceinline__ void slice_part(long long n_vec, long long slice_vecs, int r,
                                           long long* s_begin, long long* b, long long* e) {
  *s_begin = slice_vecs * r;
  const long long s_end = min(n_vec, *s_begin + slice_vecs);
  const long long n_r = max(0LL, s_end - *s_begin);
  const long long per = (n_r + gridDim.x - 1) / gridDim.x;
  *b = min(n_r, per * blockIdx.x);
  *e = min(n_r, per * (blockIdx.x + 1));
}

__global__ void __launch_bounds__(512)
allreduce_twoshot_kernel(SymmGroup g, const uint4* __restrict__ in, uint4* __restrict__ out,
                         long long n_vec, long long slice_vecs, uint32_t* done_counter,
                         int* status) {
  const uint32_t epoch0 = read_epoch(g);
  // two barriers; the call consumes three epoch values so that the next call
  // lands on the other half of the buffers
  const uint32_t e1 = epoch0 + 1, e2 = epoch0 + 2, e_end = epoch0 + 3;
  const int half = e1 & 1;
  char* my_base = static_cast<char*>(g.data[g.rank]) + half * g.half_bytes;
  uint4* stage = reinterpret_cast<uint4*>(my_base);
  const size_t red_off = static_cast<size_t>(n_vec) * sizeof(uint4);
  for (int r = 0; r < g.world; ++r) {
    long long sb, b, e;
    slice_part(n_vec, slice_vecs, r, &sb, &b, &e);
    for (long long i = b + threadIdx.x; i < e; i += blockDim.x) stage[sb + i] = in[sb + i];
  }
  bool ok = block_barrier(g, e1, status);
  if (ok) {
    long long sb, b, e;
    slice_part(n_vec, slice_vecs, g.rank, &sb, &b, &e);
    uint4* red = reinterpret_cast<uint4*>(my_base + red_off);
    const uint4* srcs[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      srcs[r] = r < g.world ? reinterpret_cast<const uint4*>(static_cast<const char*>(g.data[r]) +
                                                             half * g.half_bytes) + sb
                            : nullptr;
    // four independent vectors per thread and iteration keep more loads in flight
    long long i = b + threadIdx.x;
    for (; i + 3LL * blockDim.x < e; i += 4LL * blockDim.x) {
      uint4 v[4][kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < g.world) {
#pragma unroll
          for (int u = 0; u < 4; ++u) v[u][r] = __ldcv(srcs[r] + i + u * blockDim.x);
        }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < g.world) add8(acc, v[u][r]);
        red[i + u * blockDim.x] = pack8(acc);
      }
    }
    for (; i < e; i += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < g.world) add8(acc, __ldcv(srcs[r] + i));
      red[i] = pack8(acc);
    }
    ok = block_barrier(g, e2, status);
  }
  if (ok) {
    for (int r = 0; r < g.world; ++r) {
      long long sb, b, e;
      slice_part(n_vec, slice_vecs, r, &sb, &b, &e);
      const uint4* red = reinterpret_cast<const uint4*>(static_cast<const char*>(g.data[r]) +
                                                        half * g.half_bytes + red_off);
      long long i = b + threadIdx.x;
      for (; i + 3LL * blockDim.x < e; i += 4LL * blockDim.x) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = __ldcv(red + i + u * blockDim.x);
#pragma unroll
        for (int u = 0; u < 4; ++u) out[sb + i + u * blockDim.x] = v[u];
      }
      for (; i < e; i += blockDim.x) out[sb + i] = __ldcv(red + i);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done_counter, 1u) == gridDim.x - 1) {
      *done_counter = 0;
      *reinterpret_cast<volatile uint32_t*>(g.signal[g.rank] + kEpochWord) = e_end;
    }
  }
}

// ------------------------------------------------------------- all-gather
// out [world * n_vec] = concatenation of every rank's in [n_vec].
__global__ void __launch_bounds__(512)
allgather_kernel(SymmGroup g, const uint4* __restrict__ in, uint4* __restrict__ out, long long n_vec,
                 uint32_t* done_counter, int* status) {
  const uint32_t epoch = read_epoch(g) + 1;
  const int half = epoch & 1;
  uint4* stage = reinterpret_cast<uint4*>(static_cast<char*>(g.data[g.rank]) + half * g.half_bytes);
  const long long per = (n_vec + gridDim.x - 1) / gridDim.x;
  const long long begin = min(n_vec, per * blockIdx.x), end = min(n_vec, per * (blockIdx.x + 1));
  for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) stage[i] = in[i];
  if (block_barrier(g, epoch, status)) {
    for (int r = 0; r < g.world; ++r) {
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const char*>(g.data[r]) +
                                                        half * g.half_bytes);
      uint4* dst = out + static_cast<long long>(r) * n_vec;
      if (r == g.rank) {
        for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) dst[i] = in[i];
      } else {
        for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) dst[i] = __ldcv(src + i);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done_counter, 1u) == gridDim.x - 1) {
      *done_counter = 0;
      *reinterpret_cast<volatile uint32_t*>(g.signal[g.rank] + kEpochWord) = epoch;
    }
  }
}

// ------------------------------------------------------- bounded-wait self test
// Waits on a flag with the same acquire-poll loop and give-up path the collectives use, with a
// caller-chosen poll limit.  A flag that nothing sets makes the wait run out: the kernel records
// status 5 and returns, the context stays usable.  This is how the failure path is exercised
// without a failing peer.
__global__ void flag_wait_probe_kernel(const uint32_t* flag, uint32_t want, uint32_t max_polls, int* status,
                                       uint32_t* polls_out) {
  uint32_t i = 0;
  bool ok = true;
  while (static_cast<int32_t>(ld_acquire_sys(flag) - want) < 0) {
    if (++i > max_polls) {
      ok = false;
      break;
    }
  }
  if (!ok && status) atomicCAS(status, 0, 5);
  if (polls_out) *polls_out = i;
}

extern "C" int b200_symm_wait_probe(const void* flag, unsigned want, unsigned max_polls, int* status, void* polls_out,
                                    cudaStream_t stream) {
  if (max_polls > kMaxFlagPolls) max_polls = kMaxFlagPolls;
  flag_wait_probe_kernel<<<1, 1, 0, stream>>>(static_cast<const uint32_t*>(flag), want, max_polls, status,
                                              static_cast<uint32_t*>(polls_out));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// ------------------------------------------- staging for the fused all-gather GEMM
// Copies this rank's block into its staging half of the next epoch (where the peers' GEMM kernels
// fetch it) and into its place in the local gathered buffer; clears the per-source arrival
// counters of the GEMM; the last block to finish tells every rank (flag word kAgFlagWord + rank of
// their signal pads) and advances the epoch.  No waiting here: the GEMM that follows waits per
// source block, right before it needs it.
__global__ void __launch_bounds__(512)
ag_stage_kernel(SymmGroup g, const uint4* __restrict__ in, uint4* __restrict__ local_out, long long n_vec,
                uint32_t* ready, uint32_t* done_counter) {
  const uint32_t epoch = read_epoch(g) + 1;
  uint4* stage = reinterpret_cast<uint4*>(static_cast<char*>(g.data[g.rank]) + (epoch & 1) * g.half_bytes);
  if (blockIdx.x == 0 && threadIdx.x < g.world) ready[threadIdx.x] = 0u;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 v = in[i];
    stage[i] = v;
    local_out[i] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done_counter, 1u) == gridDim.x - 1) {
      *done_counter = 0;
      __threadfence_system();
      for (int r = 0; r < g.world; ++r) st_release_sys(g.signal[r] + kAgFlagWord + g.rank, epoch);
      *reinterpret_cast<volatile uint32_t*>(g.signal[g.rank] + kEpochWord) = epoch;
    }
  }
}

// --------------------------- second half of the fused GEMM + reduce-scatter
// The GEMM before this kernel stored every rank's partial rows into the owners' staging halves:
// stage[src][rows][row_vecs] on the owner.  Block 0 tells every rank that this rank's stores are
// done (they are: the GEMM has completed), then every block waits (bounded) for all sources and
// sums its share of the rows in rank order; optional "+ residual" and RMSNorm as in the
// all-reduce kernels.  The last block advances the epoch.
__global__ void __launch_bounds__(512)
rs_reduce_kernel(SymmGroup g, uint4* __restrict__ out, long long rows, int row_vecs, uint4* __restrict__ residual,
                 const uint4* __restrict__ norm_w, float eps, uint32_t* done_counter, int* status) {
  const uint32_t epoch = read_epoch(g) + 1;
  const uint4* stage = reinterpret_cast<const uint4*>(static_cast<const char*>(g.data[g.rank]) +
                                                      (epoch & 1) * g.half_bytes);
  if (blockIdx.x == 0 && threadIdx.x < g.world) {
    __threadfence_system();
    st_release_sys(g.signal[threadIdx.x] + kRsFlagWord + g.rank, epoch);
  }
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < g.world) {
    const uint32_t* mine = g.signal[g.rank] + kRsFlagWord + threadIdx.x;
    uint32_t i = 0;
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if (++i > kMaxFlagPolls) {
        s_ok = 0;
        if (status) atomicCAS(status, 0, 5);
        break;
      }
    }
  }
  __syncthreads();
  if (s_ok) {
    __shared__ float red[32];
    const long long slot = rows * row_vecs;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
      float vals[4][8];
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int v = threadIdx.x + k * blockDim.x;
        if (v < row_vecs) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r)
            if (r < g.world) add8(acc, __ldcv(stage + r * slot + row * row_vecs + v));
          Pack8 y;
          y.u = pack8(acc);
          if (residual) {
            Pack8 rs;
            rs.u = residual[row * row_vecs + v];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              y.h[j] = __float2bfloat16(__bfloat162float(y.h[j]) + __bfloat162float(rs.h[j]));
            if (norm_w) residual[row * row_vecs + v] = y.u;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            vals[k][j] = __bfloat162float(y.h[j]);
            ss += vals[k][j] * vals[k][j];
          }
          if (!norm_w) out[row * row_vecs + v] = y.u;
        }
      }
      if (norm_w) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        __syncthreads();
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < (blockDim.x >> 5); ++w) tot += red[w];
        const float inv = rsqrtf(tot / static_cast<float>(row_vecs * 8) + eps);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int v = threadIdx.x + k * blockDim.x;
          if (v < row_vecs) {
            Pack8 w8, o8;
            w8.u = norm_w[v];
#pragma unroll
            for (int j = 0; j < 8; ++j) o8.h[j] = __float2bfloat16(vals[k][j] * inv * __bfloat162float(w8.h[j]));
            out[row * row_vecs + v] = o8.u;
          }
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done_counter, 1u) == gridDim.x - 1) {
      *done_counter = 0;
      *reinterpret_cast<volatile uint32_t*>(g.signal[g.rank] + kEpochWord) = epoch;
    }
  }
}

// ---------------------------------------------------------- reduce-scatter
// in [world * n_vec]; out [n_vec] = sum over ranks of their chunk `rank`.
__global__ void __launch_bounds__(512)
reducescatter_kernel(SymmGroup g, const uint4* __restrict__ in, uint4* __restrict__ out,
                     long long n_vec, uint32_t* done_counter, int* status) {
  const uint32_t epoch = read_epoch(g) + 1;
  const int half = epoch & 1;
  uint4* stage = reinterpret_cast<uint4*>(static_cast<char*>(g.data[g.rank]) + half * g.half_bytes);
  const long long per = (n_vec + gridDim.x - 1) / gridDim.x;
  const long long begin = min(n_vec, per * blockIdx.x), end = min(n_vec, per * (blockIdx.x + 1));
  // stage every chunk (block b stages part b of every chunk, which is what block b of the
  // owning rank will read)
  for (int r = 0; r < g.world; ++r)
    for (long long i = begin + threadIdx.x; i < end; i += blockDim.x)
      stage[static_cast<long long>(r) * n_vec + i] = in[static_cast<long long>(r) * n_vec + i];
  if (block_barrier(g, epoch, status)) {
    for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (r < g.world) {
          const uint4* src = reinterpret_cast<const uint4*>(static_cast<const char*>(g.data[r]) +
                                                            half * g.half_bytes);
          add8(acc, __ldcv(src + static_cast<long long>(g.rank) * n_vec + i));
        }
      }
      out[i] = pack8(acc);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done_counter, 1u) == gridDim.x - 1) {
      *done_counter = 0;
      *reinterpret_cast<volatile uint32_t*>(g.signal[g.rank] + kEpochWord) = epoch;
    }
  }
}


// ------------------------------------------------------- push all-reduce ("LL")
// Latency-optimised all-reduce for small messages: no barrier at all.  Every rank
// PUSHES its vectors into a slot of every peer's receive buffer; the payload itself
// tells the receiver when it has arrived: slots are pre-filled with a sentinel bit
// pattern (the bf16 pair -0.0/-0.0 in every 32-bit word, which senders never emit: they
// turn such a word into +0.0/+0.0), and the receiver polls its OWN memory until the
// four words of a 16-byte vector differ from the sentinel.  One NVLink one-way trip is
// the whole synchronisation cost.
//
// Receive buffer of a rank: [3 slots][world source ranks][slot_vecs vectors].  Call e
// uses slot e % 3 and, at its very end, re-arms slot (e + 2) % 3 (the one call e - 1
// used): a peer can only be writing into that slot again in call e + 2, which it
// enters after receiving this rank's data of call e + 1, i.e. after this kernel (and
// its re-arming stores) completed.  The epoch lives in device memory and is advanced by
// the last block, so CUDA-graph replays need no host update.
// in/out [n_vec] vectors of 8 bf16; rows of row_vecs vectors when fused with
// "residual += sum; out = RMSNorm(residual) * w".  One block per row (fused) or per
// contiguous chunk; a thread owns up to 4 vectors of its block's range at a time.
__global__ void __launch_bounds__(512)
allreduce_ll_kernel(LLGroup g, const uint4* __restrict__ in, uint4* __restrict__ out, long long n_vec,
                    uint4* __restrict__ residual, const uint4* __restrict__ norm_w, int row_vecs, float eps,
                    uint32_t* done_counter, int* status) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(g.epoch) + 1;
  const long long slot_stride = static_cast<long long>(g.world) * g.slot_vecs;
  const long long slot_off = static_cast<long long>(epoch % 3) * slot_stride;
  const long long rearm_off = static_cast<long long>((epoch + 2) % 3) * slot_stride;
  const bool fused = norm_w != nullptr;
  long long begin, end;
  if (fused) {
    const long long rows = n_vec / row_vecs;
    const long long per = (rows + gridDim.x - 1) / gridDim.x;
    begin = min(rows, per * blockIdx.x) * row_vecs;
    end = min(rows, per * (blockIdx.x + 1)) * row_vecs;
  } else {
    const long long per = (n_vec + gridDim.x - 1) / gridDim.x;
    begin = min(n_vec, per * blockIdx.x);
    end = min(n_vec, per * (blockIdx.x + 1));
  }
  // 1) push my vectors into every rank's slot (my own included: uniform receive code)
  for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const uint4 v = ll_sanitize(in[i]);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < g.world) ll_store(g.recv[r] + slot_off + static_cast<long long>(g.rank) * g.slot_vecs + i, v);
  }
  // 2) receive + reduce (rank order, so every rank computes bit-identical sums)
  const uint4* mine = g.recv[g.rank] + slot_off;
  bool ok = true;
  if (!fused) {
    for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (r < g.world) {
          uint4 v;
          ok = ll_wait(mine + static_cast<long long>(r) * g.slot_vecs + i, v) && ok;
          add8(acc, v);
        }
      }
      out[i] = pack8(acc);
    }
  } else {
    __shared__ float red[32];
    for (long long row0 = begin; row0 < end; row0 += row_vecs) {
      float vals[4][8];
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int v = threadIdx.x + k * blockDim.x;
        if (v < row_vecs) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r) {
            if (r < g.world) {
              uint4 x;
              ok = ll_wait(mine + static_cast<long long>(r) * g.slot_vecs + row0 + v, x) && ok;
              add8(acc, x);
            }
          }
          Pack8 y;
          y.u = pack8(acc);          // the sum is rounded to bf16 before the residual add
          Pack8 rs;
          rs.u = residual[row0 + v];
          Pack8 nr;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            nr.h[j] = __float2bfloat16(__bfloat162float(y.h[j]) + __bfloat162float(rs.h[j]));
            vals[k][j] = __bfloat162float(nr.h[j]);
            ss += vals[k][j] * vals[k][j];
          }
          residual[row0 + v] = nr.u;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
      for (int w = 0; w < (blockDim.x >> 5); ++w) tot += red[w];
      __syncthreads();
      const float inv = rsqrtf(tot / static_cast<float>(row_vecs * 8) + eps);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int v = threadIdx.x + k * blockDim.x;
        if (v < row_vecs) {
          Pack8 w8, o8;
          w8.u = norm_w[v];
#pragma unroll
          for (int j = 0; j < 8; ++j) o8.h[j] = __float2bfloat16(vals[k][j] * inv * __bfloat162float(w8.h[j]));
          out[row0 + v] = o8.u;
        }
      }
    }
  }
  if (!ok && status) atomicCAS(status, 0, 5);
  // 3) re-arm the slot of the previous call for its next use (two calls from now).  How many
  //    vectors that call wrote per source rank is recorded in device memory (epoch[1 + slot]),
  //    so calls of different sizes and CUDA-graph replays in any order stay consistent.
  {
    const uint32_t prev_vecs = reinterpret_cast<volatile uint32_t*>(g.epoch)[1 + (epoch + 2) % 3];
    const uint4 s4 = make_uint4(kLLSentinel, kLLSentinel, kLLSentinel, kLLSentinel);
    uint4* rearm = g.recv[g.rank] + rearm_off;
    const long long total = static_cast<long long>(prev_vecs) * g.world;
    for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
      const long long r = idx / prev_vecs, i = idx % prev_vecs;
      rearm[r * g.slot_vecs + i] = s4;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done_counter, 1u) == gridDim.x - 1) {
      *done_counter = 0;
      volatile uint32_t* meta = reinterpret_cast<volatile uint32_t*>(g.epoch);
      meta[1 + epoch % 3] = static_cast<uint32_t>(n_vec);
      meta[0] = epoch;
    }
  }
}

__global__ void ll_fill_kernel(uint4* p, long long n) {
  const uint4 s4 = make_uint4(kLLSentinel, kLLSentinel, kLLSentinel, kLLSentinel);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    p[i] = s4;
}

}  // namespace b200

using namespace b200;

// ---- IPC plumbing (host).  The buffers are plain cudaMalloc allocations so that
// cudaIpcGetMemHandle applies to the whole allocation.
extern "C" int b200_symm_alloc(size_t bytes, void** ptr, void* handle_out_64) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return -1;
  if (cudaMemset(p, 0, bytes) != cudaSuccess) return -2;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return -3;
  memcpy(handle_out_64, &h, sizeof(h));
  *ptr = p;
  return 0;
}

extern "C" int b200_symm_open(const void* handle_64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_64, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return -1;
  *ptr = p;
  return 0;
}

extern "C" int b200_symm_close(void* ptr) {
  return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -1;
}

extern "C" int b200_symm_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -1; }

extern "C" int b200_symm_signal_words() { return kRsFlagWord + kMaxRanks + 4; }
extern "C" int b200_symm_epoch_word() { return kEpochWord; }
extern "C" int b200_symm_ag_flag_word() { return kAgFlagWord; }

static SymmGroup make_group(void* const* data, void* const* signal, int world, int rank,
                            size_t half_bytes) {
  SymmGroup g{};
  for (int r = 0; r < kMaxRanks; ++r) {
    g.data[r] = r < world ? data[r] : nullptr;
    g.signal[r] = r < world ? static_cast<uint32_t*>(signal[r]) : nullptr;
  }
  g.world = world;
  g.rank = rank;
  g.half_bytes = half_bytes;
  return g;
}

static int pick_blocks(long long n_vec, int max_blocks) {
  long long b = (n_vec + 1023) / 1024;   // >= 2 vectors per thread at 512 threads
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return static_cast<int>(b);
}

// mode: 0 auto, 1 one shot, 2 two shot.  n_elems bf16 elements (multiple of 8).
// Fused add+norm (residual, norm_w non-null, row_elems = hidden size) is available in
// one-shot mode.  done_counter: a zero-initialised device word owned by the caller.
extern "C" int b200_symm_all_reduce(void* const* data, void* const* signal, int world, int rank,
                                    size_t half_bytes, const void* in, void* out, long long n_elems,
                                    void* residual, const void* norm_w, int row_elems, float eps,
                                    int mode, void* done_counter, int* status,
                                    cudaStream_t stream) {
  if (world < 2 || world > kMaxRanks) return -1;
  if ((n_elems & 7) != 0) return -2;
  const long long n_vec = n_elems >> 3;
  const size_t bytes = static_cast<size_t>(n_elems) * 2;
  const SymmGroup g = make_group(data, signal, world, rank, half_bytes);
  const bool fused = norm_w != nullptr;
  if (fused && ((row_elems & 7) != 0 || row_elems > 512 * 4 * 8 || n_elems % row_elems != 0)) return -3;
  if (mode == 0) mode = (fused || bytes <= (world <= 2 ? (8u << 20) : (world <= 4 ? (1u << 20) : (512u << 10)))) ? 1 : 2;
  if (fused) mode = 1;
  if (mode == 1) {
    if (bytes > half_bytes) return -4;
    const int blocks = fused ? static_cast<int>((n_elems / row_elems) < kMaxCommBlocks ? (n_elems / row_elems) : kMaxCommBlocks)
                             : pick_blocks(n_vec, kMaxCommBlocks);
    allreduce_oneshot_kernel<<<blocks < 1 ? 1 : blocks, 512, 0, stream>>>(
        g, static_cast<const uint4*>(in), static_cast<uint4*>(out), n_vec,
        static_cast<uint4*>(residual), static_cast<const uint4*>(norm_w), row_elems >> 3, eps,
        static_cast<uint32_t*>(done_counter), status);
  } else {
    const long long slice = (n_vec + world - 1) / world;
    if (bytes + static_cast<size_t>(slice) * 16 > half_bytes) return -4;
    const int blocks = pick_blocks(n_vec, kMaxCommBlocks);
    allreduce_twoshot_kernel<<<blocks, 512, 0, stream>>>(
        g, static_cast<const uint4*>(in), static_cast<uint4*>(out), n_vec, slice,
        static_cast<uint32_t*>(done_counter), status);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int b200_symm_all_gather(void* const* data, void* const* signal, int world, int rank,
                                    size_t half_bytes, const void* in, void* out, long long n_elems,
                                    void* done_counter, int* status, cudaStream_t stream) {
  if (world < 2 || world > kMaxRanks || (n_elems & 7) != 0) return -1;
  if (static_cast<size_t>(n_elems) * 2 > half_bytes) return -4;
  const SymmGroup g = make_group(data, signal, world, rank, half_bytes);
  const long long n_vec = n_elems >> 3;
  allgather_kernel<<<pick_blocks(n_vec, kMaxCommBlocks), 512, 0, stream>>>(
      g, static_cast<const uint4*>(in), static_cast<uint4*>(out), n_vec,
      static_cast<uint32_t*>(done_counter), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// rows x row_elems bf16 per rank (row_elems % 8 == 0, <= 16384); out [rows, row_elems].
// residual / norm_w optional: out = RMSNorm(residual += sum) * norm_w, or out = sum (+ residual).
extern "C" int b200_symm_rs_reduce(void* const* data, void* const* signal, int world, int rank, size_t half_bytes,
                                   void* out, long long rows, int row_elems, void* residual, const void* norm_w,
                                   float eps, void* done_counter, int* status, cudaStream_t stream) {
  if (world < 2 || world > kMaxRanks || (row_elems & 7) != 0 || row_elems > 512 * 4 * 8) return -1;
  if (static_cast<size_t>(rows) * row_elems * 2 * world > half_bytes) return -4;
  const SymmGroup g = make_group(data, signal, world, rank, half_bytes);
  long long blocks = rows < kMaxCommBlocks ? rows : kMaxCommBlocks;
  if (blocks < 1) blocks = 1;
  rs_reduce_kernel<<<static_cast<unsigned>(blocks), 512, 0, stream>>>(
      g, static_cast<uint4*>(out), rows, row_elems >> 3, static_cast<uint4*>(residual),
      static_cast<const uint4*>(norm_w), eps, static_cast<uint32_t*>(done_counter), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// in: this rank's block (n_elems bf16); gathered: local [world * n_elems] buffer; ready: [world] counters.
extern "C" int b200_symm_ag_stage(void* const* data, void* const* signal, int world, int rank, size_t half_bytes,
                                  const void* in, void* gathered, long long n_elems, void* ready,
                                  void* done_counter, cudaStream_t stream) {
  if (world < 2 || world > kMaxRanks || (n_elems & 7) != 0) return -1;
  if (static_cast<size_t>(n_elems) * 2 > half_bytes) return -4;
  const SymmGroup g = make_group(data, signal, world, rank, half_bytes);
  const long long n_vec = n_elems >> 3;
  ag_stage_kernel<<<pick_blocks(n_vec, kMaxCommBlocks), 512, 0, stream>>>(
      g, static_cast<const uint4*>(in), static_cast<uint4*>(gathered) + static_cast<long long>(rank) * n_vec, n_vec,
      static_cast<uint32_t*>(ready), static_cast<uint32_t*>(done_counter));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int b200_symm_reduce_scatter(void* const* data, void* const* signal, int world, int rank,
                                        size_t half_bytes, const void* in, void* out,
                                        long long n_elems_out, void* done_counter, int* status,
                                        cudaStream_t stream) {
  if (world < 2 || world > kMaxRanks || (n_elems_out & 7) != 0) return -1;
  if (static_cast<size_t>(n_elems_out) * 2 * world > half_bytes) return -4;
  const SymmGroup g = make_group(data, signal, world, rank, half_bytes);
  const long long n_vec = n_elems_out >> 3;
  reducescatter_kernel<<<pick_blocks(n_vec, kMaxCommBlocks), 512, 0, stream>>>(
      g, static_cast<const uint4*>(in), static_cast<uint4*>(out), n_vec,
      static_cast<uint32_t*>(done_counter), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}


// ---- push ("LL") all-reduce: host side
// Arms a receive buffer (3 * world * slot_vecs vectors) with the sentinel pattern.
extern "C" int b200_symm_ll_arm(void* recv, long long total_vecs, cudaStream_t stream) {
  ll_fill_kernel<<<256, 256, 0, stream>>>(static_cast<uint4*>(recv), total_vecs);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// recv: the group's peer-mapped receive buffers; epoch: four zero-initialised device words of
// this rank (epoch and the per-slot fill counts).  The message (n_elems bf16, a multiple of 8) must fit one slot region: n_elems / 8 <=
// slot_vecs.  Calls of different sizes may follow one another freely.
extern "C" int b200_symm_all_reduce_ll(void* const* recv, int world, int rank, long long slot_vecs,
                                       void* epoch, const void* in, void* out, long long n_elems,
                                       void* residual, const void* norm_w, int row_elems, float eps,
                                       void* done_counter, int* status, cudaStream_t stream) {
  if (world < 2 || world > kMaxRanks) return -1;
  if ((n_elems & 7) != 0) return -2;
  const long long n_vec = n_elems >> 3;
  if (n_vec > slot_vecs) return -4;
  const bool fused = norm_w != nullptr;
  if (fused && ((row_elems & 7) != 0 || row_elems > 512 * 4 * 8 || n_elems % row_elems != 0)) return -3;
  LLGroup g{};
  for (int r = 0; r < kMaxRanks; ++r) g.recv[r] = r < world ? static_cast<uint4*>(recv[r]) : nullptr;
  g.epoch = static_cast<uint32_t*>(epoch);
  g.world = world;
  g.rank = rank;
  g.slot_vecs = slot_vecs;
  int blocks;
  if (fused) {
    const long long rows = n_elems / row_elems;
    blocks = static_cast<int>(rows < kMaxCommBlocks ? rows : kMaxCommBlocks);
  } else {
    blocks = static_cast<int>((n_vec + 511) / 512);
    if (blocks > kMaxCommBlocks) blocks = kMaxCommBlocks;
  }
  if (blocks < 1) blocks = 1;
  allreduce_ll_kernel<<<blocks, 512, 0, stream>>>(g, static_cast<const uint4*>(in), static_cast<uint4*>(out),
                                                  n_vec, static_cast<uint4*>(residual),
                                                  static_cast<const uint4*>(norm_w), row_elems >> 3, eps,
                                                  static_cast<uint32_t*>(done_counter), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
