// Token sampling on the device, one CTA per request row:
//   * greedy arg-max (lowest index wins ties),
//   * temperature + top-k + top-p sampling by the exponential-race (Gumbel-max)
//     method: the kept set is found with radix selection over the logit bits
//     (counts for top-k, probability mass for top-p), then the winner is
//     argmax(logit / T + Gumbel noise) over the kept tokens, noise from a
//     counter-based Philox4x32-10 generator keyed per row.
// No sort, no host round trip; suitable for CUDA-graph capture.
//
// Replaces npu_top_k_top_p_sample and the exponential-noise side stream
// (omni_npu/sample/ops/topk_topp_sampler.py:41-88).

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

static constexpr int kSampleThreads = 1024;

template <typename T>
__device__ __forceinline__ float load_logit(const T* row, int i);
template <>
__device__ __forceinline__ float load_logit<float>(const float* row, int i) {
  return row[i];
}
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* row, int i) {
  return __bfloat162float(row[i]);
}

// Order-preserving map float -> uint32 (larger float = larger key).
__device__ __forceinline__ uint32_t float_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct MaxIdx {
  float v;
  int i;
};
__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ MaxIdx block_argmax(MaxIdx m, MaxIdx* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx other;
    other.v = __shfl_xor_sync(0xffffffffu, m.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, m.i, o);
    m = better(m, other);
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = m;
  __syncthreads();
  MaxIdx t = (l < (blockDim.x >> 5)) ? red[l] : MaxIdx{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx other;
    other.v = __shfl_xor_sync(0xffffffffu, t.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, t.i, o);
    t = better(t, other);
  }
  __syncthreads();
  return t;
}

__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  __syncthreads();
  return t;
}

// Philox4x32-10 (Salmon et al., SC'11): 128-bit counter, 64-bit key.
__device__ __forceinline__ uint4 philox4x32(uint4 ctr, uint2 key) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
argmax_kernel(const T* __restrict__ logits, int* __restrict__ out, int V, long long stride) {
  __shared__ MaxIdx red[32];
  const T* row = logits + static_cast<long long>(blockIdx.x) * stride;
  MaxIdx m{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = load_logit<T>(row, i);
    if (v > m.v) {
      m.v = v;
      m.i = i;
    }
  }
  m = block_argmax(m, red);
  if (threadIdx.x == 0) out[blockIdx.x] = m.i == 0x7fffffff ? 0 : m.i;
}

// Radix selection state shared by the block.
struct SelectShared {
  float hist[2048];
  uint32_t prefix;
  uint32_t prefix_mask;
  float remaining;
  int done;
};

// Finds the largest key threshold `thr` such that the total weight of elements with key >= thr
// is >= target, where weight is 1 (COUNT) or exp2(x*s - m) (mass).  Elements below
// `floor_key` are ignored.  Returns the threshold key.
template <typename T, bool MASS>
__device__ uint32_t radix_select(const T* row, int V, float target, uint32_t floor_key,
                                 float scale_log2, float max_scaled, SelectShared* sh) {
  if (threadIdx.x == 0) {
    sh->prefix = 0;
    sh->prefix_mask = 0;
    sh->remaining = target;
  }
  const int shifts[3] = {21, 10, 0};
  const int widths[3] = {11, 11, 10};
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = shifts[pass];
    const int bins = 1 << widths[pass];
    for (int i = threadIdx.x; i < 2048; i += blockDim.x) sh->hist[i] = 0.f;
    __syncthreads();
    const uint32_t prefix = sh->prefix, mask = sh->prefix_mask;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float x = load_logit<T>(row, i);
      const uint32_t key = float_key(x);
      if (key < floor_key || (key & mask) != prefix) continue;
      const int b = (key >> shift) & (bins - 1);
      const float wgt = MASS ? exp2f(x * scale_log2 - max_scaled) : 1.f;
      atomicAdd(&sh->hist[b], wgt);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float rem = sh->remaining;
      int b = bins - 1;
      for (; b > 0; --b) {
        const float h = sh->hist[b];
        if (h >= rem) break;
        rem -= h;
      }
      sh->remaining = rem;
      sh->prefix = prefix | (static_cast<uint32_t>(b) << shift);
      sh->prefix_mask = mask | (static_cast<uint32_t>(bins - 1) << shift);
    }
    __syncthreads();
  }
  return sh->prefix;
}

template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const T* __restrict__ logits, int* __restrict__ out, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const long long* __restrict__ seeds, const long long* __restrict__ step_offset, int V,
              long long stride) {
  __shared__ MaxIdx red_mi[32];
  __shared__ float red_f[32];
  __shared__ SelectShared sh;
  const int rowi = blockIdx.x;
  const T* row = logits + static_cast<long long>(rowi) * stride;
  const float temp = temperature ? temperature[rowi] : 1.f;

  // pass 1: max (and greedy answer)
  MaxIdx m{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = load_logit<T>(row, i);
    if (v > m.v) {
      m.v = v;
      m.i = i;
    }
  }
  m = block_argmax(m, red_mi);
  if (temp < 1e-5f) {
    if (threadIdx.x == 0) out[rowi] = m.i == 0x7fffffff ? 0 : m.i;
    return;
  }
  const float scale_log2 = 1.4426950408889634f / temp;
  const float max_scaled = m.v * scale_log2;

  uint32_t floor_key = 0;  // keep keys >= floor_key
  const int k = top_k ? top_k[rowi] : 0;
  if (k > 0 && k < V) {
    floor_key = radix_select<T, false>(row, V, static_cast<float>(k), 0u, scale_log2, max_scaled, &sh);
  }
  const float p = top_p ? top_p[rowi] : 1.f;
  if (p < 1.f) {
    float z = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float x = load_logit<T>(row, i);
      if (float_key(x) >= floor_key) z += exp2f(x * scale_log2 - max_scaled);
    }
    z = block_reduce_sum(z, red_f);
    const uint32_t kp =
        radix_select<T, true>(row, V, p * z, floor_key, scale_log2, max_scaled, &sh);
    if (kp > floor_key) floor_key = kp;
  }

  // final pass: Gumbel-max over the kept set
  const uint64_t seed = seeds ? static_cast<uint64_t>(seeds[rowi]) : 0x9E3779B97F4A7C15ull;
  const uint64_t off = step_offset ? static_cast<uint64_t>(step_offset[0]) : 0ull;
  const uint2 key = make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
  MaxIdx best{-INFINITY, 0x7fffffff};
  for (int i4 = threadIdx.x; i4 * 4 < V; i4 += blockDim.x) {
    const uint4 r = philox4x32(make_uint4(static_cast<uint32_t>(i4), static_cast<uint32_t>(off),
                                          static_cast<uint32_t>(off >> 32), static_cast<uint32_t>(rowi)),
                               key);
    const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = i4 * 4 + j;
      if (i >= V) break;
      const float x = load_logit<T>(row, i);
      if (float_key(x) < floor_key) continue;
      // u in (0,1]; e = -log(u) ~ Exp(1); score = x/T - log(e)
      const float u = (static_cast<float>(rr[j] >> 8) + 1.0f) * (1.0f / 16777216.0f);
      const float e = -__logf(u);
      const float score = x / temp - __logf(fmaxf(e, 1e-30f));
      if (score > best.v || (score == best.v && i < best.i)) {
        best.v = score;
        best.i = i;
      }
    }
  }
  best = block_argmax(best, red_mi);
  if (threadIdx.x == 0) out[rowi] = best.i == 0x7fffffff ? (m.i == 0x7fffffff ? 0 : m.i) : best.i;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_argmax(const void* logits, int* out, int B, int V, long long stride,
                           int is_fp32, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (is_fp32)
    argmax_kernel<float><<<B, kSampleThreads, 0, stream>>>(static_cast<const float*>(logits), out, V, stride);
  else
    argmax_kernel<__nv_bfloat16><<<B, kSampleThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(logits), out, V, stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_sample(const void* logits, int* out, const float* temperature, const int* top_k,
                           const float* top_p, const long long* seeds, const long long* step_offset,
                           int B, int V, long long stride, int is_fp32, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (is_fp32)
    sample_kernel<float><<<B, kSampleThreads, 0, stream>>>(static_cast<const float*>(logits), out,
                                                           temperature, top_k, top_p, seeds,
                                                           step_offset, V, stride);
  else
    sample_kernel<__nv_bfloat16><<<B, kSampleThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(logits), out, temperature, top_k, top_p, seeds,
        step_offset, V, stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
