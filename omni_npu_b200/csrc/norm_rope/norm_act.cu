// Bandwidth-bound row kernels: RMSNorm, fused residual-add + RMSNorm, SiLU-and-mul,
// and 1x128 block-scaled fp8 (e4m3) activation quantisation.
//
// Each row is read once with 16-byte loads, kept in registers between the
// reduction and the scaling pass, and written once.
//
// Replaces npu_rms_norm / npu_add_rms_norm (omni_npu/layers/npu_rms_norm.py:21-28),
// npu_swiglu (omni_npu/layers/activation.py:11-33) and npu_dynamic_quant.

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/pdl.cuh"

namespace b200 {

static constexpr int kNormThreads = 256;
static constexpr int kMaxVecPerThread = 8;  // 8 vectors * 8 bf16 * 256 threads = 16384 columns

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  const int nw = blockDim.x >> 5;
  float t = (l < nw) ? red[l] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

union Vec8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

// One CTA per row.  ADD: x <- x + residual is written back to residual first.
template <bool ADD>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x,
               __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ w, float eps,
               int H, long long x_stride, long long out_stride, long long res_stride) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * x_stride;
  __nv_bfloat16* rr = ADD ? residual + row * res_stride : nullptr;
  __nv_bfloat16* orow = out + row * out_stride;
  const int nvec = H >> 3;
  float vals[kMaxVecPerThread][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVecPerThread; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      Vec8 a;
      a.u = reinterpret_cast<const uint4*>(xr)[v];
      if (ADD) {
        Vec8 b;
        b.u = reinterpret_cast<const uint4*>(rr)[v];
        Vec8 s;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // The sum is rounded to bf16 before it is normalised, exactly as an
          // unfused add followed by a norm would do.
          s.h[j] = __float2bfloat16(__bfloat162float(a.h[j]) + __bfloat162float(b.h[j]));
          vals[i][j] = __bfloat162float(s.h[j]);
        }
        reinterpret_cast<uint4*>(rr)[v] = s.u;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[i][j] = __bfloat162float(a.h[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
    }
  }
  const float tot = block_sum(ss, red);
  const float inv = rsqrtf(tot / static_cast<float>(H) + eps);
#pragma unroll
  for (int i = 0; i < kMaxVecPerThread; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      Vec8 g;
      g.u = reinterpret_cast<const uint4*>(w)[v];
      Vec8 o;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        o.h[j] = __float2bfloat16(vals[i][j] * inv * __bfloat162float(g.h[j]));
      reinterpret_cast<uint4*>(orow)[v] = o.u;
    }
  }
}

// One warp per row, for short rows (per-head q/k norms, H <= 256*... up to 2048).
__global__ void __launch_bounds__(256)
rmsnorm_warp_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x,
                    const __nv_bfloat16* __restrict__ w, float eps, int H, long long rows,
                    long long x_stride, long long out_stride) {
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* xr = x + row * x_stride;
  __nv_bfloat16* orow = out + row * out_stride;
  const int nvec = H >> 3;
  float vals[8][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int v = lane + i * 32;
    if (v < nvec) {
      Vec8 a;
      a.u = reinterpret_cast<const uint4*>(xr)[v];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        vals[i][j] = __bfloat162float(a.h[j]);
        ss += vals[i][j] * vals[i][j];
      }
    }
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / static_cast<float>(H) + eps);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int v = lane + i * 32;
    if (v < nvec) {
      Vec8 g, o;
      g.u = reinterpret_cast<const uint4*>(w)[v];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        o.h[j] = __float2bfloat16(vals[i][j] * inv * __bfloat162float(g.h[j]));
      reinterpret_cast<uint4*>(orow)[v] = o.u;
    }
  }
}

// out[t, i] = silu(x[t, i]) * x[t, I + i]
__global__ void __launch_bounds__(256)
silu_mul_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x, int I,
                long long x_stride, long long out_stride) {
  const long long row = blockIdx.y;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= (I >> 3)) return;
  Vec8 g, u, o;
  g.u = reinterpret_cast<const uint4*>(x + row * x_stride)[v];
  u.u = reinterpret_cast<const uint4*>(x + row * x_stride + I)[v];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float a = __bfloat162float(g.h[j]);
    const float b = __bfloat162float(u.h[j]);
    o.h[j] = __float2bfloat16((a / (1.f + __expf(-a))) * b);
  }
  reinterpret_cast<uint4*>(out + row * out_stride)[v] = o.u;
}

// Per-token, per-128-column dynamic quantisation to e4m3: scale = amax / 448.
// One warp per (row, 128-column group); each lane holds 4 values.
__global__ void __launch_bounds__(256)
quant_fp8_1x128_kernel(uint8_t* __restrict__ q, float* __restrict__ scales,
                       const __nv_bfloat16* __restrict__ x, long long rows, int H,
                       long long x_stride, int ue8m0) {
  const int groups = H >> 7;
  const long long gid = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (gid >= rows * groups) return;
  const long long row = gid / groups;
  const int g = static_cast<int>(gid % groups);
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* src = x + row * x_stride + g * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  float v[4] = {__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1)};
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  float scale = fmaxf(amax, 1e-10f) / 448.f;
  if (ue8m0) scale = exp2f(ceilf(log2f(scale)));  // power-of-two scale
  const float inv = 1.f / scale;
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_fp8_e4m3 f(v[j] * inv);
    packed |= static_cast<uint32_t>(f.__x) << (8 * j);
  }
  *reinterpret_cast<uint32_t*>(q + row * H + g * 128 + lane * 4) = packed;
  if (lane == 0) scales[row * groups + g] = scale;
}

// ------------------------------------------------- norm / activation fused with quantisation
__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();                       // red may still be read by the reduction before this one
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float m = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
  return m;
}

// KIND 1: e4m3, scale = amax / 448;  KIND 2: int8, scale = amax / 127 (round to nearest even).
template <int KIND>
__device__ __forceinline__ uint8_t quant_one(float v, float inv) {
  if constexpr (KIND == 1) {
    const __nv_fp8_e4m3 f(v * inv);
    return f.__x;
  } else {
    const float r = fminf(fmaxf(rintf(v * inv), -127.f), 127.f);
    return static_cast<uint8_t>(static_cast<int8_t>(r));
  }
}

// (x [+ residual]) -> RMSNorm -> per-token dynamic quantisation, one pass over the row: the row
// lives in registers between the two block reductions (sum of squares, then max |y|).  The
// normalised row is rounded to bf16 before it is quantised, as the unfused sequence would do.
// One CTA per row; optional bf16 copy of the normalised row (for consumers that are not quantised).
template <bool ADD, int KIND>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_quant_kernel(uint8_t* __restrict__ q, float* __restrict__ scales, __nv_bfloat16* __restrict__ out,
                     const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ residual,
                     const __nv_bfloat16* __restrict__ w, float eps, int H, long long x_stride,
                     long long out_stride, long long res_stride) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * x_stride;
  __nv_bfloat16* rr = ADD ? residual + row * res_stride : nullptr;
  const int nvec = H >> 3;
  float vals[kMaxVecPerThread][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVecPerThread; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      Vec8 a;
      a.u = reinterpret_cast<const uint4*>(xr)[v];
      if (ADD) {
        Vec8 b, s;
        b.u = reinterpret_cast<const uint4*>(rr)[v];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s.h[j] = __float2bfloat16(__bfloat162float(a.h[j]) + __bfloat162float(b.h[j]));
          vals[i][j] = __bfloat162float(s.h[j]);
        }
        reinterpret_cast<uint4*>(rr)[v] = s.u;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[i][j] = __bfloat162float(a.h[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
    }
  }
  const float tot = block_sum(ss, red);
  const float inv_rms = rsqrtf(tot / static_cast<float>(H) + eps);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVecPerThread; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      Vec8 g, o;
      g.u = reinterpret_cast<const uint4*>(w)[v];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o.h[j] = __float2bfloat16(vals[i][j] * inv_rms * __bfloat162float(g.h[j]));
        vals[i][j] = __bfloat162float(o.h[j]);
        amax = fmaxf(amax, fabsf(vals[i][j]));
      }
      if (out) reinterpret_cast<uint4*>(out + row * out_stride)[v] = o.u;
    }
  }
  amax = block_max(amax, red);
  const float scale = fmaxf(amax, 1e-10f) / (KIND == 1 ? 448.f : 127.f);
  const float inv = 1.f / scale;
  if (threadIdx.x == 0) scales[row] = scale;
  uint8_t* qr = q + row * static_cast<long long>(H);
#pragma unroll
  for (int i = 0; i < kMaxVecPerThread; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        lo |= static_cast<uint32_t>(quant_one<KIND>(vals[i][j], inv)) << (8 * j);
        hi |= static_cast<uint32_t>(quant_one<KIND>(vals[i][4 + j], inv)) << (8 * j);
      }
      reinterpret_cast<uint2*>(qr)[v] = make_uint2(lo, hi);
    }
  }
}

// silu(x[:, :I]) * x[:, I:] -> per-token dynamic quantisation.  One CTA per row, two sweeps over
// the row (the second one hits L1/L2): max |y| first, then quantise.  y is rounded to bf16 first.
template <int KIND>
__global__ void __launch_bounds__(256)
silu_mul_quant_kernel(uint8_t* __restrict__ q, float* __restrict__ scales, const __nv_bfloat16* __restrict__ x,
                      int I, long long x_stride) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const long long row = blockIdx.x;
  const uint4* g4 = reinterpret_cast<const uint4*>(x + row * x_stride);
  const uint4* u4 = reinterpret_cast<const uint4*>(x + row * x_stride + I);
  const int nvec = I >> 3;
  float amax = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    Vec8 g, u;
    g.u = g4[v];
    u.u = u4[v];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = __bfloat162float(g.h[j]);
      const float y = __bfloat162float(__float2bfloat16((a / (1.f + __expf(-a))) * __bfloat162float(u.h[j])));
      amax = fmaxf(amax, fabsf(y));
    }
  }
  amax = block_max(amax, red);
  const float scale = fmaxf(amax, 1e-10f) / (KIND == 1 ? 448.f : 127.f);
  const float inv = 1.f / scale;
  if (threadIdx.x == 0) scales[row] = scale;
  uint2* qr = reinterpret_cast<uint2*>(q + row * static_cast<long long>(I));
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    Vec8 g, u;
    g.u = g4[v];
    u.u = u4[v];
    uint32_t w2[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = __bfloat162float(g.h[j]);
      const float y = __bfloat162float(__float2bfloat16((a / (1.f + __expf(-a))) * __bfloat162float(u.h[j])));
      w2[j >> 2] |= static_cast<uint32_t>(quant_one<KIND>(y, inv)) << (8 * (j & 3));
    }
    qr[v] = make_uint2(w2[0], w2[1]);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_rmsnorm(void* out, const void* x, void* residual, const void* w, float eps,
                            long long rows, int H, long long x_stride, long long out_stride,
                            long long res_stride, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((H & 7) != 0) return -1;
  if (residual == nullptr && H <= 2048) {
    const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
    rmsnorm_warp_kernel<<<blocks, 256, 0, stream>>>(
        static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(x),
        static_cast<const __nv_bfloat16*>(w), eps, H, rows, x_stride, out_stride);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
  }
  if (H > kNormThreads * kMaxVecPerThread * 8) return -2;
  if (residual) {
    launch_pdl(rmsnorm_kernel<true>, dim3(static_cast<unsigned>(rows)), dim3(kNormThreads), 0, stream, 1,
               static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(x),
               static_cast<__nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(w), eps, H,
               x_stride, out_stride, res_stride);
  } else {
    launch_pdl(rmsnorm_kernel<false>, dim3(static_cast<unsigned>(rows)), dim3(kNormThreads), 0, stream, 1,
               static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(x),
               static_cast<__nv_bfloat16*>(nullptr), static_cast<const __nv_bfloat16*>(w), eps, H, x_stride,
               out_stride, 0LL);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_silu_mul(void* out, const void* x, long long rows, int I, long long x_stride,
                             long long out_stride, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((I & 7) != 0 || rows > 65535LL * 65535LL) return -1;
  // grid.y is limited to 65535: fold very tall inputs by launching in slabs.
  const int nvec = I >> 3;
  long long done = 0;
  while (done < rows) {
    const long long n = rows - done > 65535 ? 65535 : rows - done;
    dim3 grid((nvec + 255) / 256, static_cast<unsigned>(n));
    silu_mul_kernel<<<grid, 256, 0, stream>>>(
        static_cast<__nv_bfloat16*>(out) + done * out_stride,
        static_cast<const __nv_bfloat16*>(x) + done * x_stride, I, x_stride, out_stride);
    done += n;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ---------------------------------------------------------------- int8 per token
// Dynamic symmetric quantisation of activations: one scale per row,
// q = round(x / scale), scale = max|x| / 127.  One CTA per row.
__global__ void __launch_bounds__(256)
quant_int8_per_token_kernel(int8_t* __restrict__ q, float* __restrict__ scales,
                            const __nv_bfloat16* __restrict__ x, int H, long long x_stride) {
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * x_stride;
  __shared__ float red[8];
  float amax = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) amax = fmaxf(amax, fabsf(__bfloat162float(xr[i])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) amax = fmaxf(amax, red[w]);
  const float scale = fmaxf(amax, 1e-10f) / 127.f;
  const float inv = 1.f / scale;
  if (threadIdx.x == 0) scales[row] = scale;
  int8_t* qr = q + row * static_cast<long long>(H);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = rintf(__bfloat162float(xr[i]) * inv);
    qr[i] = static_cast<int8_t>(fminf(fmaxf(v, -127.f), 127.f));
  }
}

extern "C" int b200_quant_int8_per_token(void* q, void* scales, const void* x, long long rows, int H,
                                         long long x_stride, cudaStream_t stream) {
  if (rows <= 0) return 0;
  quant_int8_per_token_kernel<<<static_cast<unsigned>(rows), 256, 0, stream>>>(
      static_cast<int8_t*>(q), static_cast<float*>(scales), static_cast<const __nv_bfloat16*>(x), H, x_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_quant_fp8_1x128(void* q, void* scales, const void* x, long long rows, int H,
                                    long long x_stride, int ue8m0, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((H & 127) != 0) return -1;
  const long long groups = rows * (H >> 7);
  const unsigned blocks = static_cast<unsigned>((groups + 7) / 8);
  quant_fp8_1x128_kernel<<<blocks, 256, 0, stream>>>(static_cast<uint8_t*>(q),
                                                     static_cast<float*>(scales),
                                                     static_cast<const __nv_bfloat16*>(x), rows, H,
                                                     x_stride, ue8m0);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// RMSNorm (optionally with residual add, written back to `residual`) fused with per-token
// quantisation.  kind 1: e4m3 (scale = amax/448), 2: int8 (scale = amax/127).  out may be null.
extern "C" int b200_rmsnorm_quant(void* q, void* scales, void* out, const void* x, void* residual, const void* w,
                                  float eps, long long rows, int H, long long x_stride, long long out_stride,
                                  long long res_stride, int kind, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((H & 7) != 0 || (kind != 1 && kind != 2)) return -1;
  if (H > kNormThreads * kMaxVecPerThread * 8) return -2;
  const dim3 grid(static_cast<unsigned>(rows)), block(kNormThreads);
  auto* qq = static_cast<uint8_t*>(q);
  auto* sc = static_cast<float*>(scales);
  auto* o = static_cast<__nv_bfloat16*>(out);
  auto* xx = static_cast<const __nv_bfloat16*>(x);
  auto* rr = static_cast<__nv_bfloat16*>(residual);
  auto* ww = static_cast<const __nv_bfloat16*>(w);
  cudaError_t e;
  if (residual) {
    e = kind == 1 ? launch_pdl(rmsnorm_quant_kernel<true, 1>, grid, block, 0, stream, 1, qq, sc, o, xx, rr, ww, eps, H,
                               x_stride, out_stride, res_stride)
                  : launch_pdl(rmsnorm_quant_kernel<true, 2>, grid, block, 0, stream, 1, qq, sc, o, xx, rr, ww, eps, H,
                               x_stride, out_stride, res_stride);
  } else {
    e = kind == 1 ? launch_pdl(rmsnorm_quant_kernel<false, 1>, grid, block, 0, stream, 1, qq, sc, o, xx, rr, ww, eps,
                               H, x_stride, out_stride, res_stride)
                  : launch_pdl(rmsnorm_quant_kernel<false, 2>, grid, block, 0, stream, 1, qq, sc, o, xx, rr, ww, eps,
                               H, x_stride, out_stride, res_stride);
  }
  return e == cudaSuccess ? 0 : -3;
}

extern "C" int b200_silu_mul_quant(void* q, void* scales, const void* x, long long rows, int I, long long x_stride,
                                   int kind, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((I & 7) != 0 || (kind != 1 && kind != 2)) return -1;
  const dim3 grid(static_cast<unsigned>(rows)), block(256);
  auto* qq = static_cast<uint8_t*>(q);
  auto* sc = static_cast<float*>(scales);
  auto* xx = static_cast<const __nv_bfloat16*>(x);
  const cudaError_t e = kind == 1 ? launch_pdl(silu_mul_quant_kernel<1>, grid, block, 0, stream, 1, qq, sc, xx, I, x_stride)
                                  : launch_pdl(silu_mul_quant_kernel<2>, grid, block, 0, stream, 1, qq, sc, xx, I, x_stride);
  return e == cudaSuccess ? 0 : -3;
}
