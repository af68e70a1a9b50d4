// Rotary position embedding and paged KV-cache writes.
//
//  * rope_qk:         in-place RoPE on q [T,Hq,D] and k [T,Hk,D] (neox or gpt-j
//                     pairing, partial rotary dim, optional 3-section M-RoPE).
//  * rope_cache_gqa:  RoPE on q and k, then k and v stored into the paged cache
//                     at slot_mapping in the same pass (one read of qkv).
//  * mla_kv_rmsnorm_rope_cache: for multi-head latent attention: RMSNorm of the
//                     512-wide compressed KV, RoPE of the 64-wide shared key,
//                     both written into the paged latent cache row (576 wide),
//                     optionally also an indexer key row.
//  * paged_kv_scatter: plain copy of rows into cache slots.
//
// GQA cache layout: [num_blocks, kv_heads, block_size, D]; slot = block * block_size + offset.
// MLA cache layout: [num_blocks, block_size, 576].
//
// Replaces npu_apply_rotary_pos_emb / npu_interleave_rope / npu_rotary_mul /
// npu_scatter_nd_update_ / npu_kv_rmsnorm_rope_cache
// (omni_npu/attention/backends/attention.py:216-262, omni_npu/v1/layers/attention/npu_mla.py:196).

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/pdl.cuh"

namespace b200 {

__device__ __forceinline__ void rotate_pair(__nv_bfloat16* base, int i0, int i1, float c, float s) {
  const float x0 = __bfloat162float(base[i0]);
  const float x1 = __bfloat162float(base[i1]);
  base[i0] = __float2bfloat16(x0 * c - x1 * s);
  base[i1] = __float2bfloat16(x1 * c + x0 * s);
}

// cos_sin: [max_pos, rot_dim] fp32, first half cos, second half sin.
// mrope_sections: null, or 3 ints (t,h,w) that partition rot_dim/2; positions is
// then [3, T] and frequency index i takes its position from the section it falls in.
__global__ void __launch_bounds__(256)
rope_qk_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
               const int* __restrict__ positions, const float* __restrict__ cos_sin, int T, int Hq,
               int Hk, int D, int rot_dim, int neox, long long q_stride, long long k_stride,
               int sec_t, int sec_h, int interleaved_mrope) {
  const int t = blockIdx.x;
  const int half = rot_dim >> 1;
  const int total = (Hq + Hk) * half;
  for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
    const int head = idx / half;
    const int i = idx - head * half;
    int pos;
    if (sec_t < 0) {
      pos = positions[t];
    } else {
      int axis;
      if (interleaved_mrope) {
        // t,h,w frequencies interleaved (period 3) while the h / w sections last.
        const int m = i % 3;
        axis = (m == 1 && i < 3 * sec_h) ? 1 : ((m == 2 && i < 3 * (half - sec_t - sec_h)) ? 2 : 0);
      } else {
        axis = i < sec_t ? 0 : (i < sec_t + sec_h ? 1 : 2);
      }
      pos = positions[axis * T + t];
    }
    const float c = cos_sin[static_cast<long long>(pos) * rot_dim + i];
    const float s = cos_sin[static_cast<long long>(pos) * rot_dim + half + i];
    __nv_bfloat16* base = head < Hq ? q + t * q_stride + static_cast<long long>(head) * D
                                    : k + t * k_stride + static_cast<long long>(head - Hq) * D;
    if (neox) {
      rotate_pair(base, i, i + half, c, s);
    } else {
      rotate_pair(base, 2 * i, 2 * i + 1, c, s);
    }
  }
}

// q, k, v are views into one [T, (Hq + 2 Hk) * D] projection output.
__global__ void __launch_bounds__(256)
rope_cache_gqa_kernel(__nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                      const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ k_cache,
                      __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ positions,
                      const int* __restrict__ slot_mapping, const float* __restrict__ cos_sin,
                      int Hq, int Hk, int D, int rot_dim, int neox, long long q_stride,
                      long long k_stride, long long v_stride, int block_size) {
  b200::pdl_trigger();
  b200::pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int slot = slot_mapping[t];
  const int half = rot_dim >> 1;
  const float* cs = cos_sin + static_cast<long long>(pos) * rot_dim;
  // q heads in place.
  for (int idx = threadIdx.x; idx < Hq * half; idx += blockDim.x) {
    const int head = idx / half;
    const int i = idx - head * half;
    __nv_bfloat16* base = q + t * q_stride + static_cast<long long>(head) * D;
    if (neox) {
      rotate_pair(base, i, i + half, cs[i], cs[half + i]);
    } else {
      rotate_pair(base, 2 * i, 2 * i + 1, cs[i], cs[half + i]);
    }
  }
  if (slot < 0) return;  // padded token: nothing to store
  const long long blk = slot / block_size;
  const int off = slot - static_cast<int>(blk) * block_size;
  // k heads: rotate and store; dims beyond rot_dim are copied.
  for (int idx = threadIdx.x; idx < Hk * (D >> 1); idx += blockDim.x) {
    const int head = idx / (D >> 1);
    const int i = idx - head * (D >> 1);
    const __nv_bfloat16* src = k + t * k_stride + static_cast<long long>(head) * D;
    __nv_bfloat16* dst = k_cache + ((blk * Hk + head) * block_size + off) * D;
    int i0, i1;
    bool rot;
    if (neox) {
      // pair (i, i + half) for i < half; the remaining dims in order.
      if (i < half) {
        i0 = i;
        i1 = i + half;
        rot = true;
      } else {
        i0 = rot_dim + 2 * (i - half);
        i1 = i0 + 1;
        rot = false;
      }
    } else {
      i0 = 2 * i;
      i1 = 2 * i + 1;
      rot = i < half;
    }
    const float x0 = __bfloat162float(src[i0]);
    const float x1 = __bfloat162float(src[i1]);
    if (rot) {
      const float c = cs[i], s = cs[half + i];
      dst[i0] = __float2bfloat16(x0 * c - x1 * s);
      dst[i1] = __float2bfloat16(x1 * c + x0 * s);
    } else {
      dst[i0] = src[i0];
      dst[i1] = src[i1];
    }
  }
  // v heads: 16-byte copies.
  const int vec_per_head = D >> 3;
  for (int idx = threadIdx.x; idx < Hk * vec_per_head; idx += blockDim.x) {
    const int head = idx / vec_per_head;
    const int i = idx - head * vec_per_head;
    const uint4 val =
        reinterpret_cast<const uint4*>(v + t * v_stride + static_cast<long long>(head) * D)[i];
    reinterpret_cast<uint4*>(v_cache + ((blk * Hk + head) * block_size + off) * D)[i] = val;
  }
}

// ---- the same operation with 16-byte accesses -----------------------------------------------
// A token's work is cut into items of eight elements: rotary items of q (in place), rotary items
// of k (stored into the cache), the k dims past rot_dim and all of v (copies).  A thread loads
// two items before it stores either, so a decode step (one CTA per token, a few hundred items)
// costs one round trip to memory instead of one per pair of elements.
struct RopeItem {
  uint4 a, b;
  float4 c0, c1, s0, s1;
  __nv_bfloat16* dst_a;
  __nv_bfloat16* dst_b;
  int kind;     // 0 nothing, 1 rotate (i, i + half), 2 rotate (2i, 2i + 1), 3 copy
};

struct RopeVecArgs {
  __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  const float* cs;          // this token's cos | sin row
  long long cache_row;      // (block * Hk) * block_size + offset, in rows of D; head h adds h * block_size
  int Hq, Hk, D, rot_dim, half, neox, block_size;
  int per_rot, nq, nk, nkp, nv;
};

__device__ __forceinline__ void rope_item_load(const RopeVecArgs& g, int idx, RopeItem& it) {
  it.kind = 0;
  const __nv_bfloat16* src;
  __nv_bfloat16* dst;
  int j;
  if (idx < g.nq + g.nk) {
    const bool is_q = idx < g.nq;
    const int local = is_q ? idx : idx - g.nq;
    const int head = local / g.per_rot;
    j = local - head * g.per_rot;
    if (is_q) {
      dst = g.q + static_cast<long long>(head) * g.D;
      src = dst;
    } else {
      src = g.k + static_cast<long long>(head) * g.D;
      dst = g.k_cache + (g.cache_row + static_cast<long long>(head) * g.block_size) * g.D;
    }
    if (g.neox) {
      it.kind = 1;
      it.a = *reinterpret_cast<const uint4*>(src + 8 * j);
      it.b = *reinterpret_cast<const uint4*>(src + g.half + 8 * j);
      it.c0 = *reinterpret_cast<const float4*>(g.cs + 8 * j);
      it.c1 = *reinterpret_cast<const float4*>(g.cs + 8 * j + 4);
      it.s0 = *reinterpret_cast<const float4*>(g.cs + g.half + 8 * j);
      it.s1 = *reinterpret_cast<const float4*>(g.cs + g.half + 8 * j + 4);
      it.dst_a = dst + 8 * j;
      it.dst_b = dst + g.half + 8 * j;
    } else {
      it.kind = 2;
      it.a = *reinterpret_cast<const uint4*>(src + 8 * j);
      it.c0 = *reinterpret_cast<const float4*>(g.cs + 4 * j);
      it.s0 = *reinterpret_cast<const float4*>(g.cs + g.half + 4 * j);
      it.dst_a = dst + 8 * j;
    }
    return;
  }
  idx -= g.nq + g.nk;
  if (idx < g.nkp) {
    const int per = (g.D - g.rot_dim) >> 3;
    const int head = idx / per;
    j = idx - head * per;
    it.kind = 3;
    it.a = *reinterpret_cast<const uint4*>(g.k + static_cast<long long>(head) * g.D + g.rot_dim + 8 * j);
    it.dst_a = g.k_cache + (g.cache_row + static_cast<long long>(head) * g.block_size) * g.D + g.rot_dim + 8 * j;
    return;
  }
  idx -= g.nkp;
  if (idx < g.nv) {
    const int per = g.D >> 3;
    const int head = idx / per;
    j = idx - head * per;
    it.kind = 3;
    it.a = *reinterpret_cast<const uint4*>(g.v + static_cast<long long>(head) * g.D + 8 * j);
    it.dst_a = g.v_cache + (g.cache_row + static_cast<long long>(head) * g.block_size) * g.D + 8 * j;
  }
}

__device__ __forceinline__ void rope_item_store(RopeItem& it) {
  if (it.kind == 0) return;
  if (it.kind == 3) {
    *reinterpret_cast<uint4*>(it.dst_a) = it.a;
    return;
  }
  __nv_bfloat162* pa = reinterpret_cast<__nv_bfloat162*>(&it.a);
  if (it.kind == 1) {
    __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&it.b);
    const float c[8] = {it.c0.x, it.c0.y, it.c0.z, it.c0.w, it.c1.x, it.c1.y, it.c1.z, it.c1.w};
    const float sn[8] = {it.s0.x, it.s0.y, it.s0.z, it.s0.w, it.s1.x, it.s1.y, it.s1.z, it.s1.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x0 = __bfloat1622float2(pa[e]);
      const float2 x1 = __bfloat1622float2(pb[e]);
      pa[e] = __floats2bfloat162_rn(x0.x * c[2 * e] - x1.x * sn[2 * e], x0.y * c[2 * e + 1] - x1.y * sn[2 * e + 1]);
      pb[e] = __floats2bfloat162_rn(x1.x * c[2 * e] + x0.x * sn[2 * e], x1.y * c[2 * e + 1] + x0.y * sn[2 * e + 1]);
    }
    *reinterpret_cast<uint4*>(it.dst_a) = it.a;
    *reinterpret_cast<uint4*>(it.dst_b) = it.b;
    return;
  }
  const float c[4] = {it.c0.x, it.c0.y, it.c0.z, it.c0.w};
  const float sn[4] = {it.s0.x, it.s0.y, it.s0.z, it.s0.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 x = __bfloat1622float2(pa[e]);
    pa[e] = __floats2bfloat162_rn(x.x * c[e] - x.y * sn[e], x.y * c[e] + x.x * sn[e]);
  }
  *reinterpret_cast<uint4*>(it.dst_a) = it.a;
}

__global__ void __launch_bounds__(256)
rope_cache_gqa_vec_kernel(__nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                          const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ k_cache,
                          __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ positions,
                          const int* __restrict__ slot_mapping, const float* __restrict__ cos_sin,
                          int Hq, int Hk, int D, int rot_dim, int neox, long long q_stride,
                          long long k_stride, long long v_stride, int block_size) {
  b200::pdl_trigger();
  b200::pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int slot = slot_mapping[t];
  RopeVecArgs g;
  g.q = q + t * q_stride;
  g.k = k + t * k_stride;
  g.v = v + t * v_stride;
  g.k_cache = k_cache;
  g.v_cache = v_cache;
  g.cs = cos_sin + static_cast<long long>(pos) * rot_dim;
  g.Hq = Hq, g.Hk = Hk, g.D = D, g.rot_dim = rot_dim, g.half = rot_dim >> 1, g.neox = neox;
  g.block_size = block_size;
  g.per_rot = neox ? (rot_dim >> 4) : (rot_dim >> 3);
  g.nq = Hq * g.per_rot;
  const bool store = slot >= 0;     // a padded token rotates q only
  g.nk = store ? Hk * g.per_rot : 0;
  g.nkp = store ? Hk * ((D - rot_dim) >> 3) : 0;
  g.nv = store ? Hk * (D >> 3) : 0;
  const long long blk = store ? slot / block_size : 0;
  g.cache_row = blk * Hk * block_size + (store ? slot - blk * block_size : 0);
  const int total = g.nq + g.nk + g.nkp + g.nv;
  for (int idx = threadIdx.x; idx < total; idx += 2 * blockDim.x) {
    RopeItem i0, i1;
    rope_item_load(g, idx, i0);
    i1.kind = 0;
    if (idx + static_cast<int>(blockDim.x) < total) rope_item_load(g, idx + blockDim.x, i1);
    rope_item_store(i0);
    rope_item_store(i1);
  }
}

// MLA: kv_c [T, L] (L = 512) is RMS-normalised with weight w; k_pe [T, R] (R = 64)
// gets RoPE (gpt-j/interleaved or neox pairing); the row [norm(kv_c) | rope(k_pe)]
// is written to cache[slot].  kv_c_out / k_pe_out (optional) receive the same
// values in token order for the prefill path.
__global__ void __launch_bounds__(128)
mla_kv_rmsnorm_rope_cache_kernel(const __nv_bfloat16* __restrict__ kv_c,
                                 const __nv_bfloat16* __restrict__ k_pe,
                                 const __nv_bfloat16* __restrict__ w,
                                 __nv_bfloat16* __restrict__ cache,
                                 __nv_bfloat16* __restrict__ kv_c_out,
                                 __nv_bfloat16* __restrict__ k_pe_out,
                                 const int* __restrict__ positions,
                                 const int* __restrict__ slot_mapping,
                                 const float* __restrict__ cos_sin, float eps, int L, int R,
                                 int neox, long long kvc_stride, long long kpe_stride,
                                 long long cache_row_stride) {
  __shared__ float red[4];
  const int t = blockIdx.x;
  const int slot = slot_mapping[t];
  const __nv_bfloat16* src = kv_c + t * kvc_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < L; i += blockDim.x) {
    const float x = __bfloat162float(src[i]);
    ss += x * x;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  const float tot = red[0] + red[1] + red[2] + red[3];
  const float inv = rsqrtf(tot / static_cast<float>(L) + eps);
  __nv_bfloat16* crow = slot >= 0 ? cache + static_cast<long long>(slot) * cache_row_stride : nullptr;
  for (int i = threadIdx.x; i < L; i += blockDim.x) {
    const __nv_bfloat16 y =
        __float2bfloat16(__bfloat162float(src[i]) * inv * __bfloat162float(w[i]));
    if (crow) crow[i] = y;
    if (kv_c_out) kv_c_out[static_cast<long long>(t) * L + i] = y;
  }
  const int half = R >> 1;
  const int pos = positions[t];
  const float* cs = cos_sin + static_cast<long long>(pos) * R;
  const __nv_bfloat16* pe = k_pe + t * kpe_stride;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const int i0 = neox ? i : 2 * i;
    const int i1 = neox ? i + half : 2 * i + 1;
    const float x0 = __bfloat162float(pe[i0]);
    const float x1 = __bfloat162float(pe[i1]);
    const float c = cs[i], s = cs[half + i];
    const __nv_bfloat16 y0 = __float2bfloat16(x0 * c - x1 * s);
    const __nv_bfloat16 y1 = __float2bfloat16(x1 * c + x0 * s);
    if (crow) {
      crow[L + i0] = y0;
      crow[L + i1] = y1;
    }
    if (k_pe_out) {
      k_pe_out[static_cast<long long>(t) * R + i0] = y0;
      k_pe_out[static_cast<long long>(t) * R + i1] = y1;
    }
  }
}

// dst[slot_mapping[t], :] = src[t, :]  (row_elems a multiple of 8).
__global__ void __launch_bounds__(128)
paged_scatter_rows_kernel(__nv_bfloat16* __restrict__ dst, const __nv_bfloat16* __restrict__ src,
                          const int* __restrict__ slot_mapping, int row_elems,
                          long long src_stride, long long dst_row_stride) {
  const int t = blockIdx.x;
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const uint4* s = reinterpret_cast<const uint4*>(src + t * src_stride);
  uint4* d = reinterpret_cast<uint4*>(dst + static_cast<long long>(slot) * dst_row_stride);
  for (int i = threadIdx.x; i < (row_elems >> 3); i += blockDim.x) d[i] = s[i];
}

// GQA cache write without RoPE (k already rotated): used by models whose rope is
// applied elsewhere.
__global__ void __launch_bounds__(128)
gqa_cache_write_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                       __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                       const int* __restrict__ slot_mapping, int Hk, int D, int Dv,
                       long long k_stride, long long v_stride, int block_size) {
  const int t = blockIdx.x;
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const long long blk = slot / block_size;
  const int off = slot - static_cast<int>(blk) * block_size;
  const int kvec = D >> 3, vvec = Dv >> 3;
  for (int idx = threadIdx.x; idx < Hk * kvec; idx += blockDim.x) {
    const int head = idx / kvec, i = idx - head * kvec;
    reinterpret_cast<uint4*>(k_cache + ((blk * Hk + head) * block_size + off) * D)[i] =
        reinterpret_cast<const uint4*>(k + t * k_stride + static_cast<long long>(head) * D)[i];
  }
  for (int idx = threadIdx.x; idx < Hk * vvec; idx += blockDim.x) {
    const int head = idx / vvec, i = idx - head * vvec;
    reinterpret_cast<uint4*>(v_cache + ((blk * Hk + head) * block_size + off) * Dv)[i] =
        reinterpret_cast<const uint4*>(v + t * v_stride + static_cast<long long>(head) * Dv)[i];
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_rope_qk(void* q, void* k, const int* positions, const float* cos_sin, int T,
                            int Hq, int Hk, int D, int rot_dim, int neox, long long q_stride,
                            long long k_stride, int sec_t, int sec_h, int interleaved_mrope,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  rope_qk_kernel<<<T, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(q),
                                        static_cast<__nv_bfloat16*>(k), positions, cos_sin, T, Hq,
                                        Hk, D, rot_dim, neox, q_stride, k_stride, sec_t, sec_h,
                                        interleaved_mrope);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_rope_cache_gqa(void* q, const void* k, const void* v, void* k_cache,
                                   void* v_cache, const int* positions, const int* slot_mapping,
                                   const float* cos_sin, int T, int Hq, int Hk, int D, int rot_dim,
                                   int neox, long long q_stride, long long k_stride,
                                   long long v_stride, int block_size, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((D & 7) != 0 || (rot_dim & 1) != 0 || rot_dim > D) return -1;
  const auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = (rot_dim & 15) == 0 && ((q_stride | k_stride | v_stride) & 7) == 0 && al16(q) && al16(k) &&
                   al16(v) && al16(k_cache) && al16(v_cache) && al16(cos_sin);
  b200::launch_pdl(vec ? rope_cache_gqa_vec_kernel : rope_cache_gqa_kernel, dim3(T), dim3(256), 0, stream, 1,
                   static_cast<__nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
                   static_cast<const __nv_bfloat16*>(v), static_cast<__nv_bfloat16*>(k_cache),
                   static_cast<__nv_bfloat16*>(v_cache), positions, slot_mapping, cos_sin, Hq, Hk, D, rot_dim,
                   neox, q_stride, k_stride, v_stride, block_size);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_mla_kv_rmsnorm_rope_cache(const void* kv_c, const void* k_pe, const void* w,
                                              void* cache, void* kv_c_out, void* k_pe_out,
                                              const int* positions, const int* slot_mapping,
                                              const float* cos_sin, float eps, int T, int L, int R,
                                              int neox, long long kvc_stride, long long kpe_stride,
                                              long long cache_row_stride, cudaStream_t stream) {
  if (T <= 0) return 0;
  mla_kv_rmsnorm_rope_cache_kernel<<<T, 128, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(kv_c), static_cast<const __nv_bfloat16*>(k_pe),
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(cache),
      static_cast<__nv_bfloat16*>(kv_c_out), static_cast<__nv_bfloat16*>(k_pe_out), positions,
      slot_mapping, cos_sin, eps, L, R, neox, kvc_stride, kpe_stride, cache_row_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_paged_scatter_rows(void* dst, const void* src, const int* slot_mapping, int T,
                                       int row_elems, long long src_stride,
                                       long long dst_row_stride, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((row_elems & 7) != 0) return -1;
  paged_scatter_rows_kernel<<<T, 128, 0, stream>>>(static_cast<__nv_bfloat16*>(dst),
                                                   static_cast<const __nv_bfloat16*>(src),
                                                   slot_mapping, row_elems, src_stride,
                                                   dst_row_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_gqa_cache_write(const void* k, const void* v, void* k_cache, void* v_cache,
                                    const int* slot_mapping, int T, int Hk, int D, int Dv,
                                    long long k_stride, long long v_stride, int block_size,
                                    cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((D & 7) != 0 || (Dv & 7) != 0) return -1;
  gqa_cache_write_kernel<<<T, 128, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
      static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), slot_mapping, Hk,
      D, Dv, k_stride, v_stride, block_size);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
