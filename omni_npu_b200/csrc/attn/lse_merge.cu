// Merging partial attention results by their log-sum-exp, and gathering a paged cache.
//
//   merge:  out = sum_i exp(lse_i - lse) * out_i,   lse = log(sum_i exp(lse_i))
// for N partial results over disjoint key sets (chunked context, split-KV across ranks in
// decode context parallelism).  Partials with lse = -inf (no keys) contribute nothing.
// One warp per (token, head); head_dim is streamed in 16-byte vectors.
//
//   gather: rows of a paged cache [blocks, block_size, width] named by a block table are
// copied into a contiguous [total_tokens, width] tensor (sequence after sequence).
//
// Device counterparts of merge_attn_states / attention_update_torch /
// gather_and_maybe_dequant_cache (omni_npu/attention/ops.py:5-141).

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace b200 {

union MergePack8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

// outs [N][T][H][D] bf16 (stride_n elements between partials), lses [N][T][H] fp32
__global__ void __launch_bounds__(128)
lse_merge_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ lse_out, const __nv_bfloat16* __restrict__ outs,
                 const float* __restrict__ lses, int N, long long TH, int D, long long stride_n_out,
                 long long stride_n_lse) {
  const long long idx = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (idx >= TH) return;
  const int lane = threadIdx.x & 31;
  float m = -INFINITY;
  for (int i = 0; i < N; ++i) m = fmaxf(m, lses[i * stride_n_lse + idx]);
  float denom = 0.f;
  for (int i = 0; i < N; ++i) {
    const float l = lses[i * stride_n_lse + idx];
    denom += (l == -INFINITY) ? 0.f : __expf(l - m);
  }
  const bool empty = (m == -INFINITY) || denom == 0.f;
  if (lane == 0 && lse_out) lse_out[idx] = empty ? -INFINITY : m + __logf(denom);
  const float inv = empty ? 0.f : 1.f / denom;
  for (int v = lane; v * 8 < D; v += 32) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < N; ++i) {
      const float l = lses[i * stride_n_lse + idx];
      if (l == -INFINITY) continue;
      const float w = __expf(l - m) * inv;
      MergePack8 p;
      p.u = *reinterpret_cast<const uint4*>(outs + i * stride_n_out + idx * D + v * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += w * __bfloat162float(p.h[j]);
    }
    MergePack8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.h[j] = __float2bfloat16(acc[j]);
    *reinterpret_cast<uint4*>(out + idx * D + v * 8) = o.u;
  }
}

// cache [blocks][block_size][width] (16-byte multiples), block_tables [B][max_blocks],
// cu_seq [B+1] exclusive prefix sums of the sequence lengths; one CTA per (sequence, block).
__global__ void __launch_bounds__(128)
gather_cache_kernel(uint4* __restrict__ dst, const uint4* __restrict__ cache, const int* __restrict__ block_tables,
                    const int* __restrict__ cu_seq, int max_blocks, int block_size, int row_vecs) {
  const int b = blockIdx.y, blk = blockIdx.x;
  const int len = cu_seq[b + 1] - cu_seq[b];
  const int first = blk * block_size;
  if (first >= len) return;
  const int rows = min(block_size, len - first);
  const long long src0 = static_cast<long long>(block_tables[static_cast<long long>(b) * max_blocks + blk]) *
                         block_size * row_vecs;
  const long long dst0 = (static_cast<long long>(cu_seq[b]) + first) * row_vecs;
  const int n = rows * row_vecs;
  for (int i = threadIdx.x; i < n; i += blockDim.x) dst[dst0 + i] = cache[src0 + i];
}

}  // namespace b200

extern "C" int b200_lse_merge(void* out, float* lse_out, const void* outs, const float* lses, int N, long long T,
                              int H, int D, long long stride_n_out, long long stride_n_lse, cudaStream_t stream) {
  if (N <= 0 || T <= 0) return 0;
  if ((D & 7) != 0) return -1;
  const long long th = T * H;
  b200::lse_merge_kernel<<<static_cast<unsigned>((th + 3) / 4), 128, 0, stream>>>(
      static_cast<__nv_bfloat16*>(out), lse_out, static_cast<const __nv_bfloat16*>(outs), lses, N, th, D,
      stride_n_out, stride_n_lse);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_gather_cache(void* dst, const void* cache, const int* block_tables, const int* cu_seq, int B,
                                 int max_blocks, int block_size, int row_bytes, int max_seq_len,
                                 cudaStream_t stream) {
  if (B <= 0) return 0;
  if ((row_bytes & 15) != 0) return -1;
  const int nblk = (max_seq_len + block_size - 1) / block_size;
  if (nblk <= 0) return 0;
  dim3 grid(nblk, B);
  b200::gather_cache_kernel<<<grid, 128, 0, stream>>>(static_cast<uint4*>(dst), static_cast<const uint4*>(cache),
                                                      block_tables, cu_seq, max_blocks, block_size, row_bytes >> 4);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
