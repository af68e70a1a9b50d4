// Block-scaled e4m3 GEMM for sm_100a (the DeepSeek-V3 checkpoint format):
//
//   C[m, n] = sum_kb  a_s[m, kb] * w_s[n / 128, kb] * sum_{k in block kb} A[m, k] * W[n, k]
//
// A [M, K] e4m3 with one fp32 scale per (row, 128 columns); W [N, K] e4m3 with one fp32
// scale per (128 rows, 128 columns).  One 128-byte K slab of e4m3 is exactly one scale block,
// so every slab's product needs its own scale before it may be added to the others.
//
// Per CTA: a persistent loop over 128 x 128 output tiles.  Warp 0 streams A and W slabs
// with TMA into a shared-memory ring; warp 1 issues, per slab, four tcgen05.mma
// (kind::f8f6f4, K = 32 each) into one of TWO partial accumulators in TMEM (fresh, not
// accumulating across slabs); warps 2-5 read a finished partial from TMEM, multiply it by
// the slab's scale pair and add it to the tile's fp32 accumulator, which lives in their
// registers (one output row of 128 columns per thread).  The tensor core works on slab
// k + 1 while the promotion of slab k runs.  Epilogue: bias, residual, bf16 / fp32 store.
// All waits are bounded and report through the status word.
//
// Replaces the reference's closed quantised-matmul op for this format
// (torch_npu.npu_quant_matmul, omni_npu/layers/quantization/...; scale layout
// [N/128, K/128] of HF `weight_scale_inv`).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>

#include "../common/pdl.cuh"
#include "../common/ptx.cuh"
#include "../common/tensormap.h"
#include "../common/device_once.h"

namespace b200 {

constexpr int kFbBM = 128, kFbBN = 128, kFbSlab = 128;   // tile and K slab (bytes = elements for e4m3)
// WG = number of epilogue warp groups = tile width / 128.  One group: 128 x 128 tiles, six stages.
// Two groups: 128 x 256 tiles (each group promotes its own 128 columns, so the promotion time per MMA
// cycle halves), four stages, all 512 TMEM columns for the two partial accumulators.
template <int WG> struct FbCfg {
  static constexpr int TN = kFbBN * WG;
  static constexpr int STAGES = WG == 1 ? 6 : 4;
  static constexpr int STAGE_BYTES = (kFbBM + TN) * kFbSlab;
  static constexpr int THREADS = 64 + 128 * WG;
  static constexpr int TMEM_COLS = 2 * TN;
  static constexpr size_t SMEM_BASE = 1024 + static_cast<size_t>(STAGES) * STAGE_BYTES + (2 * STAGES + 4) * 8 + 32;
};

struct Fp8BlockParams {
  int M, N, K;
  int k_iters;              // K / 128
  int num_m_blocks, num_n_blocks;
  const float* a_scales;    // [M, k_iters]
  const float* w_scales;    // [ceil(N/128), k_iters]
  void* C;
  int ldc;
  int out_fp32;
  const __nv_bfloat16* bias;       // [N] or null
  const __nv_bfloat16* residual;   // [M, ldc] or null
  int* status;
  // grouped (mixture-of-experts) mode, num_experts > 0: A holds every expert's rows back to back,
  // expert e owns rows expert_offsets[e] .. expert_offsets[e + 1] (device array); W [E, N, K];
  // w_scales [E, scale_rows, k_iters].
  const int* expert_offsets;
  int num_experts;
  int scale_rows;           // rows of one expert's scale matrix
  // swiglu: W rows hold gate / up interleaved in groups of 8 (rows 16g .. 16g+7 gate, +8 .. +15 up);
  // their scale blocks are not interleaved: gate block b at scale row b, up block b at up_scale_row0 + b.
  // C [.., N / 2] = silu(gate) * up.
  int swiglu;
  int up_scale_row0;
};

constexpr int kFbMaxExperts = 512;

struct FbTile {
  int m0, m_end, n0, nb, expert;
};

// Tile t of this problem; grouped: n is the fast index so that concurrently running CTAs share
// an expert's rows.  s_prefix[e] = number of 128-row blocks of the experts before e.
__device__ __forceinline__ void fb_decode(const Fp8BlockParams& p, const int* s_prefix, long long t, int& cursor,
                                          FbTile& tc, int tile_n) {
  if (p.num_experts == 0) {
    tc.m0 = static_cast<int>(t % p.num_m_blocks) * kFbBM;
    tc.m_end = p.M;
    tc.nb = static_cast<int>(t / p.num_m_blocks);
    tc.expert = 0;
  } else {
    const int mblk = static_cast<int>(t / p.num_n_blocks);
    tc.nb = static_cast<int>(t % p.num_n_blocks);
    while (cursor + 1 < p.num_experts && s_prefix[cursor + 1] <= mblk) ++cursor;
    tc.expert = cursor;
    tc.m0 = p.expert_offsets[cursor] + (mblk - s_prefix[cursor]) * kFbBM;
    tc.m_end = p.expert_offsets[cursor + 1];
  }
  tc.n0 = tc.nb * tile_n;
}

template <int WG>
__global__ void __launch_bounds__(FbCfg<WG>::THREADS)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                      const Fp8BlockParams p) {
  using Cfg = FbCfg<WG>;
  constexpr int kFbStages = Cfg::STAGES;
  constexpr int kFbStageBytes = Cfg::STAGE_BYTES;
  constexpr int TN = Cfg::TN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* s_a = smem;                                   // [stages][128 x 128 B]
  uint8_t* s_w = smem + kFbStages * kFbBM * kFbSlab;     // [stages][128 x 128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kFbStages * kFbStageBytes);
  uint64_t* full = bars;                     // [stages]
  uint64_t* empty = bars + kFbStages;        // [stages]
  uint64_t* part_full = empty + kFbStages;   // [2]
  uint64_t* part_empty = part_full + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(part_empty + 2);
  int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);
  int* s_prefix = s_abort + 1;               // [num_experts + 1] (grouped)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (p.num_experts > 0) pdl_wait();         // the expert offsets come from the routing kernels ahead
  if (threadIdx.x == 0) {
    for (int s = 0; s < kFbStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&part_full[i], 1);
      mbar_init(&part_empty[i], 4 * WG);
    }
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_w);
  }
  if (p.num_experts > 0 && threadIdx.x == 64) {
    int acc = 0;
    for (int e = 0; e < p.num_experts; ++e) {
      s_prefix[e] = acc;
      acc += (p.expert_offsets[e + 1] - p.expert_offsets[e] + kFbBM - 1) / kFbBM;
    }
    s_prefix[p.num_experts] = acc;
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  volatile int* abort_flag = s_abort;
  pdl_trigger();
  pdl_wait();
  const long long tiles = p.num_experts > 0 ? static_cast<long long>(s_prefix[p.num_experts]) * p.num_n_blocks
                                            : static_cast<long long>(p.num_m_blocks) * p.num_n_blocks;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      int cursor = 0;
      FbTile tc;
      for (long long t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
        fb_decode(p, s_prefix, t, cursor, tc, TN);
        const int m0 = tc.m0, n0 = tc.n0;
        for (int kb = 0; kb < p.k_iters; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            atomicCAS(p.status, 0, kStatusTimeoutEmptyBarrier);
            *abort_flag = 1;
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full[stage], static_cast<uint32_t>(kFbStageBytes));
          tma_load_2d(s_a + stage * kFbBM * kFbSlab, &tm_a, &full[stage], kb * kFbSlab, m0);
          if (p.num_experts > 0)
            tma_load_3d(s_w + stage * TN * kFbSlab, &tm_w, &full[stage], kb * kFbSlab, n0, tc.expert);
          else
            tma_load_2d(s_w + stage * TN * kFbSlab, &tm_w, &full[stage], kb * kFbSlab, n0);
          ++issued;
          if (++stage == kFbStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // no bulk copy may land after the CTA retires: wait (bounded) for the loads in flight
        const int pending = issued < kFbStages ? static_cast<int>(issued) : kFbStages;
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) {
            s = kFbStages - 1;
            ph ^= 1;
          }
          mbar_wait(&full[s], ph);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(0, 0, kFbBM, TN);          // e4m3 x e4m3 -> fp32
      const uint32_t a_lo0 = (smem_u32(s_a) & 0x3FFFF) >> 4, w_lo0 = (smem_u32(s_w) & 0x3FFFF) >> 4;
      int stage = 0, pb = 0;
      uint32_t phase = 0, pph = 0;
      bool ok = true;
      for (long long t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
        for (int kb = 0; kb < p.k_iters; ++kb) {
          if (*abort_flag || !mbar_wait(&full[stage], phase) || !mbar_wait(&part_empty[pb], pph ^ 1)) {
            if (!*abort_flag) atomicCAS(p.status, 0, kStatusTimeoutFullBarrier);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t d = tmem_base + static_cast<uint32_t>(pb * TN);
          const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(stage * (kFbBM * kFbSlab >> 4));
          const uint32_t w_lo = w_lo0 + static_cast<uint32_t>(stage * (TN * kFbSlab >> 4));
          umma_first<kKindFP8>(d, a_lo, w_lo, idesc, 0u);
#pragma unroll
          for (int kk = 1; kk < 4; ++kk) umma_acc<kKindFP8>(d, a_lo + kk * 2, w_lo + kk * 2, idesc);
          tc_commit(&empty[stage]);
          tc_commit(&part_full[pb]);
          if (++stage == kFbStages) {
            stage = 0;
            phase ^= 1;
          }
          if (++pb == 2) {
            pb = 0;
            pph ^= 1;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------ promotion + epilogue
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int cb = ((warp - 2) >> 2) * kFbBN;     // this warp group's 128 columns inside the tile
    int pb = 0;
    uint32_t pph = 0;
    bool ok = true;
    int cursor = 0;
    FbTile tc;
    for (long long t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
      fb_decode(p, s_prefix, t, cursor, tc, TN);
      const int n0 = tc.n0 + cb;                   // first column of this thread's block (may lie beyond N)
      const int n0s = min(n0, p.N - 1);            // for scale lookups only
      const int row = tc.m0 + r;
      const bool row_ok = row < tc.m_end;
      const float* a_s = p.a_scales + static_cast<long long>(row_ok ? row : 0) * p.k_iters;
      const float* w_base = p.w_scales + static_cast<long long>(tc.expert) * p.scale_rows * p.k_iters;
      // scale row of the block's columns; with SwiGLU the gate and the up columns have one each
      const float* w_s = w_base + static_cast<long long>(p.swiglu ? (n0s >> 1) / 128 : n0s / 128) * p.k_iters;
      const float* w_s2 = p.swiglu ? w_base + static_cast<long long>(p.up_scale_row0 + (n0s >> 1) / 128) * p.k_iters
                                   : w_s;
      float acc[kFbBN];
#pragma unroll
      for (int c = 0; c < kFbBN; ++c) acc[c] = 0.f;
      const float a0 = row_ok ? a_s[0] : 0.f;
      float s_next = a0 * w_s[0], s2_next = a0 * w_s2[0];
      for (int kb = 0; kb < p.k_iters; ++kb) {
        const float s = s_next, s2 = s2_next;
        if (kb + 1 < p.k_iters) {                     // off the critical path
          const float a1 = row_ok ? a_s[kb + 1] : 0.f;
          s_next = a1 * w_s[kb + 1];
          s2_next = a1 * w_s2[kb + 1];
        }
        // every warp of the group decides alike: they all wait on the same barrier phase
        const bool mine = !*abort_flag && mbar_wait(&part_full[pb], pph);
        if (!__all_sync(0xffffffffu, mine)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                               static_cast<uint32_t>(pb * TN + cb);
#pragma unroll
        for (int c0 = 0; c0 < kFbBN; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(c0), v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)      // columns 8..15 of every 16 are "up" columns under SwiGLU
            acc[c0 + i] = fmaf(((i >> 3) & 1) ? s2 : s, __uint_as_float(v[i]), acc[c0 + i]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&part_empty[pb]);
        if (++pb == 2) {
          pb = 0;
          pph ^= 1;
        }
      }
      if (!ok) break;
      if (row_ok && p.swiglu) {
        // 64 outputs per row: silu(gate) * up, gate / up interleaved in groups of 8 columns (N % 16 == 0)
        __nv_bfloat16* crow = static_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + (n0 >> 1);
        const int nout = min(kFbBN, p.N - n0) >> 1;
#pragma unroll
        for (int g = 0; g < kFbBN / 16; ++g) {
          if (g * 8 < nout) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float gt = acc[g * 16 + i];
              o[i] = (gt / (1.f + __expf(-gt))) * acc[g * 16 + 8 + i];
            }
            uint4 pk;
            pk.x = pack_bf16x2(o[0], o[1]);
            pk.y = pack_bf16x2(o[2], o[3]);
            pk.z = pack_bf16x2(o[4], o[5]);
            pk.w = pack_bf16x2(o[6], o[7]);
            *reinterpret_cast<uint4*>(crow + g * 8) = pk;
          }
        }
      } else if (row_ok) {
        const int ncols = min(kFbBN, p.N - n0);
        if (p.out_fp32) {
          float* crow = static_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + n0;
#pragma unroll
          for (int c = 0; c < kFbBN; ++c) {      // fully unrolled: the accumulator stays in registers
            if (c < ncols) {
              float v = acc[c];
              if (p.bias) v += __bfloat162float(p.bias[n0 + c]);
              if (p.residual) v += __bfloat162float(p.residual[static_cast<long long>(row) * p.ldc + n0 + c]);
              crow[c] = v;
            }
          }
        } else {
          __nv_bfloat16* crow = static_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + n0;
          const bool vec_ok = ncols == kFbBN && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0);
#pragma unroll
          for (int c = 0; c < kFbBN; c += 8) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              v[i] = acc[c + i];
              if (c + i < ncols) {
                if (p.bias) v[i] += __bfloat162float(p.bias[n0 + c + i]);
                if (p.residual)
                  v[i] += __bfloat162float(p.residual[static_cast<long long>(row) * p.ldc + n0 + c + i]);
              }
            }
            if (vec_ok) {
              uint4 o;
              o.x = pack_bf16x2(v[0], v[1]);
              o.y = pack_bf16x2(v[2], v[3]);
              o.z = pack_bf16x2(v[4], v[5]);
              o.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(crow + c) = o;
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (c + i < ncols) crow[c + i] = __float2bfloat16(v[i]);
            }
          }
        }
      }
    }
    if (!ok && lane == 0) {
      if (!*abort_flag) atomicCAS(p.status, 0, kStatusTimeoutTmemFull);
      *abort_flag = 1;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace b200

using namespace b200;

template <int WG>
static int fb_launch_wg(const CUtensorMap& ta, const CUtensorMap& tw, const Fp8BlockParams& p, long long tiles,
                        int max_ctas, cudaStream_t stream) {
  using Cfg = FbCfg<WG>;
  const size_t smem = Cfg::SMEM_BASE + (static_cast<size_t>(p.num_experts) + 2) * 4;
  if (smem > 227u * 1024u) return -23;
  static DeviceOnce once;
  int cur = 0;
  if (once.needed(&cur)) {
    if (cudaFuncSetAttribute(gemm_fp8_block_kernel<WG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             227 * 1024) != cudaSuccess)
      return -20;
    once.mark(cur);
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = sms;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = static_cast<int>(tiles);
  if (grid < 1) grid = 1;
  return launch_pdl(gemm_fp8_block_kernel<WG>, dim3(grid), dim3(Cfg::THREADS), smem, stream, 1, ta, tw, p) ==
                 cudaSuccess
             ? 0
             : -21;
}

// 256-wide tiles pay off once there are enough of them to fill the GPU; small problems keep the
// narrow tile (more CTAs).  OMNI_B200_FP8_BLOCK_WG=1|2 forces a variant.
static int fb_pick_wg(long long rows, int N) {
  static const int forced = [] {
    const char* e = getenv("OMNI_B200_FP8_BLOCK_WG");
    return e ? atoi(e) : 0;
  }();
  if (forced == 1 || forced == 2) return N >= 256 || forced == 1 ? forced : 1;
  const long long wide_tiles = ((rows + kFbBM - 1) / kFbBM) * ((N + 255) / 256);
  return (N >= 256 && wide_tiles >= 148) ? 2 : 1;
}

// A [M, K] e4m3 (pitch lda bytes), a_scales [M, K/128]; W [N, K] e4m3 (pitch ldw), w_scales
// [ceil(N/128), K/128]; C [M, N] bf16 or fp32 (pitch ldc elements).  K must be a multiple of 128.
extern "C" int b200_gemm_fp8_block(const void* A, const float* a_scales, const void* W, const float* w_scales,
                                   void* C, const void* bias, const void* residual, int M, int N, int K, int lda,
                                   int ldw, int ldc, int out_fp32, int* status, int max_ctas,
                                   cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % kFbSlab) != 0) return -10;
  Fp8BlockParams p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.k_iters = K / kFbSlab;
  const int wg = fb_pick_wg(M, N);
  const int tn = kFbBN * wg;
  p.num_m_blocks = (M + kFbBM - 1) / kFbBM;
  p.num_n_blocks = (N + tn - 1) / tn;
  p.a_scales = a_scales;
  p.w_scales = w_scales;
  p.C = C;
  p.ldc = ldc;
  p.out_fp32 = out_fp32;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.status = status;
  p.scale_rows = (N + kFbBN - 1) / kFbBN;
  CUtensorMap ta, tw;
  int r = make_tensormap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, M, K, lda, kFbBM, kFbSlab,
                            CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r;
  r = make_tensormap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, W, N, K, ldw, tn, kFbSlab,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 1000;
  const long long tiles = static_cast<long long>(p.num_m_blocks) * p.num_n_blocks;
  return wg == 2 ? fb_launch_wg<2>(ta, tw, p, tiles, max_ctas, stream) : fb_launch_wg<1>(ta, tw, p, tiles, max_ctas, stream);
}

// Grouped (mixture-of-experts) variant.  A [total_rows, K] e4m3 holds every expert's rows back to
// back (expert_offsets [E + 1] on the device), a_scales [total_rows, K/128]; W [E, N, K] e4m3,
// w_scales [E, scale_rows, K/128].  swiglu = 1: W's gate / up rows are interleaved in groups of 8
// and C [total_rows, N/2] = silu(gate) * up; the scale rows are gate blocks 0.., then up blocks
// from row up_scale_row0.  C is bf16.
extern "C" int b200_grouped_gemm_fp8_block(const void* A, const float* a_scales, const void* W, const float* w_scales,
                                           void* C, const int* expert_offsets, int num_experts, int total_rows,
                                           int N, int K, int lda, int ldc, int scale_rows, int swiglu,
                                           int up_scale_row0, int* status, int max_ctas, cudaStream_t stream) {
  if (total_rows <= 0 || num_experts <= 0) return 0;
  if (num_experts > kFbMaxExperts) return -13;
  if ((K % kFbSlab) != 0) return -10;
  if (swiglu && (N % 16) != 0) return -11;
  Fp8BlockParams p{};
  p.M = total_rows;
  p.N = N;
  p.K = K;
  p.k_iters = K / kFbSlab;
  const int wg = fb_pick_wg(total_rows, N);
  const int tn = kFbBN * wg;
  p.num_m_blocks = 0;
  p.num_n_blocks = (N + tn - 1) / tn;
  p.a_scales = a_scales;
  p.w_scales = w_scales;
  p.C = C;
  p.ldc = ldc;
  p.status = status;
  p.expert_offsets = expert_offsets;
  p.num_experts = num_experts;
  p.scale_rows = scale_rows;
  p.swiglu = swiglu;
  p.up_scale_row0 = up_scale_row0;
  CUtensorMap ta, tw;
  int r = make_tensormap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, total_rows, K, lda, kFbBM, kFbSlab,
                            CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r;
  r = make_tensormap_3d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, W, num_experts, N, K,
                        static_cast<uint64_t>(N) * K, K, tn, kFbSlab, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 1000;
  // upper bound on the tiles (the kernel computes the exact count from the offsets)
  const long long tiles = (static_cast<long long>(total_rows) / kFbBM + num_experts) * p.num_n_blocks;
  return wg == 2 ? fb_launch_wg<2>(ta, tw, p, tiles, max_ctas, stream) : fb_launch_wg<1>(ta, tw, p, tiles, max_ctas, stream);
}
