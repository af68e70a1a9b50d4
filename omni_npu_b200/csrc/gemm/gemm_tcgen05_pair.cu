// Dense GEMM for large M on CTA pairs:  C[M,N] = A[M,K] * W[N,K]^T, bf16 / fp8 in,
// fp32 accumulate.  Two CTAs of a cluster (the two SMs of a TPC) compute one
// 256 x BN tile with tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A
// and HALF of the W tile, so the shared-memory traffic per SM and MMA drops from
// (128 + BN) rows to (128 + BN/2) rows.  On one CTA per SM that traffic (tensor-core
// reads plus TMA writes) is what capped the 128 x 256 kernel at ~0.7 of peak.
//
// Per CTA (192 threads): warp 0 TMA producer, warp 1 MMA issuer (leader CTA only
// issues; both allocate TMEM), warps 2..5 epilogue.  Barriers:
//   full[s]        leader's copy only: one arrive.expect_tx by the leader's producer,
//                  transaction bytes from BOTH CTAs' TMA loads;
//   empty[s]       one per CTA, the leader commits to both after the MMAs of a stage;
//   tmem_full[a]   one per CTA, the leader commits to both after a tile;
//   tmem_empty[a]  leader's copy only, 8 arrivals (4 epilogue warps of each CTA).
// TMA loads are plain per-CTA loads (no multicast).  All waits are bounded, and they use the
// CTA-scope try_wait: the cluster-scope acquire form costs ~300 cycles per call even on a
// completed barrier, which made the single producer / MMA threads the bottleneck.

#include <cstdlib>

#include "../common/ptx.cuh"
#include "../common/tensormap.h"
#include "../common/device_once.h"

namespace b200 {

static constexpr int kPBM = 128;        // rows of A per CTA (256 per pair)
static constexpr int kPRowBytes = 128;
static constexpr int kPThreads = 192;

// cycle counters of CTA 0's MMA and producer threads, written only with diagnostics bit 64:
// [0] cycles waiting for full barriers, [1] issuing MMAs, [2] committing, [3] waiting for a free
// accumulator, [4] full waits, [5] of which already complete, [6] producer cycles waiting for
// empty barriers, [7] empty barriers already free, [8] stages issued
__device__ long long g_pair_prof[16];

struct PairParams {
  int M, N, K;
  int BN;              // tile width (multiple of 32, <= 256); each CTA stages BN/2 rows of W
  int stages;
  int ksub;            // 128-byte K slabs per stage (1 or 2): more MMAs per barrier round trip
  int k_iters;
  int num_m_blocks;    // blocks of 256 rows
  int num_n_blocks;
  int elem_bytes;
  int tmem_cols, acc_stride;
  int ldc, out_fp32, swiglu;
  // timing diagnostics only (results are wrong), a bit mask: 1 stages are loaded once and then reused,
  // 2 no MMAs are issued, 4 the MMA thread does not wait for full barriers, 8 no empty-barrier
  // hand-back (the producer does not wait for it either), 16 one lane per epilogue warp polls,
  // 64 CTA 0 records cycle counters in g_pair_prof
  int diag;
  void* C;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int* status;
};

template <bool FP8>
__global__ void __launch_bounds__(kPThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                 const PairParams p) {
  // The diagnostic modes (wrong results by design) exist only in builds with -DB200_GEMM_DIAG;
  // otherwise `diag` is a constant zero and every branch on it is compiled out.
#ifdef B200_GEMM_DIAG
  const int diag = p.diag;
#else
  constexpr int diag = 0;
#endif
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int a_sub_bytes = kPBM * kPRowBytes;
  const int w_sub_bytes = (p.BN / 2) * kPRowBytes;
  const int a_stage_bytes = p.ksub * a_sub_bytes;
  const int w_stage_bytes = p.ksub * w_sub_bytes;
  uint8_t* smem_a = smem;
  uint8_t* smem_w = smem + p.stages * a_stage_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_w + p.stages * w_stage_bytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + p.stages;
  uint64_t* tmem_full = bars + 2 * p.stages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* drain_bar = tmem_empty + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  int* s_flags = reinterpret_cast<int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta_rank = static_cast<int>(cluster_ctarank());
  const bool leader = cta_rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full[0], 1);
    mbar_init(&tmem_full[1], 1);
    mbar_init(&tmem_empty[0], 8);
    mbar_init(&tmem_empty[1], 8);
    mbar_init(drain_bar, 1);
    s_flags[0] = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_base_slot, static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers exist before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;
  const long long total_tiles = static_cast<long long>(p.num_m_blocks) * p.num_n_blocks;
  const long long t_first = blockIdx.x >> 1;
  const long long t_stride = gridDim.x >> 1;
  volatile int* abort_flag = s_flags;

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      const bool prof = (diag & 64) && blockIdx.x == 0;
      long long c_empty = 0, n_empty_ready = 0;
      for (long long t = t_first; ok && t < total_tiles; t += t_stride) {
        const int mb = static_cast<int>(t % p.num_m_blocks), nb = static_cast<int>(t / p.num_m_blocks);
        const int m0 = mb * 2 * kPBM + cta_rank * kPBM;
        const int n0 = nb * p.BN + cta_rank * (p.BN / 2);
        for (int k = 0; k < p.k_iters; ++k) {
          const long long tp0 = prof ? clock64() : 0;
          if (prof && mbar_test(&empty_bar[stage], phase ^ 1)) ++n_empty_ready;
          if ((diag & 4) && issued >= p.stages) {
            ok = false;   // nobody waits for full barriers: the producer is done after the first fill
            break;
          }
          if (!(diag & 8) && !mbar_wait(&empty_bar[stage], phase ^ 1)) {
            atomicCAS(p.status, 0, kStatusTimeoutEmptyBarrier);
            *abort_flag = 1;
            ok = false;
            break;
          }
          if (prof) c_empty += clock64() - tp0;
          // the leader's barrier collects the bytes of both CTAs
          const uint32_t full_leader = mapa_shared(smem_u32(&full_bar[stage]), 0);
          if ((diag & 1) && issued >= p.stages) {
            // diagnostics: hand the stage back without reloading it
            if (leader) mbar_arrive_expect_tx(&full_bar[stage], 0u);
            ++issued;
            if (++stage == p.stages) {
              stage = 0;
              phase ^= 1;
            }
            continue;
          }
          if (leader)
            mbar_arrive_expect_tx(&full_bar[stage], static_cast<uint32_t>(2 * (a_stage_bytes + w_stage_bytes)));
          const int slab_elems = kPRowBytes / p.elem_bytes;
          for (int j = 0; j < p.ksub; ++j) {
            const int kcoord = (k * p.ksub + j) * slab_elems;
            tma_load_2d_pair(smem_a + stage * a_stage_bytes + j * a_sub_bytes, &tmap_a, full_leader, kcoord, m0);
            tma_load_2d_pair(smem_w + stage * w_stage_bytes + j * w_sub_bytes, &tmap_w, full_leader, kcoord, n0);
          }
          ++issued;
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (prof) {
        g_pair_prof[6] = c_empty;
        g_pair_prof[7] = n_empty_ready;
        g_pair_prof[8] = issued;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (leader && lane == 0) {
      const uint32_t idesc = FP8 ? make_idesc(0, 0, 2 * kPBM, p.BN) : make_idesc(1, 1, 2 * kPBM, p.BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const bool no_mma = (diag & 2) != 0;
      // low words of the shared-memory descriptors (start address >> 4) and their strides
      const uint32_t a_lo0 = (smem_u32(smem_a) & 0x3FFFF) >> 4, w_lo0 = (smem_u32(smem_w) & 0x3FFFF) >> 4;
      const uint32_t a_sub_lo = static_cast<uint32_t>(a_sub_bytes) >> 4, w_sub_lo = static_cast<uint32_t>(w_sub_bytes) >> 4;
      const uint32_t a_stage_lo = static_cast<uint32_t>(a_stage_bytes) >> 4, w_stage_lo = static_cast<uint32_t>(w_stage_bytes) >> 4;
      const bool prof = (diag & 64) && blockIdx.x == 0;
      long long c_wait = 0, c_issue = 0, c_commit = 0, c_tmem = 0, n_wait = 0, n_ready = 0;
      for (long long t = t_first; ok && t < total_tiles; t += t_stride) {
        long long t0 = prof ? clock64() : 0;
        if (*abort_flag || !mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          if (!*abort_flag) atomicCAS(p.status, 0, kStatusTimeoutTmemEmpty);
          *abort_flag = 1;
          break;
        }   // (once per tile; the per-stage waits below do not read the flag)
        if (prof) c_tmem += clock64() - t0;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * p.acc_stride);
        for (int k = 0; k < p.k_iters; ++k) {
          if (prof) {
            t0 = clock64();
            ++n_wait;
            if (mbar_test(&full_bar[stage], phase)) ++n_ready;
          }
          if (!(diag & 4) && !mbar_wait(&full_bar[stage], phase)) {
            atomicCAS(p.status, 0, kStatusTimeoutFullBarrier);
            *abort_flag = 1;
            ok = false;
            break;
          }
          if (prof) {
            const long long t1 = clock64();
            c_wait += t1 - t0;
            t0 = t1;
          }
          tc_fence_after_sync();
          if (!no_mma) {
            uint32_t a_lo = a_lo0 + static_cast<uint32_t>(stage) * a_stage_lo;
            uint32_t w_lo = w_lo0 + static_cast<uint32_t>(stage) * w_stage_lo;
            for (int j = 0; j < p.ksub; ++j) {
              // 32 bytes of K per MMA: the start-address field advances by 2
              umma_pair_first<FP8>(d_tmem, a_lo, w_lo, idesc, (k > 0 || j > 0) ? 1u : 0u);
              umma_pair_acc<FP8>(d_tmem, a_lo + 2, w_lo + 2, idesc);
              umma_pair_acc<FP8>(d_tmem, a_lo + 4, w_lo + 4, idesc);
              umma_pair_acc<FP8>(d_tmem, a_lo + 6, w_lo + 6, idesc);
              a_lo += a_sub_lo;
              w_lo += w_sub_lo;
            }
          }
          if (prof) {
            const long long t1 = clock64();
            c_issue += t1 - t0;
            t0 = t1;
          }
          // the stage is free in both CTAs once these MMAs retire
          if (!(diag & 8)) tc_commit_pair_both(smem_u32(&empty_bar[stage]));
          if (prof) c_commit += clock64() - t0;
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit_pair_both(smem_u32(&tmem_full[acc]));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
      if (prof) {
        g_pair_prof[0] = c_wait;
        g_pair_prof[1] = c_issue;
        g_pair_prof[2] = c_commit;
        g_pair_prof[3] = c_tmem;
        g_pair_prof[4] = n_wait;
        g_pair_prof[5] = n_ready;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (long long t = t_first; t < total_tiles; t += t_stride) {
      const int mb = static_cast<int>(t % p.num_m_blocks), nb = static_cast<int>(t / p.num_m_blocks);
      const int m0 = mb * 2 * kPBM + cta_rank * kPBM;
      const int n0 = nb * p.BN;
      bool ok = true;
      if (!(diag & 16) || lane == 0) ok = !*abort_flag && mbar_wait(&tmem_full[acc], acc_phase);
      if (diag & 16) ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      {
        uint32_t all_ok;
        asm volatile(
            "{\n\t"
            ".reg .pred p, q;\n\t"
            "setp.ne.u32 q, %1, 0;\n\t"
            "bar.red.and.pred p, 1, 128, q;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}"
            : "=r"(all_ok)
            : "r"(ok ? 1u : 0u)
            : "memory");
        ok = all_ok != 0;
      }
      if (!ok) {
        if (lane == 0 && !*abort_flag) atomicCAS(p.status, 0, kStatusTimeoutTmemFull);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(acc * p.acc_stride);
      for (int c = 0; c < p.BN; c += 16) {
        uint32_t r[16];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
              "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
              "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(t_row + static_cast<uint32_t>(c))
            : "memory");
        tmem_ld_wait();
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
        const int col = n0 + c;
        if (!row_ok || col >= p.N) continue;
        if (p.swiglu) {
          const int ocol = col >> 1;
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float g = v[i];
            o[i] = (g / (1.f + __expf(-g))) * v[8 + i];
          }
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + ocol;
          uint4 pk;
          pk.x = pack_bf16x2(o[0], o[1]);
          pk.y = pack_bf16x2(o[2], o[3]);
          pk.z = pack_bf16x2(o[4], o[5]);
          pk.w = pack_bf16x2(o[6], o[7]);
          *reinterpret_cast<uint4*>(dst) = pk;
          continue;
        }
        const int ncols = min(16, p.N - col);
        if (p.bias) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (i < ncols) v[i] += __bfloat162float(p.bias[col + i]);
        }
        if (p.residual) {
          const __nv_bfloat16* rsd = p.residual + static_cast<size_t>(row) * p.ldc + col;
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (i < ncols) v[i] += __bfloat162float(rsd[i]);
        }
        if (p.out_fp32) {
          float* dst = reinterpret_cast<float*>(p.C) + static_cast<size_t>(row) * p.ldc + col;
          if (ncols == 16 && (p.ldc & 3) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          } else {
            for (int i = 0; i < ncols; ++i) dst[i] = v[i];
          }
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col;
          if (ncols == 16 && (p.ldc & 7) == 0) {
            uint4 pk0, pk1;
            pk0.x = pack_bf16x2(v[0], v[1]);
            pk0.y = pack_bf16x2(v[2], v[3]);
            pk0.z = pack_bf16x2(v[4], v[5]);
            pk0.w = pack_bf16x2(v[6], v[7]);
            pk1.x = pack_bf16x2(v[8], v[9]);
            pk1.y = pack_bf16x2(v[10], v[11]);
            pk1.z = pack_bf16x2(v[12], v[13]);
            pk1.w = pack_bf16x2(v[14], v[15]);
            reinterpret_cast<uint4*>(dst)[0] = pk0;
            reinterpret_cast<uint4*>(dst)[1] = pk1;
          } else {
            for (int i = 0; i < ncols; ++i) dst[i] = __float2bfloat16(v[i]);
          }
        }
      }
      // hand the accumulator back to the leader's MMA warp (8 arrivals: 4 warps x 2 CTAs)
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty[acc]), 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (leader && warp == 1 && lane == 0 && *abort_flag) {
    tc_commit_pair(smem_u32(drain_bar));
    mbar_wait(drain_bar, 0);
  }
  // neither CTA may retire (or free TMEM) while its peer can still signal it or the
  // leader's MMAs can still write its TMEM
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}

static int pair_stages(int BN, int ksub) {
  const int stage_bytes = ksub * (kPBM * kPRowBytes + (BN / 2) * kPRowBytes);
  int st = (222 * 1024) / stage_bytes;
  if (st > 8) st = 8;
  return st < 2 ? 2 : st;
}

static size_t pair_smem(int BN, int stages, int ksub) {
  return 1024 + static_cast<size_t>(stages) * ksub * (kPBM * kPRowBytes + (BN / 2) * kPRowBytes) +
         (2 * stages + 5) * 8 + 64;
}

template <bool FP8>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tw, const PairParams& p, int max_ctas,
                       cudaStream_t stream) {
  auto kern = gemm_pair_kernel<FP8>;
  static DeviceOnce once;
  static int max_pairs = 0;      // the same for every B200 of a machine
  int dev = 0;
  const bool configured = !once.needed(&dev);
  const size_t smem = pair_smem(p.BN, p.stages, p.ksub);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kPThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return -20;
    cfg.gridDim = dim3(2 * sm_count(), 1, 1);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = sm_count() / 2;
    }
    max_pairs = n;
    once.mark(dev);
  }
  long long tiles = static_cast<long long>(p.num_m_blocks) * p.num_n_blocks;
  int pairs = max_pairs;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  if (tiles < pairs) pairs = static_cast<int>(tiles);
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  return cudaLaunchKernelEx(&cfg, kern, ta, tw, p) == cudaSuccess ? 0 : -22;
}

}  // namespace b200

using namespace b200;

// Copies the diagnostics counters (see g_pair_prof) to the host.
extern "C" int b200_gemm_pair_prof(long long* out16) {
  return cudaMemcpyFromSymbol(out16, g_pair_prof, sizeof(long long) * 16) == cudaSuccess ? 0 : -1;
}

// Same contract as b200_gemm (no split-K).  BN: multiple of 32 in [32, 256].
extern "C" int b200_gemm_pair(const void* A, const void* W, void* C, const void* bias, const void* residual,
                              int M, int N, int K, int lda, int ldw, int ldc, int dtype_fp8, int out_fp32,
                              int swiglu, int BN, int* status, int max_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int eb = dtype_fp8 ? 1 : 2;
  if (BN < 32 || BN > 256 || (BN % 32) != 0) return -10;
  if (swiglu && (N % 16) != 0) return -11;
  PairParams p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.BN = BN;
  p.elem_bytes = eb;
  {
    static const int ksub_env = [] {
      const char* e = getenv("OMNI_B200_GEMM_PAIR_KSUB");
      return e ? atoi(e) : 0;
    }();
    p.ksub = ksub_env == 1 || ksub_env == 2 ? ksub_env : (K * eb > 2 * kPRowBytes ? 2 : 1);
  }
  p.k_iters = (K * eb + kPRowBytes * p.ksub - 1) / (kPRowBytes * p.ksub);
  p.num_m_blocks = (M + 2 * kPBM - 1) / (2 * kPBM);
  p.num_n_blocks = (N + BN - 1) / BN;
  p.stages = pair_stages(BN, p.ksub);
  p.acc_stride = BN <= 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256));
  p.tmem_cols = 2 * p.acc_stride < 32 ? 32 : 2 * p.acc_stride;
  p.ldc = ldc;
  p.out_fp32 = out_fp32;
  p.swiglu = swiglu;
  p.C = C;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.status = status;
  p.diag = 0;
#ifdef B200_GEMM_DIAG
  {
    static const int diag = [] {
      const char* e = getenv("OMNI_B200_GEMM_DIAG");
      return e ? atoi(e) : 0;
    }();
    p.diag = diag;
  }
#endif
  CUtensorMap ta, tw;
  const CUtensorMapDataType dt = dtype_fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int box_k = kPRowBytes / eb;
  int r = make_tensormap_2d(&ta, dt, eb, A, M, K, lda, kPBM, box_k, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r;
  r = make_tensormap_2d(&tw, dt, eb, W, N, K, ldw, BN / 2, box_k, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 1000;
  if (dtype_fp8) return launch_pair<true>(ta, tw, p, max_ctas, stream);
  return launch_pair<false>(ta, tw, p, max_ctas, stream);
}
