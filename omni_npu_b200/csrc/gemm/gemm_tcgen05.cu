// Dense and grouped (per-expert) GEMM for sm_100a on the 5th-generation
// tensor cores:   C[M,N] = A[M,K] * W[N,K]^T   (bf16 or fp8-e4m3 in, fp32 accumulate).
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the A tile (128 x 64
//               elements... 128 bytes per row) and the W tile (BN rows) into a
//               ring of 128B-swizzled shared-memory stages.  Plain per-CTA loads
//               only; no cluster multicast anywhere.
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN,
//               K=16 for bf16 / 32 for fp8) with the accumulator in TMEM.  Two
//               accumulator buffers let the epilogue of tile i overlap the
//               main loop of tile i+1.
//   warps 2..5  epilogue: tcgen05.ld the accumulator, apply bias / residual /
//               SwiGLU, convert and store.  With split-K the partial sums go to
//               an fp32 workspace and the last CTA to finish a tile reduces them.
//
// BN is a run-time value (multiple of 16, 16..256) so the host can pick a tile
// width that fills the 148 SMs in a whole number of waves.
//
// Every barrier wait is bounded; on a timeout the kernel records a status code,
// drains what it has in flight, frees its TMEM columns and returns.
//
// Replaces the reference's torch.matmul / npu_quant_matmul / npu_grouped_matmul
// call sites (omni_npu/v1/layers/linear.py:124-130,
// omni_npu/layers/fused_moe/npu_moe_permute_unpermute.py:108-149).

#include <cstdlib>
#include <type_traits>

#include "../common/pdl.cuh"
#include "../common/ptx.cuh"
#include "../common/tensormap.h"
#include "../common/device_once.h"
#include "../comm/ll_protocol.cuh"

namespace b200 {

static constexpr int kBM = 128;          // rows of A per tile (UMMA M)
static constexpr int kRowBytes = 128;    // bytes of K per stage row (one swizzle span)
static constexpr int kThreads = 192;

// Build with -DB200_GEMM_TIMELINE to record, per CTA, the global timer at eight points of the
// kernel (entry, set-up done, first slab landed, last MMA issued, accumulator complete, partial
// tiles of all K slices staged, output stored, exit); read them back with b200_gemm_timeline().
#ifdef B200_GEMM_TIMELINE
__device__ unsigned long long g_timeline[1024 * 8];
__device__ long long g_timeline_clk[1024 * 8];        // SM cycle counter at the same points
__device__ __forceinline__ void timeline_mark(int i) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  if (blockIdx.x < 1024) {
    g_timeline[blockIdx.x * 8 + i] = t;
    g_timeline_clk[blockIdx.x * 8 + i] = clock64();
  }
}
#define B200_TL(i) timeline_mark(i)
#else
#define B200_TL(i)
#endif
static constexpr int kMaxExperts = 512;
static constexpr int kRsPitch = 144;                 // bytes per staged row (64 bf16 columns + padding)
static constexpr int kRsWarpBytes = 32 * kRsPitch;   // staging of one epilogue warp

struct GemmParams {
  int M, N, K;            // problem (grouped: M = total packed rows)
  int BN;                 // tile width
  int stages;             // shared-memory ring depth (128-byte K slabs)
  int ksub;               // slabs per barrier round trip (1 or 2); stages is a multiple of it
  int k_iters;            // ceil(K_bytes / 128)
  int splits;             // split-K factor (>=1)
  int num_m_blocks;       // dense only
  int num_n_blocks;
  int elem_bytes;         // 2 (bf16) or 1 (fp8)
  int tmem_cols;          // power of two >= 2*acc stride
  int acc_stride;         // TMEM column distance between the two accumulators
  int ldc;                // row pitch of C in elements
  int out_fp32;           // 1: C is fp32, 0: bf16
  int swiglu;             // 1: C[:, n/2] = silu(acc[gate]) * acc[up], gate/up interleaved per 16 cols
  int num_experts;        // grouped: number of local experts (0 = dense)
  int cluster_split;      // 1: the `splits` CTAs of a cluster share one tile and reduce over DSMEM
  void* C;
  const __nv_bfloat16* bias;       // [N] or null
  const __nv_bfloat16* residual;   // [M, ldc] or null
  float* workspace;                // split-K partials [splits][M_pad][N_pad]
  int* tile_counters;              // split-K arrival counters, one per (m,n) tile, zero at rest
  const int* expert_offsets;       // grouped: [E+1] row offsets into A / C (device)
  const float* a_scales;           // quantised inputs: [M] per-row scales or null (direct epilogue only)
  const float* w_scales;           // quantised inputs: [N] per-column scales (with a_scales)
  int* status;                     // error word (0 = ok)
  // ---- fused tensor-parallel tail (ar_world > 1): the epilogue pushes the bf16 tile to every
  // rank's receive buffer (ll_protocol.cuh) instead of writing C; once a CTA has finished its
  // tiles it reduces whole rows that have arrived from all ranks, adds the residual and applies
  // RMSNorm.  C then receives the normed rows, `residual` is updated in place.
  LLGroup ar;                      // peer receive buffers, epoch words, world, rank
  int ar_world;                    // 0 / 1 = off
  const __nv_bfloat16* ar_norm_w;  // [N] RMSNorm weight, or null: C = all-reduced sum (+residual)
  float ar_eps;
  uint32_t* ar_done;               // zero-initialised device counter
  // ---- fused all-gather of A (ag_world > 1): A [M = ag_world * ag_rows, K] is a LOCAL buffer whose
  // own block was filled by the staging kernel.  The epilogue warps of every CTA, idle until the
  // first accumulator is ready, pull this CTA's share of every foreign block from the owner's
  // staging buffer over NVLink (once: a tile re-read per N block would cross the link every time)
  // and bump a per-source counter; the producer walks the row blocks own-first and waits (bounded)
  // until a foreign block's counter shows that all CTAs delivered their share.
  void* ag_data[kMaxRanks];        // peer-mapped staging buffers (both halves)
  long long ag_half_bytes;
  const uint32_t* ag_signal;       // this rank's signal pad: word ag_epoch_word = epoch, ag_flag_word + r = rank r staged
  uint32_t* ag_ready;              // [ag_world] local counters, zeroed by the staging kernel
  const void* ag_local;            // the local gathered A buffer (same memory tmap_a describes)
  int ag_world, ag_rank;
  int ag_rows;                     // rows per rank, a multiple of 128
  int ag_epoch_word, ag_flag_word;
  // ---- fused reduce-scatter of C (rs_world > 1): every rank computes a partial [M, N]; rank r
  // owns rows [r * rs_rows, (r + 1) * rs_rows).  The epilogue stores each bf16 tile row straight
  // into its owner's staging buffer (slot of this rank: [rs_rank][rs_rows][N]) with plain peer
  // stores, so the transfer overlaps the tensor-core work; a small kernel then signals, waits for
  // all sources and sums the slots (rs_reduce_kernel in the collectives file).
  void* rs_data[kMaxRanks];        // peer-mapped staging buffers (both halves)
  const uint32_t* rs_signal;       // this rank's signal pad (epoch word)
  long long rs_half_bytes;
  int rs_world, rs_rank, rs_rows;
  int rs_epoch_word;
};

struct TileCoord {
  int m0;        // first row in A / C
  int m_end;     // one past the last valid row
  int n0;        // first column
  int expert;    // weight slab
  int k_begin;   // first k iteration
  int k_end;     // one past last k iteration
  int split;     // split index
  int mn_index;  // index of the (m,n) tile for split-K bookkeeping
  int a_src;     // fused all-gather: rank whose staging buffer holds the A rows (-1: plain A)
  int a_row0;    // fused all-gather: first row inside that buffer
};

template <bool GROUPED>
__device__ __forceinline__ bool decode_tile(const GemmParams& p, const int* s_tile_prefix,
                                            int total_mn_tiles, long long t, int cta_rank,
                                            int& cursor, TileCoord& tc) {
  int split, mn;
  if (p.cluster_split) {
    // every CTA of a cluster walks the same (m,n) tiles; its rank picks the K slice
    if (t >= total_mn_tiles) return false;
    split = cta_rank;
    mn = static_cast<int>(t);
  } else {
    const long long total = static_cast<long long>(total_mn_tiles) * p.splits;
    if (t >= total) return false;
    split = static_cast<int>(t % p.splits);
    mn = static_cast<int>(t / p.splits);
  }
  tc.split = split;
  tc.mn_index = mn;
  const int per = (p.k_iters + p.splits - 1) / p.splits;
  tc.k_begin = split * per;
  tc.k_end = min(p.k_iters, tc.k_begin + per);
  tc.a_src = -1;
  tc.a_row0 = 0;
  if constexpr (!GROUPED) {
    int mb = mn % p.num_m_blocks;
    int nb = mn / p.num_m_blocks;
    if (p.ag_world > 1) {
      // walk the row blocks rank by rank, own rows first: all (m, n) tiles of one rank's block
      // before the next rank's, so remote rows are first needed 1/world of the way in
      const int chunk = p.ag_rows / kBM;
      const int per_chunk = chunk * p.num_n_blocks;
      const int c = mn / per_chunk, rem = mn - c * per_chunk;
      const int src = (p.ag_rank + c) % p.ag_world;
      nb = rem / chunk;
      const int mb_in = rem - nb * chunk;
      mb = src * chunk + mb_in;
      tc.a_src = src;
      tc.a_row0 = mb_in * kBM;
    }
    tc.m0 = mb * kBM;
    tc.m_end = min(p.M, tc.m0 + kBM);
    tc.n0 = nb * p.BN;
    tc.expert = 0;
  } else {
    // s_tile_prefix[e] = number of m-blocks of experts < e.  n is fastest so the
    // CTAs that run together share one expert's A rows and sweep its weights.
    const int mblk_global = mn / p.num_n_blocks;
    const int nb = mn % p.num_n_blocks;
    while (cursor + 1 < p.num_experts && s_tile_prefix[cursor + 1] <= mblk_global) ++cursor;
    const int e = cursor;
    const int mb = mblk_global - s_tile_prefix[e];
    const int row0 = p.expert_offsets[e];
    const int row1 = p.expert_offsets[e + 1];
    tc.m0 = row0 + mb * kBM;
    tc.m_end = min(row1, tc.m0 + kBM);
    tc.n0 = nb * p.BN;
    tc.expert = e;
  }
  return true;
}

template <bool GROUPED, int KIND>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_w, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the 128B swizzle atoms.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int a_stage_bytes = kBM * kRowBytes;
  const int w_stage_bytes = p.BN * kRowBytes;
  uint8_t* smem_a = smem;
  uint8_t* smem_w = smem + p.stages * a_stage_bytes;
  // receive area of the cluster reduction, or staging of the reduce-scatter push
  float* red_buf = reinterpret_cast<float*>(smem_w + p.stages * w_stage_bytes);
  const int red_bytes = p.cluster_split ? kBM * p.BN * 4 : (p.rs_world > 1 ? 4 * kRsWarpBytes : 0);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_w + p.stages * w_stage_bytes + red_bytes);
  uint64_t* full_bar = bars;                    // [stages]
  uint64_t* empty_bar = bars + p.stages;        // [stages]
  uint64_t* tmem_full = bars + 2 * p.stages;    // [2]
  uint64_t* tmem_empty = tmem_full + 2;         // [2]
  uint64_t* drain_bar = tmem_empty + 2;         // [1]
  uint64_t* red_ready = drain_bar + 1;          // [1] all K slices staged (cluster split-K)
  uint64_t* red_done = red_ready + 1;           // [1] parked partial tile sent (cluster split-K): the ring is free again
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(red_done + 1);
  int* s_flags = reinterpret_cast<int*>(tmem_base_slot + 1);  // [0]=abort, [1]=is_last
  int* s_tile_prefix = s_flags + 2;                           // [num_experts + 1] (grouped)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    B200_TL(0);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full[0], 1);
    mbar_init(&tmem_full[1], 1);
    mbar_init(&tmem_empty[0], 4);
    mbar_init(&tmem_empty[1], 4);
    mbar_init(drain_bar, 1);
    mbar_init(red_ready, 1);      // armed below with the bytes of my band from every K slice
    mbar_init(red_done, 1);
    s_flags[0] = 0;
    s_flags[1] = 0;
    fence_barrier_init();
    if (p.cluster_split) mbar_arrive_expect_tx(red_ready, static_cast<uint32_t>(kBM * p.BN * 4));
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_w);
  }
  int total_mn_tiles;
  if constexpr (GROUPED) {
    pdl_wait();      // the expert offsets are written by the routing kernel ahead of this one
    if (threadIdx.x == 32) {
      int acc = 0;
      for (int e = 0; e < p.num_experts; ++e) {
        s_tile_prefix[e] = acc;
        const int rows = p.expert_offsets[e + 1] - p.expert_offsets[e];
        acc += (rows + kBM - 1) / kBM;
      }
      s_tile_prefix[p.num_experts] = acc;
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  int cta_rank = 0;
  long long t_first = blockIdx.x, t_stride = gridDim.x;
  if (p.cluster_split) {
    cta_rank = static_cast<int>(cluster_ctarank());
    t_first = blockIdx.x / p.splits;
    t_stride = gridDim.x / p.splits;
    // peers' barriers must be initialised before anyone signals them: arrive now, wait right
    // before this thread's first remote access (or at the end of its role)
    cluster_arrive_release();
  }
  const uint32_t tmem_base = *tmem_base_slot;
  if constexpr (GROUPED) {
    total_mn_tiles = s_tile_prefix[p.num_experts] * p.num_n_blocks;
  } else {
    total_mn_tiles = p.num_m_blocks * p.num_n_blocks;
  }

  volatile int* abort_flag = s_flags;
  const int groups = p.stages / p.ksub;   // barrier pairs in use
  // Dependent launch: the next kernel of the stream may start its own prologue now.  This
  // kernel's weights are written by no earlier kernel, so the producer thread of a dense
  // problem streams the first ring of weight slabs before it waits for the kernels ahead;
  // every other thread waits here, before it reads anything those kernels produced.
  pdl_trigger();
  const bool w_preload = !GROUPED && threadIdx.x == 0;
  uint32_t ar_epoch = 0;
  long long ar_slot_off = 0;
  if (!w_preload) {
    pdl_wait();
    if (p.ar_world > 1) {
      ar_epoch = *reinterpret_cast<volatile uint32_t*>(p.ar.epoch) + 1;
      ar_slot_off = static_cast<long long>(ar_epoch % 3) * p.ar_world * p.ar.slot_vecs;
    }
  }

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int cursor = 0;
      long long issued = 0;
      long long preloaded = 0;     // leading barrier groups whose weight slabs are already in flight
      bool ok = true;
      TileCoord tc;
      if constexpr (!GROUPED) {
        int c0 = 0;
        if (decode_tile<GROUPED>(p, s_tile_prefix, total_mn_tiles, t_first, cta_rank, c0, tc)) {
          int g = 0;
          for (int k = tc.k_begin; k < tc.k_end && g < groups; k += p.ksub, ++g) {
            const int ns = tc.k_end - k < p.ksub ? tc.k_end - k : p.ksub;
            mbar_arrive_expect_tx(&full_bar[g], static_cast<uint32_t>(ns * (a_stage_bytes + w_stage_bytes)));
            for (int j = 0; j < ns; ++j)
              tma_load_2d(smem_w + (g * p.ksub + j) * w_stage_bytes, &tmap_w, &full_bar[g],
                          (k + j) * (kRowBytes / p.elem_bytes), tc.n0);
          }
          preloaded = g;
        }
        pdl_wait();
        if (p.ar_world > 1) {
          ar_epoch = *reinterpret_cast<volatile uint32_t*>(p.ar.epoch) + 1;
          ar_slot_off = static_cast<long long>(ar_epoch % 3) * p.ar_world * p.ar.slot_vecs;
        }
      }
      uint32_t ag_have = p.ag_world > 1 ? (1u << p.ag_rank) : 0u;
      for (long long t = t_first; ok && decode_tile<GROUPED>(p, s_tile_prefix, total_mn_tiles, t,
                                                                cta_rank, cursor, tc);
           t += t_stride) {
        const CUtensorMap* map_a = &tmap_a;
        const int a_row = tc.m0;
        if (tc.a_src >= 0 && !((ag_have >> tc.a_src) & 1u)) {
          // first tile of a foreign block: every CTA must have delivered its share of it
          const volatile uint32_t* cnt = p.ag_ready + tc.a_src;
          uint32_t polls = 0;
          while (*cnt < gridDim.x) {
            if (*abort_flag || ++polls > (1u << 24)) {
              ok = false;
              break;
            }
            __nanosleep(64);
          }
          if (!ok) {
            atomicCAS(p.status, 0, kStatusTimeoutPeerFlag);
            *abort_flag = 1;
            break;
          }
          __threadfence();
          fence_proxy_async();
          ag_have |= 1u << tc.a_src;
        }
        for (int k = tc.k_begin; k < tc.k_end; k += p.ksub) {
          // one barrier round trip covers up to ksub slabs (`stage` counts groups of slabs)
          const int ns = tc.k_end - k < p.ksub ? tc.k_end - k : p.ksub;
          const bool w_in_flight = issued < preloaded;     // first ring of the first tile: only A is missing
          if (!w_in_flight) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
              atomicCAS(p.status, 0, kStatusTimeoutEmptyBarrier);
              *abort_flag = 1;
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&full_bar[stage],
                                  static_cast<uint32_t>(ns * (a_stage_bytes + w_stage_bytes)));
          }
          for (int j = 0; j < ns; ++j) {
            const int slab = stage * p.ksub + j;
            const int kcoord = (k + j) * (kRowBytes / p.elem_bytes);
            tma_load_2d(smem_a + slab * a_stage_bytes, map_a, &full_bar[stage], kcoord, a_row);
            if constexpr (GROUPED) {
              tma_load_3d(smem_w + slab * w_stage_bytes, &tmap_w, &full_bar[stage], kcoord, tc.n0,
                          tc.expert);
            } else {
              if (!w_in_flight)
                tma_load_2d(smem_w + slab * w_stage_bytes, &tmap_w, &full_bar[stage], kcoord, tc.n0);
            }
          }
          ++issued;
          if (++stage == groups) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // Abort path: wait (bounded) until the loads already issued have landed
        // so that no bulk copy writes into shared memory after the CTA retires.
        if (issued < preloaded)      // weight slabs in flight whose barrier will never complete: let them land
          for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        const int pending = issued < groups ? static_cast<int>(issued) : groups;
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) {
            s = groups - 1;
            ph ^= 1;
          }
          mbar_wait(&full_bar[s], ph);
        }
      }
    }
    __syncwarp();
    if (p.cluster_split) cluster_wait_acquire();
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = KIND == kKindI8 ? make_idesc_i8(kBM, p.BN)
                             : (KIND == kKindFP8 ? make_idesc(0, 0, kBM, p.BN) : make_idesc(1, 1, kBM, p.BN));
      // low words of the shared-memory descriptors (start address >> 4) and the slab pitch
      const uint32_t a_lo0 = (smem_u32(smem_a) & 0x3FFFF) >> 4, w_lo0 = (smem_u32(smem_w) & 0x3FFFF) >> 4;
      const uint32_t a_slab_lo = static_cast<uint32_t>(a_stage_bytes) >> 4, w_slab_lo = static_cast<uint32_t>(w_stage_bytes) >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      int cursor = 0;
      bool ok = true;
      TileCoord tc;
      for (long long t = t_first; ok && decode_tile<GROUPED>(p, s_tile_prefix, total_mn_tiles, t,
                                                                cta_rank, cursor, tc);
           t += t_stride) {
        if (*abort_flag || !mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          if (!*abort_flag) atomicCAS(p.status, 0, kStatusTimeoutTmemEmpty);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * p.acc_stride);
        for (int k = tc.k_begin; k < tc.k_end; k += p.ksub) {
          const int ns = tc.k_end - k < p.ksub ? tc.k_end - k : p.ksub;
          // (the abort flag is not read here: shared-memory reads by this thread queue behind
          // the tensor core's operand traffic and cost ~100 cycles each)
          if (!mbar_wait(&full_bar[stage], phase)) {
            atomicCAS(p.status, 0, kStatusTimeoutFullBarrier);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          uint32_t a_lo = a_lo0 + static_cast<uint32_t>(stage * p.ksub) * a_slab_lo;
          uint32_t w_lo = w_lo0 + static_cast<uint32_t>(stage * p.ksub) * w_slab_lo;
          for (int j = 0; j < ns; ++j) {
            // 32 bytes of K per instruction: the start-address field advances by 2
            umma_first<KIND>(d_tmem, a_lo, w_lo, idesc, (k > tc.k_begin || j > 0) ? 1u : 0u);
            umma_acc<KIND>(d_tmem, a_lo + 2, w_lo + 2, idesc);
            umma_acc<KIND>(d_tmem, a_lo + 4, w_lo + 4, idesc);
            umma_acc<KIND>(d_tmem, a_lo + 6, w_lo + 6, idesc);
            a_lo += a_slab_lo;
            w_lo += w_slab_lo;
          }
          tc_commit(&empty_bar[stage]);  // slabs reusable once these MMAs retire
          if (++stage == groups) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit(&tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
    __syncwarp();
    if (p.cluster_split) cluster_wait_acquire();
  } else {
    // ------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 belong to this warp
    bool cluster_met = false;      // this thread has completed the cluster barrier opened at set-up
    int acc = 0;
    uint32_t acc_phase = 0;
    int cursor = 0;
    int tile_iter = 0;
    // ---- all-gather pull: this CTA's slice of every foreign block, nearest rank first.  One block
    // is pulled before the first tile's epilogue and one more before every later tile, which is
    // the order and roughly the pace at which the producer needs them; what is left is pulled
    // after the last tile (other CTAs wait for this CTA's share of every block).
    int ag_next = 1, ag_part = 0, ag_parts = 1;
    uint32_t ag_epoch = 0;
    long long ag_begin = 0, ag_end = 0, ag_nvec = 0, ag_half_off = 0;
    if (p.ag_world > 1) {
      ag_epoch = *reinterpret_cast<const volatile uint32_t*>(p.ag_signal + p.ag_epoch_word);
      ag_half_off = static_cast<long long>(ag_epoch & 1u) * p.ag_half_bytes;
      ag_nvec = (static_cast<long long>(p.ag_rows) * p.K * p.elem_bytes) >> 4;
      const long long per = (ag_nvec + gridDim.x - 1) / gridDim.x;
      ag_begin = min(ag_nvec, per * blockIdx.x);
      ag_end = min(ag_nvec, per * (blockIdx.x + 1));
      // a block is pulled in as many pieces as this CTA has own-row tiles to hide them behind (minus one)
      const long long own_tiles = static_cast<long long>(p.ag_rows / kBM) * p.num_n_blocks;
      ag_parts = static_cast<int>(own_tiles / gridDim.x) - 1;
      if (ag_parts < 1) ag_parts = 1;
      if (ag_parts > 8) ag_parts = 8;
    }
    // one piece of foreign block c; returns true when the block is finished (or given up)
    auto ag_pull = [&](int c, int part) -> bool {
      const long long ag_begin_all = ag_begin, this_end = ag_end;
      const int et = threadIdx.x - 64;
      const int src = (p.ag_rank + c) % p.ag_world;
      if (part == 0) {
       if (et == 0) {
        uint32_t staged = *abort_flag ? 0u : 1u;
        const volatile uint32_t* flag = p.ag_signal + p.ag_flag_word + src;
        uint32_t polls = 0;
        while (staged && static_cast<int32_t>(*flag - ag_epoch) < 0) {     // flags only grow
          if (++polls > (1u << 24)) staged = 0u;
          else __nanosleep(64);
        }
        __threadfence_system();
        if (!staged && !*abort_flag) {
          atomicCAS(p.status, 0, kStatusTimeoutPeerFlag);
          *abort_flag = 1;
        }
        s_flags[1] = static_cast<int>(staged);
       }
       asm volatile("bar.sync 1, 128;" ::: "memory");
       const bool staged = s_flags[1] != 0;
       asm volatile("bar.sync 1, 128;" ::: "memory");
       if (!staged) return true;
      }
      const uint4* from = reinterpret_cast<const uint4*>(static_cast<const char*>(p.ag_data[src]) + ag_half_off);
      uint4* to = reinterpret_cast<uint4*>(const_cast<void*>(p.ag_local)) + static_cast<long long>(src) * ag_nvec;
      const long long piece = (this_end - ag_begin_all + ag_parts - 1) / ag_parts;
      const long long stop = min(this_end, ag_begin_all + piece * (part + 1));
      long long i = ag_begin_all + piece * part + et;
      // eight 16-byte loads in flight per thread: 16 KB per CTA, which at ~3 us of NVLink round trip
      // is what it takes for 148 CTAs together to keep the link busy (four gave half the rate)
      for (; i + 7 * 128 < stop; i += 8 * 128) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __ldcv(from + i + u * 128);
#pragma unroll
        for (int u = 0; u < 8; ++u) to[i + u * 128] = v[u];
      }
      for (; i < stop; i += 128) to[i] = __ldcv(from + i);
      if (part + 1 < ag_parts) return false;
      __threadfence();
      fence_proxy_async();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (et == 0) atomicAdd(p.ag_ready + src, 1u);
      return true;
    };
    // advance the pull by one piece
    auto ag_step = [&]() {
      if (ag_pull(ag_next, ag_part)) {
        ++ag_next;
        ag_part = 0;
      } else {
        ++ag_part;
      }
    };
    long long rs_half_off = 0;     // fused reduce-scatter: staging half of the epoch this call opens
    if (p.rs_world > 1) {
      const uint32_t e = *reinterpret_cast<const volatile uint32_t*>(p.rs_signal + p.rs_epoch_word) + 1u;
      rs_half_off = static_cast<long long>(e & 1u) * p.rs_half_bytes;
    }
    TileCoord tc;
    for (long long t = t_first;
         decode_tile<GROUPED>(p, s_tile_prefix, total_mn_tiles, t, cta_rank, cursor, tc); t += t_stride) {
      if (ag_next < p.ag_world) ag_step();
      bool ok = !*abort_flag && mbar_wait(&tmem_full[acc], acc_phase);
      {
        // The four epilogue warps take the decision together (barrier + AND
        // reduction) so that none of them is left alone at a later barrier.
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
      if (threadIdx.x == 64) B200_TL(4);
      const int row = tc.m0 + quarter * 32 + lane;
      const bool row_ok = row < tc.m_end;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(acc * p.acc_stride);
      if (p.cluster_split) {
        // ---- split-K inside a cluster (one tile per CTA).  Rows of the tile are dealt out in bands
        // of kBM / splits, band b to cluster rank b.  Every thread parks its row of the partial tile
        // in shared memory (the operand ring is idle by now; 16-byte chunks XOR-swizzled against
        // bank conflicts); one thread then sends each band with ONE bulk copy into its owner's
        // receive area, completing on the owner's barrier, and the owner sums the slots of its band
        // out of its own shared memory.  Measured on the way here: per-thread 16-byte stores of the
        // rows (into a peer's shared memory or to an L2 workspace alike) took 3.6-3.8 us for a
        // 64 KB tile, and a release arrival on each of four peers' barriers 0.3 us apiece.
        // Receive area: [source rank][row of the band][BN] fp32, chunk c of row r at c ^ (r & swz).
        bool okc = true;
        if (!cluster_met) {
          cluster_wait_acquire();
          cluster_met = true;
        }
        const int rows_per = kBM / p.splits;
        const int nch = p.BN >> 2;
        const int swz = (nch & 7) == 0 ? 7 : 3;
        float* park = reinterpret_cast<float*>(smem_a);     // [128 rows][BN] fp32 <= 64 KB <= two stages
        {
          const int my_row = quarter * 32 + lane;
          float4* park_row = reinterpret_cast<float4*>(park + my_row * p.BN);
          const int rx = my_row & swz;
          {
            // 32 columns per TMEM load; the load of the next 32 is in flight while these are stored
            // (one warp per scheduler runs this: every dependent instruction costs its full latency)
            auto ld_cols = [&](uint32_t (&r)[32], int c) {
              if (c + 32 <= p.BN) {
                tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(c), r);
              } else {
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                      "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                      "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                    : "r"(t_row + static_cast<uint32_t>(c))
                    : "memory");
              }
            };
            auto st_cols = [&](const uint32_t (&r)[32], int c) {
              const int n4 = (p.BN - c) >= 32 ? 8 : 4;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                if (i < n4)
                  park_row[((c >> 2) + i) ^ rx] =
                      make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                  __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
              }
            };
            uint32_t ra[32], rb[32];
            ld_cols(ra, 0);
            for (int c = 0; c < p.BN; c += 64) {
              tmem_ld_wait();
              if (c + 32 < p.BN) ld_cols(rb, c + 32);
              st_cols(ra, c);
              if (c + 32 < p.BN) {
                tmem_ld_wait();
                if (c + 64 < p.BN) ld_cols(ra, c + 64);
                st_cols(rb, c + 32);
              }
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[acc]);
          if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1;
          }
          fence_proxy_async();                              // the parked rows are read by bulk copies
          if (threadIdx.x == 64) B200_TL(1);
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (threadIdx.x == 64) {
            const uint32_t band_bytes = static_cast<uint32_t>(rows_per * p.BN * 4);
            const uint32_t recv = smem_u32(red_buf) + static_cast<uint32_t>(cta_rank) * band_bytes;
            const uint32_t bar = smem_u32(red_ready);
            for (int o = 0; o < p.splits; ++o)
              bulk_push_cluster(mapa_shared(recv, static_cast<uint32_t>(o)),
                                reinterpret_cast<const char*>(park) + static_cast<size_t>(o) * band_bytes, band_bytes,
                                mapa_shared(bar, static_cast<uint32_t>(o)));
            B200_TL(3);
          }
        }
        okc = okc && mbar_wait(red_ready, 0);      // all K slices of my band have landed
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
              : "r"(okc ? 1u : 0u)
              : "memory");
          okc = all_ok != 0;
        }
        if (!okc) {
          if (lane == 0 && !*abort_flag) atomicCAS(p.status, 0, kStatusTimeoutPeerFlag);
          *abort_flag = 1;
          break;
        }
        if (threadIdx.x == 64) B200_TL(5);
        {
          const int r_begin = cta_rank * rows_per;
          const int et = threadIdx.x - 64;
          // one reduced 16-byte chunk (4 columns of one row) to its destination
          auto emit = [&](int rl_now, int c, float4 sum) {
            const int orow = tc.m0 + r_begin + rl_now;
            const int col = tc.n0 + c;
            if (orow >= tc.m_end || col >= p.N) return;
            float v[4] = {sum.x, sum.y, sum.z, sum.w};
            const int ncols = min(4, p.N - col);
            if (p.ar_world > 1) {
              // fused tensor-parallel tail: push 4 columns (half a 16-byte vector) to every rank;
              // N is a multiple of 8 here, so the 4 columns are all valid
              if (p.bias && p.ar.rank == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] += __bfloat162float(p.bias[col + i]);
              }
              uint32_t w0 = pack_bf16x2(v[0], v[1]), w1 = pack_bf16x2(v[2], v[3]);
              if (w0 == kLLSentinel) w0 = 0u;
              if (w1 == kLLSentinel) w1 = 0u;
              const long long word = (static_cast<long long>(orow) * p.N + col) >> 1;     // 32-bit words
#pragma unroll
              for (int r = 0; r < kMaxRanks; ++r) {
                if (r < p.ar_world) {
                  uint32_t* dst = reinterpret_cast<uint32_t*>(p.ar.recv[r] + ar_slot_off +
                                                              static_cast<long long>(p.ar.rank) * p.ar.slot_vecs) + word;
                  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(w0), "r"(w1) : "memory");
                }
              }
              return;
            }
            for (int i = 0; i < ncols; ++i) {
              if (p.bias) v[i] += __bfloat162float(p.bias[col + i]);
              if (p.residual)
                v[i] += __bfloat162float(p.residual[static_cast<size_t>(orow) * p.ldc + col + i]);
            }
            if (p.out_fp32) {
              float* dst = reinterpret_cast<float*>(p.C) + static_cast<size_t>(orow) * p.ldc + col;
              for (int i = 0; i < ncols; ++i) dst[i] = v[i];
            } else {
              __nv_bfloat16* dst =
                  reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(orow) * p.ldc + col;
              if (ncols == 4 && (p.ldc & 3) == 0) {
                uint2 pk;
                pk.x = pack_bf16x2(v[0], v[1]);
                pk.y = pack_bf16x2(v[2], v[3]);
                *reinterpret_cast<uint2*>(dst) = pk;
              } else {
                for (int i = 0; i < ncols; ++i) dst[i] = __float2bfloat16(v[i]);
              }
            }
          };
          // item = (row of the band, 16-byte chunk); a thread walks items et, et + 128, ... without
          // dividing: 128 = row_step * nch + ch_step.  Consecutive threads read consecutive chunks.
          const int row_step = 128 / nch, ch_step = 128 - row_step * nch;
          const float4* band = reinterpret_cast<const float4*>(red_buf);
          const int slot_vecs = rows_per * nch;
          const int items = (rows_per * nch + 127 - et) / 128;      // items of this thread
          auto advance = [&](int& r_, int& c_) {
            c_ += ch_step;
            r_ += row_step;
            if (c_ >= nch) {
              c_ -= nch;
              ++r_;
            }
          };
          auto sum_band = [&](auto sp_tag) {
            constexpr int SP = decltype(sp_tag)::value;
            int rl = et / nch;
            int chl = et - rl * nch;
            for (int i0 = 0; i0 < items; ++i0) {
              const float4* src = band + rl * nch + (chl ^ ((r_begin + rl) & swz));
              float4 x[SP];
#pragma unroll
              for (int s2 = 0; s2 < SP; ++s2) x[s2] = src[s2 * slot_vecs];
              float4 sum = x[0];
#pragma unroll
              for (int s2 = 1; s2 < SP; ++s2) {
                sum.x += x[s2].x;
                sum.y += x[s2].y;
                sum.z += x[s2].z;
                sum.w += x[s2].w;
              }
              emit(rl, chl * 4, sum);
              advance(rl, chl);
            }
          };
          if (p.splits == 2) sum_band(std::integral_constant<int, 2>{});
          else if (p.splits == 4) sum_band(std::integral_constant<int, 4>{});
          else sum_band(std::integral_constant<int, 8>{});
        }
        if (threadIdx.x == 64) B200_TL(6);
        ++tile_iter;
        continue;
      }
      const bool partial = p.splits > 1;
      float* ws_col = nullptr;
      if (partial) {
        // workspace layout: [split][mn_tile][BN cols][128 rows]: for one column the 32
        // lanes of a warp (32 consecutive rows) touch 128 contiguous bytes.
        ws_col = p.workspace +
                 (static_cast<size_t>(tc.split) * total_mn_tiles + tc.mn_index) * kBM * p.BN +
                 (quarter * 32 + lane);
      }
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
        for (int i = 0; i < 16; ++i) {
          if constexpr (KIND == kKindI8) v[i] = static_cast<float>(static_cast<int>(r[i]));
          else v[i] = __uint_as_float(r[i]);
        }
        const int col = tc.n0 + c;
        if (p.a_scales != nullptr && row_ok && !partial) {
          // per-row (token) times per-column (output channel) scales of a quantised product
          const float sa = p.a_scales[row];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (col + i < p.N) v[i] *= sa * p.w_scales[col + i];
        }
        if (partial) {
#pragma unroll
          for (int i = 0; i < 16; ++i) ws_col[static_cast<size_t>(c + i) * kBM] = v[i];
          continue;
        }
        if (p.rs_world > 1) {
          // ---- reduce-scatter push.  Rows of the tile belong to different owners and a thread holds
          // one row, so direct stores would be 32-byte pieces at a row pitch apart.  Instead the warp
          // parks 64 columns of its 32 rows in shared memory and writes them out as 128-byte row
          // segments (8 lanes per row, 4 rows per store instruction) into the owners' staging slots.
          if (p.bias && p.rs_rank == 0) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col + i < p.N) v[i] += __bfloat162float(p.bias[col + i]);
          }
          uint8_t* rs_stage = reinterpret_cast<uint8_t*>(red_buf) + quarter * kRsWarpBytes;
          uint4* mine = reinterpret_cast<uint4*>(rs_stage + lane * kRsPitch + (c & 63) * 2);
          uint4 pk0, pk1;
          pk0.x = pack_bf16x2(v[0], v[1]);
          pk0.y = pack_bf16x2(v[2], v[3]);
          pk0.z = pack_bf16x2(v[4], v[5]);
          pk0.w = pack_bf16x2(v[6], v[7]);
          pk1.x = pack_bf16x2(v[8], v[9]);
          pk1.y = pack_bf16x2(v[10], v[11]);
          pk1.z = pack_bf16x2(v[12], v[13]);
          pk1.w = pack_bf16x2(v[14], v[15]);
          mine[0] = pk0;
          mine[1] = pk1;
          if ((c & 63) == 48 || c + 16 >= p.BN) {
            __syncwarp();
            const int c64 = c & ~63;
            const int segs = (min(64, p.BN - c64)) >> 3;          // 16-byte segments per row in this group
            for (int idx = lane; idx < 32 * segs; idx += 32) {
              const int rowi = idx / segs, seg = idx - rowi * segs;
              const int grow = tc.m0 + quarter * 32 + rowi;
              const int gcol = tc.n0 + c64 + seg * 8;
              if (grow < tc.m_end && gcol < p.N) {
                const int owner = grow / p.rs_rows;
                const int row_local = grow - owner * p.rs_rows;
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(p.rs_data[owner]) + rs_half_off) +
                                     (static_cast<long long>(p.rs_rank) * p.rs_rows + row_local) * p.N + gcol;
                *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(rs_stage + rowi * kRsPitch + seg * 16);
              }
            }
            __syncwarp();
          }
          continue;
        }
        if (!row_ok || col >= p.N) continue;
        if (p.ar_world > 1) {
          // push 16 columns (two 16-byte vectors) of this row to every rank; rank 0 adds the bias
          if (p.bias && p.ar.rank == 0) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col + i < p.N) v[i] += __bfloat162float(p.bias[col + i]);
          }
          uint4 pk0, pk1;
          pk0.x = pack_bf16x2(v[0], v[1]);
          pk0.y = pack_bf16x2(v[2], v[3]);
          pk0.z = pack_bf16x2(v[4], v[5]);
          pk0.w = pack_bf16x2(v[6], v[7]);
          pk1.x = pack_bf16x2(v[8], v[9]);
          pk1.y = pack_bf16x2(v[10], v[11]);
          pk1.z = pack_bf16x2(v[12], v[13]);
          pk1.w = pack_bf16x2(v[14], v[15]);
          pk0 = ll_sanitize(pk0);
          pk1 = ll_sanitize(pk1);
          const long long vec = (static_cast<long long>(row) * p.N + col) >> 3;
          const bool second = col + 8 < p.N;
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r) {
            if (r < p.ar_world) {
              uint4* dst = p.ar.recv[r] + ar_slot_off + static_cast<long long>(p.ar.rank) * p.ar.slot_vecs + vec;
              ll_store(dst, pk0);
              if (second) ll_store(dst + 1, pk1);
            }
          }
          continue;
        }
        if (p.swiglu) {
          // Columns [c, c+8) hold gate values, [c+8, c+16) the matching up values.
          const int ocol = col >> 1;
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float g = v[i];
            o[i] = (g / (1.f + __expf(-g))) * v[8 + i];
          }
          __nv_bfloat16* dst =
              reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + ocol;
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
              reinterpret_cast<float4*>(dst)[i] =
                  make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          } else {
            for (int i = 0; i < ncols; ++i) dst[i] = v[i];
          }
        } else {
          __nv_bfloat16* dst =
              reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col;
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
      // Accumulator buffer is free for the MMA warp again.
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }

      if (partial) {
        // Split-K fix-up: the last CTA to arrive at this (m,n) tile sums the
        // partials in split order (deterministic) and writes the result.
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          const int old = atomicAdd(&p.tile_counters[tc.mn_index], 1);
          const int last = (old == p.splits - 1) ? 1 : 0;
          if (last) p.tile_counters[tc.mn_index] = 0;  // leave the counter at rest
          s_flags[1] = last;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool is_last = s_flags[1] != 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (is_last) {
          __threadfence();
          const size_t split_stride = static_cast<size_t>(total_mn_tiles) * kBM * p.BN;
          const float* base =
              p.workspace + static_cast<size_t>(tc.mn_index) * kBM * p.BN + (quarter * 32 + lane);
          for (int c = 0; c < p.BN; c += 8) {
            const int col = tc.n0 + c;
            if (col >= p.N) break;
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
            for (int sp = 0; sp < p.splits; ++sp) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                v[i] += __ldcg(base + sp * split_stride + static_cast<size_t>(c + i) * kBM);
            }
            if (!row_ok) continue;
            const int ncols = min(8, p.N - col);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (i < ncols) {
                if (p.bias) v[i] += __bfloat162float(p.bias[col + i]);
                if (p.residual)
                  v[i] += __bfloat162float(p.residual[static_cast<size_t>(row) * p.ldc + col + i]);
              }
            }
            if (p.out_fp32) {
              float* dst = reinterpret_cast<float*>(p.C) + static_cast<size_t>(row) * p.ldc + col;
              for (int i = 0; i < ncols; ++i) dst[i] = v[i];
            } else {
              __nv_bfloat16* dst =
                  reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col;
              if (ncols == 8 && (p.ldc & 7) == 0) {
                uint4 pk;
                pk.x = pack_bf16x2(v[0], v[1]);
                pk.y = pack_bf16x2(v[2], v[3]);
                pk.z = pack_bf16x2(v[4], v[5]);
                pk.w = pack_bf16x2(v[6], v[7]);
                *reinterpret_cast<uint4*>(dst) = pk;
              } else {
                for (int i = 0; i < ncols; ++i) dst[i] = __float2bfloat16(v[i]);
              }
            }
          }
        }
      }
    }
    // foreign blocks this CTA has not delivered its share of yet (fewer tiles than sources, or an abort)
    while (ag_next < p.ag_world) ag_step();
    if (p.cluster_split && !cluster_met) cluster_wait_acquire();
  }

  // ------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (p.ar_world > 1) {
    // ---- fused tail: reduce rows that have arrived from every rank (data-carried flags: no
    // barrier between the ranks), + residual, RMSNorm.  Row r belongs to CTA r % gridDim.
    // (the operand stages are idle by now: every load has landed and every MMA has retired)
    float* ar_red = reinterpret_cast<float*>(smem_a);
    const int nvec_row = p.N >> 3;
    const uint4* mine = p.ar.recv[p.ar.rank] + ar_slot_off;
    bool ar_ok = *abort_flag == 0;
    for (int row = blockIdx.x; ar_ok && row < p.M; row += gridDim.x) {
      // a thread owns vectors tid, tid + 192, ...; values are kept for the second pass
      float ss = 0.f;
      for (int vb = 0; vb < nvec_row; vb += kThreads) {
        const int vi = vb + threadIdx.x;
        if (vi < nvec_row) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r) {
            if (r < p.ar_world) {
              uint4 x;
              ar_ok = ll_wait(mine + static_cast<long long>(r) * p.ar.slot_vecs +
                                  static_cast<long long>(row) * nvec_row + vi, x) && ar_ok;
              add8(acc, x);
            }
          }
          Pack8 y;
          y.u = pack8(acc);            // the sum is rounded to bf16 before the residual add
          Pack8 nr = y;
          if (p.residual) {
            uint4* rp = reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(p.residual)) +
                        static_cast<long long>(row) * nvec_row + vi;
            Pack8 rs;
            rs.u = *rp;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              nr.h[j] = __float2bfloat16(__bfloat162float(y.h[j]) + __bfloat162float(rs.h[j]));
            if (p.ar_norm_w) *rp = nr.u;      // the residual stream carries the pre-norm sum
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float f = __bfloat162float(nr.h[j]);
            ss += f * f;
          }
          // first pass result parked in C (bf16); rewritten below when a norm follows
          reinterpret_cast<uint4*>(p.C)[static_cast<long long>(row) * (p.ldc >> 3) + vi] = nr.u;
        }
      }
      if (p.ar_norm_w) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) ar_red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < kThreads / 32; ++w) tot += ar_red[w];
        const float inv = rsqrtf(tot / static_cast<float>(p.N) + p.ar_eps);
        for (int vb = 0; vb < nvec_row; vb += kThreads) {
          const int vi = vb + threadIdx.x;
          if (vi < nvec_row) {
            uint4* cp = reinterpret_cast<uint4*>(p.C) + static_cast<long long>(row) * (p.ldc >> 3) + vi;
            Pack8 x, w8, o8;
            x.u = *cp;                       // written by this same thread above
            w8.u = reinterpret_cast<const uint4*>(p.ar_norm_w)[vi];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              o8.h[j] = __float2bfloat16(__bfloat162float(x.h[j]) * inv * __bfloat162float(w8.h[j]));
            *cp = o8.u;
          }
        }
        __syncthreads();
      }
    }
    if (!ar_ok) atomicCAS(p.status, 0, kStatusTimeoutPeerFlag);
    // re-arm the slot of the previous call, then the last CTA advances the epoch
    {
      volatile uint32_t* meta = reinterpret_cast<volatile uint32_t*>(p.ar.epoch);
      const uint32_t prev_vecs = meta[1 + (ar_epoch + 2) % 3];
      const uint4 s4 = make_uint4(kLLSentinel, kLLSentinel, kLLSentinel, kLLSentinel);
      uint4* rearm = p.ar.recv[p.ar.rank] + static_cast<long long>((ar_epoch + 2) % 3) * p.ar_world * p.ar.slot_vecs;
      const long long total = static_cast<long long>(prev_vecs) * p.ar_world;
      for (long long idx = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; idx < total;
           idx += static_cast<long long>(gridDim.x) * kThreads)
        rearm[(idx / prev_vecs) * p.ar.slot_vecs + idx % prev_vecs] = s4;
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(p.ar_done, 1u) == gridDim.x - 1) {
          *p.ar_done = 0;
          meta[1 + ar_epoch % 3] = static_cast<uint32_t>((static_cast<long long>(p.M) * p.N) >> 3);
          meta[0] = ar_epoch;
        }
      }
    }
  }
  // Split-K in a cluster: the bulk copies out of this CTA's shared memory report completion to
  // their destinations only, so no CTA leaves before every owner has its band (each arrives here
  // after its sum; after an abort, peers either arrive or have exited).
  if (p.cluster_split) cluster_sync_all();
  if (threadIdx.x == 0) B200_TL(7);
  if (warp == 1) {
    if (*abort_flag && lane == 0) {
      // Give MMAs still in flight a bounded time to retire before TMEM goes away.
      tc_commit(drain_bar);
      mbar_wait(drain_bar, 0);
    }
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}

// ------------------------------------------------------------------ host side

struct GemmPlan {
  int BN;
  int splits;
  int stages;
  int cluster;   // 1: split-K inside a thread-block cluster (DSMEM reduction)
};

static inline int round_up(int x, int m) { return (x + m - 1) / m * m; }

// Bytes of the staging region that follows the pipeline stages.  mode 1: cluster split-K partial
// tile (fp32); mode 2: reduce-scatter push, per epilogue warp 32 rows x 64 bf16 columns at a
// 144-byte pitch.
static constexpr int kRsStageBytes = 4 * kRsWarpBytes;
static size_t red_bytes_for(int BN, int cluster_split) {
  if (cluster_split == 2) return kRsStageBytes;
  return cluster_split ? static_cast<size_t>(kBM) * BN * 4 : 0;     // receive area of the cluster reduction
}

static size_t smem_bytes_for(int BN, int stages, int num_experts, int cluster_split = 0) {
  return 1024 + static_cast<size_t>(stages) * (kBM * kRowBytes + BN * kRowBytes) +
         red_bytes_for(BN, cluster_split) + (2 * stages + 7) * 8 + 16 + (num_experts + 2) * 4 + 64;
}

// Slabs per barrier round trip: two when that still leaves three groups in flight.  The
// producer and MMA threads each spend several hundred cycles per round trip (their
// shared-memory accesses queue behind the tensor core's), so fewer, larger rounds keep
// them off the critical path.
static int ksub_for(int stages) {
  static const int forced = [] {
    const char* e = getenv("OMNI_B200_GEMM_KSUB");
    return e ? atoi(e) : 0;
  }();
  if (forced == 1 || (forced == 2 && stages >= 4)) return forced;
  return stages >= 6 ? 2 : 1;
}

static int stages_for(int BN, int cluster_split) {
  const int stage_bytes = kBM * kRowBytes + BN * kRowBytes;
  int stages = static_cast<int>((226 * 1024 - 2048 - red_bytes_for(BN, cluster_split)) / stage_bytes);
  if (stages > 8) stages = 8;
  if (stages < 2) stages = 2;
  return stages;
}

// Cost model used to choose the tile width and split-K factor.  All rates are
// per SM; the model only has to rank candidates, not predict time.
static GemmPlan plan_gemm(int M, int N, int K, int elem_bytes, int sms, bool allow_split,
                          bool swiglu) {
  const int k_iters = (K * elem_bytes + kRowBytes - 1) / kRowBytes;
  const int m_blocks = (M + kBM - 1) / kBM;
  const double sm_ingest = 90e9;                              // bytes/s one SM can pull from L2
  const double sm_flops = (elem_bytes == 1 ? 2.8e15 : 1.4e15) / 148.0;
  const double hbm = 6.5e12;
  double best = 1e30;
  GemmPlan bestp{128, 1, 4, 0};
  for (int bn = 256; bn >= 32; bn -= 16) {
    if (bn > round_up(N, 16) && bn != 32) continue;
    const int n_blocks = (N + bn - 1) / bn;
    const long long tiles = static_cast<long long>(m_blocks) * n_blocks;
    const int max_split = allow_split ? 8 : 1;
    for (int sp = 1; sp <= max_split; ++sp) {
      const int per = (k_iters + sp - 1) / sp;
      if (sp > 1 && (per < 8 || (sp - 1) * per >= k_iters)) continue;
      const long long ctas = tiles * sp;
      const double rows_a = M < kBM ? M : kBM;
      const double bytes_cta = (rows_a + bn) * per * static_cast<double>(kRowBytes);
      const double flops_cta = 2.0 * kBM * bn * per * (kRowBytes / elem_bytes);
      double t_cta = bytes_cta / sm_ingest;
      const double t_f = flops_cta / sm_flops;
      if (t_f > t_cta) t_cta = t_f;
      t_cta += 1.5e-6 + (sp > 1 ? 1.0e-6 : 0.0);
      const double waves = static_cast<double>((ctas + sms - 1) / sms);
      double t = waves * t_cta;
      double unique = (static_cast<double>(M) * K + static_cast<double>(N) * K) * elem_bytes +
                      static_cast<double>(M) * N * 2;
      if (sp > 1) unique += 2.0 * sp * static_cast<double>(m_blocks) * kBM * n_blocks * bn * 4;
      const double t_hbm = unique / hbm;
      if (t_hbm > t) t = t_hbm;
      if (sp > 1) t += 2.0 * sp * static_cast<double>(m_blocks) * kBM * n_blocks * bn * 4 / hbm * 0.5;
      if (t < best * 0.999) {
        best = t;
        bestp.BN = bn;
        bestp.splits = sp;
      }
    }
  }
  bestp.stages = stages_for(bestp.BN, 0);
  return bestp;
}

static int next_pow2_cols(int x) {
  int c = 32;
  while (c < x) c <<= 1;
  return c;
}

template <bool GROUPED, int KIND>
static int launch(const CUtensorMap& ta, const CUtensorMap& tw, const GemmParams& p, int grid,
                  size_t smem, cudaStream_t stream) {
  auto kern = gemm_tcgen05_kernel<GROUPED, KIND>;
  static DeviceOnce once;
  int dev = 0;
  if (once.needed(&dev)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return -20;
    once.mark(dev);
  }
  const int cluster_x = p.cluster_split ? p.splits : 1;
  return launch_pdl(kern, dim3(grid, 1, 1), dim3(kThreads, 1, 1), smem, stream, cluster_x, ta, tw, p) == cudaSuccess
             ? 0
             : (p.cluster_split ? -22 : -21);
}

// How many clusters of `size` CTAs of this kernel can be resident at once.
static int max_active_clusters(int size, size_t smem) {
  static int cache[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  if (size < 1 || size > 8) return 0;
  if (cache[size] > 0) return cache[size];
  auto kern = gemm_tcgen05_kernel<false, false>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(size * 148, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = size;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    n = sm_count() / size - (size > 2 ? 2 : 0);
  }
  cache[size] = n;
  return n;
}

}  // namespace b200

using namespace b200;

// Small-M (weight-streaming) problems: split K across the CTAs of a cluster so
// that every SM streams a slab of the weights, and reduce on chip.
static bool plan_small_m(int M, int N, int K, int elem_bytes, bool allow_split, GemmPlan* out) {
  const int k_iters = (K * elem_bytes + kRowBytes - 1) / kRowBytes;
  const int m_blocks = (M + kBM - 1) / kBM;
  const double sm_ingest = 110e9, hbm = 6.5e12;
  double best = 1e30;
  bool found = false;
  for (int bn = 256; bn >= 64; bn -= 16) {
    if (bn > ((N + 15) / 16) * 16) continue;
    const int n_blocks = (N + bn - 1) / bn;
    const int clusters = m_blocks * n_blocks;
    const int max_sp = (allow_split && bn <= 128) ? 8 : 1;
    for (int sp = 1; sp <= max_sp; ++sp) {
      if (kBM % sp != 0) continue;            // row bands of the cluster reduction: 1, 2, 4 or 8 K slices
      const int per = (k_iters + sp - 1) / sp;
      if (sp > 1 && (per < 4 || (sp - 1) * per >= k_iters)) continue;
      const int stages = stages_for(bn, sp > 1);
      const int cap = sp > 1 ? max_active_clusters(sp, smem_bytes_for(bn, stages, 0, 1)) : sm_count();
      if (cap <= 0) continue;
      const int waves = (clusters + cap - 1) / cap;
      // (the full 128-row slab is charged whatever M is: the plan, and with it the order in which
      // a row's products are summed, must not depend on how many other rows share the launch:
      // a decode step padded to a captured graph size gives the same numbers as the unpadded one)
      const double rows_a = kBM;
      double t_cta = (rows_a + bn) * per * static_cast<double>(kRowBytes) / sm_ingest + 2.5e-6;
      if (sp > 1) t_cta += 1.5e-6;
      double t = waves * t_cta;
      const double t_hbm = (static_cast<double>(N) * K * elem_bytes) / hbm;
      if (t_hbm > t) t = t_hbm;
      t += 0.1 * waves * t_cta;  // among HBM-bound candidates prefer the best SM fill
      if (t < best * 0.999) {
        best = t;
        out->BN = bn;
        out->splits = sp;
        out->cluster = sp > 1 ? 1 : 0;
        out->stages = stages;
        found = true;
      }
    }
  }
  return found;
}

// Chooses tile width / split-K for a problem.  out_cluster = 1 means the splits run
// as one thread-block cluster (no workspace needed); otherwise split-K uses the
// caller's fp32 workspace (bytes) and per-tile counters.
#ifdef B200_GEMM_TIMELINE
extern "C" int b200_gemm_timeline(unsigned long long* host, int ctas) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_timeline, sizeof(unsigned long long) * 8 * ctas));
}
extern "C" int b200_gemm_timeline_cycles(long long* host, int ctas) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_timeline_clk, sizeof(long long) * 8 * ctas));
}
#endif

extern "C" void b200_gemm_plan(int M, int N, int K, int elem_bytes, int swiglu, int force_bn,
                               int force_splits, int* out_bn, int* out_splits,
                               size_t* out_ws_bytes, int* out_counters, int* out_cluster) {
  GemmPlan pl = plan_gemm(M, N, K, elem_bytes, sm_count(), false, swiglu != 0);
  pl.cluster = 0;
  if (M <= 256 && force_bn <= 0 && force_splits <= 0) {
    GemmPlan small = pl;
    if (plan_small_m(M, N, K, elem_bytes, !swiglu, &small)) pl = small;
  }
  if (force_bn > 0) pl.BN = force_bn;
  if (force_splits > 0) {
    pl.splits = force_splits;
    // a forced split count runs as a cluster when it can
    pl.cluster = (force_splits > 1 && force_splits <= 8 && (kBM % force_splits) == 0 && pl.BN <= 128 && !swiglu) ? 1 : 0;
  }
  if (force_splits < 0) {  // negative: force the workspace (non-cluster) split-K with |splits|
    pl.splits = -force_splits;
    pl.cluster = 0;
  }
  const int m_blocks = (M + kBM - 1) / kBM;
  const int n_blocks = (N + pl.BN - 1) / pl.BN;
  *out_bn = pl.BN;
  *out_splits = pl.splits;
  *out_cluster = pl.cluster;
  *out_counters = m_blocks * n_blocks;
  *out_ws_bytes = (pl.splits > 1 && !pl.cluster)
                      ? static_cast<size_t>(pl.splits) * m_blocks * n_blocks * kBM * pl.BN * 4
                      : 0;
}

// Dense GEMM.  A [M,K] (pitch lda), W [N,K] (pitch ldw), C [M,N or N/2 with
// swiglu] (pitch ldc).  dtype_fp8 = 0: bf16 inputs; 1: e4m3 inputs (no scale
// handling here; callers fold scales, see the block-scaled wrapper).
// workspace / counters may be null when splits == 1 or cluster_split == 1.
// Returns 0 on success.
struct ArArgs;
static int gemm_impl(const void* A, const void* W, void* C, const void* bias, const void* residual, int M,
                     int N, int K, int lda, int ldw, int ldc, int dtype_fp8, int out_fp32, int swiglu, int BN,
                     int splits, int cluster_split, void* workspace, int* counters, int* status,
                     int max_ctas, cudaStream_t stream, const float* a_scales, const float* w_scales,
                     const ArArgs* ar = nullptr, const struct AgArgs* ag = nullptr,
                     const struct RsArgs* rs = nullptr);

extern "C" int b200_gemm(const void* A, const void* W, void* C, const void* bias,
                         const void* residual, int M, int N, int K, int lda, int ldw, int ldc,
                         int dtype_fp8, int out_fp32, int swiglu, int BN, int splits,
                         int cluster_split, void* workspace, int* counters, int* status,
                         int max_ctas, cudaStream_t stream) {
  return gemm_impl(A, W, C, bias, residual, M, N, K, lda, ldw, ldc, dtype_fp8, out_fp32, swiglu, BN, splits,
                   cluster_split, workspace, counters, status, max_ctas, stream, nullptr, nullptr);
}

// Quantised product with per-row (a_scales[M]) and per-column (w_scales[N]) scales applied to
// the accumulator: kind 1 = e4m3 operands, 2 = int8 operands (s32 accumulate).  No split-K.
extern "C" int b200_gemm_scaled(const void* A, const void* W, void* C, const float* a_scales,
                                const float* w_scales, const void* bias, const void* residual, int M, int N,
                                int K, int lda, int ldw, int ldc, int kind, int out_fp32, int BN, int* status,
                                int max_ctas, cudaStream_t stream) {
  if (kind != 1 && kind != 2) return -15;
  if (a_scales == nullptr || w_scales == nullptr) return -16;
  return gemm_impl(A, W, C, bias, residual, M, N, K, lda, ldw, ldc, kind, out_fp32, 0, BN, 1, 0, nullptr,
                   nullptr, status, max_ctas, stream, a_scales, w_scales);
}

struct RsArgs {
  void* const* data = nullptr;      // peer-mapped staging buffers
  const void* signal = nullptr;     // this rank's signal pad
  long long half_bytes = 0;
  int world = 0, rank = 0, rows = 0;
  int epoch_word = 0;
};

struct AgArgs {
  void* const* data = nullptr;      // peer-mapped staging buffers
  long long half_bytes = 0;
  const void* signal = nullptr;     // this rank's signal pad
  void* ready = nullptr;            // [world] local counters
  int world = 0, rank = 0, rows = 0;
  int epoch_word = 0, flag_word = 0;
};

struct ArArgs {
  void* const* recv = nullptr;
  int world = 0, rank = 0;
  long long slot_vecs = 0;
  void* epoch = nullptr;
  const void* norm_w = nullptr;
  float eps = 0.f;
  void* done = nullptr;
};

static int gemm_impl(const void* A, const void* W, void* C, const void* bias, const void* residual, int M,
                     int N, int K, int lda, int ldw, int ldc, int dtype_fp8, int out_fp32, int swiglu, int BN,
                     int splits, int cluster_split, void* workspace, int* counters, int* status,
                     int max_ctas, cudaStream_t stream, const float* a_scales, const float* w_scales,
                     const ArArgs* ar, const struct AgArgs* ag, const struct RsArgs* rs);

// Row-parallel projection of a tensor-parallel layer in ONE kernel: C = RMSNorm(residual +=
// sum over ranks of (A @ W^T)) * norm_w  (norm_w null: C = sum (+ residual), residual untouched).
// Output tiles are pushed to every rank's receive buffer (data-carried flags, no barrier);
// the CTAs then reduce the rows as they arrive.  bf16, M * N * 2 bytes <= slot size, N % 8 == 0.
extern "C" int b200_gemm_all_reduce(const void* A, const void* W, void* C, const void* bias, void* residual,
                                    const void* norm_w, float eps, int M, int N, int K, int lda, int ldw,
                                    int BN, void* const* recv, int world, int rank, long long slot_vecs,
                                    void* epoch, void* done_counter, int* status, int max_ctas,
                                    cudaStream_t stream) {
  if (world < 2 || world > kMaxRanks) return -30;
  if ((N & 7) != 0 || (static_cast<long long>(M) * N >> 3) > slot_vecs) return -31;
  ArArgs ar;
  ar.recv = recv;
  ar.world = world;
  ar.rank = rank;
  ar.slot_vecs = slot_vecs;
  ar.epoch = epoch;
  ar.norm_w = norm_w;
  ar.eps = eps;
  ar.done = done_counter;
  int splits = 1, cluster = 0;
  if (BN <= 0) {
    // same plan as the stand-alone decode GEMM: K split over the CTAs of a cluster when that
    // spreads the weight stream over more SMs (the cluster's reduced tile is what gets pushed)
    GemmPlan pl{128, 1, 4, 0};
    if (!plan_small_m(M, N, K, 2, true, &pl)) pl = GemmPlan{128, 1, 4, 0};
    BN = pl.BN;
    splits = pl.splits;
    cluster = pl.cluster;
  }
  return gemm_impl(A, W, C, bias, residual, M, N, K, lda, ldw, N, 0, 0, 0, BN, splits, cluster, nullptr, nullptr,
                   status, max_ctas, stream, nullptr, nullptr, &ar, nullptr);
}

// Row-parallel projection whose result is reduce-scattered, first half of the pair: the partial
// product A @ W^T (M = world * rows) is stored tile by tile into the row owners' staging buffers
// (slot of this rank) while the GEMM runs.  b200_symm_rs_reduce (collectives file) must follow on
// the same stream: it signals the peers, waits for all sources and sums the slots.
extern "C" int b200_gemm_reduce_scatter_push(const void* A, const void* W, const void* bias, int M, int N, int K,
                                             int lda, int ldw, void* const* data, const void* signal_local,
                                             long long half_bytes, int world, int rank, int epoch_word,
                                             int* status, int max_ctas, cudaStream_t stream) {
  if (world < 2 || world > kMaxRanks || M % world != 0) return -30;
  if (static_cast<long long>(M) * N * 2 > half_bytes) return -31;
  RsArgs rs;
  rs.data = data;
  rs.signal = signal_local;
  rs.half_bytes = half_bytes;
  rs.world = world;
  rs.rank = rank;
  rs.rows = M / world;
  rs.epoch_word = epoch_word;
  GemmPlan pl = plan_gemm(M, N, K, 2, sm_count(), false, false);
  // C is never written in this mode; pass the local staging buffer as a valid placeholder
  return gemm_impl(A, W, data[rank], bias, nullptr, M, N, K, lda, ldw, N, 0, 0, 0, pl.BN, 1, 0, nullptr, nullptr,
                   status, max_ctas, stream, nullptr, nullptr, nullptr, nullptr, &rs);
}

// Column-parallel projection of a sequence-sharded activation in ONE GEMM kernel:
// C [world * rows, N] = concat_r(A_r) @ W^T.  `gathered` [world * rows, K] bf16 is local memory
// whose own block (and every rank's staging buffer) the staging kernel has filled.  While the
// tensor cores work on the own rows, the epilogue warps of all CTAs pull the foreign blocks from
// their owners' staging buffers over NVLink, each byte once; tiles of a foreign block start when
// its counter shows it complete.  swiglu: C [.., N/2] = silu(gate) * up (interleaved weight layout).
extern "C" int b200_gemm_all_gather(void* gathered, void* const* data, long long half_bytes,
                                    const void* signal_local, void* ready, const void* W, void* C,
                                    const void* bias, int rows, int N, int K, int ldw, int ldc, int swiglu,
                                    int world, int rank, int epoch_word, int flag_word, int* status,
                                    int max_ctas, cudaStream_t stream) {
  if (world < 2 || world > kMaxRanks) return -30;
  if ((static_cast<long long>(rows) * K * 2) % 16 != 0) return -31;
  AgArgs ag;
  ag.data = data;
  ag.half_bytes = half_bytes;
  ag.signal = signal_local;
  ag.ready = ready;
  ag.world = world;
  ag.rank = rank;
  ag.rows = rows;
  ag.epoch_word = epoch_word;
  ag.flag_word = flag_word;
  const int M = rows * world;
  GemmPlan pl = plan_gemm(M, N, K, 2, sm_count(), false, swiglu != 0);
  return gemm_impl(gathered, W, C, bias, nullptr, M, N, K, K, ldw, ldc, 0, 0, swiglu, pl.BN, 1, 0, nullptr, nullptr,
                   status, max_ctas, stream, nullptr, nullptr, nullptr, &ag);
}

static int gemm_impl(const void* A, const void* W, void* C, const void* bias, const void* residual, int M,
                     int N, int K, int lda, int ldw, int ldc, int dtype_fp8, int out_fp32, int swiglu, int BN,
                     int splits, int cluster_split, void* workspace, int* counters, int* status,
                     int max_ctas, cudaStream_t stream, const float* a_scales, const float* w_scales,
                     const ArArgs* ar, const AgArgs* ag, const RsArgs* rs) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int eb = dtype_fp8 ? 1 : 2;
  if (BN < 16 || BN > 256 || (BN % 16) != 0) return -10;
  if (swiglu && ((N % 16) != 0 || splits != 1)) return -11;
  if (splits <= 1) cluster_split = 0;
  if (cluster_split && (splits > 8 || BN > 128 || (kBM % splits) != 0)) return -14;
  if (splits > 1 && !cluster_split && (workspace == nullptr || counters == nullptr)) return -12;

  GemmParams p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.BN = BN;
  p.elem_bytes = eb;
  p.k_iters = (K * eb + kRowBytes - 1) / kRowBytes;
  p.splits = splits;
  p.cluster_split = cluster_split;
  p.num_m_blocks = (M + kBM - 1) / kBM;
  p.num_n_blocks = (N + BN - 1) / BN;
  const int smem_mode = cluster_split ? 1 : ((rs != nullptr && rs->world > 1) ? 2 : 0);
  p.stages = stages_for(BN, smem_mode);
  p.ksub = ksub_for(p.stages);
  p.stages -= p.stages % p.ksub;
  p.acc_stride = BN <= 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256));
  p.tmem_cols = next_pow2_cols(2 * p.acc_stride);
  p.ldc = ldc;
  p.out_fp32 = out_fp32;
  p.swiglu = swiglu;
  p.num_experts = 0;
  p.C = C;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.workspace = static_cast<float*>(workspace);
  p.tile_counters = counters;
  p.expert_offsets = nullptr;
  p.status = status;
  p.a_scales = a_scales;
  p.w_scales = w_scales;
  if (ar != nullptr && ar->world > 1) {
    for (int r = 0; r < kMaxRanks; ++r) p.ar.recv[r] = r < ar->world ? static_cast<uint4*>(ar->recv[r]) : nullptr;
    p.ar.epoch = static_cast<uint32_t*>(ar->epoch);
    p.ar.world = ar->world;
    p.ar.rank = ar->rank;
    p.ar.slot_vecs = ar->slot_vecs;
    p.ar_world = ar->world;
    p.ar_norm_w = static_cast<const __nv_bfloat16*>(ar->norm_w);
    p.ar_eps = ar->eps;
    p.ar_done = static_cast<uint32_t*>(ar->done);
  }
  if (ag != nullptr && ag->world > 1) {
    if (splits != 1 || ag->rows <= 0 || (ag->rows % kBM) != 0 || ag->rows * ag->world != M) return -17;
    for (int r = 0; r < kMaxRanks; ++r) p.ag_data[r] = r < ag->world ? ag->data[r] : nullptr;
    p.ag_half_bytes = ag->half_bytes;
    p.ag_ready = static_cast<uint32_t*>(ag->ready);
    p.ag_local = A;
    p.ag_signal = static_cast<const uint32_t*>(ag->signal);
    p.ag_world = ag->world;
    p.ag_rank = ag->rank;
    p.ag_rows = ag->rows;
    p.ag_epoch_word = ag->epoch_word;
    p.ag_flag_word = ag->flag_word;
  }
  if (rs != nullptr && rs->world > 1) {
    if (splits != 1 || swiglu || out_fp32 || dtype_fp8 || rs->rows <= 0 || rs->rows * rs->world != M || (N % 16) != 0)
      return -18;
    for (int r = 0; r < kMaxRanks; ++r) p.rs_data[r] = r < rs->world ? rs->data[r] : nullptr;
    p.rs_signal = static_cast<const uint32_t*>(rs->signal);
    p.rs_half_bytes = rs->half_bytes;
    p.rs_world = rs->world;
    p.rs_rank = rs->rank;
    p.rs_rows = rs->rows;
    p.rs_epoch_word = rs->epoch_word;
  }
  CUtensorMap ta, tw;
  const CUtensorMapDataType dt = dtype_fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int box_k = kRowBytes / eb;
  int r = make_tensormap_2d(&ta, dt, eb, A, M, K, lda, kBM, box_k, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r;
  r = make_tensormap_2d(&tw, dt, eb, W, N, K, ldw, BN, box_k, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 1000;
  const size_t smem = smem_bytes_for(BN, p.stages, 0, smem_mode);
  int grid;
  if (cluster_split) {
    const long long clusters = static_cast<long long>(p.num_m_blocks) * p.num_n_blocks;
    if (max_active_clusters(splits, smem) <= 0) return -15;
    // one tile per CTA: the reduction's barriers and receive area are used once per launch, and
    // clusters beyond what fits at once simply start as earlier ones retire (max_ctas is not
    // honoured by this variant)
    if (clusters * splits > 0x7fffffffLL) return -15;
    grid = static_cast<int>(clusters) * splits;
  } else {
    const long long tiles = static_cast<long long>(p.num_m_blocks) * p.num_n_blocks * splits;
    grid = sm_count();
    if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
    if (tiles < grid) grid = static_cast<int>(tiles);
  }
  if (dtype_fp8 == 2) return launch<false, kKindI8>(ta, tw, p, grid, smem, stream);
  if (dtype_fp8) return launch<false, kKindFP8>(ta, tw, p, grid, smem, stream);
  return launch<false, kKindBF16>(ta, tw, p, grid, smem, stream);
}

// Grouped GEMM over E experts.  A [total_rows, K] holds each expert's rows
// contiguously, expert e owning rows expert_offsets[e] .. expert_offsets[e+1]
// (device array, so no host synchronisation is needed to learn the counts).
// W [E, N, K].  C [total_rows, N (or N/2 with swiglu)].
extern "C" int b200_grouped_gemm(const void* A, const void* W, void* C, const int* expert_offsets,
                                 int num_experts, int total_rows, int N, int K, int lda, int ldc,
                                 int dtype_fp8, int swiglu, int BN, int* status, int max_ctas,
                                 cudaStream_t stream) {
  if (total_rows <= 0 || num_experts <= 0) return 0;
  if (num_experts > kMaxExperts) return -13;
  const int eb = dtype_fp8 ? 1 : 2;
  if (BN < 16 || BN > 256 || (BN % 16) != 0) return -10;
  if (swiglu && (N % 16) != 0) return -11;
  GemmParams p{};
  p.M = total_rows;
  p.N = N;
  p.K = K;
  p.BN = BN;
  p.elem_bytes = eb;
  p.k_iters = (K * eb + kRowBytes - 1) / kRowBytes;
  p.splits = 1;
  p.num_m_blocks = 0;
  p.num_n_blocks = (N + BN - 1) / BN;
  const int stages = stages_for(BN, 0);
  p.ksub = ksub_for(stages);
  p.stages = stages - stages % p.ksub;
  p.cluster_split = 0;
  p.acc_stride = BN <= 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256));
  p.tmem_cols = next_pow2_cols(2 * p.acc_stride);
  p.ldc = ldc;
  p.out_fp32 = 0;
  p.swiglu = swiglu;
  p.num_experts = num_experts;
  p.C = C;
  p.expert_offsets = expert_offsets;
  p.status = status;
  CUtensorMap ta, tw;
  const CUtensorMapDataType dt = dtype_fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int box_k = kRowBytes / eb;
  int r = make_tensormap_2d(&ta, dt, eb, A, total_rows, K, lda, kBM, box_k, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r;
  r = make_tensormap_3d(&tw, dt, eb, W, num_experts, N, K, static_cast<uint64_t>(N) * K, K, BN,
                        box_k, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 1000;
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  const size_t smem = smem_bytes_for(BN, stages, num_experts);
  if (dtype_fp8) return launch<true, kKindFP8>(ta, tw, p, grid, smem, stream);
  return launch<true, kKindBF16>(ta, tw, p, grid, smem, stream);
}
