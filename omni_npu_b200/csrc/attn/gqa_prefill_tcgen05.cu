// Paged GQA prefill attention on the 5th-generation tensor cores (head size 128, bf16).
//
// One CTA = 128 query rows of one (sequence, query head).  Both products of every 64-key tile
// run as tcgen05.mma with the accumulators in tensor memory:
//   S = Q K^T   M = 128 rows, N = 64 keys, K = 128 (Q and the K tile are K-major 128B-swizzled
//               shared-memory operands; the K tile comes straight from the paged cache by TMA);
//               two S buffers in TMEM so that the product of tile j + 1 is issued while the
//               softmax of tile j runs;
//   O += P V    M = 128, N = 128 (two MMAs of N = 64), K = 64 keys.  P is written by the softmax
//               threads as a K-major bf16 operand; V is used as it lies in the cache
//               (keys x head dim, head dim contiguous) through an MN-major operand descriptor.
// Softmax: four warps, one thread per query row (tcgen05.ld gives a thread its row), so row
// maxima and sums need no shuffles; when a maximum moves, the row of O in TMEM is rescaled with
// tcgen05.ld / tcgen05.st.  TMEM use is 256 columns and shared memory 112 KB, so two CTAs share
// an SM and one CTA's tensor work overlaps the other's softmax.
//
// Warp roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2..5 softmax.
// Every wait is bounded; on expiry the CTA records a status code, stops issuing, waits for what
// is in flight, frees its TMEM and returns (its output rows are then not valid).
//
// Same operation as gqa_prefill_kernel (which stays for other head sizes, sliding windows and
// sinks); replaces npu_fused_infer_attention_score in its TND paged prefill form
// (omni_npu/attention/backends/attention.py:216-281).

#include <cstdlib>

#include "attn_params.cuh"
#include "../common/device_once.h"
#include "../common/pdl.cuh"
#include "../common/ptx.cuh"
#include "../common/tensormap.h"

namespace b200 {

namespace tcp {
constexpr int BM = 128;                 // query rows per CTA
constexpr int BN = 64;                  // keys per tile
constexpr int DV = 128;                 // value head size
constexpr int THREADS = 192;
constexpr int SLAB = BM * 128;          // 128 rows x 128 bytes
constexpr int KV_SLAB = BN * 128;       // 64 keys x 128 bytes
constexpr int P_BYTES = SLAB;           // 128 rows x 64 keys bf16
constexpr int STAGES = 2;
constexpr int NUM_BARS = 1 + 4 * STAGES + 2 * 2 + 3;   // q_full; k/v full+empty; s_full/s_empty[2]; p_full, o_done, drain
constexpr int TMEM_COLS = 256;          // S0 [0,64) S1 [64,128) O [128,256)
constexpr int COL_S = 0, COL_O = 128;

// DQK: query / key head size, 128 (GQA models) or 192 (non-absorbed latent attention: 128 nope + 64 rope)
template <int DQK>
struct Cfg {
  static constexpr int QK_SLABS = DQK / 64;
  static constexpr int Q_BYTES = QK_SLABS * SLAB;
  static constexpr int K_BYTES = QK_SLABS * KV_SLAB;
  static constexpr int V_BYTES = 2 * KV_SLAB;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + STAGES * K_BYTES;
  static constexpr int OFF_P = OFF_V + STAGES * V_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int SMEM = OFF_BAR + NUM_BARS * 8 + 16;
  static constexpr int CTAS_PER_SM = SMEM <= 115 * 1024 ? 2 : 1;
};
}  // namespace tcp

enum : int { kStatusPrefillTimeout = 41, kStatusPrefillSmemAlign = 42 };

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
        "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// K-major, 128-byte rows, 128B swizzle (what TMA writes): 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t smem_addr) {
  return make_smem_desc_sw128(smem_addr);
}
// MN-major, 128B swizzle: a "row" is one K index holding 64 MN elements (128 bytes); 8 K rows form a
// 1024-byte atom; the next 8 K rows follow at the stride byte offset (1024), the next 64 MN elements at
// the leading byte offset.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Launch bounds name 256 threads although 192 are launched: the register file is split over the
// four sub-partitions of an SM, and two CTAs of six warps put four warps on one of them, which only
// fits with at most 128 registers per thread (the bound a 256-thread, two-per-SM kernel gets).
template <int DQK>
__global__ void __launch_bounds__(256, tcp::Cfg<DQK>::CTAS_PER_SM)
gqa_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const AttnParams p, const int box_rows,
                      const int m_tiles) {
  using namespace tcp;
  using C = Cfg<DQK>;
  constexpr int OFF_Q = C::OFF_Q, OFF_K = C::OFF_K, OFF_V = C::OFF_V, OFF_P = C::OFF_P, OFF_BAR = C::OFF_BAR;
  constexpr int Q_BYTES = C::Q_BYTES, K_BYTES = C::K_BYTES, V_BYTES = C::V_BYTES, D = DV;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;              // [STAGES]
  uint64_t* k_empty = k_full + STAGES;
  uint64_t* v_full = k_empty + STAGES;
  uint64_t* v_empty = v_full + STAGES;
  uint64_t* s_full = v_empty + STAGES;      // [2]
  uint64_t* s_empty = s_full + 2;           // [2]
  uint64_t* p_full = s_empty + 2;
  uint64_t* o_done = p_full + 1;
  uint64_t* drain_bar = o_done + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  // heavy tiles (late query rows see the most keys) first
  const int mt = m_tiles - 1 - static_cast<int>(blockIdx.x);
  const int h = blockIdx.y;
  const int b = blockIdx.z;

  if ((smem_u32(smem) & 1023u) != 0u) {      // the operand layouts need 1024-byte aligned slabs
    if (tid == 0 && p.status) atomicCAS(p.status, 0, kStatusPrefillSmemAlign);
    return;
  }
  if (tid == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(o_done, 1);
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  {
    // key rows of a partly filled tile that no copy writes must hold finite values
    uint4* z = reinterpret_cast<uint4*>(smem + OFF_K);
    for (int i = tid; i < STAGES * (K_BYTES + V_BYTES) / 16; i += THREADS) z[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  fence_proxy_async();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  pdl_trigger();
  pdl_wait();          // q and the cache rows of this step come from earlier kernels

  const int q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_begin;
  const int m0 = mt * BM;
  const int kv_len = p.seq_lens[b];
  const int ctx = kv_len - q_len;
  const bool active = m0 < q_len;
  const int kvh = h / (p.Hq / p.Hk);
  // keys this tile can see: causal rows reach position ctx + m0 + BM - 1 at most
  const int kv_hi = p.causal ? min(kv_len, ctx + m0 + BM) : kv_len;
  const int n_tiles = active ? (kv_hi + BN - 1) / BN : 0;

  int issued = 0;          // tiles whose copies were started (producer lane only)
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && n_tiles > 0) {
      const int* bt = p.block_tables + static_cast<long long>(b) * p.max_blocks;
      mbar_arrive_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int sl = 0; sl < C::QK_SLABS; ++sl)
        tma_load_2d(smem + OFF_Q + sl * SLAB, &tm_q, q_full, h * DQK + sl * 64, q_begin + m0);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % STAGES;
        if (j >= STAGES) {
          const uint32_t par = static_cast<uint32_t>(((j / STAGES) - 1) & 1);
          if (*abort_flag || !mbar_wait(&k_empty[st], par) || !mbar_wait(&v_empty[st], par)) {
            if (!*abort_flag && p.status) atomicCAS(p.status, 0, kStatusPrefillTimeout);
            *abort_flag = 1;
            break;
          }
        }
        const int n0 = j * BN;
        const int nvalid = min(BN, kv_len - n0);
        const int nboxes = (nvalid + box_rows - 1) / box_rows;
        const uint32_t box_bytes = static_cast<uint32_t>(nboxes * box_rows * 128);
        mbar_arrive_expect_tx(&k_full[st], box_bytes * C::QK_SLABS);
        mbar_arrive_expect_tx(&v_full[st], box_bytes * 2);
        for (int i = 0; i < nboxes; ++i) {
          const int key = n0 + i * box_rows;
          const int blk = bt[key / p.block_size];
          const int row = (blk * p.Hk + kvh) * p.block_size + key % p.block_size;
#pragma unroll
          for (int sl = 0; sl < C::QK_SLABS; ++sl)
            tma_load_2d(smem + OFF_K + st * K_BYTES + sl * KV_SLAB + i * box_rows * 128, &tm_k, &k_full[st],
                        sl * 64, row);
#pragma unroll
          for (int sl = 0; sl < 2; ++sl)
            tma_load_2d(smem + OFF_V + st * V_BYTES + sl * KV_SLAB + i * box_rows * 128, &tm_v, &v_full[st],
                        sl * 64, row);
        }
        issued = j + 1;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_tiles > 0) {
      const uint32_t idesc_s = make_idesc(1, 1, BM, BN);                       // K-major A and B
      const uint32_t idesc_o = make_idesc(1, 1, BM, 64) | (1u << 16);          // B (V) MN-major
      const uint32_t q_addr = smem_u32(smem + OFF_Q);
      const uint32_t p_addr = smem_u32(smem + OFF_P);
      bool ok = mbar_wait(q_full, 0);
      auto issue_pv = [&](int j) -> bool {
        const int st = j % STAGES;
        if (!mbar_wait(p_full, static_cast<uint32_t>(j & 1)) ||
            !mbar_wait(&v_full[st], static_cast<uint32_t>((j / STAGES) & 1)))
          return false;
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(smem + OFF_V + st * V_BYTES);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {
            // A: P rows, 16 keys = 32 bytes along the swizzled row; B: 16 keys = 16 rows of 128 bytes
            umma_f16(tmem_base + COL_O + half * 64, desc_kmajor(p_addr + kk * 32),
                     desc_mnmajor(v_addr + half * KV_SLAB + kk * 16 * 128, KV_SLAB), idesc_o,
                     (j > 0 || kk > 0) ? 1u : 0u);
          }
        }
        tc_commit(o_done);
        tc_commit(&v_empty[st]);
        return true;
      };
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int st = j % STAGES;
        const int sb = j & 1;
        ok = !*abort_flag && mbar_wait(&k_full[st], static_cast<uint32_t>((j / STAGES) & 1));
        if (ok && j >= 2) ok = mbar_wait(&s_empty[sb], static_cast<uint32_t>(((j >> 1) - 1) & 1));
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(smem + OFF_K + st * K_BYTES);
#pragma unroll
        for (int kk = 0; kk < DQK / 16; ++kk) {
          const int slab = kk >> 2, off = (kk & 3) * 32;
          umma_f16(tmem_base + COL_S + sb * BN, desc_kmajor(q_addr + slab * SLAB + off),
                   desc_kmajor(k_addr + slab * KV_SLAB + off), idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[sb]);
        tc_commit(&k_empty[st]);
        if (j >= 1) ok = issue_pv(j - 1);
      }
      if (ok) ok = issue_pv(n_tiles - 1);
      if (!ok) {
        if (!*abort_flag && p.status) atomicCAS(p.status, 0, kStatusPrefillTimeout);
        *abort_flag = 1;
      }
    }
  } else if (n_tiles > 0) {
    // ------------------------------------------------------------ softmax (one thread per row)
    const int quarter = warp & 3;                         // TMEM lanes this warp may touch
    const int r = quarter * 32 + lane;                    // row within the tile
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const int q_pos = ctx + m0 + r;                       // position of this row's token
    const bool row_valid = m0 + r < q_len;
    float row_max = -INFINITY, row_sum = 0.f;
    uint8_t* p_row = smem + OFF_P + r * 128;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      ok = !*abort_flag && mbar_wait(&s_full[sb], static_cast<uint32_t>((j >> 1) & 1));
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t sv[2][32];
      tmem_ld_32x32b_x32(tmem_base + lane_base + COL_S + sb * BN, sv[0]);
      tmem_ld_32x32b_x32(tmem_base + lane_base + COL_S + sb * BN + 32, sv[1]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);
      const int n0 = j * BN;
      float tile_max = -INFINITY;
      float s[64];
      // tiles that lie entirely below the diagonal and inside the sequence need no mask
      const int row_lo = ctx + m0 + quarter * 32;                      // smallest position in this warp
      const bool interior = n0 + BN <= kv_len && (!p.causal || n0 + BN - 1 <= row_lo);
      if (interior) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const float v = __uint_as_float(sv[c >> 5][c & 31]) * p.scale_log2;
          s[c] = v;
          tile_max = fmaxf(tile_max, v);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int key = n0 + c;
          const bool keep = key < kv_len && (!p.causal || key <= q_pos);
          const float v = keep ? __uint_as_float(sv[c >> 5][c & 31]) * p.scale_log2 : -INFINITY;
          s[c] = v;
          tile_max = fmaxf(tile_max, v);
        }
      }
      // The reference maximum only moves when the tile's maximum exceeds it by more than 2^8: P then
      // stays below 256 (exact in bf16 relative terms, far from fp32 overflow in the sums), the
      // result is the same after the final division, and the costly rescale of O in tensor memory
      // becomes rare instead of happening on most early tiles.
      float new_max = row_max;
      if (tile_max > row_max + 8.f || row_max == -INFINITY) new_max = fmaxf(row_max, tile_max);
      const float corr = (new_max == -INFINITY || row_max == new_max) ? 1.f : exp2f(row_max - new_max);
      const float m_use = new_max == -INFINITY ? 0.f : new_max;
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        s[c] = exp2f(s[c] - m_use);
        sum += s[c];
      }
      row_sum = row_sum * corr + sum;
      row_max = new_max;
      if (j >= 1) {
        // P of tile j - 1 has been consumed and O is at rest once its product has completed
        ok = !*abort_flag && mbar_wait(o_done, static_cast<uint32_t>((j - 1) & 1));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t ov[32];
            tmem_ld_32x32b_x32(tmem_base + lane_base + COL_O + c * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
            tmem_st_32x32b_x32(tmem_base + lane_base + COL_O + c * 32, ov);
          }
          tmem_st_wait();
        }
      }
      // P as a K-major bf16 operand: 8 chunks of 16 bytes per row, chunk c at position c ^ (row & 7)
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 v;
        v.x = pack_bf16x2(s[c * 8 + 0], s[c * 8 + 1]);
        v.y = pack_bf16x2(s[c * 8 + 2], s[c * 8 + 3]);
        v.z = pack_bf16x2(s[c * 8 + 4], s[c * 8 + 5]);
        v.w = pack_bf16x2(s[c * 8 + 6], s[c * 8 + 7]);
        *reinterpret_cast<uint4*>(p_row + ((c ^ (r & 7)) << 4)) = v;
      }
      fence_proxy_async();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok) {
      ok = !*abort_flag && mbar_wait(o_done, static_cast<uint32_t>((n_tiles - 1) & 1));
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after_sync();
      const float inv = row_sum > 0.f ? 1.f / row_sum : 0.f;
      __nv_bfloat16* dst = p.out + static_cast<long long>(q_begin + m0 + r) * p.out_stride +
                           static_cast<long long>(h) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t ov[32];
        tmem_ld_32x32b_x32(tmem_base + lane_base + COL_O + c * 32, ov);
        tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(ov[i * 8 + 0]) * inv, __uint_as_float(ov[i * 8 + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(ov[i * 8 + 2]) * inv, __uint_as_float(ov[i * 8 + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(ov[i * 8 + 4]) * inv, __uint_as_float(ov[i * 8 + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(ov[i * 8 + 6]) * inv, __uint_as_float(ov[i * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = v;
          }
        }
      }
      if (p.lse && row_valid)
        p.lse[static_cast<long long>(q_begin + m0 + r) * p.Hq + h] =
            row_sum > 0.f ? (row_max + log2f(row_sum)) / kLog2e : -INFINITY;
    } else if (lane == 0) {
      if (!*abort_flag && p.status) atomicCAS(p.status, 0, kStatusPrefillTimeout);
      *abort_flag = 1;
    }
  }

  // ---- teardown: nothing may still be writing shared or tensor memory when the CTA leaves
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag && warp == 0 && lane == 0) {
    // copies still in flight land in this CTA's shared memory: wait (bounded) for the last tiles issued
    if (n_tiles > 0) mbar_wait(q_full, 0);
    for (int j = issued > tcp::STAGES ? issued - tcp::STAGES : 0; j < issued; ++j) {
      mbar_wait(&k_full[j % tcp::STAGES], static_cast<uint32_t>((j / tcp::STAGES) & 1));
      mbar_wait(&v_full[j % tcp::STAGES], static_cast<uint32_t>((j / tcp::STAGES) & 1));
    }
  }
  if (warp == 1) {
    if (*abort_flag && lane == 0) {
      // products still in flight write tensor memory: wait (bounded) for them before it is freed
      tc_commit(drain_bar);
      mbar_wait(drain_bar, 0);
    }
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, tcp::TMEM_COLS);
  }
}

}  // namespace b200

using namespace b200;

// CTAs of the kernel that fit one SM (2 for head size 128: 112 KB of shared memory, 256 TMEM columns each).
// smem_bytes = 0: the kernel's own size; another value asks what a CTA of that size would get.
extern "C" int b200_gqa_prefill_tc_ctas_per_sm(int smem_bytes) {
  int n = 0;
  auto kern = gqa_prefill_tc_kernel<128>;
  if (smem_bytes <= 0) smem_bytes = tcp::Cfg<128>::SMEM;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tcp::Cfg<128>::SMEM);
  cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, tcp::THREADS, smem_bytes) != cudaSuccess) return -1;
  return n;
}

// What the occupancy figure is made of: out[0..7] = registers per thread, static shared bytes, max dynamic
// shared bytes, shared memory per SM, registers per SM, reserved shared bytes per block, max blocks per SM,
// local (spill) bytes per thread.
extern "C" int b200_gqa_prefill_tc_resources(int* out) {
  cudaFuncAttributes fa{};
  if (cudaFuncGetAttributes(&fa, gqa_prefill_tc_kernel<128>) != cudaSuccess) return -1;
  int dev = 0, v = 0;
  cudaGetDevice(&dev);
  out[0] = fa.numRegs;
  out[1] = static_cast<int>(fa.sharedSizeBytes);
  out[2] = fa.maxDynamicSharedSizeBytes;
  cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
  out[3] = v;
  cudaDeviceGetAttribute(&v, cudaDevAttrMaxRegistersPerMultiprocessor, dev);
  out[4] = v;
  cudaDeviceGetAttribute(&v, cudaDevAttrReservedSharedMemoryPerBlock, dev);
  out[5] = v;
  cudaDeviceGetAttribute(&v, cudaDevAttrMaxBlocksPerMultiprocessor, dev);
  out[6] = v;
  out[7] = static_cast<int>(fa.localSizeBytes);
  return 0;
}

template <int DQK>
static int launch_prefill_tc(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p,
                             int box_rows, dim3 grid, cudaStream_t stream) {
  auto kern = gqa_prefill_tc_kernel<DQK>;
  static DeviceOnce once;
  int dev = 0;
  if (once.needed(&dev)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tcp::Cfg<DQK>::SMEM) != cudaSuccess)
      return -20;
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    once.mark(dev);
  }
  return launch_pdl(kern, grid, dim3(tcp::THREADS), tcp::Cfg<DQK>::SMEM, stream, 1, tq, tk, tv, p, box_rows,
                    static_cast<int>(grid.x)) == cudaSuccess
             ? 0
             : -21;
}

// Returns 0 when the kernel ran, 1 when the problem is not one it takes (caller falls back), < 0 on error.
// Takes query / key head sizes 128 and 192 with value head size 128, no sliding window.
extern "C" int b200_gqa_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out, float* lse,
                                   const int* block_tables, const int* cu_q, const int* seq_lens, int B,
                                   int max_q_len, int max_blocks, int block_size, int Hq, int Hk, int Dqk, int Dv,
                                   long long q_stride, long long out_stride, float scale, int causal, int window,
                                   long long total_q_rows, int num_cache_blocks, int* status, cudaStream_t stream) {
  if ((Dqk != 128 && Dqk != 192) || Dv != 128 || window != 0 || Hq % Hk != 0) return 1;
  const bool tma_ok = (block_size % 8) == 0 && (block_size <= 64 ? (64 % block_size) == 0 : (block_size % 64) == 0) &&
                      (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(q) & 15) == 0 && ((q_stride * 2) & 15) == 0 &&
                      ((out_stride * 2) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  if (!tma_ok || num_cache_blocks <= 0 || total_q_rows <= 0) return 1;
  if (B <= 0 || max_q_len <= 0) return 0;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.block_tables = block_tables;
  p.cu_q = cu_q;
  p.seq_lens = seq_lens;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  p.Hq = Hq;
  p.Hk = Hk;
  p.q_stride = q_stride;
  p.out_stride = out_stride;
  p.scale_log2 = scale * kLog2e;
  p.causal = causal;
  p.status = status;
  p.num_cache_blocks = num_cache_blocks;
  const int box_rows = block_size < 64 ? block_size : 64;
  CUtensorMap tq, tk, tv;
  int r = make_tensormap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, static_cast<uint64_t>(total_q_rows),
                            static_cast<uint64_t>(Hq) * Dqk, static_cast<uint64_t>(q_stride), tcp::BM, 64,
                            CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 1000;
  const uint64_t rows = static_cast<uint64_t>(num_cache_blocks) * Hk * block_size;
  r = make_tensormap_2d(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k_cache, rows, Dqk, Dqk, box_rows, 64,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 2000;
  r = make_tensormap_2d(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v_cache, rows, 128, 128, box_rows, 64,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 3000;
  const int m_tiles = (max_q_len + tcp::BM - 1) / tcp::BM;
  dim3 grid(m_tiles, Hq, B);
  return Dqk == 128 ? launch_prefill_tc<128>(tq, tk, tv, p, box_rows, grid, stream)
                    : launch_prefill_tc<192>(tq, tk, tv, p, box_rows, grid, stream);
}
