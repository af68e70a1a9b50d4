// Paged grouped-query attention: variable-length causal prefill (with cached
// context, so chunked prefill and prefix reuse work) and split-KV decode.
//
// K/V are read straight out of the paged cache
//   k_cache [num_blocks, kv_heads, block_size, DQK],  v_cache [.., DV]
// with 16-byte cp.async copies into swizzled shared-memory tiles, double /
// triple buffered.  The matrix products run on mma.sync m16n8k16 (bf16 in,
// fp32 accumulate); softmax is the usual online form in base 2.
//
// Prefill: one CTA = 128 query rows of one (sequence, q head); 8 warps x 16 rows.
// Decode:  one CTA = one (sequence, kv head, kv split); the q heads of the group
//          (times the query length for multi-token decode) form the 16 MMA rows;
//          4 warps take 16 keys each of every 64-key tile and merge at the end.
//          With more than one split the partial outputs and log-sum-exps go to
//          fp32 scratch and a small kernel merges them.
//
// Replaces npu_fused_infer_attention_score in its TND paged form
// (omni_npu/attention/backends/attention.py:216-281).

#include <cstdlib>

#include "attn_common.cuh"
#include "attn_params.cuh"
#include "../common/pdl.cuh"
#include "../common/tensormap.h"
#include "../common/device_once.h"

namespace b200 {


// ------------------------------------------------------------------ prefill
template <int DQK, int DV>
struct PrefillCfg {
  static constexpr int BM = 128;
  static constexpr int BN = 64;
  static constexpr int THREADS = 256;
  static constexpr int Q_BYTES = BM * DQK * 2;
  static constexpr int K_BYTES = BN * DQK * 2;
  static constexpr int V_BYTES = BN * DV * 2;
  static constexpr int SMEM = Q_BYTES + 2 * K_BYTES + 2 * V_BYTES;
};


template <int ROW_ELEMS, int ROWS, int THREADS>
__device__ __forceinline__ void load_kv_tile(uint8_t* smem_tile, const __nv_bfloat16* cache,
                                             const int* block_table, int n0, int kv_len, int kvh,
                                             int Hk, int block_size, int tid) {
  constexpr int CHUNKS = ROW_ELEMS / 8;
  constexpr int TOTAL = ROWS * CHUNKS;
  constexpr int PER_THREAD = TOTAL / THREADS;
  static_assert(TOTAL % THREADS == 0, "tile must divide evenly");
  constexpr int THREADS_PER_ROW = CHUNKS / PER_THREAD;
  static_assert(CHUNKS % PER_THREAD == 0, "row must divide evenly");
  const int row = tid / THREADS_PER_ROW;
  const int c0 = (tid % THREADS_PER_ROW) * PER_THREAD;
  const int key = n0 + row;
  const bool valid = key < kv_len;
  const __nv_bfloat16* src = cache;
  if (valid) {
    const int blk = block_table[key / block_size];
    const int off = key % block_size;
    src = cache + ((static_cast<long long>(blk) * Hk + kvh) * block_size + off) * ROW_ELEMS;
  }
  const uint32_t base = smem_u32(smem_tile);
#pragma unroll
  for (int i = 0; i < PER_THREAD; ++i) {
    const int c = c0 + i;
    const uint32_t dst = base + tile_offset<ROW_ELEMS>(row, c);
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src + c * 8),
                 "r"(sz)
                 : "memory");
  }
}

template <int DQK, int DV>
__global__ void __launch_bounds__(256, 1) gqa_prefill_kernel(const AttnParams p) {
  using Cfg = PrefillCfg<DQK, DV>;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = smem + Cfg::Q_BYTES;
  uint8_t* sV = sK + 2 * Cfg::K_BYTES;

  const int b = blockIdx.z;
  const int h = blockIdx.y;
  const int q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_begin;
  const int m0 = blockIdx.x * Cfg::BM;
  if (m0 >= q_len) return;
  const int kv_len = p.seq_lens[b];
  const int ctx = kv_len - q_len;  // tokens already cached before this step's queries
  const int kvh = h / (p.Hq / p.Hk);
  const int* bt = p.block_tables + static_cast<long long>(b) * p.max_blocks;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---- Q tile -> shared (rows beyond q_len are zero filled)
  {
    constexpr int CHUNKS = DQK / 8;
    for (int idx = tid; idx < Cfg::BM * CHUNKS; idx += Cfg::THREADS) {
      const int row = idx / CHUNKS, c = idx % CHUNKS;
      const bool valid = (m0 + row) < q_len;
      const __nv_bfloat16* src =
          p.q + (valid ? (static_cast<long long>(q_begin + m0 + row) * p.q_stride +
                          static_cast<long long>(h) * DQK + c * 8)
                       : 0);
      const uint32_t dst = smem_u32(sQ) + tile_offset<DQK>(row, c);
      const int sz = valid ? 16 : 0;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz)
                   : "memory");
    }
  }
  // Last key any row of this tile may see.
  const int last_row = min(q_len, m0 + Cfg::BM) - 1;
  const int kv_end = p.causal ? min(kv_len, ctx + last_row + 1) : kv_len;
  int kv_start = 0;
  // (with sink tokens the leading tiles must stay: no skipping then)
  if (p.window > 0 && p.sink == 0) kv_start = max(0, ctx + m0 - p.window + 1) / Cfg::BN * Cfg::BN;
  const int n_tiles = (kv_end - kv_start + Cfg::BN - 1) / Cfg::BN;

  load_kv_tile<DQK, Cfg::BN, Cfg::THREADS>(sK, p.k_cache, bt, kv_start, kv_end, kvh, p.Hk,
                                            p.block_size, tid);
  load_kv_tile<DV, Cfg::BN, Cfg::THREADS>(sV, p.v_cache, bt, kv_start, kv_end, kvh, p.Hk,
                                           p.block_size, tid);
  cp_async_commit();

  float o_acc[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY};
  float row_sum[2] = {0.f, 0.f};
  uint32_t q_frag[DQK / 16][4];

  const int row_a = warp * 16 + (lane >> 2);  // tile-local rows of this thread: row_a, row_a + 8
  const int pos_a = ctx + m0 + row_a;         // absolute position of row_a

  for (int it = 0; it < n_tiles; ++it) {
    const int stage = it & 1;
    if (it + 1 < n_tiles) {
      const int n_next = kv_start + (it + 1) * Cfg::BN;
      load_kv_tile<DQK, Cfg::BN, Cfg::THREADS>(sK + (stage ^ 1) * Cfg::K_BYTES, p.k_cache, bt,
                                                n_next, kv_end, kvh, p.Hk, p.block_size, tid);
      load_kv_tile<DV, Cfg::BN, Cfg::THREADS>(sV + (stage ^ 1) * Cfg::V_BYTES, p.v_cache, bt,
                                               n_next, kv_end, kvh, p.Hk, p.block_size, tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int ks = 0; ks < DQK / 16; ++ks) {
        const uint32_t addr =
            smem_u32(sQ) + tile_offset<DQK>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4));
        ldmatrix_x4(q_frag[ks], addr);
      }
    }
    const uint8_t* kt = sK + stage * Cfg::K_BYTES;
    const uint8_t* vt = sV + stage * Cfg::V_BYTES;
    const int n0 = kv_start + it * Cfg::BN;

    // S = Q K^T : 16 rows x 64 keys per warp
    float s[Cfg::BN / 8][4];
#pragma unroll
    for (int i = 0; i < Cfg::BN / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < DQK / 16; ++ks) {
#pragma unroll
      for (int nt = 0; nt < Cfg::BN / 16; ++nt) {
        uint32_t kf[4];
        const int krow = nt * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int kchunk = ks * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(kf, smem_u32(kt) + tile_offset<DQK>(krow, kchunk));
        mma_bf16_16816(s[2 * nt], q_frag[ks], kf[0], kf[1]);
        mma_bf16_16816(s[2 * nt + 1], q_frag[ks], kf[2], kf[3]);
      }
    }
    // mask + online softmax
    const bool need_mask = (n0 + Cfg::BN > kv_end) ||
                           (p.causal && (n0 + Cfg::BN - 1 > ctx + m0 + warp * 16)) ||
                           (p.window > 0);
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < Cfg::BN / 8; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = s[i][j] * p.scale_log2;
        if (need_mask) {
          const int key = n0 + i * 8 + (lane & 3) * 2 + (j & 1);
          const int pos = pos_a + ((j >> 1) << 3);
          bool ok = key < kv_end;
          if (p.causal) ok = ok && key <= pos;
          if (p.window > 0) ok = ok && (key > pos - p.window || key < p.sink);
          if (!ok) v = -INFINITY;
        }
        s[i][j] = v;
        tile_max[j >> 1] = fmaxf(tile_max[j >> 1], v);
      }
    }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float tm = quad_max(tile_max[r]);
      const float new_max = fmaxf(row_max[r], tm);
      corr[r] = (new_max == -INFINITY) ? 1.f : exp2f(row_max[r] - new_max);
      row_max[r] = new_max;
      row_sum[r] *= corr[r];
    }
    const float m_use[2] = {row_max[0] == -INFINITY ? 0.f : row_max[0],
                            row_max[1] == -INFINITY ? 0.f : row_max[1]};
#pragma unroll
    for (int i = 0; i < Cfg::BN / 8; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float e = exp2f(s[i][j] - m_use[j >> 1]);
        s[i][j] = e;
        row_sum[j >> 1] += e;
      }
    }
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
      o_acc[i][0] *= corr[0];
      o_acc[i][1] *= corr[0];
      o_acc[i][2] *= corr[1];
      o_acc[i][3] *= corr[1];
    }
    // O += P V
#pragma unroll
    for (int ks = 0; ks < Cfg::BN / 16; ++ks) {
      uint32_t pa[4];
      pa[0] = pack_bf16x2(s[2 * ks][0], s[2 * ks][1]);
      pa[1] = pack_bf16x2(s[2 * ks][2], s[2 * ks][3]);
      pa[2] = pack_bf16x2(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      pa[3] = pack_bf16x2(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
      for (int dt = 0; dt < DV / 16; ++dt) {
        uint32_t vf[4];
        const int vrow = ks * 16 + (lane & 15);
        const int vchunk = dt * 2 + (lane >> 4);
        ldmatrix_x4_trans(vf, smem_u32(vt) + tile_offset<DV>(vrow, vchunk));
        mma_bf16_16816(o_acc[2 * dt], pa, vf[0], vf[1]);
        mma_bf16_16816(o_acc[2 * dt + 1], pa, vf[2], vf[3]);
      }
    }
    __syncthreads();
  }

  cp_async_wait<0>();
  __syncthreads();
  // ---- finalise: O / l, stage through the Q tile, 16-byte stores
  float inv[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    row_sum[r] = quad_sum(row_sum[r]);
    inv[r] = row_sum[r] > 0.f ? 1.f / row_sum[r] : 0.f;
  }
  static_assert(DV <= DQK, "output staging reuses the Q tile");
#pragma unroll
  for (int i = 0; i < DV / 8; ++i) {
    const int col = i * 8 + (lane & 3) * 2;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = warp * 16 + (lane >> 2) + r * 8;
      const uint32_t v = pack_bf16x2(o_acc[i][2 * r] * inv[r], o_acc[i][2 * r + 1] * inv[r]);
      uint8_t* dst = sQ + tile_offset<DQK>(row, col >> 3) + (col & 7) * 2;
      *reinterpret_cast<uint32_t*>(dst) = v;
    }
  }
  if (p.lse && (lane & 3) == 0) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = m0 + warp * 16 + (lane >> 2) + r * 8;
      if (row < q_len) {
        const float l = row_sum[r] > 0.f ? (row_max[r] + log2f(row_sum[r])) / kLog2e : -INFINITY;
        p.lse[static_cast<long long>(q_begin + row) * p.Hq + h] = l;
      }
    }
  }
  __syncwarp();
  {
    constexpr int CHUNKS = DV / 8;
    // Each warp stores the 16 rows it owns.
    for (int idx = lane; idx < 16 * CHUNKS; idx += 32) {
      const int r = idx / CHUNKS, c = idx % CHUNKS;
      const int row = warp * 16 + r;
      if (m0 + row < q_len) {
        const uint4 v = *reinterpret_cast<const uint4*>(sQ + tile_offset<DQK>(row, c));
        *reinterpret_cast<uint4*>(p.out + static_cast<long long>(q_begin + m0 + row) * p.out_stride +
                                  static_cast<long long>(h) * DV + c * 8) = v;
      }
    }
  }
}

// ------------------------------------------------------------------- decode
template <int D>
struct DecodeCfg {
  static constexpr int BN = 64;
  static constexpr int STAGES = 3;
  static constexpr int THREADS = 128;
  static constexpr int Q_BYTES = 16 * D * 2;
  static constexpr int KV_BYTES = BN * D * 2;
  static constexpr int SMEM = Q_BYTES + 2 * STAGES * KV_BYTES;
};

template <int D>
__global__ void __launch_bounds__(128) gqa_decode_kernel(const AttnParams p) {
  using Cfg = DecodeCfg<D>;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = smem + Cfg::Q_BYTES;
  uint8_t* sV = sK + Cfg::STAGES * Cfg::KV_BYTES;

  const int b = blockIdx.x;
  const int kvh = blockIdx.y;
  const int split = blockIdx.z;
  const int G = p.Hq / p.Hk;
  const int rows = G * p.q_len;  // <= 16
  const int kv_len = p.seq_lens[b];
  const int* bt = p.block_tables + static_cast<long long>(b) * p.max_blocks;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  const int n_tiles_all = (kv_len + Cfg::BN - 1) / Cfg::BN;
  const int per = (n_tiles_all + p.splits - 1) / p.splits;
  const int t_begin = split * per;
  const int t_end = min(n_tiles_all, t_begin + per);
  const int n_tiles = max(0, t_end - t_begin);

  // Row r of the MMA tile = (query token r / G, q head kvh*G + r % G).
  {
    constexpr int CHUNKS = D / 8;
    for (int idx = tid; idx < 16 * CHUNKS; idx += Cfg::THREADS) {
      const int row = idx / CHUNKS, c = idx % CHUNKS;
      const bool valid = row < rows;
      const int qi = row / G, hh = kvh * G + row % G;
      const __nv_bfloat16* src =
          p.q + (valid ? (static_cast<long long>(b * p.q_len + qi) * p.q_stride +
                          static_cast<long long>(hh) * D + c * 8)
                       : 0);
      const uint32_t dst = smem_u32(sQ) + tile_offset<D>(row, c);
      const int sz = valid ? 16 : 0;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz)
                   : "memory");
    }
  }
#pragma unroll
  for (int s = 0; s < Cfg::STAGES - 1; ++s) {
    if (s < n_tiles) {
      const int n0 = (t_begin + s) * Cfg::BN;
      load_kv_tile<D, Cfg::BN, Cfg::THREADS>(sK + s * Cfg::KV_BYTES, p.k_cache, bt, n0, kv_len, kvh,
                                              p.Hk, p.block_size, tid);
      load_kv_tile<D, Cfg::BN, Cfg::THREADS>(sV + s * Cfg::KV_BYTES, p.v_cache, bt, n0, kv_len, kvh,
                                              p.Hk, p.block_size, tid);
    }
    cp_async_commit();
  }

  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY};
  float row_sum[2] = {0.f, 0.f};
  uint32_t q_frag[D / 16][4];

  const int r_a = lane >> 2;  // rows r_a and r_a + 8
  int pos_r[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r_a + 8 * r;
    pos_r[r] = kv_len - p.q_len + row / G;  // causal limit for this row's query token
  }

  for (int it = 0; it < n_tiles; ++it) {
    const int stage = it % Cfg::STAGES;
    {
      const int nxt = it + Cfg::STAGES - 1;
      if (nxt < n_tiles) {
        const int ns = nxt % Cfg::STAGES;
        const int n0 = (t_begin + nxt) * Cfg::BN;
        load_kv_tile<D, Cfg::BN, Cfg::THREADS>(sK + ns * Cfg::KV_BYTES, p.k_cache, bt, n0, kv_len,
                                                kvh, p.Hk, p.block_size, tid);
        load_kv_tile<D, Cfg::BN, Cfg::THREADS>(sV + ns * Cfg::KV_BYTES, p.v_cache, bt, n0, kv_len,
                                                kvh, p.Hk, p.block_size, tid);
      }
      cp_async_commit();
    }
    cp_async_wait<Cfg::STAGES - 1>();
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        ldmatrix_x4(q_frag[ks], smem_u32(sQ) + tile_offset<D>(lane & 15, ks * 2 + (lane >> 4)));
    }
    const uint8_t* kt = sK + stage * Cfg::KV_BYTES;
    const uint8_t* vt = sV + stage * Cfg::KV_BYTES;
    const int n0 = (t_begin + it) * Cfg::BN + warp * 16;  // this warp's 16 keys

    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t kf[4];
      const int krow = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int kchunk = ks * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(kf, smem_u32(kt) + tile_offset<D>(krow, kchunk));
      mma_bf16_16816(s[0], q_frag[ks], kf[0], kf[1]);
      mma_bf16_16816(s[1], q_frag[ks], kf[2], kf[3]);
    }
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = n0 + i * 8 + (lane & 3) * 2 + (j & 1);
        const int pos = pos_r[j >> 1];
        bool ok = key <= pos && key < kv_len;
        if (p.window > 0) ok = ok && (key > pos - p.window || key < p.sink);
        const float v = ok ? s[i][j] * p.scale_log2 : -INFINITY;
        s[i][j] = v;
        tile_max[j >> 1] = fmaxf(tile_max[j >> 1], v);
      }
    }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float tm = quad_max(tile_max[r]);
      const float new_max = fmaxf(row_max[r], tm);
      corr[r] = (new_max == -INFINITY) ? 1.f : exp2f(row_max[r] - new_max);
      row_max[r] = new_max;
      row_sum[r] *= corr[r];
    }
    const float m_use[2] = {row_max[0] == -INFINITY ? 0.f : row_max[0],
                            row_max[1] == -INFINITY ? 0.f : row_max[1]};
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float e = exp2f(s[i][j] - m_use[j >> 1]);
        s[i][j] = e;
        row_sum[j >> 1] += e;
      }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o_acc[i][0] *= corr[0];
      o_acc[i][1] *= corr[0];
      o_acc[i][2] *= corr[1];
      o_acc[i][3] *= corr[1];
    }
    uint32_t pa[4];
    pa[0] = pack_bf16x2(s[0][0], s[0][1]);
    pa[1] = pack_bf16x2(s[0][2], s[0][3]);
    pa[2] = pack_bf16x2(s[1][0], s[1][1]);
    pa[3] = pack_bf16x2(s[1][2], s[1][3]);
#pragma unroll
    for (int dt = 0; dt < D / 16; ++dt) {
      uint32_t vf[4];
      const int vrow = warp * 16 + (lane & 15);
      const int vchunk = dt * 2 + (lane >> 4);
      ldmatrix_x4_trans(vf, smem_u32(vt) + tile_offset<D>(vrow, vchunk));
      mma_bf16_16816(o_acc[2 * dt], pa, vf[0], vf[1]);
      mma_bf16_16816(o_acc[2 * dt + 1], pa, vf[2], vf[3]);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the four warps' partial results through shared memory
  float* m_buf = reinterpret_cast<float*>(sK);          // [4][16]
  float* l_buf = m_buf + 64;                            // [4][16]
  float* o_buf = l_buf + 64;                            // [4][16][D]
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    row_sum[r] = quad_sum(row_sum[r]);
    if ((lane & 3) == 0) {
      m_buf[warp * 16 + r_a + 8 * r] = row_max[r];
      l_buf[warp * 16 + r_a + 8 * r] = row_sum[r];
    }
  }
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    const int col = i * 8 + (lane & 3) * 2;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float* dst = o_buf + (static_cast<size_t>(warp) * 16 + r_a + 8 * r) * D + col;
      dst[0] = o_acc[i][2 * r];
      dst[1] = o_acc[i][2 * r + 1];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < rows * (D / 4); idx += Cfg::THREADS) {
    const int row = idx / (D / 4);
    const int c4 = (idx % (D / 4)) * 4;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, m_buf[w * 16 + row]);
    float l = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = m_buf[w * 16 + row];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
      l += l_buf[w * 16 + row] * f;
      const float4 x = *reinterpret_cast<const float4*>(o_buf + (static_cast<size_t>(w) * 16 + row) * D + c4);
      acc.x += x.x * f;
      acc.y += x.y * f;
      acc.z += x.z * f;
      acc.w += x.w * f;
    }
    const int qi = row / G, hh = kvh * G + row % G;
    if (p.splits == 1) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      uint2 pk;
      pk.x = pack_bf16x2(acc.x * inv, acc.y * inv);
      pk.y = pack_bf16x2(acc.z * inv, acc.w * inv);
      *reinterpret_cast<uint2*>(p.out + static_cast<long long>(b * p.q_len + qi) * p.out_stride +
                                static_cast<long long>(hh) * D + c4) = pk;
      if (p.lse && c4 == 0)
        p.lse[static_cast<long long>(b * p.q_len + qi) * p.Hq + hh] =
            l > 0.f ? (m + log2f(l)) / kLog2e : -INFINITY;
    } else {
      // partial: unnormalised numerator, base-2 max and sum
      const size_t pr = ((static_cast<size_t>(b) * p.Hk + kvh) * p.splits + split) * 16 + row;
      *reinterpret_cast<float4*>(p.o_part + pr * D + c4) = acc;
      if (c4 == 0) {
        p.lse_part[pr * 2] = m;
        p.lse_part[pr * 2 + 1] = l;
      }
    }
  }
}


// ------------------------------------------------------- decode, TMA-fed
// Same computation as gqa_decode_kernel, but the K/V tiles are brought in by
// the TMA engine (cp.async.bulk.tensor, 128B swizzle) instead of per-thread
// cp.async: a handful of bulk copies per tile keep far more bytes in flight
// per SM than the load/store unit allows, which is what a bandwidth-bound
// decode needs.  The cache is addressed as a 2-D tensor
// [num_blocks * kv_heads * block_size rows, D columns]; a box is
// (box_rows = min(block_size, 64)) rows x 64 columns (128 bytes).
template <int D, int NSTAGES = 3>
struct DecodeTmaCfg {
  static constexpr int BN = 64;
  static constexpr int STAGES = NSTAGES;
  static constexpr int COMPUTE_THREADS = 128;
  static constexpr int THREADS = 160;          // 4 compute warps + 1 producer warp
  static constexpr int HALVES = D / 64;
  static constexpr int HALF_BYTES = BN * 128;
  static constexpr int KV_BYTES = HALVES * HALF_BYTES;
  static constexpr int Q_BYTES = 16 * D * 2;
  static constexpr int BT_ENTRIES = 1024;      // block-table slice cached in shared memory
  static constexpr int SMEM = 1024 + 2 * STAGES * KV_BYTES + Q_BYTES + BT_ENTRIES * 4 + 128;
};

template <int D>
__device__ __forceinline__ uint32_t kv_swz(int key, int chunk) {
  return static_cast<uint32_t>((chunk >> 3) * (64 * 128) + key * 128 + (((chunk & 7) ^ (key & 7)) << 4));
}

// Build with -DB200_ATTN_TIMELINE to record, per CTA of the TMA decode kernel, the global timer at
// six points (entry, set-up done, first tile landed, last tile consumed, merged and stored, and the
// SM id); read back with b200_gqa_decode_timeline().
#ifdef B200_ATTN_TIMELINE
__device__ unsigned long long g_attn_timeline[4096 * 8];
__device__ __forceinline__ void attn_mark(int i) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  const unsigned cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  if (cta < 4096) g_attn_timeline[cta * 8 + i] = t;
}
#define B200_ATL(i) attn_mark(i)
#else
#define B200_ATL(i)
#endif

// NSTAGES / MINB: three stages and two CTAs per SM, or two stages and three CTAs per SM (more
// warps to hide the latency of the dependent ldmatrix -> mma -> softmax chains).
// One compute warp's share of a 64-key tile in the TMA-fed decode kernels: its 16 keys against the
// query rows, online softmax, and the product with its 16 value rows.  kt / vt: shared-memory
// addresses of the stage; n0: the warp's first key.  The accumulator is rescaled only when some
// row's running maximum moved (rare after the first tiles); the decision is taken by the whole warp.
//
// NR = 2: up to sixteen query rows per kv head.  S = Q K^T with the queries as the 16 MMA rows;
// lane 4 g + t holds rows g and g + 8.  o_acc[i][2 r + c]: row g + 8 r, column 8 i + 2 t + c.
//
// NR = 1: at most eight query rows per kv head (the single-token decode step of a model with a
// group of 4 or 8, or two tokens of a group of 4).  Sixteen MMA rows would be half padding, so the
// products are transposed: S^T = K Q^T (16 keys x 8 queries) and O^T = V^T P^T (head dims x 8
// queries): half the MMAs, half the exponentials, half the accumulator and query registers.  Lane
// 4 g + t holds queries 2 t and 2 t + 1.  o_acc[2 d + h][c]: head dim 16 d + g + 8 h, query 2 t + c.
// P^T reaches the operand layout of the second product through two 8 x 8 transposes (movmatrix).
// row_max / row_sum / pos_r are per row g + 8 r (NR = 2) or per query 2 t + c (NR = 1).
template <int D, int NR>
__device__ __forceinline__ void decode_warp_tile(uint32_t kt, uint32_t vt, int n0, int warp, int lane,
                                                 const uint32_t (&q_frag)[D / 16][2 * NR],
                                                 float (&o_acc)[D / 8][2 * NR], float (&row_max)[2],
                                                 float (&row_sum)[2], const int (&pos_r)[2], int kv_len,
                                                 float scale_log2, int window, int sink) {
  if constexpr (NR == 2) {
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t kf[4];
      const int krow = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int kchunk = ks * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(kf, kt + kv_swz<D>(krow, kchunk));
      mma_bf16_16816(s[0], q_frag[ks], kf[0], kf[1]);
      mma_bf16_16816(s[1], q_frag[ks], kf[2], kf[3]);
    }
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = n0 + i * 8 + (lane & 3) * 2 + (j & 1);
        const int pos = pos_r[j >> 1];
        bool keep = key <= pos && key < kv_len;
        if (window > 0) keep = keep && (key > pos - window || key < sink);
        const float v = keep ? s[i][j] * scale_log2 : -INFINITY;
        s[i][j] = v;
        tile_max[j >> 1] = fmaxf(tile_max[j >> 1], v);
      }
    }
    float corr[2], m_use[2];
    bool moved = false;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float tm = quad_max(tile_max[r]);
      const float new_max = fmaxf(row_max[r], tm);
      corr[r] = (new_max == -INFINITY) ? 1.f : exp2f(row_max[r] - new_max);
      moved = moved || new_max != row_max[r];
      row_max[r] = new_max;
      row_sum[r] *= corr[r];
      m_use[r] = new_max == -INFINITY ? 0.f : new_max;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float e = exp2f(s[i][j] - m_use[j >> 1]);
        s[i][j] = e;
        row_sum[j >> 1] += e;
      }
    if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o_acc[i][j] *= corr[j >> 1];
    }
    uint32_t pa[4];
    pa[0] = pack_bf16x2(s[0][0], s[0][1]);
    pa[1] = pack_bf16x2(s[0][2], s[0][3]);
    pa[2] = pack_bf16x2(s[1][0], s[1][1]);
    pa[3] = pack_bf16x2(s[1][2], s[1][3]);
#pragma unroll
    for (int dt = 0; dt < D / 16; ++dt) {
      uint32_t vf[4];
      const int vrow = warp * 16 + (lane & 15);
      const int vchunk = dt * 2 + (lane >> 4);
      ldmatrix_x4_trans(vf, vt + kv_swz<D>(vrow, vchunk));
      mma_bf16_16816(o_acc[2 * dt], pa, vf[0], vf[1]);
      mma_bf16_16816(o_acc[2 * dt + 1], pa, vf[2], vf[3]);
    }
  } else {
    // S^T in two accumulators (even and odd 16-dim slices), so that the dependent chain is half as long
    float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t kf[4];   // (keys 0-7, dims 0-7), (keys 0-7, dims 8-15), (keys 8-15, dims 0-7), (keys 8-15, dims 8-15)
      const int krow = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int kchunk = ks * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(kf, kt + kv_swz<D>(krow, kchunk));
      if (ks & 1)
        mma_bf16_16816_regs(sb[0], sb[1], sb[2], sb[3], kf[0], kf[2], kf[1], kf[3], q_frag[ks][0], q_frag[ks][1]);
      else
        mma_bf16_16816_regs(sa[0], sa[1], sa[2], sa[3], kf[0], kf[2], kf[1], kf[3], q_frag[ks][0], q_frag[ks][1]);
    }
    // s[2 h + c]: key n0 + g + 8 h, query 2 t + c
    float s[4];
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int key = n0 + (lane >> 2) + 8 * (j >> 1);
      const int pos = pos_r[j & 1];
      bool keep = key <= pos && key < kv_len;
      if (window > 0) keep = keep && (key > pos - window || key < sink);
      const float v = keep ? (sa[j] + sb[j]) * scale_log2 : -INFINITY;
      s[j] = v;
      tile_max[j & 1] = fmaxf(tile_max[j & 1], v);
    }
    float corr[2], m_use[2];
    bool moved = false;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const float tm = col_max(tile_max[c]);
      const float new_max = fmaxf(row_max[c], tm);
      corr[c] = (new_max == -INFINITY) ? 1.f : exp2f(row_max[c] - new_max);
      moved = moved || new_max != row_max[c];
      row_max[c] = new_max;
      row_sum[c] *= corr[c];
      m_use[c] = new_max == -INFINITY ? 0.f : new_max;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float e = exp2f(s[j] - m_use[j & 1]);
      s[j] = e;
      row_sum[j & 1] += e;
    }
    if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o_acc[i][0] *= corr[0];
        o_acc[i][1] *= corr[1];
      }
    }
    // P^T (16 keys x 8 queries) as the k16 x n8 operand: lane wants keys 2 t, 2 t + 1 (+ 8) of query g
    const uint32_t pb0 = movmatrix_trans(pack_bf16x2(s[0], s[1]));
    const uint32_t pb1 = movmatrix_trans(pack_bf16x2(s[2], s[3]));
#pragma unroll
    for (int dt = 0; dt < D / 16; ++dt) {
      uint32_t vf[4];   // transposed: (dims 0-7, keys 0-7), (dims 0-7, keys 8-15), (dims 8-15, keys 0-7), (dims 8-15, keys 8-15)
      const int vrow = warp * 16 + (lane & 15);
      const int vchunk = dt * 2 + (lane >> 4);
      ldmatrix_x4_trans(vf, vt + kv_swz<D>(vrow, vchunk));
      mma_bf16_16816_regs(o_acc[2 * dt][0], o_acc[2 * dt][1], o_acc[2 * dt + 1][0], o_acc[2 * dt + 1][1], vf[0],
                          vf[2], vf[1], vf[3], pb0, pb1);
    }
  }
}

template <int D, int NSTAGES, int MINB, int NR>
__global__ void __launch_bounds__(160, MINB)
gqa_decode_tma_kernel(const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const AttnParams p,
                      const int box_rows) {
  using Cfg = DecodeTmaCfg<D, NSTAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::STAGES * Cfg::KV_BYTES;
  uint8_t* sQ = sV + Cfg::STAGES * Cfg::KV_BYTES;
  int* s_bt = reinterpret_cast<int*>(sQ + Cfg::Q_BYTES);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(s_bt + Cfg::BT_ENTRIES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  int* s_abort = reinterpret_cast<int*>(empty_bar + Cfg::STAGES);

  if (threadIdx.x == 0) B200_ATL(0);
  pdl_trigger();
  pdl_wait();   // sequence lengths, block tables, q and the cache rows of this step come from earlier kernels
  const int b = blockIdx.x;
  const int kvh = blockIdx.y;
  const int split = blockIdx.z;
  const int G = p.Hq / p.Hk;
  const int rows = G * p.q_len;
  const int kv_len = p.seq_lens[b];
  const int* bt = p.block_tables + static_cast<long long>(b) * p.max_blocks;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  const int n_tiles_all = (kv_len + Cfg::BN - 1) / Cfg::BN;
  const int per = (n_tiles_all + p.splits - 1) / p.splits;
  const int t_begin = split * per;
  const int t_end = min(n_tiles_all, t_begin + per);
  const int n_tiles = max(0, t_end - t_begin);
  // Block-table entries this CTA needs: blocks [bt_first, bt_last).
  const int bt_first = (t_begin * Cfg::BN) / p.block_size;
  const int bt_last = min(p.max_blocks, (min(kv_len, t_end * Cfg::BN) + p.block_size - 1) / p.block_size);
  const bool bt_cached = (bt_last - bt_first) <= Cfg::BT_ENTRIES;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 4);
    }
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (bt_cached)
    for (int i = bt_first + tid; i < bt_last; i += Cfg::THREADS) s_bt[i - bt_first] = bt[i];
  // Zero the stages once: rows of a partly filled tile that no copy writes must
  // hold finite values (they are multiplied by zero probabilities).
  {
    uint4* z = reinterpret_cast<uint4*>(sK);
    const int n16 = 2 * Cfg::STAGES * Cfg::KV_BYTES / 16;
    for (int i = tid; i < n16; i += Cfg::THREADS) z[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  fence_proxy_async();
  __syncthreads();
  volatile int* abort_flag = s_abort;
  if (threadIdx.x == 0) {
    B200_ATL(1);
#ifdef B200_ATTN_TIMELINE
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    const unsigned cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    if (cta < 4096) g_attn_timeline[cta * 8 + 5] = smid;
#endif
  }

  if (warp == 4) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int issued = 0;
      for (int it = 0; it < n_tiles; ++it) {
        const int stage = it % Cfg::STAGES;
        if (it >= Cfg::STAGES) {
          const uint32_t parity = static_cast<uint32_t>(((it / Cfg::STAGES) - 1) & 1);
          if (*abort_flag || !mbar_wait(&empty_bar[stage], parity)) {
            if (!*abort_flag && p.status) atomicCAS(p.status, 0, kStatusTimeoutEmptyBarrier);
            *abort_flag = 1;
            break;
          }
        }
        const int n0 = (t_begin + it) * Cfg::BN;
        const int nvalid = min(Cfg::BN, kv_len - n0);
        const int nboxes = (nvalid + box_rows - 1) / box_rows;
        mbar_arrive_expect_tx(&full_bar[stage],
                              static_cast<uint32_t>(nboxes * box_rows * 128 * Cfg::HALVES * 2));
        for (int j = 0; j < nboxes; ++j) {
          const int key = n0 + j * box_rows;
          const int bi = key / p.block_size;
          const int blk = bt_cached ? s_bt[bi - bt_first] : bt[bi];
          const int row = (blk * p.Hk + kvh) * p.block_size + key % p.block_size;
#pragma unroll
          for (int h = 0; h < Cfg::HALVES; ++h) {
            const int dst = stage * Cfg::KV_BYTES + h * Cfg::HALF_BYTES + j * box_rows * 128;
            tma_load_2d(sK + dst, &tm_k, &full_bar[stage], h * 64, row);
            tma_load_2d(sV + dst, &tm_v, &full_bar[stage], h * 64, row);
          }
        }
        ++issued;
      }
      if (*abort_flag) {
        // Bounded wait for the copies still in flight before the CTA retires.
        const int first = issued > Cfg::STAGES ? issued - Cfg::STAGES : 0;
        for (int i = first; i < issued; ++i)
          mbar_wait(&full_bar[i % Cfg::STAGES], static_cast<uint32_t>((i / Cfg::STAGES) & 1));
      }
    }
    __syncthreads();   // pairs with the barrier before the merge
    __syncthreads();   // pairs with the barrier inside the merge
    return;
  }

  // -------------------------------------------------------------- consumers
  {
    constexpr int CHUNKS = D / 8;
    // Each compute warp only needs the Q rows; every warp loads the whole (small) tile part.
    for (int idx = tid; idx < 16 * CHUNKS; idx += Cfg::COMPUTE_THREADS) {
      const int row = idx / CHUNKS, c = idx % CHUNKS;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (row < rows) {
        const int qi = row / G, hh = kvh * G + row % G;
        v = *reinterpret_cast<const uint4*>(p.q + static_cast<long long>(b * p.q_len + qi) * p.q_stride +
                                            static_cast<long long>(hh) * D + c * 8);
      }
      *reinterpret_cast<uint4*>(sQ + tile_offset<D>(row, c)) = v;
    }
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");

  float o_acc[D / 8][2 * NR];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 2 * NR; ++j) o_acc[i][j] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY};
  float row_sum[2] = {0.f, 0.f};
  uint32_t q_frag[D / 16][2 * NR];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    uint32_t f[4];
    ldmatrix_x4(f, smem_u32(sQ) + tile_offset<D>(lane & 15, ks * 2 + (lane >> 4)));
    if constexpr (NR == 2) {
#pragma unroll
      for (int j = 0; j < 4; ++j) q_frag[ks][j] = f[j];
    } else {
      q_frag[ks][0] = f[0];   // query lane / 4, dims 16 ks + 2 (lane % 4), + 1
      q_frag[ks][1] = f[2];   // the same query, dims + 8
    }
  }

  // the two rows this lane keeps statistics for: fragment rows g and g + 8 (NR = 2), queries
  // 2 t and 2 t + 1 (NR = 1)
  const int r_a = lane >> 2;
  const int row_of[2] = {NR == 2 ? r_a : (lane & 3) * 2, NR == 2 ? r_a + 8 : (lane & 3) * 2 + 1};
  int pos_r[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) pos_r[r] = kv_len - p.q_len + row_of[r] / G;

  // (Issuing the scores of tile it + 1 before the softmax of tile it was tried: the warp then holds
  // two stages of the ring at once, which leaves the producer one stage less to fill, and the kernel
  // got slower, 161 us against 133 us on 128 sequences x 1152 keys x 8 kv heads.)
  for (int it = 0; it < n_tiles; ++it) {
    const int stage = it % Cfg::STAGES;
    bool ok = !*abort_flag &&
              mbar_wait(&full_bar[stage], static_cast<uint32_t>((it / Cfg::STAGES) & 1));
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
      if (lane == 0) {
        if (!*abort_flag && p.status) atomicCAS(p.status, 0, kStatusTimeoutFullBarrier);
        *abort_flag = 1;
      }
      break;
    }
    if (it == 0 && threadIdx.x == 0) B200_ATL(2);
    decode_warp_tile<D, NR>(smem_u32(sK + stage * Cfg::KV_BYTES), smem_u32(sV + stage * Cfg::KV_BYTES),
                            (t_begin + it) * Cfg::BN + warp * 16, warp, lane, q_frag, o_acc, row_max,
                            row_sum, pos_r, kv_len, p.scale_log2, p.window, p.sink);
    // This warp is done reading the stage.
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[stage]);
  }
  __syncthreads();   // every warp (and the producer) is past the main loop
  if (threadIdx.x == 0) B200_ATL(3);
  if (*abort_flag) {
    __syncthreads();
    return;
  }

  // ---- merge the four warps' partial results through shared memory
  float* m_buf = reinterpret_cast<float*>(sK);
  float* l_buf = m_buf + 64;
  float* o_buf = l_buf + 64;
  if constexpr (NR == 2) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      row_sum[r] = quad_sum(row_sum[r]);
      if ((lane & 3) == 0) {
        m_buf[warp * 16 + r_a + 8 * r] = row_max[r];
        l_buf[warp * 16 + r_a + 8 * r] = row_sum[r];
      }
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int col = i * 8 + (lane & 3) * 2;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float* dst = o_buf + (static_cast<size_t>(warp) * 16 + r_a + 8 * r) * (D + 4) + col;
        *reinterpret_cast<float2*>(dst) = make_float2(o_acc[i][2 * r], o_acc[i][2 * r + 1]);
      }
    }
  } else {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      row_sum[c] = col_sum(row_sum[c]);
      if (r_a == 0) {
        m_buf[warp * 16 + row_of[c]] = row_max[c];
        l_buf[warp * 16 + row_of[c]] = row_sum[c];
      }
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int dim = (i >> 1) * 16 + r_a + 8 * (i & 1);
#pragma unroll
      for (int c = 0; c < 2; ++c)
        o_buf[(static_cast<size_t>(warp) * 16 + row_of[c]) * (D + 4) + dim] = o_acc[i][c];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < rows * (D / 4); idx += Cfg::COMPUTE_THREADS) {
    const int row = idx / (D / 4);
    const int c4 = (idx % (D / 4)) * 4;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, m_buf[w * 16 + row]);
    float l = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = m_buf[w * 16 + row];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
      l += l_buf[w * 16 + row] * f;
      const float4 x =
          *reinterpret_cast<const float4*>(o_buf + (static_cast<size_t>(w) * 16 + row) * (D + 4) + c4);
      acc.x += x.x * f;
      acc.y += x.y * f;
      acc.z += x.z * f;
      acc.w += x.w * f;
    }
    const int qi = row / G, hh = kvh * G + row % G;
    if (p.splits == 1) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      uint2 pk;
      pk.x = pack_bf16x2(acc.x * inv, acc.y * inv);
      pk.y = pack_bf16x2(acc.z * inv, acc.w * inv);
      *reinterpret_cast<uint2*>(p.out + static_cast<long long>(b * p.q_len + qi) * p.out_stride +
                                static_cast<long long>(hh) * D + c4) = pk;
      if (p.lse && c4 == 0)
        p.lse[static_cast<long long>(b * p.q_len + qi) * p.Hq + hh] =
            l > 0.f ? (m + log2f(l)) / kLog2e : -INFINITY;
    } else {
      const size_t pr = ((static_cast<size_t>(b) * p.Hk + kvh) * p.splits + split) * 16 + row;
      *reinterpret_cast<float4*>(p.o_part + pr * D + c4) = acc;
      if (c4 == 0) {
        p.lse_part[pr * 2] = m;
        p.lse_part[pr * 2 + 1] = l;
      }
    }
  }
  if (threadIdx.x == 0) B200_ATL(4);
}

// ------------------------------------------------- decode, persistent CTAs
// Same math and the same TMA-fed ring as gqa_decode_tma_kernel, but a CTA does not end with
// its (sequence, kv head, split) item: the grid is sized to what is resident at once and every
// CTA walks a list of items.  The producer warp runs ahead ACROSS items (its ring of K/V tiles,
// the next item's query rows and block-table slice are in flight while the compute warps still
// work on the current item), so the per-item prologue (query load, first-tile latency) and the
// epilogue (merge of the four warps, output store) overlap with streaming, and no barrier or
// stage is re-initialised between items.  Items are handed out through a device counter
// (p.work_counter: ticket word + finished-CTA word, both zero at rest; the last CTA to finish
// puts them back to zero, so graph replays need no host reset) or, without a counter, by
// striding.  q_len rows x group heads <= 16 as in the other decode kernels.
//
// Balanced mode (p.persistent == 2).  Whole items leave the last round of a grid part empty: 1024
// items of 18 tiles on 444 resident CTAs take three rounds for 2.3 rounds of work.  Here the tiles
// of all items, laid end to end (sequence, then kv head, then tile), are cut into gridDim.x equal
// ranges, one per CTA.  A range covers whole items, which the CTA finishes and stores itself, and at
// most two pieces of items that continue in a neighbour: the piece its range starts in and the piece
// it ends in.  Pieces go to the fp32 scratch (slot 2 x CTA for the first segment of a CTA, 2 x CTA + 1
// for a later one) and gqa_decode_merge_balanced_kernel, which derives the same cut from the
// sequence lengths, joins them.  A sequence of length zero counts as one (fully masked) tile, so
// that its output rows are written.
template <int D, int NSTAGES>
struct DecodePersistCfg {
  static constexpr int BN = 64;
  static constexpr int STAGES = NSTAGES;
  static constexpr int COMPUTE_THREADS = 128;
  static constexpr int THREADS = 160;
  static constexpr int HALVES = D / 64;
  static constexpr int HALF_BYTES = BN * 128;
  static constexpr int KV_BYTES = HALVES * HALF_BYTES;
  static constexpr int BT_ENTRIES = 256;       // block-table slice of one item (per buffer)
  static constexpr int META_INTS = 8;
  // dynamic: 2 query buffers of rows x D bf16 and two fold slots of rows x D fp32 (the four warps'
  // results are joined 2, 3 -> 0, 1 and then 1 -> 0), their maxima and sums
  static constexpr size_t smem(int rows) {
    return 1024 + 2 * static_cast<size_t>(STAGES) * KV_BYTES + 2 * static_cast<size_t>(rows) * D * 2 +
           2 * static_cast<size_t>((rows + 1) & ~1) * D * 4 + 4 * static_cast<size_t>(rows) * 4 +
           2 * BT_ENTRIES * 4 + 2 * META_INTS * 4 + (2 * STAGES + 4) * 8 + 64;
  }
};

// Tiles that a sequence of kv_len keys counts for in the balanced cut (never zero).
__device__ __forceinline__ int balanced_tiles(int kv_len) {
  const int n = (kv_len + 63) >> 6;
  return n > 0 ? n : 1;
}
// Tiles per CTA range: equal parts, at least two tiles (a piece of one tile costs more in set-up and
// merge than it streams).
__device__ __forceinline__ long long balanced_per(long long total_tiles, int ctas) {
  const long long per = (total_tiles + ctas - 1) / ctas;
  return per < 2 ? 2 : per;
}

template <int D, int NSTAGES, int MINB, int NR>
__global__ void __launch_bounds__(160, MINB)
gqa_decode_persist_kernel(const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v, const AttnParams p,
                          const int box_rows, const int total_items) {
  using Cfg = DecodePersistCfg<D, NSTAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int G = p.Hq / p.Hk;
  const int rows = G * p.q_len;
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::STAGES * Cfg::KV_BYTES;
  uint8_t* sQ = sV + Cfg::STAGES * Cfg::KV_BYTES;                       // [2][rows][D] bf16, linear
  float* s_fold = reinterpret_cast<float*>(sQ + 2 * rows * D * 2);      // [2][D / 8][rows][4] float2, then maxima [2][rows], sums [2][rows]
  int* s_bt = reinterpret_cast<int*>(s_fold + 2 * ((rows + 1) & ~1) * D + 4 * rows);  // [2][BT_ENTRIES]
  int* s_meta = s_bt + 2 * Cfg::BT_ENTRIES;                             // [2][META_INTS]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(s_meta + 2 * Cfg::META_INTS);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  uint64_t* q_full = empty_bar + Cfg::STAGES;                           // [2]
  uint64_t* q_empty = q_full + 2;                                       // [2]
  int* s_abort = reinterpret_cast<int*>(q_empty + 2);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 4);
    }
    mbar_init(&q_full[0], 1);
    mbar_init(&q_full[1], 1);
    mbar_init(&q_empty[0], 4);
    mbar_init(&q_empty[1], 4);
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  {
    // rows of a partly filled tile that no copy ever wrote must hold finite values
    uint4* z = reinterpret_cast<uint4*>(sK);
    const int n16 = 2 * Cfg::STAGES * Cfg::KV_BYTES / 16;
    for (int i = tid; i < n16; i += Cfg::THREADS) z[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  fence_proxy_async();
  __syncthreads();
  pdl_trigger();
  pdl_wait();   // q, the cache rows of this step, lengths and block tables come from earlier kernels
  volatile int* abort_flag = s_abort;

  if (warp == 4) {
    // ------------------------------------------------------------ producer
    int item = blockIdx.x;
    uint32_t g = 0;            // tiles issued so far (ring position), identical in all lanes
    // balanced mode: position in the end-to-end tile sequence (all lanes hold the same values)
    const bool balanced = p.persistent == 2;
    const int n_seqs = total_items / p.Hk;
    long long bx = 0, bx_end = 0;
    int bal_b = 0, bal_kvh = 0, bal_t = 0, bal_nb = 1;
    if (balanced) {
      int total = 0;
      for (int i = lane; i < n_seqs; i += 32) total += balanced_tiles(p.seq_lens[i]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
      const long long all_tiles = static_cast<long long>(total) * p.Hk;
      const long long per = balanced_per(all_tiles, static_cast<int>(gridDim.x));
      bx = static_cast<long long>(blockIdx.x) * per;
      bx_end = bx + per < all_tiles ? bx + per : all_tiles;
      if (bx < bx_end) {
        // the sequence that tile bx belongs to: 32 sequences per pass, inclusive scan of their tiles
        long long before = 0;      // tiles of the sequences ahead of the pass, times kv heads
        for (int c0 = 0; c0 < n_seqs; c0 += 32) {
          const int n = c0 + lane < n_seqs ? balanced_tiles(p.seq_lens[c0 + lane]) : 0;
          int incl = n;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
          }
          const unsigned past = __ballot_sync(0xffffffffu, before + static_cast<long long>(incl) * p.Hk > bx);
          if (past != 0u) {
            const int l = __ffs(static_cast<int>(past)) - 1;
            const int incl_l = __shfl_sync(0xffffffffu, incl, l);
            bal_nb = __shfl_sync(0xffffffffu, n, l);
            bal_b = c0 + l;
            before += static_cast<long long>(incl_l - bal_nb) * p.Hk;
            break;
          }
          before += static_cast<long long>(__shfl_sync(0xffffffffu, incl, 31)) * p.Hk;
        }
        const int off = static_cast<int>(bx - before);      // < bal_nb * Hk
        bal_kvh = off / bal_nb;
        bal_t = off % bal_nb;
      }
    }
    for (int k = 0;; ++k) {
      const int par = k & 1;
      int next_item = item + static_cast<int>(gridDim.x);
      if (p.work_counter != nullptr && lane == 0)
        next_item = static_cast<int>(gridDim.x) + atomicAdd(p.work_counter, 1);
      bool ok = true;
      if (k >= 2 && lane == 0) ok = mbar_wait(&q_empty[par], static_cast<uint32_t>(((k >> 1) - 1) & 1));
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0 && !*abort_flag;
      if (!ok) {
        if (lane == 0) {
          if (!*abort_flag && p.status) atomicCAS(p.status, 0, kStatusTimeoutEmptyBarrier);
          *abort_flag = 1;
        }
        break;
      }
      const bool valid = balanced ? bx < bx_end : item < total_items;
      int b = 0, kvh = 0, split = 0, kv_len = 0, t_begin = 0, n_tiles = 0, bt_first = 0, bt_last = 0;
      int slot = -1;             // scratch slot of a partial result; -1: the output is final
      const int* bt = p.block_tables;
      if (valid && balanced) {
        b = bal_b;
        kvh = bal_kvh;
        kv_len = p.seq_lens[b];
        bt = p.block_tables + static_cast<long long>(b) * p.max_blocks;
        t_begin = bal_t;
        const long long left = bx_end - bx;
        n_tiles = bal_nb - bal_t < left ? bal_nb - bal_t : static_cast<int>(left);
        const int t_end = t_begin + n_tiles;
        if (t_begin != 0 || n_tiles != bal_nb) slot = 2 * static_cast<int>(blockIdx.x) + (k == 0 ? 0 : 1);
        item = b * p.Hk + kvh;
        bt_first = (t_begin * Cfg::BN) / p.block_size;
        bt_last = min(p.max_blocks, (min(kv_len, t_end * Cfg::BN) + p.block_size - 1) / p.block_size);
        // next segment
        bx += n_tiles;
        bal_t += n_tiles;
        if (bal_t == bal_nb) {
          bal_t = 0;
          if (++bal_kvh == p.Hk) {
            bal_kvh = 0;
            ++bal_b;
            bal_nb = bal_b < n_seqs ? balanced_tiles(p.seq_lens[bal_b]) : 1;
          }
        }
      } else if (valid) {
        split = item % p.splits;
        kvh = (item / p.splits) % p.Hk;
        b = item / (p.splits * p.Hk);
        kv_len = p.seq_lens[b];
        bt = p.block_tables + static_cast<long long>(b) * p.max_blocks;
        const int n_tiles_all = (kv_len + Cfg::BN - 1) / Cfg::BN;
        const int per = (n_tiles_all + p.splits - 1) / p.splits;
        t_begin = split * per;
        const int t_end = min(n_tiles_all, t_begin + per);
        n_tiles = max(0, t_end - t_begin);
        bt_first = (t_begin * Cfg::BN) / p.block_size;
        bt_last = min(p.max_blocks, (min(kv_len, t_end * Cfg::BN) + p.block_size - 1) / p.block_size);
        if (p.splits > 1) slot = (b * p.Hk + kvh) * p.splits + split;
      }
      const bool bt_cached = (bt_last - bt_first) <= Cfg::BT_ENTRIES;
      int* my_bt = s_bt + par * Cfg::BT_ENTRIES;
      if (valid && bt_cached)
        for (int i = bt_first + lane; i < bt_last; i += 32) my_bt[i - bt_first] = bt[i];
      __syncwarp();
      if (lane == 0) {
        int* meta = s_meta + par * Cfg::META_INTS;
        meta[0] = valid ? item : -1;
        meta[1] = kv_len;
        meta[2] = t_begin;
        meta[3] = n_tiles;
        meta[4] = slot;
        if (!valid) {
          mbar_arrive(&q_full[par]);
        } else {
          mbar_arrive_expect_tx(&q_full[par], static_cast<uint32_t>(rows * D * 2));
          for (int qi = 0; qi < p.q_len; ++qi)
            bulk_load_1d(sQ + (par * rows + qi * G) * D * 2,
                         p.q + static_cast<long long>(b * p.q_len + qi) * p.q_stride +
                             static_cast<long long>(kvh) * G * D,
                         static_cast<uint32_t>(G * D * 2), &q_full[par]);
          for (int it = 0; it < n_tiles; ++it, ++g) {
            const int stage = static_cast<int>(g % Cfg::STAGES);
            if (g >= Cfg::STAGES) {
              const uint32_t parity = static_cast<uint32_t>(((g / Cfg::STAGES) - 1) & 1);
              if (*abort_flag || !mbar_wait(&empty_bar[stage], parity)) {
                if (!*abort_flag && p.status) atomicCAS(p.status, 0, kStatusTimeoutEmptyBarrier);
                *abort_flag = 1;
                break;
              }
            }
            const int n0 = (t_begin + it) * Cfg::BN;
            const int nvalid = min(Cfg::BN, kv_len - n0);
            const int nboxes = (nvalid + box_rows - 1) / box_rows;
            mbar_arrive_expect_tx(&full_bar[stage],
                                  static_cast<uint32_t>(nboxes * box_rows * 128 * Cfg::HALVES * 2));
            for (int j = 0; j < nboxes; ++j) {
              const int key = n0 + j * box_rows;
              const int bi = key / p.block_size;
              const int blk = bt_cached ? my_bt[bi - bt_first] : bt[bi];
              const int row = (blk * p.Hk + kvh) * p.block_size + key % p.block_size;
#pragma unroll
              for (int h = 0; h < Cfg::HALVES; ++h) {
                const int dst = stage * Cfg::KV_BYTES + h * Cfg::HALF_BYTES + j * box_rows * 128;
                tma_load_2d(sK + dst, &tm_k, &full_bar[stage], h * 64, row);
                tma_load_2d(sV + dst, &tm_v, &full_bar[stage], h * 64, row);
              }
            }
          }
        }
      }
      g = __shfl_sync(0xffffffffu, g, 0);
      if (!valid || *abort_flag) break;
      item = __shfl_sync(0xffffffffu, next_item, 0);
    }
    if (lane == 0) {
      if (*abort_flag) {
        // bounded wait for the copies still in flight before the CTA retires
        const uint32_t first = g > Cfg::STAGES ? g - Cfg::STAGES : 0;
        for (uint32_t i = first; i < g; ++i)
          mbar_wait(&full_bar[i % Cfg::STAGES], static_cast<uint32_t>((i / Cfg::STAGES) & 1));
      }
      if (p.work_counter != nullptr) {
        // the last CTA to finish puts the ticket and finished-CTA words back to zero
        __threadfence();
        if (atomicAdd(p.work_counter + 1, 1) == static_cast<int>(gridDim.x) - 1) {
          p.work_counter[0] = 0;
          p.work_counter[1] = 0;
        }
      }
    }
    return;
  }

  // -------------------------------------------------------------- consumers
  const int r_a = lane >> 2;
  uint32_t g = 0;
  volatile int* s_dec = s_abort + 1;
  float* m_buf = s_fold + 2 * ((rows + 1) & ~1) * D;   // [2][rows] maxima, then [2][rows] sums
  float* l_buf = m_buf + 2 * rows;
  for (int k = 0;; ++k) {
    const int par = k & 1;
    bool ok = !*abort_flag && mbar_wait(&q_full[par], static_cast<uint32_t>((k >> 1) & 1));
    ok = __all_sync(0xffffffffu, ok);
    if (!ok && lane == 0) {
      if (!*abort_flag && p.status) atomicCAS(p.status, 0, kStatusTimeoutFullBarrier);
      *abort_flag = 1;
    }
    // The four compute warps leave the loop together or not at all: a warp that gave up on a wait
    // must not exit while the others sit in a named barrier.  This barrier also frees the merge
    // buffer of the previous item.
    // The decision to leave is taken by one thread and read by all after the barrier (two slots:
    // one per barrier of the loop body), so it is the same for every warp even when the flag
    // changes while they cross the barrier.
    if (tid == 0) s_dec[0] = *abort_flag;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (s_dec[0]) break;
    const int* meta = s_meta + par * Cfg::META_INTS;
    const int item = meta[0];
    if (item < 0) break;
    const int kv_len = meta[1], t_begin = meta[2], n_tiles = meta[3], slot = meta[4];
    const int kvh = (item / p.splits) % p.Hk;
    const int b = item / (p.splits * p.Hk);

    // query fragments straight from the linear rows (rows beyond `rows` are zero).  NR = 2:
    // {a0, a1, a2, a3} = (row, col), (row + 8, col), (row, col + 8), (row + 8, col + 8) with row =
    // lane / 4; NR = 1: the operand of the transposed product, {(row, col), (row, col + 8)}.
    uint32_t q_frag[D / 16][2 * NR];
    {
      const uint8_t* qb = sQ + par * rows * D * 2;
      const int c0 = (lane & 3) * 2;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int col = ks * 16 + c0;
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          const int row = r_a + 8 * r;
          q_frag[ks][r] = row < rows ? *reinterpret_cast<const uint32_t*>(qb + (row * D + col) * 2) : 0u;
          q_frag[ks][NR + r] = row < rows ? *reinterpret_cast<const uint32_t*>(qb + (row * D + col + 8) * 2) : 0u;
        }
      }
    }
    // the query buffer and the meta words of this parity may be rewritten from here on
    __syncwarp();
    if (lane == 0) mbar_arrive(&q_empty[par]);

    float o_acc[D / 8][2 * NR];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
      for (int j = 0; j < 2 * NR; ++j) o_acc[i][j] = 0.f;
    float row_max[2] = {-INFINITY, -INFINITY};
    float row_sum[2] = {0.f, 0.f};
    // the two rows this lane keeps statistics for: fragment rows g and g + 8 (NR = 2), queries
    // 2 t and 2 t + 1 (NR = 1)
    const int row_of[2] = {NR == 2 ? r_a : (lane & 3) * 2, NR == 2 ? r_a + 8 : (lane & 3) * 2 + 1};
    int pos_r[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) pos_r[r] = kv_len - p.q_len + row_of[r] / G;

    for (int it = 0; it < n_tiles; ++it, ++g) {
      const int stage = static_cast<int>(g % Cfg::STAGES);
      bool okt = !*abort_flag && mbar_wait(&full_bar[stage], static_cast<uint32_t>((g / Cfg::STAGES) & 1));
      okt = __all_sync(0xffffffffu, okt);
      if (!okt) {
        if (lane == 0) {
          if (!*abort_flag && p.status) atomicCAS(p.status, 0, kStatusTimeoutFullBarrier);
          *abort_flag = 1;
        }
        break;
      }
      decode_warp_tile<D, NR>(smem_u32(sK + stage * Cfg::KV_BYTES), smem_u32(sV + stage * Cfg::KV_BYTES),
                              (t_begin + it) * Cfg::BN + warp * 16, warp, lane, q_frag, o_acc, row_max,
                              row_sum, pos_r, kv_len, p.scale_log2, p.window, p.sink);
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
    }

    // ---- join the four warps' results (rows < `rows` only): warps 2 and 3 hand theirs to warps 0
    // and 1, then warp 1 hands the sum to warp 0, which stores.  The same lane of every warp holds
    // the same positions of the output, so a slot is indexed by accumulator register and lane: as
    // float2 [register pair i][row][lane % 4] (NR = 2: the pair of row g + 8 r) or
    // [i][lane / 4][lane % 4 < tq] (NR = 1: the two queries of the lane, tq = ceil(rows / 2)).
    const int tq = (rows + 1) >> 1;
#pragma unroll
    for (int r = 0; r < 2; ++r) row_sum[r] = NR == 2 ? quad_sum(row_sum[r]) : col_sum(row_sum[r]);
    const bool stat_lane = NR == 2 ? (lane & 3) == 0 : r_a == 0;      // writes the row's maximum and sum
    const bool acc_lane = NR == 2 || (lane & 3) < tq;
    auto fold_at = [&](int fs, int i, int r) -> float2* {
      const int idx = NR == 2 ? ((fs * (D / 8) + i) * rows + row_of[r]) * 4 + (lane & 3)
                              : ((fs * (D / 8) + i) * 8 + r_a) * tq + (lane & 3);
      return reinterpret_cast<float2*>(s_fold) + idx;
    };
    auto put = [&](int fs) {
#pragma unroll
      for (int r = 0; r < 2; ++r)
        if (stat_lane && row_of[r] < rows) {
          m_buf[fs * rows + row_of[r]] = row_max[r];
          l_buf[fs * rows + row_of[r]] = row_sum[r];
        }
      if constexpr (NR == 2) {
#pragma unroll
        for (int r = 0; r < 2; ++r)
          if (row_of[r] < rows) {
#pragma unroll
            for (int i = 0; i < D / 8; ++i) *fold_at(fs, i, r) = make_float2(o_acc[i][2 * r], o_acc[i][2 * r + 1]);
          }
      } else if (acc_lane) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) *fold_at(fs, i, 0) = make_float2(o_acc[i][0], o_acc[i][1]);
      }
    };
    auto take = [&](int fs) {
      float fa[2], fb[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        fa[r] = 1.f;
        fb[r] = 0.f;
        if (row_of[r] < rows) {
          const float mo = m_buf[fs * rows + row_of[r]];
          const float m = fmaxf(row_max[r], mo);
          fa[r] = row_max[r] == -INFINITY ? 0.f : exp2f(row_max[r] - m);
          fb[r] = mo == -INFINITY ? 0.f : exp2f(mo - m);
          row_sum[r] = row_sum[r] * fa[r] + l_buf[fs * rows + row_of[r]] * fb[r];
          row_max[r] = m;
        }
      }
      if constexpr (NR == 2) {
#pragma unroll
        for (int r = 0; r < 2; ++r)
          if (row_of[r] < rows) {
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
              const float2 x = *fold_at(fs, i, r);
              o_acc[i][2 * r] = o_acc[i][2 * r] * fa[r] + x.x * fb[r];
              o_acc[i][2 * r + 1] = o_acc[i][2 * r + 1] * fa[r] + x.y * fb[r];
            }
          }
      } else if (acc_lane) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          const float2 x = *fold_at(fs, i, 0);
          o_acc[i][0] = o_acc[i][0] * fa[0] + x.x * fb[0];
          o_acc[i][1] = o_acc[i][1] * fa[1] + x.y * fb[1];
        }
      }
    };
    if (warp >= 2) put(warp - 2);
    if (tid == 0) s_dec[1] = *abort_flag;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (s_dec[1]) break;
    if (warp < 2) take(warp);
    if (warp == 1) put(1);     // slot 1 was read by this warp alone
    if (tid == 0) s_dec[2] = *abort_flag;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (s_dec[2]) break;
    if (warp == 0) {
      take(1);
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int row = row_of[r];
        if (row >= rows) continue;
        const float m = row_max[r], l = row_sum[r];
        const int qi = row / G, hh = kvh * G + row % G;
        const float inv = slot < 0 ? (l > 0.f ? 1.f / l : 0.f) : 1.f;
        __nv_bfloat16* dst_o = p.out + static_cast<long long>(b * p.q_len + qi) * p.out_stride +
                               static_cast<long long>(hh) * D;
        float* dst_p = p.o_part + (static_cast<size_t>(slot < 0 ? 0 : slot) * 16 + row) * D;
        if constexpr (NR == 2) {
#pragma unroll
          for (int i = 0; i < D / 8; ++i) {
            const int col = i * 8 + (lane & 3) * 2;
            if (slot < 0)
              *reinterpret_cast<uint32_t*>(dst_o + col) =
                  pack_bf16x2(o_acc[i][2 * r] * inv, o_acc[i][2 * r + 1] * inv);
            else
              *reinterpret_cast<float2*>(dst_p + col) = make_float2(o_acc[i][2 * r], o_acc[i][2 * r + 1]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < D / 8; ++i) {
            const int dim = (i >> 1) * 16 + r_a + 8 * (i & 1);
            if (slot < 0)
              dst_o[dim] = __float2bfloat16(o_acc[i][r] * inv);
            else
              dst_p[dim] = o_acc[i][r];
          }
        }
        if (stat_lane) {
          if (slot < 0) {
            if (p.lse)
              p.lse[static_cast<long long>(b * p.q_len + qi) * p.Hq + hh] =
                  l > 0.f ? (m + log2f(l)) / kLog2e : -INFINITY;
          } else {
            const size_t pr = static_cast<size_t>(slot) * 16 + row;
            p.lse_part[pr * 2] = m;
            p.lse_part[pr * 2 + 1] = l;
          }
        }
      }
    }
  }
}

// Merge of split-KV partials: one warp per (sequence, kv head, row).
template <int D>
__global__ void __launch_bounds__(128) gqa_decode_merge_kernel(const AttnParams p, int B) {
  const int G = p.Hq / p.Hk;
  const int rows = G * p.q_len;
  const long long gw = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  const long long total = static_cast<long long>(B) * p.Hk * rows;
  if (gw >= total) return;
  const int lane = threadIdx.x & 31;
  const int row = static_cast<int>(gw % rows);
  const int kvh = static_cast<int>((gw / rows) % p.Hk);
  const int b = static_cast<int>(gw / (static_cast<long long>(rows) * p.Hk));
  const size_t base = (static_cast<size_t>(b) * p.Hk + kvh) * p.splits;
  float m = -INFINITY;
  for (int s = 0; s < p.splits; ++s) m = fmaxf(m, p.lse_part[((base + s) * 16 + row) * 2]);
  float l = 0.f;
  float acc[D / 32];
#pragma unroll
  for (int i = 0; i < D / 32; ++i) acc[i] = 0.f;
  for (int s = 0; s < p.splits; ++s) {
    const size_t pr = (base + s) * 16 + row;
    const float ms = p.lse_part[pr * 2];
    const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
    l += p.lse_part[pr * 2 + 1] * f;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) acc[i] += p.o_part[pr * D + i * 32 + lane] * f;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  const int qi = row / G, hh = kvh * G + row % G;
  __nv_bfloat16* dst = p.out + static_cast<long long>(b * p.q_len + qi) * p.out_stride +
                       static_cast<long long>(hh) * D;
#pragma unroll
  for (int i = 0; i < D / 32; ++i) dst[i * 32 + lane] = __float2bfloat16(acc[i] * inv);
  if (p.lse && lane == 0)
    p.lse[static_cast<long long>(b * p.q_len + qi) * p.Hq + hh] =
        l > 0.f ? (m + log2f(l)) / kLog2e : -INFINITY;
}

// Joins the pieces that the balanced persistent kernel left in the scratch: one warp per
// (sequence, kv head, row).  The warp recomputes the cut (tiles ahead of its item, tiles per CTA
// range), finds the CTAs that its item's tiles fell to, and returns at once when that is a single
// CTA (which then stored the final output itself).
template <int D>
__global__ void __launch_bounds__(128) gqa_decode_merge_balanced_kernel(const AttnParams p, int B, int ctas) {
  const int G = p.Hq / p.Hk;
  const int rows = G * p.q_len;
  const long long gw = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  const long long total = static_cast<long long>(B) * p.Hk * rows;
  if (gw >= total) return;
  const int lane = threadIdx.x & 31;
  const int row = static_cast<int>(gw % rows);
  const int kvh = static_cast<int>((gw / rows) % p.Hk);
  const int b = static_cast<int>(gw / (static_cast<long long>(rows) * p.Hk));
  int ahead = 0, all = 0;
  for (int i = lane; i < B; i += 32) {
    const int n = balanced_tiles(p.seq_lens[i]);
    all += n;
    if (i < b) ahead += n;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    all += __shfl_xor_sync(0xffffffffu, all, o);
    ahead += __shfl_xor_sync(0xffffffffu, ahead, o);
  }
  const int nb = balanced_tiles(p.seq_lens[b]);
  const long long per = balanced_per(static_cast<long long>(all) * p.Hk, ctas);
  const long long x0 = static_cast<long long>(ahead) * p.Hk + static_cast<long long>(kvh) * nb;
  const int c0 = static_cast<int>(x0 / per), c1 = static_cast<int>((x0 + nb - 1) / per);
  if (c0 == c1) return;
  // the piece in CTA c0 is that CTA's first segment only when the item starts its range
  const int first_slot = 2 * c0 + (x0 == static_cast<long long>(c0) * per ? 0 : 1);
  float m = -INFINITY;
  for (int c = c0; c <= c1; ++c) {
    const size_t pr = static_cast<size_t>(c == c0 ? first_slot : 2 * c) * 16 + row;
    m = fmaxf(m, p.lse_part[pr * 2]);
  }
  float l = 0.f;
  float acc[D / 32];
#pragma unroll
  for (int i = 0; i < D / 32; ++i) acc[i] = 0.f;
  for (int c = c0; c <= c1; ++c) {
    const size_t pr = static_cast<size_t>(c == c0 ? first_slot : 2 * c) * 16 + row;
    const float ms = p.lse_part[pr * 2];
    const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
    l += p.lse_part[pr * 2 + 1] * f;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) acc[i] += p.o_part[pr * D + i * 32 + lane] * f;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  const int qi = row / G, hh = kvh * G + row % G;
  __nv_bfloat16* dst = p.out + static_cast<long long>(b * p.q_len + qi) * p.out_stride +
                       static_cast<long long>(hh) * D;
#pragma unroll
  for (int i = 0; i < D / 32; ++i) dst[i * 32 + lane] = __float2bfloat16(acc[i] * inv);
  if (p.lse && lane == 0)
    p.lse[static_cast<long long>(b * p.q_len + qi) * p.Hq + hh] =
        l > 0.f ? (m + log2f(l)) / kLog2e : -INFINITY;
}

template <int DQK, int DV>
static int launch_prefill(const AttnParams& p, int B, int max_q_len, cudaStream_t stream) {
  using Cfg = PrefillCfg<DQK, DV>;
  auto kern = gqa_prefill_kernel<DQK, DV>;
  static DeviceOnce once;
  int dev = 0;
  if (once.needed(&dev)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) !=
        cudaSuccess)
      return -20;
    once.mark(dev);
  }
  dim3 grid((max_q_len + Cfg::BM - 1) / Cfg::BM, p.Hq, B);
  kern<<<grid, Cfg::THREADS, Cfg::SMEM, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

template <int D, int NSTAGES, int MINB, int NR>
static int launch_decode_tma_rows(const AttnParams& p, dim3 grid, cudaStream_t stream) {
  using Cfg = DecodeTmaCfg<D, NSTAGES>;
  auto kern = gqa_decode_tma_kernel<D, NSTAGES, MINB, NR>;
  static DeviceOnce once;
  int dev = 0;
  if (once.needed(&dev)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess)
      return -20;
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    once.mark(dev);
  }
  const int box_rows = p.block_size < 64 ? p.block_size : 64;
  CUtensorMap tk, tv;
  // Unknown cache size (callers on the raw C ABI): describe a view large enough for
  // any block index; only the boxes named by the block table are ever touched.
  const uint64_t rows = p.num_cache_blocks > 0
                            ? static_cast<uint64_t>(p.num_cache_blocks) * p.Hk * p.block_size
                            : (1ull << 31);
  int r = make_tensormap_2d(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.k_cache, rows, D, D, box_rows, 64,
                            CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 2000;
  r = make_tensormap_2d(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.v_cache, rows, D, D, box_rows, 64,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 3000;
  if (launch_pdl(kern, grid, dim3(Cfg::THREADS), Cfg::SMEM, stream, 1, tk, tv, p, box_rows) != cudaSuccess)
    return -21;
  if (p.splits > 1) {
    const long long warps = static_cast<long long>(grid.x) * p.Hk * (p.Hq / p.Hk) * p.q_len;
    gqa_decode_merge_kernel<D><<<static_cast<unsigned>((warps + 3) / 4), 128, 0, stream>>>(p, static_cast<int>(grid.x));
    if (cudaGetLastError() != cudaSuccess) return -22;
  }
  return 0;
}

// CTAs of the balanced persistent kernel: what is resident at once (three per SM when the shared
// memory of a CTA allows it, else two).  The scratch holds two slots per CTA.
static int balanced_ctas_per_sm(int D, int rows) {
  return DecodePersistCfg<128, 2>::smem(rows) <= 75 * 1024 && D <= 128 ? 3 : 2;
}
static int device_sms() {
  static const int sms = [] {
    int dev = 0, n = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
  }();
  return sms;
}

// At most eight query rows per kv head: the kernel variant that keeps half of every fragment.
template <int D, int NSTAGES, int MINB>
static int launch_decode_tma(const AttnParams& p, dim3 grid, cudaStream_t stream) {
  return (p.Hq / p.Hk) * p.q_len <= 8 ? launch_decode_tma_rows<D, NSTAGES, MINB, 1>(p, grid, stream)
                                      : launch_decode_tma_rows<D, NSTAGES, MINB, 2>(p, grid, stream);
}

template <int D, int NSTAGES, int MINB>
static int launch_decode_persist(const AttnParams& p, int B, cudaStream_t stream) {
  using Cfg = DecodePersistCfg<D, NSTAGES>;
  const int rows = (p.Hq / p.Hk) * p.q_len;
  // at most eight query rows per kv head: the variant that keeps half of every fragment
  auto kern = rows <= 8 ? gqa_decode_persist_kernel<D, NSTAGES, MINB, 1> : gqa_decode_persist_kernel<D, NSTAGES, MINB, 2>;
  const size_t smem = Cfg::smem(rows);
  static DeviceOnce once;
  static int sms = 148;
  int dev = 0;
  if (once.needed(&dev)) {
    if (cudaFuncSetAttribute(gqa_decode_persist_kernel<D, NSTAGES, MINB, 1>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(Cfg::smem(8))) != cudaSuccess ||
        cudaFuncSetAttribute(gqa_decode_persist_kernel<D, NSTAGES, MINB, 2>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(Cfg::smem(16))) != cudaSuccess)
      return -20;
    cudaFuncSetAttribute(gqa_decode_persist_kernel<D, NSTAGES, MINB, 1>,
                         cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    cudaFuncSetAttribute(gqa_decode_persist_kernel<D, NSTAGES, MINB, 2>,
                         cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    once.mark(dev);
  }
  const int box_rows = p.block_size < 64 ? p.block_size : 64;
  CUtensorMap tk, tv;
  const uint64_t cache_rows = p.num_cache_blocks > 0
                                  ? static_cast<uint64_t>(p.num_cache_blocks) * p.Hk * p.block_size
                                  : (1ull << 31);
  int r = make_tensormap_2d(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.k_cache, cache_rows, D, D, box_rows, 64,
                            CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 2000;
  r = make_tensormap_2d(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.v_cache, cache_rows, D, D, box_rows, 64,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 3000;
  const long long items = static_cast<long long>(B) * p.Hk * p.splits;
  if (p.persistent == 2) {
    const int grid = MINB * sms;
    if (launch_pdl(kern, dim3(grid), dim3(Cfg::THREADS), smem, stream, 1, tk, tv, p, box_rows,
                   static_cast<int>(items)) != cudaSuccess)
      return -21;
    const long long warps = static_cast<long long>(B) * p.Hk * rows;
    gqa_decode_merge_balanced_kernel<D><<<static_cast<unsigned>((warps + 3) / 4), 128, 0, stream>>>(p, B, grid);
    return cudaGetLastError() != cudaSuccess ? -22 : 0;
  }
  const int grid = static_cast<int>(items < 2LL * sms ? items : 2LL * sms);
  if (launch_pdl(kern, dim3(grid), dim3(Cfg::THREADS), smem, stream, 1, tk, tv, p, box_rows,
                 static_cast<int>(items)) != cudaSuccess)
    return -21;
  if (p.splits > 1) {
    const long long warps = static_cast<long long>(B) * p.Hk * (p.Hq / p.Hk) * p.q_len;
    gqa_decode_merge_kernel<D><<<static_cast<unsigned>((warps + 3) / 4), 128, 0, stream>>>(p, B);
    if (cudaGetLastError() != cudaSuccess) return -22;
  }
  return 0;
}

// Whether the persistent decode kernel can take this problem: TMA-compatible cache layout, at
// most 16 query rows per kv head, and query rows that a bulk copy can fetch (16-byte aligned).
static bool persist_ok(const AttnParams& p) {
  const int rows = (p.Hq / p.Hk) * p.q_len;
  const bool tma = (p.block_size % 8) == 0 && (p.block_size <= 64 ? (64 % p.block_size) == 0
                                                                   : (p.block_size % 64) == 0) &&
                   (reinterpret_cast<uintptr_t>(p.k_cache) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(p.v_cache) & 15) == 0;
  return tma && rows <= 16 && (reinterpret_cast<uintptr_t>(p.q) & 15) == 0 && ((p.q_stride * 2) & 15) == 0;
}

template <int D>
static int launch_decode(const AttnParams& p, int B, cudaStream_t stream) {
  if (p.persistent && persist_ok(p)) {
    const int rows = (p.Hq / p.Hk) * p.q_len;
    if (p.persistent == 2) {
      if (balanced_ctas_per_sm(D, rows) == 3) return launch_decode_persist<D, 2, 3>(p, B, stream);
      return rows <= 8 ? launch_decode_persist<D, 3, 2>(p, B, stream) : launch_decode_persist<D, 2, 2>(p, B, stream);
    }
    return rows <= 4 ? launch_decode_persist<D, 3, 2>(p, B, stream) : launch_decode_persist<D, 2, 2>(p, B, stream);
  }
  const bool use_tma = (p.block_size % 8) == 0 && (p.block_size <= 64 ? (64 % p.block_size) == 0
                                                                       : (p.block_size % 64) == 0) &&
                       (reinterpret_cast<uintptr_t>(p.k_cache) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(p.v_cache) & 15) == 0;
  dim3 grid(B, p.Hk, p.splits);
  if (use_tma) {
    static const int occ3 = [] {
      const char* e = getenv("OMNI_B200_DECODE_OCC3");
      return e ? atoi(e) : -1;
    }();
    // Two variants: three CTAs per SM with a two-stage ring, or two per SM with a three-stage ring.
    // A wave of the first costs about 1.3x a wave of the second (the SM's bandwidth is shared by more
    // CTAs), so it wins exactly when it saves whole waves.  Measured (B = 128, ctx 1152, us, 3/SM vs
    // 2/SM): 1024 CTAs 127 / 131, 512 CTAs 86 / 72, 384 CTAs 32 / 38, 256 CTAs 56 / 48.
    const long ctas = (long)B * p.Hk * p.splits;
    static const int sms = [] {
      int dev = 0, n = 148;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
      return n;
    }();
    const long waves2 = (ctas + 2L * sms - 1) / (2L * sms), waves3 = (ctas + 3L * sms - 1) / (3L * sms);
    const bool shallow = occ3 < 0 ? (13 * waves3 < 10 * waves2) : occ3 != 0;
    if (shallow) return launch_decode_tma<D, 2, 3>(p, grid, stream);
    return launch_decode_tma<D, 3, 2>(p, grid, stream);
  } else {
    using Cfg = DecodeCfg<D>;
    auto kern = gqa_decode_kernel<D>;
    static DeviceOnce once;
    int dev = 0;
    if (once.needed(&dev)) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) !=
          cudaSuccess)
        return -20;
      once.mark(dev);
    }
    kern<<<grid, Cfg::THREADS, Cfg::SMEM, stream>>>(p);
  }
  if (cudaGetLastError() != cudaSuccess) return -21;
  if (p.splits > 1) {
    const long long warps = static_cast<long long>(B) * p.Hk * (p.Hq / p.Hk) * p.q_len;
    gqa_decode_merge_kernel<D><<<static_cast<unsigned>((warps + 3) / 4), 128, 0, stream>>>(p, B);
    if (cudaGetLastError() != cudaSuccess) return -22;
  }
  return 0;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gqa_prefill(const void* q, const void* k_cache, const void* v_cache, void* out,
                                float* lse, const int* block_tables, const int* cu_q,
                                const int* seq_lens, int B, int max_q_len, int max_blocks,
                                int block_size, int Hq, int Hk, int Dqk, int Dv, long long q_stride,
                                long long out_stride, float scale, int causal, int window,
                                cudaStream_t stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (Hq % Hk != 0) return -1;
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
  p.window = window & 0xFFFFF;   // low 20 bits: sliding window; upper bits: leading sink tokens
  p.sink = window >> 20;
  p.q_len = 0;
  p.splits = 1;
  if (Dqk == 128 && Dv == 128) return launch_prefill<128, 128>(p, B, max_q_len, stream);
  if (Dqk == 64 && Dv == 64) return launch_prefill<64, 64>(p, B, max_q_len, stream);
  if (Dqk == 192 && Dv == 128) return launch_prefill<192, 128>(p, B, max_q_len, stream);
  return -2;
}

// Scratch needed by the decode kernel for a given split count (bytes).
extern "C" size_t b200_gqa_decode_scratch_bytes(int B, int Hk, int D, int splits) {
  if (splits <= 1) return 0;
  return static_cast<size_t>(B) * Hk * splits * 16 * (static_cast<size_t>(D) + 2) * sizeof(float);
}

// Scratch of the balanced persistent decode kernel: two slots of 16 rows per CTA.
extern "C" size_t b200_gqa_decode_balanced_scratch_bytes(int D, int rows) {
  const size_t slots = 2 * static_cast<size_t>(balanced_ctas_per_sm(D, rows)) * device_sms();
  return slots * 16 * (static_cast<size_t>(D) + 2) * sizeof(float);
}

// persistent: 0 = one CTA per (sequence, kv head, split) item; 1 = persistent CTAs that take items
// from a counter (work_counter: two ints, zero at rest, or null for striding); 2 = persistent CTAs
// over a balanced cut of the tiles (splits is ignored, scratch of
// b200_gqa_decode_balanced_scratch_bytes required).  1 and 2 fall back to 0 when the problem does
// not fit the persistent kernel.
extern "C" int b200_gqa_decode_ex(const void* q, const void* k_cache, const void* v_cache, void* out,
                                  float* lse, const int* block_tables, const int* seq_lens, int B,
                                  int q_len, int max_blocks, int block_size, int Hq, int Hk, int D,
                                  long long q_stride, long long out_stride, float scale, int window,
                                  int splits, void* scratch, int num_cache_blocks, int* status,
                                  int persistent, int* work_counter, cudaStream_t stream);

extern "C" int b200_gqa_decode(const void* q, const void* k_cache, const void* v_cache, void* out,
                               float* lse, const int* block_tables, const int* seq_lens, int B,
                               int q_len, int max_blocks, int block_size, int Hq, int Hk, int D,
                               long long q_stride, long long out_stride, float scale, int window,
                               int splits, void* scratch, int num_cache_blocks, int* status,
                               cudaStream_t stream) {
  return b200_gqa_decode_ex(q, k_cache, v_cache, out, lse, block_tables, seq_lens, B, q_len, max_blocks,
                            block_size, Hq, Hk, D, q_stride, out_stride, scale, window, splits, scratch,
                            num_cache_blocks, status, 0, nullptr, stream);
}

extern "C" int b200_gqa_decode_ex(const void* q, const void* k_cache, const void* v_cache, void* out,
                                  float* lse, const int* block_tables, const int* seq_lens, int B,
                                  int q_len, int max_blocks, int block_size, int Hq, int Hk, int D,
                                  long long q_stride, long long out_stride, float scale, int window,
                                  int splits, void* scratch, int num_cache_blocks, int* status,
                                  int persistent, int* work_counter, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (Hq % Hk != 0 || (Hq / Hk) * q_len > 16 || q_len < 1) return -1;
  if (splits < 1) splits = 1;
  if (persistent == 2) splits = 1;
  if ((splits > 1 || persistent == 2) && scratch == nullptr) return -3;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.block_tables = block_tables;
  p.cu_q = nullptr;
  p.seq_lens = seq_lens;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  p.Hq = Hq;
  p.Hk = Hk;
  p.q_stride = q_stride;
  p.out_stride = out_stride;
  p.scale_log2 = scale * kLog2e;
  p.causal = 1;
  p.window = window & 0xFFFFF;   // low 20 bits: sliding window; upper bits: leading sink tokens
  p.sink = window >> 20;
  p.q_len = q_len;
  p.splits = splits;
  p.status = status;
  p.num_cache_blocks = num_cache_blocks;
  p.persistent = persistent;
  p.work_counter = work_counter;
  if (splits > 1) {
    p.o_part = static_cast<float*>(scratch);
    p.lse_part = p.o_part + static_cast<size_t>(B) * Hk * splits * 16 * D;
  }
  if (persistent == 2) {
    if (!persist_ok(p)) {
      p.persistent = 0;       // one CTA per item, keys not split
    } else {
      const size_t slots = 2 * static_cast<size_t>(balanced_ctas_per_sm(D, (Hq / Hk) * q_len)) * device_sms();
      p.o_part = static_cast<float*>(scratch);
      p.lse_part = p.o_part + slots * 16 * D;
    }
  }
  if (D == 128) return launch_decode<128>(p, B, stream);
  if (D == 64) return launch_decode<64>(p, B, stream);
  return -2;
}

#ifdef B200_ATTN_TIMELINE
extern "C" int b200_gqa_decode_timeline(unsigned long long* host, int ctas) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, b200::g_attn_timeline, sizeof(unsigned long long) * 8 * ctas));
}
#endif
