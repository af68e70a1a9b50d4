// Multi-head latent attention, absorbed (MQA) form, over the paged latent cache.
//
//   cache row  = [ c_kv (512) | k_pe (64) ]                 one row per token, shared by all heads
//   query row  = [ q_nope . W_UK (512) | q_pe (64) ]       per head
//   out[h]     = softmax(q[h] . cache^T * scale) . c_kv     (512 wide; W_UV is applied by the caller)
//
// One CTA handles 16 query rows (heads) of one sequence (and one query token for
// multi-token decode) over one split of the keys.  K tiles of 64 tokens x 576
// dims come in through TMA (nine 64-column slabs, 128B swizzle) into a two-stage
// ring, issued by a producer warp.  Four compute warps:
//   QK^T : warp w scores keys 16w..16w+15 of the tile (K = 576),
//   softmax: tile-wide row max / sum through shared memory, P stored as bf16,
//   P.V  : warp w accumulates output columns 128w..128w+127 over all 64 keys.
// Split-KV partials are merged by a second kernel.  All waits are bounded.
//
// Replaces the decode call of npu_fused_infer_attention_score over the latent
// cache (omni_npu/attention/backends/mla.py:695-804,
// omni_npu/v1/layers/attention/npu_mla.py:169-242) and, restricted to selected
// tokens, npu_sparse_flash_attention (omni_npu/v1/layers/attention/npu_dsa.py:341,570).

#include "attn_common.cuh"
#include "../common/tensormap.h"
#include "../common/device_once.h"

namespace b200 {

static constexpr float kMlaLog2e = 1.4426950408889634f;
static constexpr int kLat = 512;
static constexpr int kRope = 64;
static constexpr int kRow = kLat + kRope;     // 576
static constexpr int kSlabs = kRow / 64;      // 9
static constexpr int kMlaBN = 64;
static constexpr int kMlaStages = 2;
static constexpr int kSlabBytes = kMlaBN * 128;           // 8 KB
static constexpr int kTileBytes = kSlabs * kSlabBytes;    // 72 KB
static constexpr int kQBytes = kSlabs * 16 * 128;         // 18 KB
static constexpr int kPBytes = 16 * kMlaBN * 2;           // 2 KB
static constexpr int kMlaSmem = 1024 + kMlaStages * kTileBytes + kQBytes + kPBytes + 4096;

struct MlaParams {
  const __nv_bfloat16* q;        // [T, N, 576]
  __nv_bfloat16* out;            // [T, N, 512]
  float* lse;                    // [T, N] or null
  const int* block_tables;       // [B, max_blocks]
  const int* seq_lens;           // [B]
  const int* topk_indices;       // sparse mode: [T, topk] token positions (-1 = none) or null
  int topk;
  int max_blocks, block_size;
  int N;                         // heads
  int q_len;                     // query tokens per sequence (uniform)
  long long q_stride, out_stride;  // elements between tokens
  float scale_log2;
  int splits;
  float* o_part;                 // [B*q_len, head_tiles, splits, 16, 512]
  float* ml_part;                // [.., 16, 2]
  int* status;
};

// offset of 16-byte chunk `chunk` (0..71) of row `row` in a slab-major swizzled tile
__device__ __forceinline__ uint32_t mla_off(int row, int chunk, int rows_per_slab) {
  return static_cast<uint32_t>((chunk >> 3) * rows_per_slab * 128 + row * 128 +
                               (((chunk & 7) ^ (row & 7)) << 4));
}

__global__ void __launch_bounds__(160)
mla_decode_kernel(const __grid_constant__ CUtensorMap tm_c, const MlaParams p, const int box_rows) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sKV = smem;
  uint8_t* sQ = sKV + kMlaStages * kTileBytes;
  uint8_t* sP = sQ + kQBytes;                                  // [16][64] bf16, swizzled rows of 128 B
  float* s_red = reinterpret_cast<float*>(sP + kPBytes);       // [2][4][16] max / sum exchange
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(s_red + 128);
  uint64_t* empty_bar = full_bar + kMlaStages;
  int* s_abort = reinterpret_cast<int*>(empty_bar + kMlaStages);
  int* s_bt = s_abort + 4;                                     // up to 512 block-table entries

  const int tok = blockIdx.x;                 // b * q_len + qi
  const int b = tok / p.q_len;
  const int qi = tok % p.q_len;
  const int head0 = blockIdx.y * 16;
  const int split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int seq_len = p.seq_lens[b];
  const int kv_len = p.topk_indices ? p.topk : (seq_len - p.q_len + qi + 1);   // causal limit
  const int* bt = p.block_tables + static_cast<long long>(b) * p.max_blocks;
  const int* sel = p.topk_indices ? p.topk_indices + static_cast<long long>(tok) * p.topk : nullptr;

  const int n_tiles_all = (max(kv_len, 0) + kMlaBN - 1) / kMlaBN;
  const int per = (n_tiles_all + p.splits - 1) / p.splits;
  const int t_begin = split * per;
  const int t_end = min(n_tiles_all, t_begin + per);
  const int n_tiles = max(0, t_end - t_begin);

  if (tid == 0) {
    for (int s = 0; s < kMlaStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 4);
    }
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_c);
  }
  {
    uint4* z = reinterpret_cast<uint4*>(sKV);
    for (int i = tid; i < kMlaStages * kTileBytes / 16; i += 160) z[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  const int bt_first = sel ? 0 : (t_begin * kMlaBN) / p.block_size;
  const int bt_last = sel ? 0 : min(p.max_blocks, (min(kv_len, t_end * kMlaBN) + p.block_size - 1) / p.block_size);
  const bool bt_cached = !sel && (bt_last - bt_first) <= 512;
  if (bt_cached)
    for (int i = bt_first + tid; i < bt_last; i += 160) s_bt[i - bt_first] = bt[i];
  fence_proxy_async();
  __syncthreads();
  volatile int* abort_flag = s_abort;

  if (warp == 4) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int issued = 0;
      for (int it = 0; it < n_tiles; ++it) {
        const int stage = it % kMlaStages;
        if (it >= kMlaStages) {
          const uint32_t parity = static_cast<uint32_t>(((it / kMlaStages) - 1) & 1);
          if (*abort_flag || !mbar_wait(&empty_bar[stage], parity)) {
            if (!*abort_flag && p.status) atomicCAS(p.status, 0, kStatusTimeoutEmptyBarrier);
            *abort_flag = 1;
            break;
          }
        }
        const int n0 = (t_begin + it) * kMlaBN;
        const int nvalid = min(kMlaBN, kv_len - n0);
        uint8_t* dst_tile = sKV + stage * kTileBytes;
        if (!sel) {
          const int nboxes = (nvalid + box_rows - 1) / box_rows;
          mbar_arrive_expect_tx(&full_bar[stage], static_cast<uint32_t>(nboxes * box_rows * 128 * kSlabs));
          for (int j = 0; j < nboxes; ++j) {
            const int key = n0 + j * box_rows;
            const int bi = key / p.block_size;
            const int blk = bt_cached ? s_bt[bi - bt_first] : bt[bi];
            const int row = blk * p.block_size + key % p.block_size;
#pragma unroll
            for (int s = 0; s < kSlabs; ++s)
              tma_load_2d(dst_tile + s * kSlabBytes + j * box_rows * 128, &tm_c, &full_bar[stage], s * 64, row);
          }
        } else {
          // sparse: one row per selected token (negative index = hole, left zero-scored)
          int nrows = 0;
          for (int j = 0; j < nvalid; ++j) nrows += sel[n0 + j] >= 0 ? 1 : 0;
          mbar_arrive_expect_tx(&full_bar[stage], static_cast<uint32_t>(nrows * 128 * kSlabs));
          for (int j = 0; j < nvalid; ++j) {
            const int pos = sel[n0 + j];
            if (pos < 0) continue;
            const int row = bt[pos / p.block_size] * p.block_size + pos % p.block_size;
#pragma unroll
            for (int s = 0; s < kSlabs; ++s)
              tma_load_2d(dst_tile + s * kSlabBytes + j * 128, &tm_c, &full_bar[stage], s * 64, row);
          }
        }
        ++issued;
      }
      if (*abort_flag) {
        const int first = issued > kMlaStages ? issued - kMlaStages : 0;
        for (int i = first; i < issued; ++i)
          mbar_wait(&full_bar[i % kMlaStages], static_cast<uint32_t>((i / kMlaStages) & 1));
      }
    }
    __syncthreads();
    return;
  }

  // -------------------------------------------------------------- consumers
  for (int idx = tid; idx < 16 * 72; idx += 128) {
    const int row = idx / 72, c = idx % 72;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (head0 + row < p.N)
      v = *reinterpret_cast<const uint4*>(p.q + static_cast<long long>(tok) * p.q_stride +
                                          static_cast<long long>(head0 + row) * kRow + c * 8);
    *reinterpret_cast<uint4*>(sQ + mla_off(row, c, 16)) = v;
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");

  float o_acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY};
  float row_sum[2] = {0.f, 0.f};
  const int r_a = lane >> 2;

  for (int it = 0; it < n_tiles; ++it) {
    const int stage = it % kMlaStages;
    bool ok = !*abort_flag && mbar_wait(&full_bar[stage], static_cast<uint32_t>((it / kMlaStages) & 1));
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
      if (lane == 0) {
        if (!*abort_flag && p.status) atomicCAS(p.status, 0, kStatusTimeoutFullBarrier);
        *abort_flag = 1;
      }
    }
    // the decision must be uniform across the four warps (they share barriers below)
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
      if (!all_ok) break;
    }
    const uint32_t kt = smem_u32(sKV + stage * kTileBytes);
    const int n0 = (t_begin + it) * kMlaBN;

    // ---- S = Q K^T for this warp's 16 keys
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 4
    for (int ks = 0; ks < kRow / 16; ++ks) {
      uint32_t qf[4], kf[4];
      ldmatrix_x4(qf, smem_u32(sQ) + mla_off(lane & 15, ks * 2 + (lane >> 4), 16));
      const int krow = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
      ldmatrix_x4(kf, kt + mla_off(krow, ks * 2 + ((lane >> 3) & 1), kMlaBN));
      mma_bf16_16816(s[0], qf, kf[0], kf[1]);
      mma_bf16_16816(s[1], qf, kf[2], kf[3]);
    }
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = n0 + warp * 16 + i * 8 + (lane & 3) * 2 + (j & 1);
        bool keep = key < kv_len;
        if (sel && keep) keep = sel[key] >= 0;
        const float v = keep ? s[i][j] * p.scale_log2 : -INFINITY;
        s[i][j] = v;
        tmax[j >> 1] = fmaxf(tmax[j >> 1], v);
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tmax[r] = quad_max(tmax[r]);
      if ((lane & 3) == 0) s_red[warp * 16 + r_a + 8 * r] = tmax[r];
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = r_a + 8 * r;
      const float tm = fmaxf(fmaxf(s_red[row], s_red[16 + row]), fmaxf(s_red[32 + row], s_red[48 + row]));
      const float nm = fmaxf(row_max[r], tm);
      corr[r] = (nm == -INFINITY) ? 1.f : exp2f(row_max[r] - nm);
      row_max[r] = nm;
      m_use[r] = nm == -INFINITY ? 0.f : nm;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float e = exp2f(s[i][j] - m_use[j >> 1]);
        s[i][j] = e;
        psum[j >> 1] += e;
      }
    // P (bf16) -> shared: row r, keys warp*16 + i*8 + (lane&3)*2
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int row = r_a + 8 * r;
        const int key = warp * 16 + i * 8 + (lane & 3) * 2;
        const uint32_t v = pack_bf16x2(s[i][2 * r], s[i][2 * r + 1]);
        *reinterpret_cast<uint32_t*>(sP + row * 128 + (((key >> 3) ^ (row & 7)) << 4) + (key & 7) * 2) = v;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      psum[r] = quad_sum(psum[r]);
      if ((lane & 3) == 0) s_red[64 + warp * 16 + r_a + 8 * r] = psum[r];
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = r_a + 8 * r;
      row_sum[r] = row_sum[r] * corr[r] + s_red[64 + row] + s_red[80 + row] + s_red[96 + row] + s_red[112 + row];
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o_acc[i][0] *= corr[0];
      o_acc[i][1] *= corr[0];
      o_acc[i][2] *= corr[1];
      o_acc[i][3] *= corr[1];
    }
    // ---- O[:, 128w : 128w+128] += P V
#pragma unroll
    for (int ks = 0; ks < kMlaBN / 16; ++ks) {
      uint32_t pf[4];
      {
        const int prow = lane & 15;
        const int pchunk = ks * 2 + (lane >> 4);
        ldmatrix_x4(pf, smem_u32(sP) + prow * 128 + ((pchunk ^ (prow & 7)) << 4));
      }
#pragma unroll
      for (int dt = 0; dt < 8; ++dt) {
        uint32_t vf[4];
        const int vrow = ks * 16 + (lane & 15);
        const int vchunk = warp * 16 + dt * 2 + (lane >> 4);
        ldmatrix_x4_trans(vf, kt + mla_off(vrow, vchunk, kMlaBN));
        mma_bf16_16816(o_acc[2 * dt], pf, vf[0], vf[1]);
        mma_bf16_16816(o_acc[2 * dt + 1], pf, vf[2], vf[3]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[stage]);
    // P and the reduction scratch are rewritten next tile: everyone must be done reading
    asm volatile("bar.sync 1, 128;" ::: "memory");
  }
  __syncthreads();
  if (*abort_flag) return;

  // ---- write: every thread owns rows r_a, r_a+8 and 32 columns of its warp's slice
  const size_t part_row = ((static_cast<size_t>(tok) * gridDim.y + blockIdx.y) * p.splits + split) * 16;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r_a + 8 * r;
    if (head0 + row >= p.N) continue;
    const float l = row_sum[r];
    if (p.splits == 1) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + static_cast<long long>(tok) * p.out_stride +
                           static_cast<long long>(head0 + row) * kLat + warp * 128;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int col = i * 8 + (lane & 3) * 2;
        *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16x2(o_acc[i][2 * r] * inv, o_acc[i][2 * r + 1] * inv);
      }
      if (p.lse && warp == 0 && (lane & 3) == 0)
        p.lse[static_cast<long long>(tok) * p.N + head0 + row] =
            l > 0.f ? (row_max[r] + log2f(l)) / kMlaLog2e : -INFINITY;
    } else {
      float* dst = p.o_part + (part_row + row) * kLat + warp * 128;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int col = i * 8 + (lane & 3) * 2;
        *reinterpret_cast<float2*>(dst + col) = make_float2(o_acc[i][2 * r], o_acc[i][2 * r + 1]);
      }
      if (warp == 0 && (lane & 3) == 0) {
        p.ml_part[(part_row + row) * 2] = row_max[r];
        p.ml_part[(part_row + row) * 2 + 1] = l;
      }
    }
  }
}

// one warp per (token, head): merge split partials
__global__ void __launch_bounds__(128)
mla_merge_kernel(const MlaParams p, int total_tokens, int head_tiles) {
  const long long gw = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (gw >= static_cast<long long>(total_tokens) * p.N) return;
  const int lane = threadIdx.x & 31;
  const int head = static_cast<int>(gw % p.N);
  const int tok = static_cast<int>(gw / p.N);
  const size_t base = ((static_cast<size_t>(tok) * head_tiles + head / 16) * p.splits) * 16 + head % 16;
  float m = -INFINITY;
  for (int s = 0; s < p.splits; ++s) m = fmaxf(m, p.ml_part[(base + static_cast<size_t>(s) * 16) * 2]);
  float l = 0.f;
  float acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.f;
  for (int s = 0; s < p.splits; ++s) {
    const size_t pr = base + static_cast<size_t>(s) * 16;
    const float ms = p.ml_part[pr * 2];
    const float f = ms == -INFINITY ? 0.f : exp2f(ms - m);
    l += p.ml_part[pr * 2 + 1] * f;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] += p.o_part[pr * kLat + i * 32 + lane] * f;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  __nv_bfloat16* dst = p.out + static_cast<long long>(tok) * p.out_stride + static_cast<long long>(head) * kLat;
#pragma unroll
  for (int i = 0; i < 16; ++i) dst[i * 32 + lane] = __float2bfloat16(acc[i] * inv);
  if (p.lse && lane == 0)
    p.lse[static_cast<long long>(tok) * p.N + head] = l > 0.f ? (m + log2f(l)) / kMlaLog2e : -INFINITY;
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_mla_decode_scratch_bytes(int total_tokens, int N, int splits) {
  if (splits <= 1) return 0;
  const size_t tiles = (N + 15) / 16;
  return static_cast<size_t>(total_tokens) * tiles * splits * 16 * (kLat + 2) * sizeof(float);
}

// q [T, N*576]; cache [num_blocks, block_size, 576]; out [T, N*512].  T = B * q_len.
// topk_indices (optional) [T, topk]: attend only to these token positions.
extern "C" int b200_mla_decode(const void* q, const void* cache, void* out, float* lse,
                               const int* block_tables, const int* seq_lens, const int* topk_indices,
                               int topk, int B, int q_len, int N, int max_blocks, int block_size,
                               int num_cache_blocks, long long q_stride, long long out_stride,
                               float scale, int splits, void* scratch, int* status,
                               cudaStream_t stream) {
  if (B <= 0) return 0;
  if (splits < 1) splits = 1;
  if (splits > 1 && scratch == nullptr) return -3;
  if ((block_size % 8) != 0 || !(block_size <= 64 ? (64 % block_size) == 0 : (block_size % 64) == 0)) return -4;
  static DeviceOnce once;
  int cur_dev = 0;
  if (once.needed(&cur_dev)) {
    if (cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmem) != cudaSuccess)
      return -20;
    once.mark(cur_dev);
  }
  MlaParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.block_tables = block_tables;
  p.seq_lens = seq_lens;
  p.topk_indices = topk_indices;
  p.topk = topk;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  p.N = N;
  p.q_len = q_len;
  p.q_stride = q_stride;
  p.out_stride = out_stride;
  p.scale_log2 = scale * kMlaLog2e;
  p.splits = splits;
  p.status = status;
  const int T = B * q_len;
  const int tiles = (N + 15) / 16;
  if (splits > 1) {
    p.o_part = static_cast<float*>(scratch);
    p.ml_part = p.o_part + static_cast<size_t>(T) * tiles * splits * 16 * kLat;
  }
  const int box_rows = topk_indices ? 1 : (block_size < 64 ? block_size : 64);
  CUtensorMap tm;
  const uint64_t rows = num_cache_blocks > 0 ? static_cast<uint64_t>(num_cache_blocks) * block_size : (1ull << 31);
  int r = make_tensormap_2d(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, cache, rows, kRow, kRow, box_rows, 64,
                            CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 2000;
  dim3 grid(T, tiles, splits);
  mla_decode_kernel<<<grid, 160, kMlaSmem, stream>>>(tm, p, box_rows);
  if (cudaGetLastError() != cudaSuccess) return -21;
  if (splits > 1) {
    const long long warps = static_cast<long long>(T) * N;
    mla_merge_kernel<<<static_cast<unsigned>((warps + 3) / 4), 128, 0, stream>>>(p, T, tiles);
    if (cudaGetLastError() != cudaSuccess) return -22;
  }
  return 0;
}
