// Sparse-attention indexer for sm_100a: index scores on the tensor cores, then a radix
// select of the best `topk` key positions per query token.
//
//   score[t, j] = sum_h  w[t, h] * relu( q[t, h, :] . k[j, :] )        j <= position of t
//
// q [T, H, 128] bf16 (H heads of 128 dims, H * tokens-per-MMA <= 256), w [T, H] fp32 (the
// caller folds the softmax scale and H^-1/2 into it), k: a paged cache of 128-dim bf16 keys
// addressed through the sequences' block tables.
//
// Score kernel.  One CTA owns a run of 128-key tiles of one sequence.  A key tile is the
// M operand of tcgen05.mma (128 keys x 128 dims, two 128-byte-swizzled K slabs written by
// one TMA box per cache page), a group of `ntok` query tokens is the N operand
// (ntok * H head rows x 128 dims); the accumulator [128 keys x ntok * H] lives in TMEM,
// double buffered.  Warp 0 issues TMA, warp 1 issues MMA, warps 2-5 read the accumulator
// (each thread owns one key row), apply relu and the head weights, sum over heads in
// registers and store one score per (token, key): no cross-thread reduction at all.
// Key tiles above a token's position are never visited for that token.
//
// Select kernel.  One CTA per query token: four 8-bit histogram passes over the valid
// prefix of the score row find the exact value of the topk-th best score, a last pass emits
// the positions (unordered; ties at the threshold are broken arbitrarily).  Rows with at
// most topk valid keys select every key.  Unused slots are -1.
//
// Every wait is bounded; a timeout records a status code and the CTA drains and exits.
//
// Counterpart of the reference's closed indexer ops (torch.ops.custom.npu_lightning_indexer,
// omni_npu/v1/layers/attention/npu_dsa.py:37-142).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/pdl.cuh"
#include "../common/ptx.cuh"
#include "../common/tensormap.h"
#include "../common/device_once.h"

namespace b200 {

constexpr int kIdxD = 128;                 // index head dim (two 64-element slabs)
constexpr int kIdxBK = 128;                // keys per tile = MMA M
constexpr int kIdxSlabBytes = kIdxBK * 128;  // one K slab of a key tile
constexpr int kIdxKeyBytes = 2 * kIdxSlabBytes;
constexpr int kIdxThreads = 192;

struct IndexerParams {
  const float* w;          // [T, H]
  float* scores;           // [T, ld]
  long long ld;
  const int* block_tables;  // [B, max_blocks]
  int max_blocks;
  int block_size;
  int box_rows;            // rows per TMA box of the key cache
  const int* cu_q;         // [B + 1] first query token of every sequence, or null: b * q_len
  const int* positions;    // [T] absolute position of every query token
  int q_len;
  int H;
  int ntok;                // query tokens per MMA: N = ntok * H
  int tiles_per_cta;
  int q_split;             // grid.z: the token groups of a sequence are divided over this many CTAs
  int tmem_cols;
  int* status;
};

__global__ void __launch_bounds__(kIdxThreads)
dsa_indexer_scores_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_q,
                          const IndexerParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int N = p.ntok * p.H;
  const int q_slab_bytes = N * 128;
  const int q_bytes = 2 * q_slab_bytes;
  uint8_t* s_keys = smem;                                   // [2][kIdxKeyBytes]
  uint8_t* s_q = s_keys + 2 * kIdxKeyBytes;                 // [2][q_bytes]
  float* s_w = reinterpret_cast<float*>(s_q + 2 * q_bytes);  // [2][N]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_w + 2 * N);
  uint64_t* key_full = bars;          // [2]
  uint64_t* key_empty = bars + 2;     // [2]
  uint64_t* q_full = bars + 4;        // [2]
  uint64_t* q_empty = bars + 6;       // [2]
  uint64_t* acc_full = bars + 8;      // [2]
  uint64_t* acc_empty = bars + 10;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);

  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.y;
  const int qs = p.cu_q ? p.cu_q[b] : b * p.q_len;
  const int qe = p.cu_q ? p.cu_q[b + 1] : (b + 1) * p.q_len;
  const int nq = qe - qs;
  if (nq <= 0) return;
  const int pos0 = p.positions[qs];
  const int kv_limit = pos0 + nq;                           // keys 0 .. position of the last query token
  const int n_key_tiles = (kv_limit + kIdxBK - 1) / kIdxBK;
  const int kt_begin = blockIdx.x * p.tiles_per_cta;
  const int kt_end = min(n_key_tiles, kt_begin + p.tiles_per_cta);
  if (pos0 < 0 || kt_begin >= kt_end) return;               // uniform over the CTA: nothing allocated yet
  const int groups_all = (nq + p.ntok - 1) / p.ntok;
  // this CTA's share of the token groups: [gz0, groups)
  const int per_z = (groups_all + p.q_split - 1) / p.q_split;
  const int gz0 = blockIdx.z * per_z;
  const int groups = min(groups_all, gz0 + per_z);
  if (gz0 >= groups) return;
  const bool single_q = groups - gz0 == 1;                  // the one query group stays resident
  const int* bt = p.block_tables + static_cast<long long>(b) * p.max_blocks;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&key_full[i], 1);
      mbar_init(&key_empty[i], 1);
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);
    }
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_q);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int acc_stride = p.tmem_cols >> 1;
  volatile int* abort_flag = s_abort;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int ks = 0, qst = 0;
      uint32_t kph = 0, qph = 0;
      bool q_loaded = false, ok = true;
      uint64_t* last_bar = nullptr;
      uint32_t last_par = 0;
      for (int kt = kt_begin; ok && kt < kt_end; ++kt) {
        const int k0 = kt * kIdxBK;
        const int g_begin = max(max(0, k0 - pos0) / p.ntok, gz0);
        if (g_begin >= groups) continue;           // none of this CTA's tokens sees the tile
        if (!mbar_wait(&key_empty[ks], kph ^ 1)) {
          ok = false;
          break;
        }
        const int nvalid = min(kIdxBK, kv_limit - k0);
        const int nboxes = (nvalid + p.box_rows - 1) / p.box_rows;
        mbar_arrive_expect_tx(&key_full[ks], static_cast<uint32_t>(nboxes * p.box_rows * 128 * 2));
        for (int j = 0; j < nboxes; ++j) {
          const int key = k0 + j * p.box_rows;
          const int row = bt[key / p.block_size] * p.block_size + key % p.block_size;
          uint8_t* dst = s_keys + ks * kIdxKeyBytes + j * p.box_rows * 128;
          tma_load_2d(dst, &tm_k, &key_full[ks], 0, row);
          tma_load_2d(dst + kIdxSlabBytes, &tm_k, &key_full[ks], 64, row);
        }
        last_bar = &key_full[ks];
        last_par = kph;
        for (int g = g_begin; ok && g < groups; ++g) {
          if (single_q && q_loaded) break;
          if (!mbar_wait(&q_empty[qst], qph ^ 1)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&q_full[qst], static_cast<uint32_t>(q_bytes));
          const int row = (qs + g * p.ntok) * p.H;
          tma_load_2d(s_q + qst * q_bytes, &tm_q, &q_full[qst], 0, row);
          tma_load_2d(s_q + qst * q_bytes + q_slab_bytes, &tm_q, &q_full[qst], 64, row);
          q_loaded = true;
          if (++qst == 2) {
            qst = 0;
            qph ^= 1;
          }
        }
        if (++ks == 2) {
          ks = 0;
          kph ^= 1;
        }
      }
      if (!ok) {
        atomicCAS(p.status, 0, kStatusTimeoutEmptyBarrier);
        *abort_flag = 1;
        if (last_bar) mbar_wait(last_bar, last_par);   // no bulk copy may land after the CTA retires
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(1, 1, kIdxBK, static_cast<uint32_t>(N));
      int ks = 0, qst = 0, acc = 0;
      uint32_t kph = 0, qph = 0, aph = 0;
      bool q_seen = false, ok = true;
      for (int kt = kt_begin; ok && kt < kt_end; ++kt) {
        const int k0 = kt * kIdxBK;
        const int g_begin = max(max(0, k0 - pos0) / p.ntok, gz0);
        if (g_begin >= groups) continue;
        if (*abort_flag || !mbar_wait(&key_full[ks], kph)) {
          ok = false;
          break;
        }
        const uint32_t a_lo0 = (smem_u32(s_keys + ks * kIdxKeyBytes) & 0x3FFFF) >> 4;
        for (int g = g_begin; g < groups; ++g) {
          if (!(single_q && q_seen)) {
            if (*abort_flag || !mbar_wait(&q_full[qst], qph)) {
              ok = false;
              break;
            }
            q_seen = true;
          }
          if (!mbar_wait(&acc_empty[acc], aph ^ 1)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const int qbuf = single_q ? 0 : qst;
          const uint32_t b_lo0 = (smem_u32(s_q + qbuf * q_bytes) & 0x3FFFF) >> 4;
          const uint32_t d = tmem_base + static_cast<uint32_t>(acc * acc_stride);
#pragma unroll
          for (int s = 0; s < 2; ++s) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(s * (kIdxSlabBytes >> 4) + kk * 2);
              const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(s * (q_slab_bytes >> 4) + kk * 2);
              if (s == 0 && kk == 0) umma_first<kKindBF16>(d, a_lo, b_lo, idesc, 0u);
              else umma_acc<kKindBF16>(d, a_lo, b_lo, idesc);
            }
          }
          tc_commit(&acc_full[acc]);
          if (!single_q) {
            tc_commit(&q_empty[qst]);
            if (++qst == 2) {
              qst = 0;
              qph ^= 1;
            }
          }
          if (g == groups - 1) tc_commit(&key_empty[ks]);
          if (++acc == 2) {
            acc = 0;
            aph ^= 1;
          }
        }
        if (++ks == 2) {
          ks = 0;
          kph ^= 1;
        }
      }
      if (!ok) {
        atomicCAS(p.status, 0, kStatusTimeoutFullBarrier);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    const int et = threadIdx.x - 64;                 // 0..127 over the four epilogue warps
    const int r = quarter * 32 + lane;               // key row inside the tile
    int acc = 0;
    uint32_t aph = 0;
    bool ok = true;
    for (int kt = kt_begin; ok && kt < kt_end; ++kt) {
      const int k0 = kt * kIdxBK;
      const int key = k0 + r;
      const int g_begin = max(max(0, k0 - pos0) / p.ntok, gz0);
      for (int g = g_begin; g < groups; ++g) {
        const int t0 = g * p.ntok;                   // first token of the group, relative to qs
        float* wbuf = s_w + acc * N;
        for (int i = et; i < N; i += 128) {
          const int tok = t0 + i / p.H;
          wbuf[i] = tok < nq ? p.w[static_cast<long long>(qs + tok) * p.H + (i % p.H)] : 0.f;
        }
        {
          // one verdict for all four warps (they meet at the barrier either way), so that
          // no warp leaves the loop while another still expects it at the next barrier
          const bool mine = !*abort_flag && mbar_wait(&acc_full[acc], aph);
          uint32_t all_ok;
          asm volatile(
              "{\n\t"
              ".reg .pred p, q;\n\t"
              "setp.ne.u32 q, %1, 0;\n\t"
              "bar.red.and.pred p, 1, 128, q;\n\t"
              "selp.u32 %0, 1, 0, p;\n\t"
              "}"
              : "=r"(all_ok)
              : "r"(mine ? 1u : 0u)
              : "memory");
          if (!all_ok) {
            ok = false;
            break;
          }
        }
        tc_fence_after_sync();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                               static_cast<uint32_t>(acc * acc_stride);
        for (int j = 0; j < p.ntok; ++j) {
          float sum = 0.f;
          if ((p.H & 63) == 0) {
            // 64 columns in flight per wait: the load latency is paid once per 64 heads
            for (int c = 0; c < p.H; c += 64) {
              uint32_t v0[32], v1[32];
              tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(j * p.H + c), v0);
              tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(j * p.H + c + 32), v1);
              tmem_ld_wait();
              const float* wj = wbuf + j * p.H + c;
#pragma unroll
              for (int i = 0; i < 32; ++i) sum += wj[i] * fmaxf(__uint_as_float(v0[i]), 0.f);
#pragma unroll
              for (int i = 0; i < 32; ++i) sum += wj[32 + i] * fmaxf(__uint_as_float(v1[i]), 0.f);
            }
          } else {
            for (int c = 0; c < p.H; c += 16) {
              uint32_t v[16];
              asm volatile(
                  "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                  "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                  : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                    "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
                    "=r"(v[15])
                  : "r"(t_row + static_cast<uint32_t>(j * p.H + c))
                  : "memory");
              tmem_ld_wait();
              const float* wj = wbuf + j * p.H + c;
#pragma unroll
              for (int i = 0; i < 16; ++i) sum += wj[i] * fmaxf(__uint_as_float(v[i]), 0.f);
            }
          }
          const int tok = t0 + j;
          if (tok < nq && key < p.ld)
            p.scores[static_cast<long long>(qs + tok) * p.ld + key] = key <= pos0 + tok ? sum : -INFINITY;
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        if (++acc == 2) {
          acc = 0;
          aph ^= 1;
        }
      }
    }
    if (!ok && lane == 0) {
      atomicCAS(p.status, 0, kStatusTimeoutTmemFull);
      *abort_flag = 1;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}

// ------------------------------------------------------------------------ radix select
__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);     // larger float <=> larger key
}

constexpr int kSelThreads = 512;

// Adds 1 to hist[bin] for every active lane; lanes that hit the same bin are combined into one
// shared-memory atomic (scores of one row share their leading bytes, so without this the first
// passes serialise thousands of atomics on two or three addresses).
__device__ __forceinline__ void hist_add(uint32_t* hist, uint32_t bin, bool active) {
  const uint32_t peers = __match_any_sync(0xffffffffu, active ? bin : 0xffffffffu);
  if (active && (__ffs(peers) - 1) == static_cast<int>(threadIdx.x & 31)) atomicAdd(&hist[bin], __popc(peers));
}

// Slot reservation for the lanes with `take` set: one atomic per warp, lanes get consecutive slots.
__device__ __forceinline__ uint32_t warp_reserve(uint32_t* counter, bool take) {
  const uint32_t mask = __ballot_sync(0xffffffffu, take);
  uint32_t base = 0;
  if (mask != 0u) {
    const int leader = __ffs(mask) - 1;
    if (static_cast<int>(threadIdx.x & 31) == leader) base = atomicAdd(counter, __popc(mask));
    base = __shfl_sync(0xffffffffu, base, leader);
  }
  return base + __popc(mask & ((1u << (threadIdx.x & 31)) - 1u));
}

__global__ void __launch_bounds__(kSelThreads)
dsa_indexer_select_kernel(int* __restrict__ out, const float* __restrict__ scores, long long ld,
                          const int* __restrict__ positions, int topk) {
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_mask, s_krem, s_cnt, s_eq;
  pdl_trigger();
  pdl_wait();
  const long long t = blockIdx.x;
  const float* row = scores + t * ld;
  int* o = out + t * topk;
  const int pos = positions[t];
  const int n = static_cast<int>(min(static_cast<long long>(max(pos + 1, 0)), ld));
  if (n <= topk) {
    for (int i = threadIdx.x; i < topk; i += kSelThreads) o[i] = i < n ? i : -1;
    return;
  }
  if (threadIdx.x == 0) {
    s_prefix = 0u;
    s_mask = 0u;
    s_krem = static_cast<uint32_t>(topk);
    s_cnt = 0u;
    s_eq = 0u;
  }
  const int n_round = (n + kSelThreads - 1) / kSelThreads * kSelThreads;   // whole warps take part in every step
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += kSelThreads) hist[i] = 0u;
    __syncthreads();
    const uint32_t prefix = s_prefix, mask = s_mask;
    if (pass < 2) {
      // leading bytes (sign, exponent, top of the mantissa) are shared by most of the row: combine per warp
      for (int i = threadIdx.x; i < n_round; i += kSelThreads) {
        const uint32_t u = i < n ? order_key(row[i]) : 0u;
        hist_add(hist, (u >> shift) & 255u, i < n && (u & mask) == prefix);
      }
    } else {
      // trailing bytes are spread over the bins and few elements still match the prefix: plain atomics
      for (int i = threadIdx.x; i < n; i += kSelThreads) {
        const uint32_t u = order_key(row[i]);
        if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & 255u], 1u);
      }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // warp 0 scans the 256 bins from the top: lane l owns bins 255 - 8l .. 248 - 8l
      uint32_t mine[8], sum = 0u;
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        mine[b] = hist[255 - (threadIdx.x * 8 + b)];
        sum += mine[b];
      }
      uint32_t before = sum;                       // exclusive prefix over the lanes
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, before, d);
        if (static_cast<int>(threadIdx.x) >= d) before += v;
      }
      before -= sum;
      const uint32_t k = s_krem;
      if (before < k && before + sum >= k) {       // the k-th best value falls into one of my bins
        uint32_t cum = before;
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          if (cum < k && cum + mine[b] >= k) {
            s_prefix = prefix | (static_cast<uint32_t>(255 - (threadIdx.x * 8 + b)) << shift);
            s_mask = mask | (255u << shift);
            s_krem = k - cum;
          }
          cum += mine[b];
        }
      }
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix, krem = s_krem;
  for (int i = threadIdx.x; i < n_round; i += kSelThreads) {
    const uint32_t u = i < n ? order_key(row[i]) : 0u;
    const bool above = i < n && u > thr;
    const bool equal = i < n && u == thr;
    const uint32_t e = warp_reserve(&s_eq, equal);
    const bool take = above || (equal && e < krem);
    const uint32_t slot = warp_reserve(&s_cnt, take);
    if (take) o[slot] = i;
  }
}

}  // namespace b200

using namespace b200;

static int pow2_cols(int x) {
  int c = 32;
  while (c < x) c <<= 1;
  return c;
}

// Scores (and, with topk > 0, the selection) of the indexer for a batch of sequences.
//   q [T, H, 128] bf16, w [T, H] fp32, cache [num_blocks, block_size, 128] bf16,
//   block_tables [B, max_blocks], cu_q [B + 1] or null (then every sequence has q_len query
//   tokens), positions [T], scores [T, ld] fp32 scratch (ld >= longest context, multiple of 4),
//   topk_out [T, topk] int32 or null.
// Returns 0, or a negative code: -1 bad shape, -2 unsupported page size, -2xxx/-3xxx tensor map.
extern "C" int b200_dsa_indexer(const void* q, const float* w, const void* cache, const int* block_tables,
                                const int* cu_q, const int* positions, float* scores, int* topk_out, int T,
                                int B, int H, int q_len, long long num_blocks, int block_size, int max_blocks,
                                long long ld, int max_ctx, int max_q, int topk, int* status,
                                cudaStream_t stream) {
  if (T <= 0 || B <= 0) return 0;
  if (H <= 0 || (H % 16) != 0 || H > 256) return -1;
  if ((block_size % 8) != 0 || !(block_size >= kIdxBK ? (block_size % kIdxBK) == 0 : (kIdxBK % block_size) == 0))
    return -2;
  IndexerParams p{};
  p.w = w;
  p.scores = scores;
  p.ld = ld;
  p.block_tables = block_tables;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  p.box_rows = block_size < kIdxBK ? block_size : kIdxBK;
  p.cu_q = cu_q;
  p.positions = positions;
  p.q_len = q_len;
  p.H = H;
  // tokens per MMA: as many as fit N <= 256, but no more than a sequence can have
  int ntok = 256 / H;
  if (ntok > 4) ntok = 4;
  while (ntok > 1 && ntok > max_q) ntok >>= 1;
  p.ntok = ntok;
  const int N = ntok * H;
  p.tmem_cols = pow2_cols(2 * N);
  p.status = status;
  const int key_tiles = (max_ctx + kIdxBK - 1) / kIdxBK;
  // enough CTAs for a few waves; a CTA keeps its query group resident across its key tiles
  int chunks = (4 * 148 + B - 1) / B;
  if (chunks > key_tiles) chunks = key_tiles;
  if (chunks < 1) chunks = 1;
  p.tiles_per_cta = (key_tiles + chunks - 1) / chunks;
  chunks = (key_tiles + p.tiles_per_cta - 1) / p.tiles_per_cta;
  // long query runs (prefill): also divide the token groups, so that a few sequences fill the GPU
  const int groups_max = (max_q + ntok - 1) / ntok;
  int q_split = (2 * 148 + chunks * B - 1) / (chunks * B);
  if (q_split > groups_max / 8) q_split = groups_max / 8;      // keep >= 8 groups per CTA per key tile
  if (q_split < 1) q_split = 1;
  if (q_split > 64) q_split = 64;
  p.q_split = q_split;
  const size_t smem = 1024 + 2 * kIdxKeyBytes + 2 * (2 * static_cast<size_t>(N) * 128) + 2 * N * 4 + 12 * 8 + 16;
  if (smem > 227u * 1024u) return -23;
  static DeviceOnce once;
  int cur = 0;
  if (once.needed(&cur)) {
    if (cudaFuncSetAttribute(dsa_indexer_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             227 * 1024) != cudaSuccess)
      return -20;
    once.mark(cur);
  }
  CUtensorMap tk, tq;
  int r = make_tensormap_2d(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, cache,
                            static_cast<uint64_t>(num_blocks) * block_size, kIdxD, kIdxD, p.box_rows, 64,
                            CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 2000;
  r = make_tensormap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, static_cast<uint64_t>(T) * H, kIdxD, kIdxD, N, 64,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r - 3000;
  if (launch_pdl(dsa_indexer_scores_kernel, dim3(chunks, B, q_split), dim3(kIdxThreads), smem, stream, 1, tk, tq, p) !=
      cudaSuccess)
    return -21;
  if (topk_out && topk > 0) {
    if (launch_pdl(dsa_indexer_select_kernel, dim3(T), dim3(kSelThreads), 0, stream, 1, topk_out,
                   static_cast<const float*>(scores), ld, positions, topk) != cudaSuccess)
      return -22;
  }
  return 0;
}
