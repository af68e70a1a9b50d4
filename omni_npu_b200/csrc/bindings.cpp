// torch.ops.omni_b200.* : tensor-level entry points of the sm_100a kernels.
// The kernels themselves live in .cu files with plain C launchers (raw
// pointers + stream); this file only validates tensors and forwards.

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include <tuple>

extern "C" {
void b200_gemm_plan(int M, int N, int K, int elem_bytes, int swiglu, int force_bn, int force_splits,
                    int* out_bn, int* out_splits, size_t* out_ws_bytes, int* out_counters,
                    int* out_cluster);
int b200_gemm(const void* A, const void* W, void* C, const void* bias, const void* residual, int M,
              int N, int K, int lda, int ldw, int ldc, int dtype_fp8, int out_fp32, int swiglu,
              int BN, int splits, int cluster_split, void* workspace, int* counters, int* status,
              int max_ctas, cudaStream_t stream);
int b200_gemm_pair(const void* A, const void* W, void* C, const void* bias, const void* residual,
                   int M, int N, int K, int lda, int ldw, int ldc, int dtype_fp8, int out_fp32,
                   int swiglu, int BN, int* status, int max_ctas, cudaStream_t stream);
int b200_grouped_gemm(const void* A, const void* W, void* C, const int* expert_offsets,
                      int num_experts, int total_rows, int N, int K, int lda, int ldc,
                      int dtype_fp8, int swiglu, int BN, int* status, int max_ctas,
                      cudaStream_t stream);
int b200_lse_merge(void* out, float* lse_out, const void* outs, const float* lses, int N, long long T, int H, int D,
                   long long stride_n_out, long long stride_n_lse, cudaStream_t stream);
int b200_gather_cache(void* dst, const void* cache, const int* block_tables, const int* cu_seq, int B,
                      int max_blocks, int block_size, int row_bytes, int max_seq_len, cudaStream_t stream);
int b200_spec_verify(const int* draft, const int* target, const int* bonus, const int* cu, int* out,
                     int* num_out, int B, int max_spec, cudaStream_t stream);
int b200_rmsnorm(void* out, const void* x, void* residual, const void* w, float eps, long long rows,
                 int H, long long x_stride, long long out_stride, long long res_stride,
                 cudaStream_t stream);
int b200_silu_mul(void* out, const void* x, long long rows, int I, long long x_stride,
                  long long out_stride, cudaStream_t stream);
int b200_quant_fp8_1x128(void* q, void* scales, const void* x, long long rows, int H,
                         long long x_stride, int ue8m0, cudaStream_t stream);
int b200_quant_int8_per_token(void* q, void* scales, const void* x, long long rows, int H,
                              long long x_stride, cudaStream_t stream);
int b200_gemm_fp8_block(const void* A, const float* a_scales, const void* W, const float* w_scales, void* C,
                        const void* bias, const void* residual, int M, int N, int K, int lda, int ldw, int ldc,
                        int out_fp32, int* status, int max_ctas, cudaStream_t stream);
int b200_grouped_gemm_fp8_block(const void* A, const float* a_scales, const void* W, const float* w_scales, void* C,
                                const int* expert_offsets, int num_experts, int total_rows, int N, int K, int lda,
                                int ldc, int scale_rows, int swiglu, int up_scale_row0, int* status, int max_ctas,
                                cudaStream_t stream);
int b200_dsa_indexer(const void* q, const float* w, const void* cache, const int* block_tables, const int* cu_q,
                     const int* positions, float* scores, int* topk_out, int T, int B, int H, int q_len,
                     long long num_blocks, int block_size, int max_blocks, long long ld, int max_ctx, int max_q,
                     int topk, int* status, cudaStream_t stream);
int b200_rmsnorm_quant(void* q, void* scales, void* out, const void* x, void* residual, const void* w, float eps,
                       long long rows, int H, long long x_stride, long long out_stride, long long res_stride,
                       int kind, cudaStream_t stream);
int b200_silu_mul_quant(void* q, void* scales, const void* x, long long rows, int I, long long x_stride, int kind,
                        cudaStream_t stream);
int b200_gemm_scaled(const void* A, const void* W, void* C, const float* a_scales, const float* w_scales,
                     const void* bias, const void* residual, int M, int N, int K, int lda, int ldw, int ldc,
                     int kind, int out_fp32, int BN, int* status, int max_ctas, cudaStream_t stream);
int b200_rope_qk(void* q, void* k, const int* positions, const float* cos_sin, int T, int Hq,
                 int Hk, int D, int rot_dim, int neox, long long q_stride, long long k_stride,
                 int sec_t, int sec_h, int interleaved_mrope, cudaStream_t stream);
int b200_rope_cache_gqa(void* q, const void* k, const void* v, void* k_cache, void* v_cache,
                        const int* positions, const int* slot_mapping, const float* cos_sin, int T,
                        int Hq, int Hk, int D, int rot_dim, int neox, long long q_stride,
                        long long k_stride, long long v_stride, int block_size,
                        cudaStream_t stream);
int b200_mla_kv_rmsnorm_rope_cache(const void* kv_c, const void* k_pe, const void* w, void* cache,
                                   void* kv_c_out, void* k_pe_out, const int* positions,
                                   const int* slot_mapping, const float* cos_sin, float eps, int T,
                                   int L, int R, int neox, long long kvc_stride,
                                   long long kpe_stride, long long cache_row_stride,
                                   cudaStream_t stream);
int b200_paged_scatter_rows(void* dst, const void* src, const int* slot_mapping, int T,
                            int row_elems, long long src_stride, long long dst_row_stride,
                            cudaStream_t stream);
int b200_gqa_cache_write(const void* k, const void* v, void* k_cache, void* v_cache,
                         const int* slot_mapping, int T, int Hk, int D, int Dv, long long k_stride,
                         long long v_stride, int block_size, cudaStream_t stream);
int b200_gqa_prefill(const void* q, const void* k_cache, const void* v_cache, void* out, float* lse,
                     const int* block_tables, const int* cu_q, const int* seq_lens, int B,
                     int max_q_len, int max_blocks, int block_size, int Hq, int Hk, int Dqk, int Dv,
                     long long q_stride, long long out_stride, float scale, int causal, int window,
                     cudaStream_t stream);
size_t b200_gqa_decode_scratch_bytes(int B, int Hk, int D, int splits);
size_t b200_gqa_decode_balanced_scratch_bytes(int D, int rows);
int b200_gqa_decode(const void* q, const void* k_cache, const void* v_cache, void* out, float* lse,
                    const int* block_tables, const int* seq_lens, int B, int q_len, int max_blocks,
                    int block_size, int Hq, int Hk, int D, long long q_stride, long long out_stride,
                    float scale, int window, int splits, void* scratch, int num_cache_blocks,
                    int* status, cudaStream_t stream);
int b200_gqa_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out, float* lse,
                        const int* block_tables, const int* cu_q, const int* seq_lens, int B, int max_q_len,
                        int max_blocks, int block_size, int Hq, int Hk, int Dqk, int Dv, long long q_stride,
                        long long out_stride, float scale, int causal, int window, long long total_q_rows,
                        int num_cache_blocks, int* status, cudaStream_t stream);
int b200_gqa_decode_ex(const void* q, const void* k_cache, const void* v_cache, void* out, float* lse,
                       const int* block_tables, const int* seq_lens, int B, int q_len, int max_blocks,
                       int block_size, int Hq, int Hk, int D, long long q_stride, long long out_stride,
                       float scale, int window, int splits, void* scratch, int num_cache_blocks, int* status,
                       int persistent, int* work_counter, cudaStream_t stream);
int b200_kv_p2p_copy(const void* tensors, int num_tensors, const int* src_blocks, const int* dst_blocks,
                     int num_pairs, long long max_block_bytes, cudaStream_t stream);
size_t b200_mla_decode_scratch_bytes(int total_tokens, int N, int splits);
int b200_mla_decode(const void* q, const void* cache, void* out, float* lse, const int* block_tables,
                    const int* seq_lens, const int* topk_indices, int topk, int B, int q_len, int N,
                    int max_blocks, int block_size, int num_cache_blocks, long long q_stride,
                    long long out_stride, float scale, int splits, void* scratch, int* status,
                    cudaStream_t stream);
int b200_moe_topk(const float* logits, const float* bias, int* topk_ids, float* topk_w, int T, int E,
                  int k, int scoring, int n_group, int topk_group, int renorm, float scale,
                  cudaStream_t stream);
int b200_argmax(const void* logits, int* out, int B, int V, long long stride, int is_fp32,
                cudaStream_t stream);
int b200_sample(const void* logits, int* out, const float* temperature, const int* top_k,
                const float* top_p, const long long* seeds, const long long* step_offset, int B,
                int V, long long stride, int is_fp32, cudaStream_t stream);
}

namespace {

using torch::Tensor;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline void check(int rc, const char* what) {
  TORCH_CHECK(rc == 0, "omni_b200::", what, " failed with code ", rc);
}

#define CHECK_CUDA_BF16(t) \
  TORCH_CHECK((t).is_cuda() && (t).scalar_type() == at::kBFloat16, #t " must be a CUDA bf16 tensor")
#define CHECK_I32(t) \
  TORCH_CHECK((t).is_cuda() && (t).scalar_type() == at::kInt && (t).is_contiguous(), #t " must be a contiguous CUDA int32 tensor")

// Merge N partial attention results over disjoint key sets by their log-sum-exp.
// outs [N, T, H, D] bf16, lses [N, T, H] fp32 -> (out [T, H, D], lse [T, H]).
std::tuple<Tensor, Tensor> lse_merge(const Tensor& outs, const Tensor& lses) {
  CHECK_CUDA_BF16(outs);
  TORCH_CHECK(outs.dim() == 4 && outs.is_contiguous() && lses.is_cuda() && lses.scalar_type() == at::kFloat &&
                  lses.dim() == 3 && lses.is_contiguous(), "lse_merge: outs [N,T,H,D] bf16, lses [N,T,H] fp32");
  const int N = outs.size(0), H = outs.size(2), D = outs.size(3);
  const long long T = outs.size(1);
  TORCH_CHECK(lses.size(0) == N && lses.size(1) == T && lses.size(2) == H, "lse_merge: shapes");
  c10::cuda::CUDAGuard guard(outs.device());
  Tensor out = torch::empty({T, H, D}, outs.options());
  Tensor lse = torch::empty({T, H}, lses.options());
  check(b200_lse_merge(out.data_ptr(), lse.data_ptr<float>(), outs.data_ptr(), lses.data_ptr<float>(), N, T, H, D,
                       T * H * D, T * H, cur_stream()),
        "lse_merge");
  return {out, lse};
}

// Contiguous copy of the cached rows of B sequences: cache [blocks, block_size, ...],
// cu_seq [B+1] int32 -> [cu_seq[B], ...].
Tensor gather_cache(const Tensor& cache, const Tensor& block_tables, const Tensor& cu_seq, int64_t total_tokens,
                    int64_t max_seq_len) {
  TORCH_CHECK(cache.is_cuda() && cache.is_contiguous() && cache.dim() >= 3, "gather_cache: cache [blocks, bs, ...]");
  CHECK_I32(block_tables);
  CHECK_I32(cu_seq);
  const int bs = cache.size(1);
  const int64_t width = cache.numel() / (cache.size(0) * bs);
  c10::cuda::CUDAGuard guard(cache.device());
  std::vector<int64_t> shape{total_tokens};
  for (int i = 2; i < cache.dim(); ++i) shape.push_back(cache.size(i));
  Tensor dst = torch::empty(shape, cache.options());
  check(b200_gather_cache(dst.data_ptr(), cache.data_ptr(), block_tables.data_ptr<int>(), cu_seq.data_ptr<int>(),
                          (int)cu_seq.numel() - 1, (int)block_tables.size(1), bs,
                          (int)(width * cache.element_size()), (int)max_seq_len, cur_stream()),
        "gather_cache");
  return dst;
}

// Speculative decoding: accept drafts while they equal the target's tokens.
// Returns (tokens [B, max_spec+1] padded with -1, count [B]).
std::tuple<Tensor, Tensor> spec_verify(const Tensor& draft, const Tensor& target, const Tensor& bonus,
                                       const Tensor& cu, int64_t max_spec) {
  for (const Tensor* t : {&draft, &target, &bonus, &cu})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->is_contiguous(), "spec_verify: int32 CUDA");
  const int B = (int)cu.numel() - 1;
  TORCH_CHECK(bonus.numel() >= B && draft.numel() == target.numel(), "spec_verify: shapes");
  c10::cuda::CUDAGuard guard(draft.device());
  Tensor out = torch::empty({B, max_spec + 1}, draft.options());
  Tensor num = torch::empty({B}, draft.options());
  check(b200_spec_verify(draft.data_ptr<int>(), target.data_ptr<int>(), bonus.data_ptr<int>(),
                         cu.data_ptr<int>(), out.data_ptr<int>(), num.data_ptr<int>(), B, (int)max_spec,
                         cur_stream()),
        "spec_verify");
  return {out, num};
}

// (BN, splits, workspace bytes, counters, cluster flag) for a problem.
std::tuple<int64_t, int64_t, int64_t, int64_t, int64_t> gemm_plan(int64_t M, int64_t N, int64_t K,
                                                                  int64_t elem_bytes, bool swiglu,
                                                                  int64_t force_bn,
                                                                  int64_t force_splits) {
  int bn, sp, cnt, cl;
  size_t ws;
  b200_gemm_plan((int)M, (int)N, (int)K, (int)elem_bytes, swiglu ? 1 : 0, (int)force_bn,
                 (int)force_splits, &bn, &sp, &ws, &cnt, &cl);
  return {bn, sp, (int64_t)ws, cnt, cl};
}

// C = A @ W^T (+bias) (+residual).  A [M,K], W [N,K]; bf16 or float8_e4m3fn.
Tensor gemm(const Tensor& a, const Tensor& w, const c10::optional<Tensor>& bias,
            const c10::optional<Tensor>& residual, bool out_fp32, bool swiglu, int64_t bn,
            int64_t splits, bool cluster_split, const c10::optional<Tensor>& workspace,
            const c10::optional<Tensor>& counters, const Tensor& status, int64_t max_ctas) {
  TORCH_CHECK(a.is_cuda() && w.is_cuda() && a.dim() == 2 && w.dim() == 2, "gemm: 2-D CUDA tensors");
  TORCH_CHECK(a.scalar_type() == w.scalar_type(), "gemm: dtype mismatch");
  const bool fp8 = a.scalar_type() == at::kFloat8_e4m3fn;
  TORCH_CHECK(fp8 || a.scalar_type() == at::kBFloat16, "gemm: bf16 or float8_e4m3fn inputs");
  TORCH_CHECK(a.stride(1) == 1 && w.stride(1) == 1, "gemm: K must be contiguous");
  const int M = a.size(0), K = a.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K, "gemm: K mismatch");
  c10::cuda::CUDAGuard guard(a.device());
  const int n_out = swiglu ? N / 2 : N;
  Tensor c = torch::empty({M, n_out}, a.options().dtype(out_fp32 ? at::kFloat : at::kBFloat16));
  const void* bias_p = nullptr;
  const void* res_p = nullptr;
  if (bias.has_value()) {
    CHECK_CUDA_BF16(*bias);
    TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "gemm: bias [N]");
    bias_p = bias->data_ptr();
  }
  if (residual.has_value()) {
    CHECK_CUDA_BF16(*residual);
    TORCH_CHECK(residual->is_contiguous() && residual->size(0) == M && residual->size(1) == n_out,
                "gemm: residual [M,N] contiguous");
    res_p = residual->data_ptr();
  }
  void* ws_p = nullptr;
  int* cnt_p = nullptr;
  if (splits > 1 && !cluster_split) {
    TORCH_CHECK(workspace.has_value() && counters.has_value(), "gemm: split-K needs workspace");
    ws_p = workspace->data_ptr();
    cnt_p = counters->data_ptr<int>();
  }
  check(b200_gemm(a.data_ptr(), w.data_ptr(), c.data_ptr(), bias_p, res_p, M, N, K,
                  (int)a.stride(0), (int)w.stride(0), n_out, fp8 ? 1 : 0, out_fp32 ? 1 : 0,
                  swiglu ? 1 : 0, (int)bn, (int)splits, cluster_split ? 1 : 0, ws_p, cnt_p,
                  status.data_ptr<int>(),
                  (int)max_ctas, cur_stream()),
        "gemm");
  return c;
}

// Same contract as gemm() without split-K, run by CTA pairs: one 256 x BN tile per pair of SMs
// (tcgen05 cta_group::2), each SM staging half of the weight tile.
Tensor gemm_pair(const Tensor& a, const Tensor& w, const c10::optional<Tensor>& bias,
                 const c10::optional<Tensor>& residual, bool out_fp32, bool swiglu, int64_t bn,
                 const Tensor& status, int64_t max_ctas) {
  TORCH_CHECK(a.is_cuda() && w.is_cuda() && a.dim() == 2 && w.dim() == 2, "gemm_pair: 2-D CUDA tensors");
  TORCH_CHECK(a.scalar_type() == w.scalar_type(), "gemm_pair: dtype mismatch");
  const bool fp8 = a.scalar_type() == at::kFloat8_e4m3fn;
  TORCH_CHECK(fp8 || a.scalar_type() == at::kBFloat16, "gemm_pair: bf16 or float8_e4m3fn inputs");
  TORCH_CHECK(a.stride(1) == 1 && w.stride(1) == 1, "gemm_pair: K must be contiguous");
  const int M = a.size(0), K = a.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K, "gemm_pair: K mismatch");
  c10::cuda::CUDAGuard guard(a.device());
  const int n_out = swiglu ? N / 2 : N;
  Tensor c = torch::empty({M, n_out}, a.options().dtype(out_fp32 ? at::kFloat : at::kBFloat16));
  const void* bias_p = nullptr;
  const void* res_p = nullptr;
  if (bias.has_value()) {
    CHECK_CUDA_BF16(*bias);
    TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "gemm_pair: bias [N]");
    bias_p = bias->data_ptr();
  }
  if (residual.has_value()) {
    CHECK_CUDA_BF16(*residual);
    TORCH_CHECK(residual->is_contiguous() && residual->size(0) == M && residual->size(1) == n_out,
                "gemm_pair: residual [M,N] contiguous");
    res_p = residual->data_ptr();
  }
  check(b200_gemm_pair(a.data_ptr(), w.data_ptr(), c.data_ptr(), bias_p, res_p, M, N, K,
                       (int)a.stride(0), (int)w.stride(0), n_out, fp8 ? 1 : 0, out_fp32 ? 1 : 0,
                       swiglu ? 1 : 0, (int)bn, status.data_ptr<int>(), (int)max_ctas, cur_stream()),
        "gemm_pair");
  return c;
}

Tensor grouped_gemm(const Tensor& a, const Tensor& w, const Tensor& expert_offsets, bool swiglu,
                    int64_t bn, const Tensor& status, int64_t max_ctas) {
  TORCH_CHECK(a.is_cuda() && w.is_cuda() && a.dim() == 2 && w.dim() == 3, "grouped_gemm: shapes");
  TORCH_CHECK(a.scalar_type() == w.scalar_type(), "grouped_gemm: dtype mismatch");
  const bool fp8 = a.scalar_type() == at::kFloat8_e4m3fn;
  TORCH_CHECK(fp8 || a.scalar_type() == at::kBFloat16, "grouped_gemm: bf16 or fp8 inputs");
  TORCH_CHECK(a.stride(1) == 1 && w.is_contiguous(), "grouped_gemm: contiguity");
  CHECK_I32(expert_offsets);
  const int E = w.size(0), N = w.size(1), K = w.size(2), rows = a.size(0);
  TORCH_CHECK(a.size(1) == K && expert_offsets.numel() == E + 1, "grouped_gemm: size mismatch");
  c10::cuda::CUDAGuard guard(a.device());
  const int n_out = swiglu ? N / 2 : N;
  Tensor c = torch::empty({rows, n_out}, a.options().dtype(at::kBFloat16));
  check(b200_grouped_gemm(a.data_ptr(), w.data_ptr(), c.data_ptr(), expert_offsets.data_ptr<int>(),
                          E, rows, N, K, (int)a.stride(0), n_out, fp8 ? 1 : 0, swiglu ? 1 : 0,
                          (int)bn, status.data_ptr<int>(), (int)max_ctas, cur_stream()),
        "grouped_gemm");
  return c;
}

Tensor rms_norm(const Tensor& x, const Tensor& w, double eps) {
  CHECK_CUDA_BF16(x);
  CHECK_CUDA_BF16(w);
  TORCH_CHECK(x.stride(-1) == 1, "rms_norm: last dim contiguous");
  const int H = x.size(-1);
  Tensor x2 = x.dim() == 2 ? x : x.reshape({-1, H});
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty({x2.size(0), H}, x.options());
  check(b200_rmsnorm(out.data_ptr(), x2.data_ptr(), nullptr, w.data_ptr(), (float)eps, x2.size(0),
                     H, x2.stride(0), H, 0, cur_stream()),
        "rms_norm");
  return out.view(x.sizes());
}

// residual <- x + residual ; returns norm(residual) * w
Tensor fused_add_rms_norm(const Tensor& x, Tensor residual, const Tensor& w, double eps) {
  CHECK_CUDA_BF16(x);
  CHECK_CUDA_BF16(residual);
  CHECK_CUDA_BF16(w);
  TORCH_CHECK(x.dim() == 2 && residual.dim() == 2 && x.stride(1) == 1 && residual.stride(1) == 1,
              "fused_add_rms_norm: 2-D, last dim contiguous");
  const int H = x.size(1);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty({x.size(0), H}, x.options());
  check(b200_rmsnorm(out.data_ptr(), x.data_ptr(), residual.data_ptr(), w.data_ptr(), (float)eps,
                     x.size(0), H, x.stride(0), H, residual.stride(0), cur_stream()),
        "fused_add_rms_norm");
  return out;
}

Tensor silu_and_mul(const Tensor& x) {
  CHECK_CUDA_BF16(x);
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "silu_and_mul: 2-D, last dim contiguous");
  const int I = x.size(1) / 2;
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty({x.size(0), I}, x.options());
  check(b200_silu_mul(out.data_ptr(), x.data_ptr(), x.size(0), I, x.stride(0), I, cur_stream()),
        "silu_and_mul");
  return out;
}

std::tuple<Tensor, Tensor> quant_fp8_1x128(const Tensor& x, bool ue8m0) {
  CHECK_CUDA_BF16(x);
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "quant_fp8_1x128: 2-D, last dim contiguous");
  const int H = x.size(1);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor q = torch::empty({x.size(0), H}, x.options().dtype(at::kFloat8_e4m3fn));
  Tensor s = torch::empty({x.size(0), H / 128}, x.options().dtype(at::kFloat));
  check(b200_quant_fp8_1x128(q.data_ptr(), s.data_ptr(), x.data_ptr(), x.size(0), H, x.stride(0),
                             ue8m0 ? 1 : 0, cur_stream()),
        "quant_fp8_1x128");
  return {q, s};
}

std::tuple<Tensor, Tensor> quant_int8_per_token(const Tensor& x) {
  CHECK_CUDA_BF16(x);
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "quant_int8_per_token: 2-D, last dim contiguous");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor q = torch::empty({x.size(0), x.size(1)}, x.options().dtype(at::kChar));
  Tensor s = torch::empty({x.size(0)}, x.options().dtype(at::kFloat));
  check(b200_quant_int8_per_token(q.data_ptr(), s.data_ptr(), x.data_ptr(), x.size(0), (int)x.size(1),
                                  x.stride(0), cur_stream()),
        "quant_int8_per_token");
  return {q, s};
}

// Block-scaled e4m3 GEMM: a [M,K] e4m3 with a_scale [M, K/128]; w [N,K] e4m3 with w_scale
// [ceil(N/128), K/128]; every 128-wide K block's product is scaled before it is accumulated.
Tensor gemm_fp8_block(const Tensor& a, const Tensor& a_scale, const Tensor& w, const Tensor& w_scale,
                      const c10::optional<Tensor>& bias, const c10::optional<Tensor>& residual, bool out_fp32,
                      const Tensor& status, int64_t max_ctas) {
  TORCH_CHECK(a.is_cuda() && w.is_cuda() && a.dim() == 2 && w.dim() == 2, "gemm_fp8_block: 2-D CUDA tensors");
  TORCH_CHECK(a.scalar_type() == at::kFloat8_e4m3fn && w.scalar_type() == at::kFloat8_e4m3fn,
              "gemm_fp8_block: float8_e4m3fn operands");
  TORCH_CHECK(a.stride(1) == 1 && w.stride(1) == 1, "gemm_fp8_block: K must be contiguous");
  const int64_t M = a.size(0), K = a.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K && K % 128 == 0, "gemm_fp8_block: K mismatch / K must be a multiple of 128");
  const int64_t kb = K / 128, nbk = (N + 127) / 128;
  TORCH_CHECK(a_scale.is_cuda() && a_scale.scalar_type() == at::kFloat && a_scale.is_contiguous() &&
                  a_scale.numel() == M * kb, "gemm_fp8_block: a_scale fp32 [M, K/128]");
  TORCH_CHECK(w_scale.is_cuda() && w_scale.scalar_type() == at::kFloat && w_scale.is_contiguous() &&
                  w_scale.numel() == nbk * kb, "gemm_fp8_block: w_scale fp32 [ceil(N/128), K/128]");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor c = torch::empty({M, N}, a.options().dtype(out_fp32 ? at::kFloat : at::kBFloat16));
  const void* bias_p = nullptr;
  const void* res_p = nullptr;
  if (bias.has_value()) {
    CHECK_CUDA_BF16((*bias));
    TORCH_CHECK(bias->numel() == N, "gemm_fp8_block: bias [N]");
    bias_p = bias->data_ptr();
  }
  if (residual.has_value()) {
    CHECK_CUDA_BF16((*residual));
    TORCH_CHECK(residual->dim() == 2 && residual->size(0) == M && residual->size(1) == N && residual->is_contiguous(),
                "gemm_fp8_block: residual [M, N] contiguous");
    res_p = residual->data_ptr();
  }
  check(b200_gemm_fp8_block(a.data_ptr(), a_scale.data_ptr<float>(), w.data_ptr(), w_scale.data_ptr<float>(),
                            c.data_ptr(), bias_p, res_p, (int)M, (int)N, (int)K, (int)a.stride(0), (int)w.stride(0),
                            (int)N, out_fp32 ? 1 : 0, status.data_ptr<int>(), (int)max_ctas, cur_stream()),
        "gemm_fp8_block");
  return c;
}

// Grouped block-scaled e4m3 GEMM (MoE experts): a [rows, K] e4m3 + a_scale [rows, K/128]; w [E, N, K] e4m3 +
// w_scale [E, R, K/128]; expert e owns rows expert_offsets[e] .. [e + 1].  swiglu: gate / up rows of w are
// interleaved in groups of 8, their scale rows are gate blocks then up blocks (from row up_scale_row0).
Tensor grouped_gemm_fp8_block(const Tensor& a, const Tensor& a_scale, const Tensor& w, const Tensor& w_scale,
                              const Tensor& expert_offsets, bool swiglu, int64_t up_scale_row0, const Tensor& status,
                              int64_t max_ctas) {
  TORCH_CHECK(a.is_cuda() && w.is_cuda() && a.dim() == 2 && w.dim() == 3, "grouped_gemm_fp8_block: shapes");
  TORCH_CHECK(a.scalar_type() == at::kFloat8_e4m3fn && w.scalar_type() == at::kFloat8_e4m3fn,
              "grouped_gemm_fp8_block: float8_e4m3fn operands");
  TORCH_CHECK(a.stride(1) == 1 && w.is_contiguous(), "grouped_gemm_fp8_block: contiguity");
  CHECK_I32(expert_offsets);
  const int64_t E = w.size(0), N = w.size(1), K = w.size(2), rows = a.size(0);
  TORCH_CHECK(a.size(1) == K && K % 128 == 0 && expert_offsets.numel() == E + 1, "grouped_gemm_fp8_block: sizes");
  TORCH_CHECK(a_scale.is_cuda() && a_scale.scalar_type() == at::kFloat && a_scale.is_contiguous() &&
                  a_scale.numel() == rows * (K / 128), "grouped_gemm_fp8_block: a_scale fp32 [rows, K/128]");
  TORCH_CHECK(w_scale.is_cuda() && w_scale.scalar_type() == at::kFloat && w_scale.is_contiguous() &&
                  w_scale.dim() == 3 && w_scale.size(0) == E && w_scale.size(2) == K / 128,
              "grouped_gemm_fp8_block: w_scale fp32 [E, R, K/128]");
  const int64_t R = w_scale.size(1);
  TORCH_CHECK(swiglu ? (N % 256 == 0 && up_scale_row0 + (N / 2 + 127) / 128 <= R) : (N + 127) / 128 <= R,
              "grouped_gemm_fp8_block: scale rows do not cover the weight rows");
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t n_out = swiglu ? N / 2 : N;
  Tensor c = torch::empty({rows, n_out}, a.options().dtype(at::kBFloat16));
  check(b200_grouped_gemm_fp8_block(a.data_ptr(), a_scale.data_ptr<float>(), w.data_ptr(), w_scale.data_ptr<float>(),
                                    c.data_ptr(), expert_offsets.data_ptr<int>(), (int)E, (int)rows, (int)N, (int)K,
                                    (int)a.stride(0), (int)n_out, (int)R, swiglu ? 1 : 0, (int)up_scale_row0,
                                    status.data_ptr<int>(), (int)max_ctas, cur_stream()),
        "grouped_gemm_fp8_block");
  return c;
}

// Sparse-attention indexer: scores on the tensor cores + radix select of the topk best key
// positions per query token.  q [T,H,128] bf16, w [T,H] fp32, cache [blocks, block_size, 128]
// bf16, cu_q [B+1] int32 or none (then q_len tokens per sequence), positions [T] int32.
// Returns (topk indices int32 [T, topk], scores fp32 [T, ld]); entries of `scores` beyond a
// token's position are not defined.
std::tuple<Tensor, Tensor> dsa_indexer(const Tensor& q, const Tensor& w, const Tensor& cache,
                                       const Tensor& block_tables, const c10::optional<Tensor>& cu_q,
                                       const Tensor& positions, int64_t num_seqs, int64_t q_len, int64_t max_ctx,
                                       int64_t max_q, int64_t topk, const Tensor& status) {
  CHECK_CUDA_BF16(q);
  CHECK_CUDA_BF16(cache);
  TORCH_CHECK(q.dim() == 3 && q.size(2) == 128 && q.is_contiguous(), "dsa_indexer: q [T, H, 128] contiguous");
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kFloat && w.is_contiguous() && w.dim() == 2 &&
                  w.size(0) == q.size(0) && w.size(1) == q.size(1), "dsa_indexer: w fp32 [T, H]");
  TORCH_CHECK(cache.dim() == 3 && cache.size(2) == 128 && cache.is_contiguous(), "dsa_indexer: cache [blocks, bs, 128]");
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && block_tables.dim() == 2 && block_tables.is_contiguous(),
              "dsa_indexer: block_tables int32 [B, max_blocks]");
  TORCH_CHECK(positions.scalar_type() == at::kInt && positions.is_contiguous() && positions.numel() >= q.size(0),
              "dsa_indexer: positions int32 [T]");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t T = q.size(0), H = q.size(1);
  const int64_t ld = ((std::max<int64_t>(max_ctx, 1) + 127) / 128) * 128;
  Tensor scores = torch::empty({T, ld}, q.options().dtype(at::kFloat));
  Tensor sel = torch::empty({T, topk}, q.options().dtype(at::kInt));
  const int* cu = nullptr;
  if (cu_q.has_value()) {
    TORCH_CHECK(cu_q->scalar_type() == at::kInt && cu_q->is_contiguous() && cu_q->numel() >= num_seqs + 1,
                "dsa_indexer: cu_q int32 [B + 1]");
    cu = cu_q->data_ptr<int>();
  }
  check(b200_dsa_indexer(q.data_ptr(), w.data_ptr<float>(), cache.data_ptr(), block_tables.data_ptr<int>(), cu,
                         positions.data_ptr<int>(), scores.data_ptr<float>(), sel.data_ptr<int>(), (int)T,
                         (int)num_seqs, (int)H, (int)q_len, cache.size(0), (int)cache.size(1),
                         (int)block_tables.size(1), ld, (int)max_ctx, (int)max_q, (int)topk, status.data_ptr<int>(),
                         cur_stream()),
        "dsa_indexer");
  return {sel, scores};
}

// RMSNorm (+ residual add, in place on `residual`) fused with per-token quantisation.
// kind 1: e4m3, 2: int8.  Returns (q [T,H], scale [T], normalised bf16 row or empty).
std::tuple<Tensor, Tensor, Tensor> rms_norm_quant(const Tensor& x, const c10::optional<Tensor>& residual,
                                                  const Tensor& w, double eps, int64_t kind, bool want_bf16) {
  CHECK_CUDA_BF16(x);
  CHECK_CUDA_BF16(w);
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "rms_norm_quant: 2-D, last dim contiguous");
  TORCH_CHECK(kind == 1 || kind == 2, "rms_norm_quant: kind 1 (e4m3) or 2 (int8)");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t T = x.size(0), H = x.size(1);
  Tensor q = torch::empty({T, H}, x.options().dtype(kind == 1 ? at::kFloat8_e4m3fn : at::kChar));
  Tensor s = torch::empty({T}, x.options().dtype(at::kFloat));
  Tensor out = want_bf16 ? torch::empty({T, H}, x.options()) : Tensor();
  void* res_p = nullptr;
  long long res_stride = 0;
  if (residual.has_value()) {
    CHECK_CUDA_BF16((*residual));
    TORCH_CHECK(residual->dim() == 2 && residual->stride(1) == 1 && residual->size(0) == T && residual->size(1) == H,
                "rms_norm_quant: residual shape");
    res_p = residual->data_ptr();
    res_stride = residual->stride(0);
  }
  check(b200_rmsnorm_quant(q.data_ptr(), s.data_ptr(), want_bf16 ? out.data_ptr() : nullptr, x.data_ptr(), res_p,
                           w.data_ptr(), (float)eps, T, (int)H, x.stride(0), H, res_stride, (int)kind, cur_stream()),
        "rms_norm_quant");
  return {q, s, out};
}

// silu(x[:, :I]) * x[:, I:] fused with per-token quantisation (kind 1: e4m3, 2: int8).
std::tuple<Tensor, Tensor> silu_and_mul_quant(const Tensor& x, int64_t kind) {
  CHECK_CUDA_BF16(x);
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.size(1) % 16 == 0, "silu_and_mul_quant: [T, 2I], I % 8 == 0");
  TORCH_CHECK(kind == 1 || kind == 2, "silu_and_mul_quant: kind 1 (e4m3) or 2 (int8)");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t T = x.size(0), I = x.size(1) / 2;
  Tensor q = torch::empty({T, I}, x.options().dtype(kind == 1 ? at::kFloat8_e4m3fn : at::kChar));
  Tensor s = torch::empty({T}, x.options().dtype(at::kFloat));
  check(b200_silu_mul_quant(q.data_ptr(), s.data_ptr(), x.data_ptr(), T, (int)I, x.stride(0), (int)kind, cur_stream()),
        "silu_and_mul_quant");
  return {q, s};
}

// Quantised GEMM: (a_q @ w_q^T) * a_scale[:, None] * w_scale[None, :] (+bias, +residual).
// int8 x int8 (s32 accumulate) or e4m3 x e4m3 (fp32 accumulate).
Tensor gemm_scaled(const Tensor& a, const Tensor& w, const Tensor& a_scale, const Tensor& w_scale,
                   const c10::optional<Tensor>& bias, const c10::optional<Tensor>& residual, bool out_fp32,
                   int64_t bn, const Tensor& status, int64_t max_ctas) {
  TORCH_CHECK(a.is_cuda() && w.is_cuda() && a.dim() == 2 && w.dim() == 2, "gemm_scaled: 2-D CUDA tensors");
  TORCH_CHECK(a.scalar_type() == w.scalar_type(), "gemm_scaled: dtype mismatch");
  const bool i8 = a.scalar_type() == at::kChar;
  TORCH_CHECK(i8 || a.scalar_type() == at::kFloat8_e4m3fn, "gemm_scaled: int8 or float8_e4m3fn inputs");
  TORCH_CHECK(a.stride(1) == 1 && w.stride(1) == 1, "gemm_scaled: K must be contiguous");
  const int M = a.size(0), K = a.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K && K % 16 == 0, "gemm_scaled: K mismatch / K must be a multiple of 16");
  TORCH_CHECK(a_scale.is_cuda() && a_scale.scalar_type() == at::kFloat && a_scale.numel() == M &&
                  a_scale.is_contiguous(), "gemm_scaled: a_scale fp32 [M]");
  TORCH_CHECK(w_scale.is_cuda() && w_scale.scalar_type() == at::kFloat && w_scale.numel() == N &&
                  w_scale.is_contiguous(), "gemm_scaled: w_scale fp32 [N]");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor c = torch::empty({M, N}, a.options().dtype(out_fp32 ? at::kFloat : at::kBFloat16));
  const void* bias_p = nullptr;
  const void* res_p = nullptr;
  if (bias.has_value()) {
    CHECK_CUDA_BF16(*bias);
    TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "gemm_scaled: bias [N]");
    bias_p = bias->data_ptr();
  }
  if (residual.has_value()) {
    CHECK_CUDA_BF16(*residual);
    TORCH_CHECK(residual->is_contiguous() && residual->size(0) == M && residual->size(1) == N,
                "gemm_scaled: residual [M,N] contiguous");
    res_p = residual->data_ptr();
  }
  check(b200_gemm_scaled(a.data_ptr(), w.data_ptr(), c.data_ptr(), a_scale.data_ptr<float>(),
                         w_scale.data_ptr<float>(), bias_p, res_p, M, N, K, (int)a.stride(0), (int)w.stride(0),
                         N, i8 ? 2 : 1, out_fp32 ? 1 : 0, (int)bn, status.data_ptr<int>(), (int)max_ctas,
                         cur_stream()),
        "gemm_scaled");
  return c;
}

void rope_qk(Tensor q, Tensor k, const Tensor& positions, const Tensor& cos_sin, int64_t head_dim,
             int64_t rot_dim, bool neox, int64_t sec_t, int64_t sec_h, bool interleaved) {
  CHECK_CUDA_BF16(q);
  CHECK_CUDA_BF16(k);
  CHECK_I32(positions);
  TORCH_CHECK(cos_sin.is_cuda() && cos_sin.scalar_type() == at::kFloat && cos_sin.is_contiguous(),
              "rope: cos_sin must be contiguous fp32");
  TORCH_CHECK(q.dim() == 2 && k.dim() == 2 && q.stride(1) == 1 && k.stride(1) == 1, "rope: [T, H*D]");
  const int T = q.size(0);
  c10::cuda::CUDAGuard guard(q.device());
  check(b200_rope_qk(q.data_ptr(), k.data_ptr(), positions.data_ptr<int>(),
                     cos_sin.data_ptr<float>(), T, (int)(q.size(1) / head_dim),
                     (int)(k.size(1) / head_dim), (int)head_dim, (int)rot_dim, neox ? 1 : 0,
                     q.stride(0), k.stride(0), (int)sec_t, (int)sec_h, interleaved ? 1 : 0,
                     cur_stream()),
        "rope_qk");
}

void rope_cache_gqa(Tensor q, const Tensor& k, const Tensor& v, Tensor k_cache, Tensor v_cache,
                    const Tensor& positions, const Tensor& slot_mapping, const Tensor& cos_sin,
                    int64_t head_dim, int64_t rot_dim, bool neox) {
  CHECK_CUDA_BF16(q);
  CHECK_CUDA_BF16(k);
  CHECK_CUDA_BF16(v);
  CHECK_CUDA_BF16(k_cache);
  CHECK_CUDA_BF16(v_cache);
  CHECK_I32(positions);
  CHECK_I32(slot_mapping);
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous(),
              "cache: [blocks, kv_heads, block_size, D] contiguous");
  TORCH_CHECK(q.dim() == 2 && k.dim() == 2 && v.dim() == 2, "rope_cache: [T, H*D] views");
  const int T = q.size(0);
  const int Hk = k_cache.size(1), bs = k_cache.size(2);
  c10::cuda::CUDAGuard guard(q.device());
  check(b200_rope_cache_gqa(q.data_ptr(), k.data_ptr(), v.data_ptr(), k_cache.data_ptr(),
                            v_cache.data_ptr(), positions.data_ptr<int>(),
                            slot_mapping.data_ptr<int>(), cos_sin.data_ptr<float>(), T,
                            (int)(q.size(1) / head_dim), Hk, (int)head_dim, (int)rot_dim,
                            neox ? 1 : 0, q.stride(0), k.stride(0), v.stride(0), bs, cur_stream()),
        "rope_cache_gqa");
}

void mla_kv_rmsnorm_rope_cache(const Tensor& kv_c, const Tensor& k_pe, const Tensor& w, Tensor cache,
                               const c10::optional<Tensor>& kv_c_out,
                               const c10::optional<Tensor>& k_pe_out, const Tensor& positions,
                               const Tensor& slot_mapping, const Tensor& cos_sin, double eps,
                               bool neox) {
  CHECK_CUDA_BF16(kv_c);
  CHECK_CUDA_BF16(k_pe);
  CHECK_CUDA_BF16(cache);
  CHECK_I32(positions);
  CHECK_I32(slot_mapping);
  const int T = kv_c.size(0), L = kv_c.size(1), R = k_pe.size(1);
  TORCH_CHECK(cache.is_contiguous() && cache.size(-1) >= L + R, "mla cache row too small");
  c10::cuda::CUDAGuard guard(kv_c.device());
  check(b200_mla_kv_rmsnorm_rope_cache(
            kv_c.data_ptr(), k_pe.data_ptr(), w.data_ptr(), cache.data_ptr(),
            kv_c_out.has_value() ? kv_c_out->data_ptr() : nullptr,
            k_pe_out.has_value() ? k_pe_out->data_ptr() : nullptr, positions.data_ptr<int>(),
            slot_mapping.data_ptr<int>(), cos_sin.data_ptr<float>(), (float)eps, T, L, R,
            neox ? 1 : 0, kv_c.stride(0), k_pe.stride(0), cache.size(-1), cur_stream()),
        "mla_kv_rmsnorm_rope_cache");
}

void paged_scatter_rows(Tensor dst, const Tensor& src, const Tensor& slot_mapping) {
  CHECK_CUDA_BF16(dst);
  CHECK_CUDA_BF16(src);
  CHECK_I32(slot_mapping);
  TORCH_CHECK(dst.is_contiguous() && src.dim() == 2 && src.stride(1) == 1, "paged_scatter_rows");
  c10::cuda::CUDAGuard guard(src.device());
  check(b200_paged_scatter_rows(dst.data_ptr(), src.data_ptr(), slot_mapping.data_ptr<int>(),
                                (int)src.size(0), (int)src.size(1), src.stride(0), dst.size(-1),
                                cur_stream()),
        "paged_scatter_rows");
}

void gqa_cache_write(const Tensor& k, const Tensor& v, Tensor k_cache, Tensor v_cache,
                     const Tensor& slot_mapping) {
  CHECK_CUDA_BF16(k);
  CHECK_CUDA_BF16(v);
  CHECK_I32(slot_mapping);
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous(), "cache layout");
  const int Hk = k_cache.size(1), bs = k_cache.size(2), D = k_cache.size(3), Dv = v_cache.size(3);
  c10::cuda::CUDAGuard guard(k.device());
  check(b200_gqa_cache_write(k.data_ptr(), v.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                             slot_mapping.data_ptr<int>(), (int)k.size(0), Hk, D, Dv, k.stride(0),
                             v.stride(0), bs, cur_stream()),
        "gqa_cache_write");
}

std::tuple<Tensor, Tensor> gqa_prefill(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache,
                                       const Tensor& block_tables, const Tensor& cu_q,
                                       const Tensor& seq_lens, int64_t num_seqs, int64_t max_q_len,
                                       int64_t num_q_heads, double scale, bool causal,
                                       int64_t window, bool return_lse, bool use_tcgen05,
                                       const c10::optional<Tensor>& status) {
  CHECK_CUDA_BF16(q);
  CHECK_CUDA_BF16(k_cache);
  CHECK_CUDA_BF16(v_cache);
  CHECK_I32(block_tables);
  CHECK_I32(cu_q);
  CHECK_I32(seq_lens);
  TORCH_CHECK(q.dim() == 2 && q.stride(1) == 1, "gqa_prefill: q [T, Hq*D]");
  const int T = q.size(0);
  const int Hk = k_cache.size(1), bs = k_cache.size(2), Dqk = k_cache.size(3), Dv = v_cache.size(3);
  const int Hq = num_q_heads;
  TORCH_CHECK(q.size(1) == (int64_t)Hq * Dqk, "gqa_prefill: q width");
  c10::cuda::CUDAGuard guard(q.device());
  Tensor out = torch::empty({T, (int64_t)Hq * Dv}, q.options());
  Tensor lse = return_lse ? torch::empty({T, Hq}, q.options().dtype(at::kFloat)) : Tensor();
  if (use_tcgen05) {
    // head size 128 without a sliding window: both products on tcgen05 with TMEM accumulators
    const int rc = b200_gqa_prefill_tc(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
        return_lse ? lse.data_ptr<float>() : nullptr, block_tables.data_ptr<int>(), cu_q.data_ptr<int>(),
        seq_lens.data_ptr<int>(), (int)num_seqs, (int)max_q_len, (int)block_tables.size(1), bs, Hq, Hk, Dqk, Dv,
        q.stride(0), out.stride(0), (float)scale, causal ? 1 : 0, (int)window, (long long)T, (int)k_cache.size(0),
        status.has_value() ? status->data_ptr<int>() : nullptr, cur_stream());
    if (rc == 0) return {out, lse};
    TORCH_CHECK(rc == 1, "omni_b200::gqa_prefill (tcgen05) failed with code ", rc);
  }
  check(b200_gqa_prefill(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                         return_lse ? lse.data_ptr<float>() : nullptr, block_tables.data_ptr<int>(),
                         cu_q.data_ptr<int>(), seq_lens.data_ptr<int>(), (int)num_seqs,
                         (int)max_q_len, (int)block_tables.size(1), bs, Hq, Hk, Dqk, Dv,
                         q.stride(0), out.stride(0), (float)scale, causal ? 1 : 0, (int)window,
                         cur_stream()),
        "gqa_prefill");
  return {out, lse};
}

int64_t gqa_decode_scratch_bytes(int64_t B, int64_t Hk, int64_t D, int64_t splits) {
  return (int64_t)b200_gqa_decode_scratch_bytes((int)B, (int)Hk, (int)D, (int)splits);
}

Tensor gqa_decode(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache,
                  const Tensor& block_tables, const Tensor& seq_lens, int64_t num_seqs,
                  int64_t q_len, int64_t num_q_heads, double scale, int64_t window, int64_t splits,
                  const c10::optional<Tensor>& scratch, const Tensor& status, int64_t persistent,
                  const c10::optional<Tensor>& work_counter) {
  CHECK_CUDA_BF16(q);
  CHECK_CUDA_BF16(k_cache);
  CHECK_CUDA_BF16(v_cache);
  CHECK_I32(block_tables);
  CHECK_I32(seq_lens);
  const int Hk = k_cache.size(1), bs = k_cache.size(2), D = k_cache.size(3);
  const int Hq = num_q_heads;
  TORCH_CHECK(q.dim() == 2 && q.stride(1) == 1 && q.size(1) == (int64_t)Hq * D, "gqa_decode: q");
  TORCH_CHECK(q.size(0) >= num_seqs * q_len, "gqa_decode: q rows");
  c10::cuda::CUDAGuard guard(q.device());
  Tensor out = torch::empty({q.size(0), (int64_t)Hq * D}, q.options());
  void* sp = nullptr;
  if (persistent == 2) {
    TORCH_CHECK(scratch.has_value(), "gqa_decode: scratch required for the balanced kernel");
    TORCH_CHECK((int64_t)scratch->nbytes() >=
                    (int64_t)b200_gqa_decode_balanced_scratch_bytes(D, (int)((Hq / Hk) * q_len)),
                "gqa_decode: scratch too small");
    sp = scratch->data_ptr();
  } else if (splits > 1) {
    TORCH_CHECK(scratch.has_value(), "gqa_decode: scratch required for splits > 1");
    TORCH_CHECK((int64_t)scratch->nbytes() >=
                    (int64_t)b200_gqa_decode_scratch_bytes((int)num_seqs, Hk, D, (int)splits),
                "gqa_decode: scratch too small");
    sp = scratch->data_ptr();
  }
  int* wc = nullptr;
  if (work_counter.has_value()) {
    CHECK_I32((*work_counter));
    TORCH_CHECK(work_counter->numel() >= 2, "gqa_decode: work_counter needs two ints");
    wc = work_counter->data_ptr<int>();
  }
  check(b200_gqa_decode_ex(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                           nullptr, block_tables.data_ptr<int>(), seq_lens.data_ptr<int>(),
                           (int)num_seqs, (int)q_len, (int)block_tables.size(1), bs, Hq, Hk, D,
                           q.stride(0), out.stride(0), (float)scale, (int)window, (int)splits, sp,
                           (int)k_cache.size(0), status.data_ptr<int>(), (int)persistent, wc, cur_stream()),
        "gqa_decode");
  return out;
}

// Copies KV blocks between two sets of cache tensors (the source may be another GPU's,
// mapped through CUDA IPC).  desc: int64 [num_tensors, 3] = (src base, dst base, block bytes).
void kv_p2p_copy(const Tensor& desc, const Tensor& src_blocks, const Tensor& dst_blocks,
                 int64_t max_block_bytes) {
  TORCH_CHECK(desc.is_cuda() && desc.scalar_type() == at::kLong && desc.dim() == 2 && desc.size(1) == 3 &&
                  desc.is_contiguous(),
              "kv_p2p_copy: desc int64 [n,3] on the device");
  CHECK_I32(src_blocks);
  CHECK_I32(dst_blocks);
  TORCH_CHECK(src_blocks.numel() == dst_blocks.numel(), "kv_p2p_copy: block list sizes differ");
  c10::cuda::CUDAGuard guard(desc.device());
  check(b200_kv_p2p_copy(desc.data_ptr(), (int)desc.size(0), src_blocks.data_ptr<int>(),
                         dst_blocks.data_ptr<int>(), (int)src_blocks.numel(), max_block_bytes, cur_stream()),
        "kv_p2p_copy");
}

int64_t mla_decode_scratch_bytes(int64_t T, int64_t N, int64_t splits) {
  return (int64_t)b200_mla_decode_scratch_bytes((int)T, (int)N, (int)splits);
}

// Absorbed multi-head latent attention over the paged latent cache.
// q [T, N*576], cache [blocks, block_size, 576] -> out [T, N*512].
std::tuple<Tensor, Tensor> mla_decode(const Tensor& q, const Tensor& cache, const Tensor& block_tables,
                  const Tensor& seq_lens, const c10::optional<Tensor>& topk_indices,
                  int64_t num_seqs, int64_t q_len, int64_t num_heads, double scale, int64_t splits,
                  const c10::optional<Tensor>& scratch, const Tensor& status, bool return_lse) {
  CHECK_CUDA_BF16(q);
  CHECK_CUDA_BF16(cache);
  CHECK_I32(block_tables);
  CHECK_I32(seq_lens);
  TORCH_CHECK(cache.dim() == 3 && cache.size(2) == 576 && cache.is_contiguous(), "mla cache [blocks, bs, 576]");
  TORCH_CHECK(q.dim() == 2 && q.stride(1) == 1 && q.size(1) == num_heads * 576, "mla_decode: q [T, N*576]");
  const int T = num_seqs * q_len;
  TORCH_CHECK(q.size(0) >= T, "mla_decode: q rows");
  c10::cuda::CUDAGuard guard(q.device());
  Tensor out = torch::empty({q.size(0), num_heads * 512}, q.options());
  const int* tk = nullptr;
  int topk = 0;
  if (topk_indices.has_value()) {
    CHECK_I32(*topk_indices);
    TORCH_CHECK(topk_indices->dim() == 2 && topk_indices->size(0) >= T, "topk_indices [T, topk]");
    tk = topk_indices->data_ptr<int>();
    topk = topk_indices->size(1);
  }
  void* sp = nullptr;
  if (splits > 1) {
    TORCH_CHECK(scratch.has_value() &&
                    (int64_t)scratch->nbytes() >= mla_decode_scratch_bytes(T, num_heads, splits),
                "mla_decode: scratch too small");
    sp = scratch->data_ptr();
  }
  Tensor lse = return_lse ? torch::empty({q.size(0), num_heads}, q.options().dtype(at::kFloat)) : Tensor();
  check(b200_mla_decode(q.data_ptr(), cache.data_ptr(), out.data_ptr(), return_lse ? lse.data_ptr<float>() : nullptr,
                        block_tables.data_ptr<int>(), seq_lens.data_ptr<int>(), tk, topk, (int)num_seqs,
                        (int)q_len, (int)num_heads, (int)block_tables.size(1), (int)cache.size(1),
                        (int)cache.size(0), q.stride(0), out.stride(0), (float)scale, (int)splits, sp,
                        status.data_ptr<int>(), cur_stream()),
        "mla_decode");
  return {out, lse};
}

// Router: gate logits [T,E] fp32 -> (top-k ids int32 [T,k], weights fp32 [T,k]).
std::tuple<Tensor, Tensor> moe_topk(const Tensor& logits, const c10::optional<Tensor>& bias,
                                    int64_t k, bool sigmoid, int64_t n_group, int64_t topk_group,
                                    bool renorm, double scale) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.is_contiguous() &&
                  logits.dim() == 2,
              "moe_topk: logits [T,E] fp32 contiguous");
  const int T = logits.size(0), E = logits.size(1);
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor ids = torch::empty({T, k}, logits.options().dtype(at::kInt));
  Tensor w = torch::empty({T, k}, logits.options());
  const float* bp = nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == at::kFloat && bias->numel() == E && bias->is_contiguous(),
                "moe_topk: bias [E] fp32");
    bp = bias->data_ptr<float>();
  }
  check(b200_moe_topk(logits.data_ptr<float>(), bp, ids.data_ptr<int>(), w.data_ptr<float>(), T, E,
                      (int)k, sigmoid ? 1 : 0, (int)n_group, (int)topk_group, renorm ? 1 : 0,
                      (float)scale, cur_stream()),
        "moe_topk");
  return {ids, w};
}

Tensor argmax(const Tensor& logits) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "argmax: [B,V]");
  const bool f32 = logits.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || logits.scalar_type() == at::kBFloat16, "argmax: fp32 or bf16");
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor out = torch::empty({logits.size(0)}, logits.options().dtype(at::kInt));
  check(b200_argmax(logits.data_ptr(), out.data_ptr<int>(), (int)logits.size(0),
                    (int)logits.size(1), logits.stride(0), f32 ? 1 : 0, cur_stream()),
        "argmax");
  return out;
}

Tensor sample(const Tensor& logits, const c10::optional<Tensor>& temperature,
              const c10::optional<Tensor>& top_k, const c10::optional<Tensor>& top_p,
              const c10::optional<Tensor>& seeds, const c10::optional<Tensor>& step_offset) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "sample: [B,V]");
  const bool f32 = logits.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || logits.scalar_type() == at::kBFloat16, "sample: fp32 or bf16");
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor out = torch::empty({logits.size(0)}, logits.options().dtype(at::kInt));
  check(b200_sample(logits.data_ptr(), out.data_ptr<int>(),
                    temperature.has_value() ? temperature->data_ptr<float>() : nullptr,
                    top_k.has_value() ? top_k->data_ptr<int>() : nullptr,
                    top_p.has_value() ? top_p->data_ptr<float>() : nullptr,
                    seeds.has_value() ? (const long long*)seeds->data_ptr<int64_t>() : nullptr,
                    step_offset.has_value() ? (const long long*)step_offset->data_ptr<int64_t>() : nullptr,
                    (int)logits.size(0), (int)logits.size(1), logits.stride(0), f32 ? 1 : 0,
                    cur_stream()),
        "sample");
  return out;
}

}  // namespace

TORCH_LIBRARY(omni_b200, m) {
  m.def("spec_verify", &spec_verify);
  m.def("lse_merge", &lse_merge);
  m.def("gather_cache", &gather_cache);
  m.def("gemm_plan", &gemm_plan);
  m.def("gemm", &gemm);
  m.def("gemm_pair", &gemm_pair);
  m.def("gemm_scaled", &gemm_scaled);
  m.def("quant_int8_per_token", &quant_int8_per_token);
  m.def("rms_norm_quant", &rms_norm_quant);
  m.def("dsa_indexer", &dsa_indexer);
  m.def("gemm_fp8_block", &gemm_fp8_block);
  m.def("grouped_gemm_fp8_block", &grouped_gemm_fp8_block);
  m.def("silu_and_mul_quant", &silu_and_mul_quant);
  m.def("grouped_gemm", &grouped_gemm);
  m.def("rms_norm", &rms_norm);
  m.def("fused_add_rms_norm", &fused_add_rms_norm);
  m.def("silu_and_mul", &silu_and_mul);
  m.def("quant_fp8_1x128", &quant_fp8_1x128);
  m.def("rope_qk", &rope_qk);
  m.def("rope_cache_gqa", &rope_cache_gqa);
  m.def("mla_kv_rmsnorm_rope_cache", &mla_kv_rmsnorm_rope_cache);
  m.def("paged_scatter_rows", &paged_scatter_rows);
  m.def("gqa_cache_write", &gqa_cache_write);
  m.def("gqa_prefill", &gqa_prefill);
  m.def("gqa_decode_scratch_bytes", &gqa_decode_scratch_bytes);
  m.def("gqa_decode_balanced_scratch_bytes", [](int64_t D, int64_t rows) {
    return (int64_t)b200_gqa_decode_balanced_scratch_bytes((int)D, (int)rows);
  });
  m.def("gqa_decode", &gqa_decode);
  m.def("kv_p2p_copy", &kv_p2p_copy);
  m.def("mla_decode_scratch_bytes", &mla_decode_scratch_bytes);
  m.def("mla_decode", &mla_decode);
  m.def("moe_topk", &moe_topk);
  m.def("argmax", &argmax);
  m.def("sample", &sample);
}
