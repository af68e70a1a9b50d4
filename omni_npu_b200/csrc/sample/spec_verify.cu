// Speculative-decoding verification.  Request b proposed n_b = cu[b+1]-cu[b] draft
// tokens; the target model produced a token for each of those positions (sampled
// from the target distribution) plus one bonus token for the position after the last
// draft.  A draft token is accepted while it equals the target's token at the same
// position; the first mismatch emits the target's token and stops; if every draft
// matched, the bonus token is emitted as well.  One thread per request.
//
//   out[b, 0..max_spec]  accepted tokens then -1 padding
//   num_out[b]           tokens emitted for request b (1 .. n_b + 1)
//
// Same decision rule as `simple_verify` in omni_npu/sample/rejection_sampler.py:253-291,
// with the cascade made explicit (nothing after the first mismatch is emitted).

#include <cuda_runtime.h>

namespace b200 {

__global__ void spec_verify_kernel(const int* __restrict__ draft, const int* __restrict__ target,
                                   const int* __restrict__ bonus, const int* __restrict__ cu,
                                   int* __restrict__ out, int* __restrict__ num_out, int B, int max_spec) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int lo = cu[b], n = cu[b + 1] - lo;
  int* row = out + static_cast<long long>(b) * (max_spec + 1);
  int emitted = 0;
  bool all = true;
  for (int i = 0; i < n && i < max_spec; ++i) {
    const int t = target[lo + i];
    row[emitted++] = t;
    if (t != draft[lo + i]) {
      all = false;
      break;
    }
  }
  if (all) row[emitted++] = bonus[b];
  num_out[b] = emitted;
  for (int i = emitted; i <= max_spec; ++i) row[i] = -1;
}

}  // namespace b200

extern "C" int b200_spec_verify(const int* draft, const int* target, const int* bonus, const int* cu,
                                int* out, int* num_out, int B, int max_spec, cudaStream_t stream) {
  if (B <= 0) return 0;
  b200::spec_verify_kernel<<<(B + 127) / 128, 128, 0, stream>>>(draft, target, bonus, cu, out, num_out, B, max_spec);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
