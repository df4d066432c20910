// Merge of per-part (max, sum-exp, target-logit) triples.  The parts are vocabulary
// shards after the vocab-parallel exchange, or the vocabulary bands of one fused
// LM-head launch.  The reference has no sharded head; the merge is the standard
// log-sum-exp identity  lse = M + log(sum_p s_p * exp(m_p - M)),  M = max_p m_p.
#include <float.h>

#include "combine.h"
#include "host_common.h"

namespace tome {

template <bool FINAL>
__global__ void __launch_bounds__(256) combine_kernel(const float* __restrict__ m,
                                                      const float* __restrict__ s,
                                                      int64_t ms_stride, int n_parts,
                                                      const float* __restrict__ t,
                                                      int64_t t_stride, int n_t_parts,
                                                      int64_t rows, float* __restrict__ out0,
                                                      float* __restrict__ out1,
                                                      float* __restrict__ out2) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < rows;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float M = -FLT_MAX;
    for (int p = 0; p < n_parts; ++p) M = fmaxf(M, m[p * ms_stride + i]);
    float S = 0.0f;
    for (int p = 0; p < n_parts; ++p) {
      const float sp = s[p * ms_stride + i];
      // a part that saw no column keeps s = 0 and must not contribute exp(-huge) * 0 = NaN
      if (sp != 0.0f) S += sp * expf(m[p * ms_stride + i] - M);
    }
    float T = 0.0f;
    for (int q = 0; q < n_t_parts; ++q) T += t[q * t_stride + i];
    if (FINAL) {
      const float lse = M + logf(S);
      out0[i] = T - lse;
      if (out1 != nullptr) out1[i] = lse;
    } else {
      out0[i] = M;
      out1[i] = S;
      out2[i] = T;
    }
  }
}

int32_t launch_combine(bool final, const float* m, const float* s, int64_t ms_stride,
                       int32_t n_parts, const float* t, int64_t t_stride, int32_t n_t_parts,
                       int64_t rows, float* out0, float* out1, float* out2,
                       cudaStream_t stream) {
  if (rows == 0) return TOME_OK;
  const int threads = 256;
  const int64_t want = (rows + threads - 1) / threads;
  const int grid = static_cast<int>(want < 4096 ? want : 4096);
  if (final)
    combine_kernel<true><<<grid, threads, 0, stream>>>(m, s, ms_stride, n_parts, t, t_stride,
                                                       n_t_parts, rows, out0, out1, out2);
  else
    combine_kernel<false><<<grid, threads, 0, stream>>>(m, s, ms_stride, n_parts, t, t_stride,
                                                        n_t_parts, rows, out0, out1, out2);
  return check_cuda(cudaGetLastError(), "combine launch");
}

}  // namespace tome

extern "C" int32_t tome_combine_triples(const float* m, const float* s, int64_t ms_part_stride,
                                        int32_t n_parts, const float* t, int64_t t_part_stride,
                                        int32_t n_t_parts, int64_t rows, float* out_logprob,
                                        float* out_lse, void* stream) {
  using namespace tome;
  if (rows < 0 || n_parts <= 0 || n_t_parts <= 0)
    return fail(TOME_ERR_BAD_SHAPE, "rows=%lld n_parts=%d n_t_parts=%d", (long long)rows, n_parts,
                n_t_parts);
  if (rows == 0) return TOME_OK;
  if (m == nullptr || s == nullptr || t == nullptr || out_logprob == nullptr)
    return fail(TOME_ERR_NULL_POINTER, "a required pointer is NULL");
  if ((n_parts > 1 && ms_part_stride < rows) || (n_t_parts > 1 && t_part_stride < rows))
    return fail(TOME_ERR_BAD_STRIDE, "part stride smaller than rows");
  return launch_combine(true, m, s, ms_part_stride, n_parts, t, t_part_stride, n_t_parts, rows,
                        out_logprob, out_lse, nullptr, static_cast<cudaStream_t>(stream));
}
