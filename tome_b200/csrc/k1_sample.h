// Internal interface of the streaming kernel's sampling mode (see k1_logprob.cu, MODE = SAMPLE),
// the middle stage of the three-kernel sampling path of k4_sample.cu: it streams the logits
// once at HBM speed, keeps the row's (max, sum-exp) and appends every logit that reaches the
// row's threshold to the row's candidate list.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tome {

// Base and row pitch are multiples of 16 bytes and a row holds at least one 16-byte vector.
bool k1_sample_eligible(const void* logits, int32_t dtype, int64_t vocab, int64_t row_stride);

// row_thr [rows]: value thresholds; cand_count [rows] (zeroed by the caller) counts the
// candidates of each row, of which the first cand_cap are stored in cand [rows, cand_cap] as
// packed codes (sampling.cuh); out_lse [rows] receives logsumexp(x / temperature).
int32_t k1_launch_sample(const void* logits, int32_t dtype, int64_t rows, int64_t vocab,
                         int64_t row_stride, float temperature, const float* row_thr,
                         int32_t* cand_count, unsigned long long* cand, int32_t cand_cap,
                         float* out_lse, int32_t* dev_status, cudaStream_t stream);

}  // namespace tome
