// Internal interface of the streaming kernel's sampling mode (see k1_logprob.cu, MODE = SAMPLE),
// the middle stage of the three-kernel sampling path of k4_sample.cu: it streams the logits
// once at HBM speed, keeps the row's (max, sum-exp) and appends every logit that reaches the
// row's threshold, with the 16-byte vector it sits in, to the row's candidate list.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tome {

// Base and row pitch are multiples of 16 bytes and a row holds at least one 16-byte vector.
bool k1_sample_eligible(const void* logits, int32_t dtype, int64_t vocab, int64_t row_stride);

// row_thr [rows]: value thresholds.  cand_count [rows] receives the number of 16-byte vectors
// of the row that hold a logit >= the threshold (cand_cap + 1 if more than cand_cap), the
// vectors themselves go to cand_vec [rows, cand_cap] and their positions in the row (in
// 16-byte units) to cand_idx [rows, cand_cap]; a tail shorter than a vector is padded with
// -inf.  out_lse [rows] receives logsumexp(x / temperature).
int32_t k1_launch_sample(const void* logits, int32_t dtype, int64_t rows, int64_t vocab,
                         int64_t row_stride, float temperature, const float* row_thr,
                         int32_t* cand_count, uint4* cand_vec, int32_t* cand_idx,
                         int32_t cand_cap, float* out_lse, int32_t* dev_status,
                         cudaStream_t stream);

}  // namespace tome
