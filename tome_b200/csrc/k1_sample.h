// Internal interface of the streaming kernel's sampling mode (see k1_logprob.cu, MODE = SAMPLE),
// the first stage of the large-batch sampling path of k4_sample.cu: it streams the logits once
// at HBM speed, keeps the row's (max, sum-exp), derives the row's top-k threshold from the
// logits as they pass and gathers the 16-byte vectors that hold a logit reaching it.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tome {

// Base and row pitch are multiples of 16 bytes and a row holds at least one 16-byte vector.
bool k1_sample_eligible(const void* logits, int32_t dtype, int64_t vocab, int64_t row_stride);

// Candidate lists the kernel keeps per row (one per consumer warp).
int k1_sample_lists_per_row();

// Outputs, per row: row_thr [rows], a value that at least min(top_k, vocab) logits of the row
// reach; L = k1_sample_lists_per_row() lists of the 16-byte vectors that hold a logit >= the
// threshold in force when they passed (never above row_thr, so every logit >= row_thr is in a
// listed vector): cand_count [rows, L] (cand_cap + 1 if a list ran over), cand_vec
// [rows, L, cand_cap] and cand_idx [rows, L, cand_cap] (position in the row, 16-byte units);
// a tail shorter than a vector is padded with -inf.  out_lse [rows] receives
// logsumexp(x / temperature).  *zero_word (nullable) is set to 0 by the kernel (the counter of
// the stage that follows).
int32_t k1_launch_sample(const void* logits, int32_t dtype, int64_t rows, int64_t vocab,
                         int64_t row_stride, float temperature, int32_t top_k, float* row_thr,
                         int32_t* cand_count, uint4* cand_vec, int32_t* cand_idx,
                         int32_t cand_cap, float* out_lse, int32_t* zero_word,
                         int32_t* dev_status, cudaStream_t stream);

}  // namespace tome
