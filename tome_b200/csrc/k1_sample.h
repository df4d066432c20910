// Internal interface of the streaming kernel's sampling mode (see k1_logprob.cu, MODE = SAMPLE),
// the first stage of the large-batch sampling path of k4_sample.cu: it streams the logits once
// at HBM speed, keeps the row's (max, sum-exp), derives the row's top-k threshold from the
// logits as they pass and notes where the logits that reach it sit.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tome {

// Base and row pitch are multiples of 16 bytes, a row holds at least one 16-byte vector and
// fewer than 2^27 of them.
bool k1_sample_eligible(const void* logits, int32_t dtype, int64_t vocab, int64_t row_stride);

// Lists the kernel keeps per row (one per consumer warp), entries a list holds, and the
// distance (in 16-byte vectors) between the four vectors one entry speaks of.
int k1_sample_lists_per_row();
int k1_sample_list_capacity();
int k1_sample_vector_stride();

// Outputs, per row: row_thr [rows], a value that at least min(top_k, vocab) logits of the row
// reach; L = k1_sample_lists_per_row() lists of entries {(v << 4) | mask, largest}: bit j of the
// mask says that the 16-byte vector number v + j * k1_sample_vector_stride() of the row holds a
// logit >= the threshold in force when it passed (never above row_thr, so every logit >=
// row_thr sits in a vector some entry names; the elements past the row's last 16-byte boundary
// count as one more, short, vector), and `largest` is the float bits of the largest logit of the
// entry's four vectors (NaN if one of them holds a NaN): cand_count [rows, L] (cand_cap + 1 if a
// list ran over) and cand_entry [rows, L, cand_cap].  out_lse [rows] receives
// logsumexp(x / temperature).  *zero_word (nullable) is set to 0 by the kernel (the counter of
// the stage that follows).
int32_t k1_launch_sample(const void* logits, int32_t dtype, int64_t rows, int64_t vocab,
                         int64_t row_stride, float temperature, int32_t top_k, float* row_thr,
                         int32_t* cand_count, uint2* cand_entry, int32_t cand_cap,
                         float* out_lse, int32_t* zero_word, int32_t* dev_status,
                         cudaStream_t stream);

}  // namespace tome
