// Internal interface of the streaming kernel's sampling mode (see k1_logprob.cu, MODE = SAMPLE):
// top-k sampling + log-prob at HBM speed for large batches.  Rows whose candidate ring
// overflowed get token -1 and are redone by the one-CTA-per-row kernel (k4_sample.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tome {

// Base and row pitch are multiples of 16 bytes and a row holds at least one 16-byte vector.
bool k1_sample_eligible(const void* logits, int32_t dtype, int64_t vocab, int64_t row_stride);

int32_t k1_launch_sample(const void* logits, int32_t dtype, int64_t rows, int64_t vocab,
                         int64_t row_stride, float temperature, int32_t top_k, uint64_t seed,
                         uint64_t offset, int32_t* out_tokens, float* out_logprob,
                         int32_t* out_topk_idx, float* out_topk_val, int32_t* dev_status,
                         cudaStream_t stream);

}  // namespace tome
