// Internal launcher of the triple-merge kernel (see combine.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tome {

// final = true : out0 = logprob, out1 = lse (nullable), out2 unused
// final = false: out0 = M, out1 = S, out2 = T (the merged triple, still a triple)
int32_t launch_combine(bool final, const float* m, const float* s, int64_t ms_stride,
                       int32_t n_parts, const float* t, int64_t t_stride, int32_t n_t_parts,
                       int64_t rows, float* out0, float* out1, float* out2, cudaStream_t stream);

}  // namespace tome
