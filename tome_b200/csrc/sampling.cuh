// Pieces shared by the kernels that sample a token from the top-k of a row: the order-preserving
// (value, index) codes, the counter-based random generator and the categorical draw.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace tome {

constexpr int K4_MAX_K = 64;  // largest top_k

// Order-preserving map float -> uint32 (larger float <=> larger key).  NaN maps to 0.
__device__ __forceinline__ uint32_t k4_key(float x) {
  if (x != x) return 0u;
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float k4_unkey(uint32_t k) {
  const uint32_t b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(b);
}

// (value, index) as one integer whose numeric order is "larger value first, then lower index":
// every logit of a row gets a distinct code, so top-k selection has no ties to break.
__device__ __forceinline__ unsigned long long k4_pack(float x, int64_t idx) {
  return (static_cast<unsigned long long>(k4_key(x)) << 32) |
         static_cast<unsigned long long>(0xffffffffu - static_cast<uint32_t>(idx));
}
__device__ __forceinline__ float k4_value(unsigned long long pk) {
  return k4_unkey(static_cast<uint32_t>(pk >> 32));
}
__device__ __forceinline__ int32_t k4_index(unsigned long long pk) {
  return static_cast<int32_t>(0xffffffffu - static_cast<uint32_t>(pk));
}

// Philox-4x32-10: one 128-bit block for (counter, key); returns the first word.
__device__ __forceinline__ uint32_t k4_philox(uint64_t ctr_lo, uint64_t ctr_hi, uint64_t key) {
  uint32_t c0 = static_cast<uint32_t>(ctr_lo), c1 = static_cast<uint32_t>(ctr_lo >> 32);
  uint32_t c2 = static_cast<uint32_t>(ctr_hi), c3 = static_cast<uint32_t>(ctr_hi >> 32);
  uint32_t k0 = static_cast<uint32_t>(key), k1 = static_cast<uint32_t>(key >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0;
    const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2;
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ k0;
    const uint32_t n1 = static_cast<uint32_t>(p1);
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ k1;
    const uint32_t n3 = static_cast<uint32_t>(p0);
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}

// Index (0 = best) drawn from softmax(top / temperature) over the kk best codes of a row,
// `top` sorted best first (at most 64), c = log2(e) / temperature.  The draw depends only on
// (seed, offset, row): u = uniform(row, offset, seed) * sum_j e_j with e_j = 2^((top_j - top_0) c)
// summed in the order j = 0, 1, ..., and the index is the first j whose partial sum exceeds u.
// Made by a whole warp (all 32 lanes call it, all get the index): the terms are formed side by
// side, the sums are taken one term at a time so that every caller gets the same bits.
__device__ __forceinline__ int32_t k4_draw_warp(const unsigned long long* top, int32_t kk, float c,
                                                int64_t row, uint64_t seed, uint64_t offset) {
  if (kk <= 1) return 0;
  const int lane = static_cast<int>(lane_id());
  const float best = k4_value(top[0]);
  const float e_lo = (lane < kk) ? ex2f((k4_value(top[lane]) - best) * c) : 0.0f;
  const float e_hi = (lane + 32 < kk) ? ex2f((k4_value(top[lane + 32]) - best) * c) : 0.0f;
  // prefix sums in the serial order: every lane adds the terms one by one and keeps the
  // partial sums that belong to its own two places
  float acc = 0.0f, mine_lo = 0.0f, mine_hi = 0.0f;
  for (int32_t j = 0; j < kk; ++j) {
    acc += __shfl_sync(0xffffffffu, (j < 32) ? e_lo : e_hi, j & 31);
    if (j == lane) mine_lo = acc;
    if (j == lane + 32) mine_hi = acc;
  }
  const uint32_t r = k4_philox(static_cast<uint64_t>(row), offset, seed);
  const float u = (static_cast<float>(r >> 8) + 0.5f) * (1.0f / 16777216.0f) * acc;
  const uint32_t lo = __ballot_sync(0xffffffffu, lane < kk && u < mine_lo);
  const uint32_t hi = __ballot_sync(0xffffffffu, lane + 32 < kk && u < mine_hi);
  if (lo != 0u) return __ffs(lo) - 1;
  if (hi != 0u) return 32 + __ffs(hi) - 1;
  return kk - 1;
}

}  // namespace tome
