// Shared pieces of the streaming log-softmax kernels (K1): modes, launch parameters, the
// per-row result code and the exact fallback.  Included by k1_logprob.cu (pipeline and
// plain-load kernels, C entry points), k1_small.cu (small batches) and k1_full.cu
// (cluster-resident full matrix).
#pragma once
#include <cuda_bf16.h>
#include <float.h>
#include <math.h>
#include <stdlib.h>

#include <algorithm>
#include <type_traits>

#include "host_common.h"
#include "online.cuh"
#include "ptx.cuh"

namespace tome {

enum K1Mode { K1_SELECTIVE = 0, K1_DUAL = 1, K1_FULL = 2, K1_RAGGED = 3, K1_SAMPLE = 4 };

// DUAL and RAGGED score only a window [start, start + length) of each sequence.
__host__ __device__ constexpr bool k1_windowed(int mode) {
  return mode == K1_DUAL || mode == K1_RAGGED;
}

// Tuning constants (overridable at compile time for experiments).
#ifndef K1_CFG_WARPS
#define K1_CFG_WARPS 4
#endif
#ifndef K1_CFG_STAGES
#define K1_CFG_STAGES 2
#endif
#ifndef K1_CFG_CHUNK
#define K1_CFG_CHUNK 25600
#endif
#ifndef K1_CFG_CHUNK_ALIGN
#define K1_CFG_CHUNK_ALIGN 1024
#endif
#ifndef K1_CFG_CTAS_PER_SM
#define K1_CFG_CTAS_PER_SM 4
#endif
#ifndef K1_CFG_L2_HINT
#define K1_CFG_L2_HINT 1
#endif
constexpr int K1_CONSUMER_WARPS = K1_CFG_WARPS;
constexpr int K1_CONSUMERS = K1_CONSUMER_WARPS * 32;
constexpr int K1_THREADS = K1_CONSUMERS + 32;
constexpr int K1_STAGES = K1_CFG_STAGES;
constexpr int K1_CHUNK_BYTES = K1_CFG_CHUNK;
constexpr int K1_CTAS_PER_SM = K1_CFG_CTAS_PER_SM;
// bulk copies start on multiples of this many bytes from the row start (keeps them aligned
// to whole 128-byte lines when the row pitch is)
constexpr int K1_CHUNK_ALIGN = K1_CFG_CHUNK_ALIGN;
static_assert(K1_CHUNK_BYTES % K1_CHUNK_ALIGN == 0 && K1_CHUNK_ALIGN % 16 == 0, "chunk alignment");
static_assert(K1_CONSUMER_WARPS <= 32, "row-end merge reads one partial per lane");
constexpr int K1_MAX_SEQ = 1024;
constexpr int K1_POLY_DEFAULT = 2;

struct K1Params {
  const void* src[2];      // DUAL: policy, reference
  int64_t n_rows;          // SELECTIVE/FULL: rows; DUAL: n_seq * seq_len (dense row count)
  int64_t vocab;
  int64_t stride;          // elements between rows
  const int32_t* targets;  // SELECTIVE, DUAL
  float c;                 // log2(e) / temperature
  float temp;
  float inv_temp;
  float* out0;             // SELECTIVE: logprob   DUAL: policy logprob   FULL: lse (nullable)   SAMPLE: logprob of the drawn token
  float* out1;             // SELECTIVE: lse (nullable)   DUAL: reference logprob   SAMPLE: lse (scratch)
  float* out2;             // SELECTIVE: raw target logit (nullable)   DUAL: k3 KL
  void* out_full;          // FULL
  int64_t out_stride;      // FULL
  const int32_t* lengths;  // DUAL
  const int32_t* starts;   // DUAL, nullable
  int32_t n_seq;           // DUAL
  int32_t seq_len;         // DUAL
  int64_t packed_capacity; // RAGGED: entries the packed target/output arrays can hold
  int32_t* out_offsets;    // RAGGED: int32 [n_seq + 1], start of each sequence in the packed output
  float* row_thr;          // SAMPLE: out, per row (per part) the final threshold (>= top_k logits reach it)
  int32_t* cand_count;     // SAMPLE: [rows, parts, lists] entries per list (cand_cap + 1: overflow)
  uint2* cand_entry;       // SAMPLE: [rows, parts, lists, cand_cap] noted places, see K1SampleSmem
  int32_t cand_cap;        // SAMPLE: entries per list (lists per row = consumer warps)
  int32_t sample_kk;       // SAMPLE: min(top_k, vocab)
  int32_t sample_q;        // SAMPLE: ceil(top_k / consumer warps), 1 .. 32
  int32_t finish_in_kernel;  // SAMPLE: the producer warp finishes the rows
  int32_t sample_parts_log2;  // SAMPLE: a row is cut into 1, 2 or 4 parts (work items of their own)
  float2* part_ms;         // SAMPLE, rows in parts: [rows, parts] (max, sum-exp) of each part
  int32_t sample_top_k;    // SAMPLE: top_k as asked for (width of the top-k outputs)
  float sample_temperature;  // SAMPLE: as asked for; 0 = greedy (then temp is 1)
  uint64_t sample_seed, sample_offset;
  int32_t* out_tokens;     // SAMPLE: [rows]
  int32_t* out_topk_idx;   // SAMPLE: nullable, [rows, top_k]
  float* out_topk_val;     // SAMPLE: nullable, [rows, top_k]
  int32_t* marked;         // SAMPLE: number of rows left to the row kernel (see K1SampleArgs)
  int32_t* marked_rows;    // SAMPLE: their indices
  int32_t* status;         // nullable
  int32_t chunk_bytes;     // bulk-copy size (multiple of 16, <= K1_CHUNK_BYTES), set by launch
  int32_t n_chunks;        // bulk copies per row
};

// ------------------------------------------------------------------ FULL mode output
// out = T(float(x) * inv_temp) - T(lse), subtraction in T (mlx-impl/model.py:57-60).
// bf16 rows use packed forms, two logits per instruction (f32x2 multiply, bf16x2 convert and
// subtract); the rounding steps are those of the scalar forms below, one by one.  Pass 2 of
// the full-matrix kernels was bound by its instruction count: 48 -> 20 instructions per
// 16-byte vector took 4096 x 151936 bf16 from 5.43 to 5.63 TB/s (5.92 at temperature 1, where
// only the subtraction is left).
__device__ __forceinline__ uint32_t full_out_bf16x2(uint32_t w, float2 inv2, uint32_t lse2) {
  const float2 scaled = __fmul2_rn(make_float2(bf16_lo(w), bf16_hi(w)), inv2);
  uint32_t t;  // round both to bf16 (nearest even), low half = first operand of the pair
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(t) : "f"(scaled.y), "f"(scaled.x));
  const __nv_bfloat162 r = __hsub2(as_bf162(t), as_bf162(lse2));
  return *reinterpret_cast<const uint32_t*>(&r);
}

__device__ __forceinline__ uint4 full_out_vec(uint4 v, float inv_temp, float lse, __nv_bfloat16) {
  const uint32_t l16 = __bfloat16_as_ushort(__float2bfloat16_rn(lse));
  const uint32_t lse2 = l16 | (l16 << 16);
  uint4 o;
  if (inv_temp == 1.0f) {  // x * 1 rounds to x: only the subtraction is left
    const __nv_bfloat162 l2 = as_bf162(lse2);
    const __nv_bfloat162 a = __hsub2(as_bf162(v.x), l2), b = __hsub2(as_bf162(v.y), l2);
    const __nv_bfloat162 c = __hsub2(as_bf162(v.z), l2), d = __hsub2(as_bf162(v.w), l2);
    o.x = *reinterpret_cast<const uint32_t*>(&a);
    o.y = *reinterpret_cast<const uint32_t*>(&b);
    o.z = *reinterpret_cast<const uint32_t*>(&c);
    o.w = *reinterpret_cast<const uint32_t*>(&d);
    return o;
  }
  const float2 inv2 = make_float2(inv_temp, inv_temp);
  o.x = full_out_bf16x2(v.x, inv2, lse2);
  o.y = full_out_bf16x2(v.y, inv2, lse2);
  o.z = full_out_bf16x2(v.z, inv2, lse2);
  o.w = full_out_bf16x2(v.w, inv2, lse2);
  return o;
}

// fp32: scalar multiply and subtract with the rounding of each step spelt out.  (The packed
// f32x2 multiply followed by a packed add came out fused into one multiply-add, which skips
// the first rounding: an error of 1e22 on logits of -1e30.  fp32 rows are not bound by the
// instruction count anyway.)
__device__ __forceinline__ uint4 full_out_vec(uint4 v, float inv_temp, float lse, float) {
  uint4 o;
  o.x = __float_as_uint(__fsub_rn(__fmul_rn(__uint_as_float(v.x), inv_temp), lse));
  o.y = __float_as_uint(__fsub_rn(__fmul_rn(__uint_as_float(v.y), inv_temp), lse));
  o.z = __float_as_uint(__fsub_rn(__fmul_rn(__uint_as_float(v.z), inv_temp), lse));
  o.w = __float_as_uint(__fsub_rn(__fmul_rn(__uint_as_float(v.w), inv_temp), lse));
  return o;
}

__device__ __forceinline__ float full_out_scalar(float x, float inv_temp, float lse) {
  return __fsub_rn(__fmul_rn(x, inv_temp), lse);
}

__device__ __forceinline__ __nv_bfloat16 full_out_scalar(__nv_bfloat16 x, float inv_temp,
                                                         float lse) {
  return __hsub(__float2bfloat16_rn(__bfloat162float(x) * inv_temp), __float2bfloat16_rn(lse));
}

// ------------------------------------------------------------------ row results
// lse of x/T from the raw maximum m and s = sum 2^((x - m) * c).
template <int MODE>
__device__ __forceinline__ float finish_lse(float m, float s, const K1Params& p) {
  // SELECTIVE/DUAL follow node.py:401 (true division); FULL follows the Metal kernel
  // (multiplication by the reciprocal, model.py:27).
  const float ms = (MODE == K1_FULL) ? __fmul_rn(m, p.inv_temp) : __fdiv_rn(m, p.temp);
  return ms + logf(s);
}

__device__ __forceinline__ void raise_status(int32_t* status, int32_t bit) {
  if (status != nullptr) atomicOr(status, bit);
}

// DUAL: window of sequence i, clamped to the sequence.
__device__ __forceinline__ void dual_window(const K1Params& p, int i, int& start, int& len) {
  start = (p.starts != nullptr) ? p.starts[i] : 0;
  start = max(0, min(start, p.seq_len));
  len = max(0, min(p.lengths[i], p.seq_len - start));
}

// DUAL: dense row of the a-th active position; cum[] = exclusive prefix sums of the lengths.
__device__ __forceinline__ int64_t dual_row_of_item(const K1Params& p, const int32_t* cum,
                                                    int64_t a) {
  int lo = 0, hi = p.n_seq;  // find i with cum[i] <= a < cum[i+1]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cum[mid] <= a) lo = mid; else hi = mid;
  }
  int start = (p.starts != nullptr) ? p.starts[lo] : 0;
  start = max(0, min(start, p.seq_len));
  return static_cast<int64_t>(lo) * p.seq_len + start + (a - cum[lo]);
}

// Block-wide exclusive prefix sum of the window lengths into cum[0..n_seq]; returns the total.
static __device__ int64_t dual_build_prefix(const K1Params& p, int32_t* cum, int32_t* scratch) {
  const int n = p.n_seq;
  const int nt = blockDim.x;
  const int per = (n + nt - 1) / nt;
  const int b = min(n, static_cast<int>(threadIdx.x) * per);
  const int e = min(n, b + per);
  int32_t local = 0;
  for (int i = b; i < e; ++i) {
    int st, ln;
    dual_window(p, i, st, ln);
    local += ln;
  }
  scratch[threadIdx.x] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t run = 0;
    for (int t = 0; t < nt; ++t) {
      const int32_t v = scratch[t];
      scratch[t] = run;
      run += v;
    }
    cum[n] = run;
  }
  __syncthreads();
  int32_t run = scratch[threadIdx.x];
  for (int i = b; i < e; ++i) {
    int st, ln;
    dual_window(p, i, st, ln);
    cum[i] = run;
    run += ln;
  }
  __syncthreads();
  return cum[n];
}

// DUAL: zero the outputs of every position outside its sequence's window.
static __device__ void dual_zero_masked(const K1Params& p) {
  const int64_t total = p.n_rows;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx / p.seq_len);
    const int pos = static_cast<int>(idx - static_cast<int64_t>(i) * p.seq_len);
    int st, ln;
    dual_window(p, i, st, ln);
    if (pos < st || pos >= st + ln) {
      p.out0[idx] = 0.0f;
      p.out1[idx] = 0.0f;
      p.out2[idx] = 0.0f;
    }
  }
}

// Writes the per-row results once the row's (m, s) and raw target logit are known.
// Called by one thread.  `carry` holds the policy logprob between the two DUAL sub-rows.
template <int MODE>
__device__ __forceinline__ void emit_row(const K1Params& p, int64_t row, int sub, float m, float s,
                                         float x_t, bool target_ok, float& carry) {
  const float lse = finish_lse<MODE>(m, s, p);
  if (MODE == K1_FULL) {
    if (p.out0 != nullptr) p.out0[row] = lse;
    return;
  }
  float lp = __fdiv_rn(x_t, p.temp) - lse;
  if (!target_ok) lp = __int_as_float(0x7fc00000);
  if (MODE == K1_SELECTIVE || MODE == K1_RAGGED) {
    p.out0[row] = lp;
    if (p.out1 != nullptr) p.out1[row] = lse;
    if (p.out2 != nullptr) p.out2[row] = target_ok ? x_t : __int_as_float(0x7fc00000);
  } else {
    if (sub == 0) {
      carry = lp;
      p.out0[row] = lp;
    } else {
      const float d = lp - carry;  // r - p
      p.out1[row] = lp;
      p.out2[row] = expf(d) - d - 1.0f;
    }
  }
}

// Exact two-pass (max, sum 2^((x - max) * c)) of one row with plain loads, by one full warp.
// Only used for rows the streaming arithmetic cannot represent (see K1_M_FLOOR).
template <typename T>
__device__ __noinline__ void exact_row(const T* src, int64_t vocab, float c, int lane, float& m,
                                       float& s) {
  float mx = __int_as_float(0xff800000);  // -inf
  for (int64_t j = lane; j < vocab; j += 32) mx = fmaxf(mx, to_float(src[j]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.0f;
  for (int64_t j = lane; j < vocab; j += 32) sum += ex2f((to_float(src[j]) - mx) * c);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  m = mx;
  s = sum;
}

// ------------------------------------------------------------------ launchers in other files
// Small batches (k1_small.cu): if the batch is small enough for a cluster of CTAs to share
// each row, launches that kernel, sets *taken and returns its status; else leaves *taken
// false.  mode is K1_SELECTIVE or K1_FULL.
int32_t k1_small_batch_launch(const K1Params& p, int32_t dtype, int mode, cudaStream_t stream,
                              bool* taken);

// Full matrix with each row shared by a cluster of CTAs (k1_full.cu): same contract.
// bulk_ok: logits and output meet the bulk-copy alignment rules.
int32_t k1_full_cluster_launch(const K1Params& p, int32_t dtype, bool bulk_ok, int sm_count,
                                cudaStream_t stream, bool* taken);

}  // namespace tome
