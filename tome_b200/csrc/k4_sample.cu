// K4: top-k temperature sampling fused with the sampled token's full-vocabulary log-prob.
//
// Base form (k4_sample_kernel): one CTA per row.  A single sweep over the row (128-bit loads, no barrier inside) keeps the
// online (max, sum-exp) of the full vocabulary AND collects the candidates for the top-k: a
// threshold derived from the first few thousand logits rejects almost everything with one
// compare, the survivors (a few hundred for ordinary data) go to a shared-memory list, and an
// all-pairs ranking picks the exact top-k ordered by (value descending, index ascending).  If
// the list overflows (sorted or heavily tied rows) the k-th best of what was stored becomes a
// tighter (value, index) threshold and the row is swept again.  One thread then draws from
// the categorical distribution over the top-k with a counter-based generator and writes the
// token and its log-prob under the FULL softmax.  No host round trip per sequence.
//
// Replaces the per-sequence host loop of the rollout (mlx-impl/node.py:593-610):
//   token = _sample_token(logits[b, 0], temperature)       node.py:894-907 (top-k = 20)
//   lp    = float(fused_log_softmax(...)[b, token])        node.py:590, 605
// Semantics kept: temperature 0 means argmax (first maximum) scored at temperature 1; the
// reported log-prob is of the full-vocabulary softmax although sampling is truncated.
// The random stream is this library's own (Philox-4x32-10 keyed by seed, row and offset);
// MLX's generator cannot be reproduced, so parity with the reference is distributional.
#include <cuda_bf16.h>
#include <float.h>

#include <stdlib.h>

#include <algorithm>

#include "host_common.h"
#include "k1_sample.h"
#include "online.cuh"
#include "ptx.cuh"
#include "row_geom.cuh"
#include "sampling.cuh"

namespace tome {

constexpr int K4_THREADS = 512;
constexpr int K4_WARPS = K4_THREADS / 32;
constexpr int K4_CAP = 8192;       // candidate list capacity
constexpr int K4_SAMPLE = 32768;   // leading logits used to derive the first threshold
constexpr int K4_GROUPS = K4_THREADS / 4;  // sample maxima kept for the threshold
constexpr int K4_RANK_MAX = 1024;  // above this many candidates, compact before ranking
constexpr int K4_MAX_SWEEPS = 64;   // re-sweeps with a tightened threshold before giving up
// From these row counts on a batch takes the streaming path.  bf16: one row more than a full
// wave of the row kernel's CTAs (two per SM); below that the row kernel is as fast or faster
// (V = 151936, row kernel / streaming path, CUDA-graph replay: 200 rows 27.7 / 30.8 us, 296 rows
// 28.7 / 34.7; 320 rows 45.5 / 39.1) and is one launch instead of four stream operations.
// fp32: one row more than the clusters of two CTAs per row can hold on 148 SMs.  Rows of that
// length (608 KB) do not stay in L2 between the GEMM that writes them and this call, and from
// DRAM the streaming path with the rows in two parts is ahead (160 / 200 / 256 rows, L2 flushed:
// 43.1 / 45.9 / 49.8 us row kernel, 38.3 / 41.8 / 47.4 streaming); replayed from a graph over
// logits that fit L2 it is the other way round by as much (29.1 / 34.7 / 37.5 against 34.3 /
// 36.2 / 39.5).  From 297 rows on the streaming path wins either way (400 rows 63 against 51 us).
constexpr int64_t K4_STREAM_MIN_ROWS_BF16 = 297;
constexpr int64_t K4_STREAM_MIN_ROWS_F32 = 149;
constexpr int64_t K4_FINISH_IN_KERNEL_MIN_ROWS = 4096;  // fp32: rows finished inside the streaming kernel
constexpr int64_t K4_STREAM_MIN_VOCAB = 4096;  // every consumer of the streaming kernel sees logits
constexpr int K4_MAX_PARTS = 4;                // parts a row of a small streamed batch is cut into
constexpr int K4_MAX_LISTS = 16;              // lists per row (one per consumer warp and part, streaming kernel)
constexpr int K4_CODE_CAP = 256;               // logits of a row that may reach its final threshold
constexpr int K4_LIST_THREADS = 128;
constexpr int K4_SPLIT_MAX = 8;               // CTAs of a cluster that may share one row
constexpr int64_t K4_SPLIT_MIN_VOCAB = 16384; // shorter rows stay with one CTA

struct K4Params {
  const void* logits;
  int64_t rows, vocab, stride;
  float temperature;  // 0 = greedy
  int32_t top_k;
  uint64_t seed, offset;
  int32_t* out_tokens;
  float* out_logprob;
  int32_t* out_topk_idx;  // nullable, [rows, top_k]
  float* out_topk_val;    // nullable, [rows, top_k]
  int32_t only_flagged;   // redo only the rows listed in marked_rows (left over by the streaming path)
  int32_t* marked;        // with only_flagged: how many rows are listed (0: nothing to do)
  int32_t* marked_rows;   // with only_flagged: their indices
  int32_t* status;
};

struct K4Smem {
  unsigned long long cand[K4_CAP];   // candidates, packed (see k4_pack)
  unsigned long long top[K4_MAX_K];  // the top-k, best first
  uint32_t sample_key[K4_GROUPS];
  float red_f[2 * K4_WARPS];
  int32_t red_i[K4_WARPS];
  int32_t count;
  unsigned long long bcast;
  // split rows: the first CTA of the cluster receives every other rank's top-k and (m, s)
  unsigned long long inbox[K4_SPLIT_MAX * K4_MAX_K];
  float2 inbox_ms[K4_SPLIT_MAX];
  int32_t inbox_n[K4_SPLIT_MAX];
};

__device__ __forceinline__ float k4_load(const float* p, int64_t i) { return p[i]; }
__device__ __forceinline__ float k4_load(const __nv_bfloat16* p, int64_t i) {
  return __bfloat162float(p[i]);
}

// Block-wide sum of an int; every thread gets the result.  Two barriers.
__device__ int32_t k4_block_sum(int32_t v, K4Smem& sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sm.red_i[threadIdx.x >> 5] = v;
  __syncthreads();
  int32_t t = 0;
#pragma unroll
  for (int w = 0; w < K4_WARPS; ++w) t += sm.red_i[w];
  __syncthreads();
  return t;
}

// Exact k-th largest code among cand[0..n) by bisection on the bits (n >= k, codes distinct).
__device__ unsigned long long k4_kth(K4Smem& sm, int32_t n, int32_t k) {
  unsigned long long t = 0;
  for (int bit = 63; bit >= 0; --bit) {
    const unsigned long long c = t | (1ull << bit);
    int32_t cnt = 0;
    for (int32_t i = threadIdx.x; i < n; i += K4_THREADS) cnt += (sm.cand[i] >= c) ? 1 : 0;
    if (k4_block_sum(cnt, sm) >= k) t = c;
  }
  return t;
}

// Keeps exactly the k best of cand[0..n) (in arbitrary order) and returns the k-th best code.
__device__ unsigned long long k4_compact(K4Smem& sm, int32_t n, int32_t k) {
  const unsigned long long kth = k4_kth(sm, n, k);
  unsigned long long mine[K4_CAP / K4_THREADS];
  int32_t n_mine = 0;
  for (int32_t i = threadIdx.x; i < n; i += K4_THREADS) {
    const unsigned long long v = sm.cand[i];
    if (v >= kth) mine[n_mine++] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) sm.count = 0;
  __syncthreads();
  for (int32_t j = 0; j < n_mine; ++j) sm.cand[atomicAdd(&sm.count, 1)] = mine[j];
  __syncthreads();
  return kth;
}

// Exact top-kk of cand[0..n), best first, into top[] (n <= K4_RANK_MAX, codes distinct): each
// thread ranks its (at most two) candidates in one pipelined pass over the list.  Warps none of
// whose threads holds a candidate skip the pass (a few hundred candidates are the rule, so
// half the warps do), and the second candidate is only looked at by the warps that have one.
__device__ __forceinline__ void k4_rank_top(K4Smem& sm, int32_t n, int32_t kk) {
  const int tid = threadIdx.x;
  const int warp_first = tid & ~31;  // index of the candidate of this warp's first lane
  if (warp_first >= n) return;
  const unsigned long long mine0 = (tid < n) ? sm.cand[tid] : ~0ull;  // ~0 outranks everything: never placed
  int32_t rank0 = 0;
  if (warp_first + K4_THREADS < n) {
    const unsigned long long mine1 = (tid + K4_THREADS < n) ? sm.cand[tid + K4_THREADS] : ~0ull;
    int32_t rank1 = 0;
#pragma unroll 4
    for (int32_t j = 0; j < n; ++j) {
      const unsigned long long o = sm.cand[j];
      rank0 += (o > mine0) ? 1 : 0;
      rank1 += (o > mine1) ? 1 : 0;
    }
    if (tid + K4_THREADS < n && rank1 < kk) sm.top[rank1] = mine1;
  } else {
#pragma unroll 4
    for (int32_t j = 0; j < n; ++j) rank0 += (sm.cand[j] > mine0) ? 1 : 0;
  }
  if (tid < n && rank0 < kk) sm.top[rank0] = mine0;
}

// One pass over a row.  Candidate collection: a 16-byte vector is looked at element by element
// only if its largest logit reaches the threshold's value (one compare per vector); elements
// whose code is >= thr go to the candidate ring (if more than the capacity arrive, later ones
// overwrite earlier ones and the count tells).  With SOFTMAX the per-thread online softmax of
// ALL logits is updated too: the packed fast path (`fs`) for whole vectors, the exact scalar
// form (`tail`) for the elements outside them.  The vectors start `head` elements into the
// row, at its first 16-byte boundary.  No barrier inside.
template <typename T, bool VEC, bool SOFTMAX>
__device__ __forceinline__ void k4_sweep(const T* src, int64_t V, int64_t base, int64_t head,
                                         float c, unsigned long long thr, K4Smem& sm, Fast& fs,
                                         Online& tail) {
  // thr == 0 means "no threshold": every logit is a candidate
  const float thr_val = (thr == 0ull) ? __int_as_float(0xff800000) : k4_value(thr);
  auto candidate = [&](float x, int64_t i) {
    const unsigned long long code = k4_pack(x, base + i);  // index within the whole row
    if (code >= thr) {
      const uint32_t slot = static_cast<uint32_t>(atomicAdd(&sm.count, 1));
      sm.cand[slot % K4_CAP] = code;  // one aligned 8-byte store: never a torn entry
    }
  };
  auto scalar = [&](int64_t i) {
    const float x = k4_load(src, i);
    if (SOFTMAX) online_update_scalar(tail, x, c);
    if (x >= thr_val) candidate(x, i);
  };
  if (VEC) {
    constexpr int PER = 16 / static_cast<int>(sizeof(T));
    const int64_t nvec = (V - head) / PER;
    const uint4* vp = reinterpret_cast<const uint4*>(src + head);
    auto reduce = [&](const uint4& q) {  // folds a vector into the sums, returns its largest logit
      return SOFTMAX ? fast_update<0>(fs, q, c, T()) : vec_max(q, T());
    };
    // (the vector is fetched again for the look, from L1: holding four of them across the
    // updates would not fit the 64 registers two CTAs per SM leave a thread)
    auto look = [&](float vmax, int64_t v) {
      if (!(vmax < thr_val)) {  // a NaN maximum (bf16 vector holding a NaN): look inside
        const uint4 q = __ldg(vp + v);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        const int64_t i0 = head + v * PER;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (sizeof(T) == 4) {
            candidate(__uint_as_float(w[j]), i0 + j);
          } else {
            candidate(__uint_as_float(w[j] << 16), i0 + 2 * j);
            candidate(__uint_as_float(w[j] & 0xffff0000u), i0 + 2 * j + 1);
          }
        }
      }
    };
    // Four vectors per step: the loads are asked for together, the four updates of the sums run
    // as one straight piece of code, and one test tells whether any of the vectors needs a
    // look.  (Left to `#pragma unroll` the loop kept program order, load - update - candidates
    // - load, because the candidate branch stores to shared memory: four memory round trips per
    // step instead of one, and no update overlapping another.)
    int64_t v = threadIdx.x;
    for (; v + 3 * K4_THREADS < nvec; v += 4 * K4_THREADS) {
      const uint4 q0 = __ldg(vp + v);
      const uint4 q1 = __ldg(vp + v + K4_THREADS);
      const uint4 q2 = __ldg(vp + v + 2 * K4_THREADS);
      const uint4 q3 = __ldg(vp + v + 3 * K4_THREADS);
      const float m0 = reduce(q0);
      const float m1 = reduce(q1);
      const float m2 = reduce(q2);
      const float m3 = reduce(q3);
      if (!(fmax3_nan(fmax_nan(m0, m1), m2, m3) < thr_val)) {
        look(m0, v);
        look(m1, v + K4_THREADS);
        look(m2, v + 2 * K4_THREADS);
        look(m3, v + 3 * K4_THREADS);
      }
    }
    for (; v < nvec; v += K4_THREADS) {
      look(reduce(__ldg(vp + v)), v);
    }
    for (int64_t i = threadIdx.x; i < head; i += K4_THREADS) scalar(i);
    for (int64_t i = head + nvec * PER + threadIdx.x; i < V; i += K4_THREADS) scalar(i);
  } else {
#pragma unroll 4
    for (int64_t i = threadIdx.x; i < V; i += K4_THREADS) scalar(i);
  }
}

// Block-wide exact (max, sum 2^((x - max) * c)) of a row with plain loads, for rows the fast
// path cannot represent (see K1_M_FLOOR in online.cuh).  Every thread gets the result.
template <typename T>
__device__ void k4_exact_row(const T* src, int64_t V, float c, K4Smem& sm, float& row_m,
                             float& row_s) {
  float mx = __int_as_float(0xff800000);
  for (int64_t i = threadIdx.x; i < V; i += K4_THREADS) mx = fmaxf(mx, k4_load(src, i));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) sm.red_f[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = sm.red_f[0];
#pragma unroll
  for (int w = 1; w < K4_WARPS; ++w) mx = fmaxf(mx, sm.red_f[w]);
  __syncthreads();
  float sum = 0.0f;
  for (int64_t i = threadIdx.x; i < V; i += K4_THREADS) sum += ex2f((k4_load(src, i) - mx) * c);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if ((threadIdx.x & 31) == 0) sm.red_f[threadIdx.x >> 5] = sum;
  __syncthreads();
  sum = 0.0f;
#pragma unroll
  for (int w = 0; w < K4_WARPS; ++w) sum += sm.red_f[w];
  __syncthreads();
  row_m = mx;
  row_s = sum;
}

// Works through `V` logits starting at `src` (a whole row, or one CTA's part of a split row;
// `base` = index of src[0] within the row).  Afterwards sm.top[0 .. kk) holds the exact top-kk
// of the part, best first, and every thread has the part's (max, sum-exp).  kk = min(k, V),
// or the number of logits that are not NaN if that is smaller (NaN is never a candidate).
template <typename T>
__device__ void k4_segment(const T* src, const int64_t V, const int64_t base, const int32_t k,
                           const float c, K4Smem& sm, int32_t* status, int32_t& kk_out,
                           float& m_out, float& s_out) {
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int32_t kk = static_cast<int32_t>(min(static_cast<int64_t>(k), V));

  // ---- first threshold: the leading K4_SAMPLE logits are cut into 128 groups (4 adjacent
  //      threads each); the kk-th largest group maximum is a value that at least kk logits
  //      reach, so it bounds the answer from below.  Values only: ties are kept.
  // 128-bit loads from the part's first 16-byte boundary on (`head` elements in; the part
  // begins on an element boundary, so there is one unless the part is shorter than that)
  const int64_t head = static_cast<int64_t>(((16u - (reinterpret_cast<uintptr_t>(src) & 15u)) & 15u) /
                                            sizeof(T));
  const bool vec = head < V;
  const int64_t n_sample = min(static_cast<int64_t>(K4_SAMPLE), V - (vec ? head : 0));
  float lmax = __int_as_float(0xff800000);
  int64_t filled_threads;  // threads that saw at least one logit
  if (vec) {
    constexpr int PER = 16 / static_cast<int>(sizeof(T));
    const int64_t nvec_s = n_sample / PER;
    const uint4* vp = reinterpret_cast<const uint4*>(src + head);
#pragma unroll 4
    for (int64_t v = tid; v < nvec_s; v += K4_THREADS) lmax = fmaxf(lmax, vec_max(__ldg(vp + v), T()));
    filled_threads = min(nvec_s, static_cast<int64_t>(K4_THREADS));
  } else {
#pragma unroll 4
    for (int64_t i = tid; i < n_sample; i += K4_THREADS) lmax = fmaxf(lmax, k4_load(src, i));
    filled_threads = min(n_sample, static_cast<int64_t>(K4_THREADS));
  }
  lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, 1));
  lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, 2));
  if ((tid & 3) == 0) sm.sample_key[tid >> 2] = k4_key(lmax);
  if (tid == 0) {
    sm.count = 0;
    sm.bcast = 0ull;  // no usable threshold: every logit is a candidate
  }
  __syncthreads();
  const int64_t full_groups = filled_threads / 4;  // groups whose four threads all hold data
  if (tid < K4_GROUPS && full_groups >= kk && kk > 0) {
    const uint32_t mine = sm.sample_key[tid];
    int32_t rank = 0;
    for (int j = 0; j < K4_GROUPS; ++j) {
      const uint32_t o = sm.sample_key[j];
      rank += (o > mine || (o == mine && j < tid)) ? 1 : 0;
    }
    if (rank == kk - 1) sm.bcast = static_cast<unsigned long long>(mine) << 32;
  }
  __syncthreads();
  unsigned long long thr = sm.bcast;
  __syncthreads();

  // ---- sweep: online softmax of the whole part + candidate collection; swept again with a
  //      tighter threshold only if more candidates arrived than the ring holds
  Fast fs;
  fast_init(fs, c);
  Online tail;
  online_init(tail);
  int32_t n = 0;
  for (int sweep = 0; sweep < K4_MAX_SWEEPS; ++sweep) {
    if (sweep == 0) {
      if (vec) k4_sweep<T, true, true>(src, V, base, head, c, thr, sm, fs, tail);
      else k4_sweep<T, false, true>(src, V, base, 0, c, thr, sm, fs, tail);
    } else {
      if (vec) k4_sweep<T, true, false>(src, V, base, head, c, thr, sm, fs, tail);
      else k4_sweep<T, false, false>(src, V, base, 0, c, thr, sm, fs, tail);
    }
    __syncthreads();
    const int32_t total = sm.count;
    __syncthreads();
    if (total <= K4_CAP) {
      n = total;
      break;
    }
    // overflow: the ring holds CAP of the candidates (mostly the latest); their kk-th best
    // is a valid, tighter bound
    thr = k4_compact(sm, K4_CAP, kk);
    n = kk;
    if (sweep + 1 == K4_MAX_SWEEPS) {
      if (tid == 0 && status != nullptr) atomicOr(status, TOME_DEV_TIMEOUT);
      break;  // keeps the kk best of what the ring held
    }
    if (tid == 0) sm.count = 0;
    __syncthreads();
  }

  // ---- merge the online softmax across the block
  {
    const Online vecs = fast_finish(fs, c);
    const float m = fmaxf(vecs.m, tail.m);
    const float s = vecs.s * ex2f((vecs.m - m) * c) + tail.s * ex2f((tail.m - m) * c);
    float wm = m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, o));
    float ws = s * ex2f((m - wm) * c);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ws += __shfl_xor_sync(0xffffffffu, ws, o);
    if (lane == 0) {
      sm.red_f[2 * warp] = wm;
      sm.red_f[2 * warp + 1] = ws;
    }
  }
  __syncthreads();
  float row_m = -FLT_MAX, row_s = 0.0f;
#pragma unroll
  for (int w = 0; w < K4_WARPS; ++w) row_m = fmaxf(row_m, sm.red_f[2 * w]);
#pragma unroll
  for (int w = 0; w < K4_WARPS; ++w) row_s += sm.red_f[2 * w + 1] * ex2f((sm.red_f[2 * w] - row_m) * c);
  __syncthreads();
  // the true maximum contributes 2^0, so a healthy part has row_s >= ~1 (see online.cuh)
  if (V > 0 && !(row_s >= 0.5f && row_s <= FLT_MAX)) k4_exact_row(src, V, c, sm, row_m, row_s);
  m_out = row_m;
  s_out = row_s;

  // ---- exact top-kk of the candidates, best first
  if (n > K4_RANK_MAX) {
    k4_compact(sm, n, kk);
    n = kk;
  }
  const int32_t have = min(kk, n);  // n < kk: the part holds fewer than kk logits that are not NaN
  k4_rank_top(sm, n, have);
  kk_out = have;
  __syncthreads();
}

// The first warp draws the token and scores it; all write the optional top-k outputs.
__device__ void k4_finish_row(const K4Params& p, K4Smem& sm, int64_t row, int32_t kk, float c,
                              float temp, bool greedy, float lse) {
  const int tid = threadIdx.x;
  const int32_t k = p.top_k;
  if (tid < 32) {  // the first warp draws (its lanes form the terms of the sum side by side)
    if (kk > 0) {
      const int32_t pick = greedy ? 0 : k4_draw_warp(sm.top, kk, c, row, p.seed, p.offset);
      if (tid == 0) {
        p.out_tokens[row] = k4_index(sm.top[pick]);
        p.out_logprob[row] = __fdiv_rn(k4_value(sm.top[pick]), temp) - lse;
      }
    } else if (tid == 0) {  // a row of NaNs: nothing to draw from
      p.out_tokens[row] = -1;
      p.out_logprob[row] = __int_as_float(0x7fc00000);
      if (p.status != nullptr) atomicOr(p.status, TOME_DEV_NO_CANDIDATE);
    }
  }
  if (p.out_topk_idx != nullptr || p.out_topk_val != nullptr) {
    for (int32_t j = tid; j < k; j += K4_THREADS) {
      const bool have = j < kk;
      if (p.out_topk_idx != nullptr) p.out_topk_idx[row * k + j] = have ? k4_index(sm.top[j]) : -1;
      if (p.out_topk_val != nullptr)
        p.out_topk_val[row * k + j] = have ? k4_value(sm.top[j]) : -INFINITY;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(K4_THREADS, 2) k4_sample_kernel(const K4Params p) {
  extern __shared__ __align__(16) uint8_t k4_smem_raw[];
  K4Smem& sm = *reinterpret_cast<K4Smem*>(k4_smem_raw);
  const bool greedy = !(p.temperature > 0.0f);
  const float temp = greedy ? 1.0f : p.temperature;  // temperature of the reported log-prob
  const float c = LOG2E / temp;

  // after a streamed batch: the list of rows left over is complete once the kernels before
  // this one have finished (launched on its own the wait returns at once)
  griddep_wait();
  const int64_t n_items = p.only_flagged ? static_cast<int64_t>(*p.marked) : p.rows;
  for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int64_t row = p.only_flagged ? static_cast<int64_t>(p.marked_rows[item]) : item;
    const T* src = reinterpret_cast<const T*>(p.logits) + row * p.stride;
    int32_t kk;
    float row_m, row_s;
    k4_segment(src, p.vocab, 0, p.top_k, c, sm, p.status, kk, row_m, row_s);
    const float lse = __fdiv_rn(row_m, temp) + logf(row_s);
    k4_finish_row(p, sm, row, kk, c, temp, greedy, lse);
    __syncthreads();
  }
}

// Small batches: a cluster of `split` CTAs shares each row.  Every CTA finds the top-k and the
// (max, sum-exp) of its part; the parts meet in the first CTA's shared memory, which ranks the
// at most split * k survivors, merges the sums and draws.  Same tokens as the kernel above
// (the draw depends on the row's top-k only).  grid = rows * split, one row per cluster.
template <typename T>
__global__ void __launch_bounds__(K4_THREADS, 2) k4_sample_split_kernel(const K4Params p,
                                                                     const int split) {
  extern __shared__ __align__(16) uint8_t k4_smem_raw[];
  K4Smem& sm = *reinterpret_cast<K4Smem*>(k4_smem_raw);
  const int tid = threadIdx.x;
  const bool greedy = !(p.temperature > 0.0f);
  const float temp = greedy ? 1.0f : p.temperature;
  const float c = LOG2E / temp;
  const uint32_t rank = cluster_ctarank();
  const int64_t row = static_cast<int64_t>(blockIdx.x) / split;
  const T* src = reinterpret_cast<const T*>(p.logits) + row * p.stride;
  // parts begin on multiples of 8 logits, so they are as aligned as the row itself
  const int64_t units = p.vocab / 8;
  const int64_t begin = (units * rank / split) * 8;
  const int64_t end = (rank + 1 == static_cast<uint32_t>(split)) ? p.vocab
                                                                 : (units * (rank + 1) / split) * 8;
  int32_t kk;
  float part_m, part_s;
  k4_segment(src + begin, end - begin, begin, p.top_k, c, sm, p.status, kk, part_m, part_s);
  if (rank != 0) {
    const uint32_t inbox = mapa_shared(smem_u32(&sm.inbox[rank * K4_MAX_K]), 0);
    if (tid < kk) st_cluster_u64(inbox + tid * 8, sm.top[tid]);
    if (tid == 0) {
      st_cluster_f32x2(mapa_shared(smem_u32(&sm.inbox_ms[rank]), 0), part_m, part_s);
      st_cluster_u32(mapa_shared(smem_u32(&sm.inbox_n[rank]), 0), static_cast<uint32_t>(kk));
    }
  }
  cluster_sync_all();  // release/acquire: the first CTA sees what the others stored
  if (rank != 0) return;
  // gather the survivors of every part into the candidate list (at most split * k codes), part
  // after part: thread r * K4_MAX_K + j moves survivor j of part r (K4_SPLIT_MAX * K4_MAX_K =
  // K4_THREADS).  (Taking the places with an atomic counter cost the first CTA 2 - 3 us per row:
  // up to 160 shared-memory atomics in a row.)
  static_assert(K4_SPLIT_MAX * K4_MAX_K <= K4_THREADS, "one thread per survivor of any part");
  {
    const int r = tid / K4_MAX_K, j = tid % K4_MAX_K;
    int32_t before = 0, total = kk;
    for (int q = 1; q < split; ++q) {
      const int32_t n_q = sm.inbox_n[q];
      if (q <= r) before = total;
      total += n_q;
    }
    if (r == 0) {
      if (j < kk) sm.cand[j] = sm.top[j];
    } else if (r < split && j < sm.inbox_n[r]) {
      sm.cand[before + j] = sm.inbox[r * K4_MAX_K + j];
    }
    if (tid == 0) sm.count = total;
  }
  // a part without a finite logit (maximum -inf, sum NaN) adds nothing to the row's sum
  const float ninf = __int_as_float(0xff800000);
  float row_m = part_m;
  for (int r = 1; r < split; ++r) row_m = fmaxf(row_m, sm.inbox_ms[r].x);
  float row_s = (part_m == ninf) ? 0.0f : part_s * ex2f((part_m - row_m) * c);
  for (int r = 1; r < split; ++r) {
    const float2 ms = sm.inbox_ms[r];
    if (ms.x != ninf) row_s += ms.y * ex2f((ms.x - row_m) * c);
  }
  __syncthreads();
  const int32_t n = sm.count;
  // fewer survivors than top_k: the row holds fewer logits that are not NaN
  const int32_t kk_row =
      min(n, static_cast<int32_t>(min(static_cast<int64_t>(p.top_k), p.vocab)));
  __syncthreads();
  k4_rank_top(sm, n, kk_row);
  __syncthreads();
  const float lse = __fdiv_rn(row_m, temp) + logf(row_s);
  k4_finish_row(p, sm, row, kk_row, c, temp, greedy, lse);
}

// ------------------------------------------------------------------ large batches
// The streaming kernel's SAMPLE mode (k1_logprob.cu) makes one pass at HBM speed: its consumer
// warps keep (max, sum-exp), derive the row's threshold (a value that at least kk logits reach)
// from the logits as they pass and note which 16-byte vectors hold a logit that reaches it.
// The noted vectors of a row are then fetched again, their logits ranked (exact top-kk), a token
// drawn, scored and written.  A row whose lists ran
// over (sorted or heavily tied rows) or that holds fewer than kk logits that are not NaN is put
// on a list and redone by k4_sample_kernel (only_flagged).  Same tokens as the other kernels of
// this file.
//
// The last step, from the noted places to token and log-prob, exists twice: k4_finish_kernel
// after the streaming kernel, or the streaming kernel's own producer warp between two copies.
// For bf16 logits the streaming kernel is bound by its instruction count and the work costs
// more there than in a kernel of its own (4096 rows: 256 us against 238 us).  For fp32 logits
// the producer warp's version adds nothing to the streaming kernel's time (8192 x 151936: 775 ->
// 727 us when the finish kernel still read every noted entry); since the lists are compacted
// and the streaming kernel clears the counter of left-over rows itself (no memset node), the
// finish kernel is as cheap up to a few thousand rows or cheaper (297 / 800 / 2048 rows: 42.6 /
// 91.3 / 195.5 us against 46.3 / 96.5 / 200.7, CUDA-graph replay; 4096 rows 379 / 378), so the
// producer warp finishes fp32 batches from 4096 rows on only.  TOME_K4_FINISH=kernel|warp
// forces one or the other (tests).
//
// Batches with fewer rows than the streaming kernel has CTAs (4 per SM) would leave it one slow
// CTA per row, so their rows are cut into 2 or 4 parts, each a work item of that kernel with a
// threshold, a (max, sum-exp) pair and lists of its own; k4_finish_kernel puts a row's parts
// together (largest threshold, merged pair, all lists).  TOME_K4_PARTS=1|2|4 forces a count.
struct K4Lists {
  int32_t lists;          // per part (one per consumer warp of the streaming kernel)
  int32_t parts;          // per row
  int32_t cap;            // entries per list
  int32_t vec_stride;     // 16-byte vectors between the four vectors of an entry
  const float* row_thr;   // [rows, parts]
  const float* lse;       // [rows] (parts == 1)
  const float2* part_ms;  // [rows, parts] (parts > 1)
  const int32_t* count;   // [rows, parts, lists]
  const uint2* entry;     // [rows, parts, lists, cap]
};

// One warp per row (four rows per CTA at a time), nothing but warp-level synchronisation:
// the row's entries are expanded into a list of vector numbers, the vectors are fetched and
// their logits that reach the threshold become codes, the codes are ranked, the warp draws.
constexpr int K4_VEC_CAP = 512;  // vectors a row's entries may name (beyond that: row kernel)

template <typename T, int MAXL>
__global__ void __launch_bounds__(K4_LIST_THREADS)
k4_finish_kernel(const K4Params p, const K4Lists w) {
  constexpr int ROWS_PER_CTA = K4_LIST_THREADS / 32;
  __shared__ unsigned long long codes[ROWS_PER_CTA][K4_CODE_CAP];
  __shared__ unsigned long long tops[ROWS_PER_CTA][K4_MAX_K];
  __shared__ int32_t vecs[ROWS_PER_CTA][K4_VEC_CAP];
  __shared__ int32_t n_codes[ROWS_PER_CTA];
  constexpr int PER = 16 / static_cast<int>(sizeof(T));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t lanes_below = (1u << lane) - 1u;
  const bool greedy = !(p.temperature > 0.0f);
  const float temp = greedy ? 1.0f : p.temperature;
  const float c = LOG2E / temp;
  const int32_t k = p.top_k;
  const int32_t kk = static_cast<int32_t>(min(static_cast<int64_t>(k), p.vocab));
  unsigned long long* list = codes[warp];
  unsigned long long* top = tops[warp];
  int32_t* vec = vecs[warp];
  griddep_wait();               // the streaming kernel's lists are complete and visible
  griddep_launch_dependents();  // the row kernel after this one may be set up meanwhile
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * ROWS_PER_CTA + warp; row < p.rows;
       row += static_cast<int64_t>(gridDim.x) * ROWS_PER_CTA) {
    if (lane == 0) n_codes[warp] = 0;
    // ---- what the streaming kernel left for the row, asked for in one go: lane l reads the
    //      counter of list l, and the threshold and the (max, sum-exp) pair of part l
    const int32_t n_lists = w.lists * w.parts;
    int32_t my_count = (lane < n_lists) ? w.count[row * n_lists + lane] : 0;
    float thr = (lane < w.parts) ? w.row_thr[row * w.parts + lane] : __int_as_float(0xff800000);
    float lse;
    bool sick = false;  // a sum that is no number: the row kernel takes the row
    if (w.parts == 1) {
      lse = w.lse[row];
    } else {
      // rows in parts: the largest of the parts' thresholds (each a value that top_k logits of
      // the row reach) and the merged pair
      const float2 ms = (lane < w.parts) ? w.part_ms[row * w.parts + lane] : make_float2(-FLT_MAX, 0.0f);
      float m = ms.x;
#pragma unroll
      for (int o = 1; o < K4_MAX_PARTS; o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      float s = (lane < w.parts) ? ms.y * ex2f((ms.x - m) * c) : 0.0f;
#pragma unroll
      for (int o = 1; o < K4_MAX_PARTS; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      sick = !(s >= 0.5f && s <= FLT_MAX);  // a healthy row's maximum contributes 2^0
      lse = __fdiv_rn(m, temp) + logf(s);
    }
#pragma unroll
    for (int o = 1; o < K4_MAX_PARTS; o <<= 1) thr = fmaxf(thr, __shfl_xor_sync(0xffffffffu, thr, o));
    thr = __shfl_sync(0xffffffffu, thr, 0);
    lse = __shfl_sync(0xffffffffu, lse, 0);
    sick = __shfl_sync(0xffffffffu, sick ? 1 : 0, 0) != 0;
    const T* src = reinterpret_cast<const T*>(p.logits) + row * p.stride;
    const K1RowGeom geom = k1_row_geom(src, p.vocab);  // vector numbers count from the row's first 16-byte boundary
    // ---- the lists of the row, end to end: lane l knows where list l begins
    const bool overflow = __any_sync(0xffffffffu, my_count > w.cap);
    my_count = min(my_count, w.cap);
    int32_t begin = my_count;  // inclusive prefix sum over the lanes, then made exclusive
#pragma unroll
    for (int o = 1; o < MAXL; o <<= 1) {
      const int32_t up = __shfl_up_sync(0xffffffffu, begin, o);
      if (lane >= o) begin += up;
    }
    const int32_t total = __shfl_sync(0xffffffffu, begin, MAXL - 1);
    begin -= my_count;
    // ---- entries -> vector numbers.  Every logit that reaches the final threshold sits in a
    //      vector some entry names; an entry whose largest logit stays below it is dropped
    //      unread (a NaN there keeps it).  Two steps: the surviving entries are gathered (one
    //      ballot per 32 entries), then expanded (four ballots per 32 survivors).
    int32_t n_kept = 0;
    for (int32_t g0 = 0; g0 < total; g0 += 128) {  // four entries per lane and trip, asked for together
      uint2 e[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int32_t g = g0 + t * 32 + lane;
        int32_t l = 0, at = g;
#pragma unroll
        for (int q = 1; q < MAXL; ++q) {  // the last list that begins at or before g
          const int32_t b = __shfl_sync(0xffffffffu, begin, q);
          if (q < n_lists && g >= b) {
            l = q;
            at = g - b;
          }
        }
        e[t] = (g < total) ? w.entry[(row * n_lists + l) * w.cap + at] : make_uint2(0u, 0u);
      }
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const bool keep = (g0 + t * 32 + lane < total) && !(__uint_as_float(e[t].y) < thr);
        const uint32_t bal = __ballot_sync(0xffffffffu, keep);
        const int32_t to = n_kept + __popc(bal & lanes_below);
        if (keep && to < K4_VEC_CAP) vec[to] = static_cast<int32_t>(e[t].x);
        n_kept += __popc(bal);
      }
    }
    __syncwarp();
    // every surviving entry is taken into a register first; then the buffer is overwritten with
    // the vector numbers
    int32_t n_vec = 0;
    const int32_t kept = min(n_kept, K4_VEC_CAP / 4);
    uint32_t mine_e[(K4_VEC_CAP / 4 + 31) / 32];
#pragma unroll
    for (int t = 0; t < (K4_VEC_CAP / 4 + 31) / 32; ++t)
      mine_e[t] = (t * 32 + lane < kept) ? static_cast<uint32_t>(vec[t * 32 + lane]) : 0u;
    __syncwarp();
#pragma unroll
    for (int t = 0; t < (K4_VEC_CAP / 4 + 31) / 32; ++t) {
      if (t * 32 >= kept) break;
      const uint32_t e = mine_e[t];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bool bit = (e >> j) & 1u;
        const uint32_t bal = __ballot_sync(0xffffffffu, bit);
        const int32_t to = n_vec + __popc(bal & lanes_below);
        if (bit && to < K4_VEC_CAP) vec[to] = static_cast<int32_t>(e >> 4) + j * w.vec_stride;
        n_vec += __popc(bal);
      }
    }
    __syncwarp();
    // ---- vectors -> codes of the logits that reach the threshold
    for (int32_t i = lane; i < min(n_vec, K4_VEC_CAP); i += 32) {
      const int64_t e0 = geom.head + static_cast<int64_t>(vec[i]) * PER;
      if (static_cast<int64_t>(vec[i]) * 16 < geom.bulk_bytes) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(src + e0));
        const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int t = 0; t < PER; ++t) {
          const float x = (sizeof(T) == 4)
                              ? __uint_as_float(u[t])
                              : __uint_as_float((t & 1) ? (u[t >> 1] & 0xffff0000u) : (u[t >> 1] << 16));
          if (x >= thr) {
            const int32_t at = atomicAdd(&n_codes[warp], 1);
            if (at < K4_CODE_CAP) list[at] = k4_pack(x, e0 + t);
          }
        }
      } else {  // the short vector: the elements outside the row's 16-byte boundaries
        const int64_t n_ends = geom.head + (p.vocab - geom.tail_begin);
        for (int64_t j = 0; j < n_ends; ++j) {
          const int64_t t = (j < geom.head) ? j : geom.tail_begin + (j - geom.head);
          const float x = k4_load(src, t);
          if (x >= thr) {
            const int32_t at = atomicAdd(&n_codes[warp], 1);
            if (at < K4_CODE_CAP) list[at] = k4_pack(x, t);
          }
        }
      }
    }
    __syncwarp();
    const int32_t n = n_codes[warp];
    if (overflow || sick || n_kept > K4_VEC_CAP / 4 || n_vec > K4_VEC_CAP || n > K4_CODE_CAP ||
        n < kk) {
      // lists that ran over (sorted or heavily tied rows) or a row with too few logits that
      // are not NaN: left to the row kernel
      if (lane == 0) p.marked_rows[atomicAdd(p.marked, 1)] = static_cast<int32_t>(row);
      __syncwarp();
      continue;
    }
    // ---- exact top-kk by ranking every code against all (codes are distinct), two per lane
    //      and trip
    for (int32_t i0 = 0; i0 < n; i0 += 64) {
      const int32_t ia = i0 + lane, ib = i0 + 32 + lane;
      const unsigned long long a = (ia < n) ? list[ia] : ~0ull;
      const unsigned long long b = (ib < n) ? list[ib] : ~0ull;
      int32_t rank_a = 0, rank_b = 0;
#pragma unroll 4
      for (int32_t j = 0; j < n; ++j) {
        const unsigned long long o = list[j];
        rank_a += (o > a) ? 1 : 0;
        rank_b += (o > b) ? 1 : 0;
      }
      if (ia < n && rank_a < kk) top[rank_a] = a;
      if (ib < n && rank_b < kk) top[rank_b] = b;
    }
    __syncwarp();
    const int32_t pick = greedy ? 0 : k4_draw_warp(top, kk, c, row, p.seed, p.offset);
    if (lane == 0) {
      p.out_tokens[row] = k4_index(top[pick]);
      p.out_logprob[row] = __fdiv_rn(k4_value(top[pick]), temp) - lse;
    }
    if (p.out_topk_idx != nullptr || p.out_topk_val != nullptr) {
      for (int32_t j = lane; j < k; j += 32) {
        const bool have = j < kk;
        if (p.out_topk_idx != nullptr) p.out_topk_idx[row * k + j] = have ? k4_index(top[j]) : -1;
        if (p.out_topk_val != nullptr)
          p.out_topk_val[row * k + j] = have ? k4_value(top[j]) : -INFINITY;
      }
    }
    __syncwarp();
  }
}

// Scratch layout: per part of a row its (max, sum-exp) pair and its threshold, per row the
// logsumexp and a slot of the list of rows to redo, then the list counters; one counter for the
// batch; then the lists.
struct K4Workspace {
  float2* part_ms;   // [rows, parts]
  float* thr;        // [rows, parts]
  float* lse;        // [rows]
  int32_t* marked_rows;
  int32_t* count;    // [rows, parts, lists]
  int32_t* marked;   // one counter for the batch
  uint2* entry;      // [rows, parts, lists, cap]
};
static size_t k4_workspace_head(int64_t rows, int lists, int parts) {
  return (static_cast<size_t>(rows) * (8 + parts * (12 + 4 * lists)) + 4 + 15) &
         ~static_cast<size_t>(15);
}
static size_t k4_workspace_bytes(int64_t rows, int lists, int cap, int parts) {
  return k4_workspace_head(rows, lists, parts) +
         static_cast<size_t>(rows) * parts * lists * cap * sizeof(uint2);
}
static K4Workspace k4_workspace(void* base, int64_t rows, int lists, int parts) {
  K4Workspace w;
  uint8_t* b = static_cast<uint8_t*>(base);
  w.part_ms = reinterpret_cast<float2*>(b);
  w.thr = reinterpret_cast<float*>(w.part_ms + rows * parts);
  w.lse = w.thr + rows * parts;
  w.marked_rows = reinterpret_cast<int32_t*>(w.lse + rows);
  w.count = w.marked_rows + rows;
  w.marked = w.count + rows * parts * lists;
  w.entry = reinterpret_cast<uint2*>(b + k4_workspace_head(rows, lists, parts));
  return w;
}

// Parts a row of a streamed batch is cut into: two while every half row is a work item of a CTA
// of its own on a GPU of 148 SMs, four CTAs each (one CTA streams a row at 15 - 20 B/ns
// whatever runs beside it, so more and smaller items finish sooner: 256 bf16 rows leave the
// streaming kernel after 25 us whole, after 21 us in halves); not for a wide top-k, whose
// parts together would bring more logits to the finish than it holds.  Quarters (the kernels
// take them, TOME_K4_PARTS=4) shorten the streaming kernel further (128 bf16 rows: 20 -> 12 us)
// but the finish reads twice the lists and the call gains nothing.
constexpr int64_t K4_PART_SLOTS = 148 * 4;
static int k4_stream_parts(int64_t rows, int64_t vocab, int32_t dtype, int32_t top_k) {
  const int most = k1_sample_max_parts(vocab, dtype);
  if (const char* e = getenv("TOME_K4_PARTS")) {
    const int v = atoi(e);
    return (v == 1 || v == 2 || v == 4) ? std::min(v, most) : 1;
  }
  if (most >= 2 && rows * 2 <= K4_PART_SLOTS && top_k <= 48) return 2;
  return 1;
}
// The most parts any call with this many rows may use (scratch is sized for it).
static int k4_stream_parts_most(int64_t rows, int64_t vocab) {
  return std::max(k4_stream_parts(rows, vocab, TOME_F32, 1),
                  k4_stream_parts(rows, vocab, TOME_BF16, 1));
}

// Whether a batch takes the streaming path (given scratch): large batches of rows that the
// streaming kernel can read.  TOME_K4_STREAM = 1 / 0 forces it on (where possible) / off.
static bool k4_wants_stream(int64_t rows, int64_t vocab, int32_t dtype) {
  if (vocab < K4_STREAM_MIN_VOCAB) return false;
  if (const char* e = getenv("TOME_K4_STREAM")) return atoi(e) != 0;
  return rows >= (dtype == TOME_F32 ? K4_STREAM_MIN_ROWS_F32 : K4_STREAM_MIN_ROWS_BF16);
}

// Cluster size for a batch too small to fill the GPU with one CTA per row: the largest of 8,
// 4 and 2 whose clusters are all resident at once (0: do not split).
// TOME_K4_SPLIT=0 switches the split off, 2/4/8 forces a size (read at every call; tests).
static int k4_split_factor(const void* kernel, int smem, int64_t rows, int64_t vocab) {
  if (vocab < K4_SPLIT_MIN_VOCAB) return 0;
  const char* e = getenv("TOME_K4_SPLIT");
  if (e != nullptr) {
    const int v = atoi(e);
    return ((v == 2 || v == 4 || v == 8) && rows * v <= 0x7fffffffLL) ? v : 0;
  }
  // pairs too: measured at 80 - 148 rows of 151936 logits, 24 - 28 us against 29 - 30 us with one
  // CTA per row on fp32, 22 - 24 against 23 - 25 on bf16
  for (int split = K4_SPLIT_MAX; split >= 2; split >>= 1)
    if (rows <= max_active_clusters(kernel, K4_THREADS, smem, split)) return split;
  return 0;
}

// Launches a kernel of the streamed path behind the one before it in the stream with the
// programmatic-serialization attribute: its CTAs are set up while that kernel drains and wait
// in griddep_wait, which takes the launch latency (2 - 3 us each) out of a small batch's time.
// TOME_K4_PDL=0 launches them the ordinary way (read at every call; measurements).
template <typename... Args>
static int32_t k4_launch_after(const void* kernel, int grid, int block, int smem, cudaStream_t s,
                               Args... args) {
  void* argv[] = {static_cast<void*>(&args)...};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(static_cast<unsigned>(block), 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  const char* e = getenv("TOME_K4_PDL");
  const bool pdl = (e == nullptr) || atoi(e) != 0;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return check_cuda(cudaLaunchKernelExC(&cfg, kernel, argv), "k4 dependent launch");
}

}  // namespace tome

using namespace tome;

static int32_t k4_sample_impl(const void* logits, int32_t dtype, int64_t rows, int64_t vocab,
                              int64_t row_stride, float temperature, int32_t top_k,
                              uint64_t seed, uint64_t offset, int32_t* out_tokens,
                              float* out_logprob, int32_t* out_topk_idx, float* out_topk_val,
                              void* workspace, size_t ws_bytes, int32_t* dev_status,
                              void* stream) {
  if (dtype != TOME_F32 && dtype != TOME_BF16)
    return fail(TOME_ERR_BAD_DTYPE, "dtype %d is neither TOME_F32 nor TOME_BF16", dtype);
  if (rows < 0 || vocab <= 0 || vocab > 0x7fffffffLL)
    return fail(TOME_ERR_BAD_SHAPE, "rows=%lld vocab=%lld", (long long)rows, (long long)vocab);
  if (row_stride < vocab)
    return fail(TOME_ERR_BAD_STRIDE, "row_stride=%lld < vocab=%lld", (long long)row_stride,
                (long long)vocab);
  if (!(temperature >= 0.0f) || temperature > 3.0e38f)
    return fail(TOME_ERR_BAD_TEMPERATURE, "temperature=%g must be >= 0 and finite", temperature);
  if (top_k < 1 || top_k > K4_MAX_K)
    return fail(TOME_ERR_BAD_SHAPE, "top_k=%d must be in [1, %d]", top_k, K4_MAX_K);
  if (rows == 0) return TOME_OK;
  if (logits == nullptr || out_tokens == nullptr || out_logprob == nullptr)
    return fail(TOME_ERR_NULL_POINTER, "a required pointer is NULL");
  const size_t es = (dtype == TOME_F32) ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(logits) % es) != 0)
    return fail(TOME_ERR_MISALIGNED, "logits is not aligned to its element size");
  DeviceInfo info;
  int32_t st = current_device_info(&info);
  if (st != TOME_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool streamed = workspace != nullptr && k4_wants_stream(rows, vocab, dtype) &&
                        k1_sample_eligible(logits, dtype, vocab, row_stride);
  const int lists = k1_sample_lists_per_row();
  const int list_cap = k1_sample_list_capacity();
  const int parts = streamed ? k4_stream_parts(rows, vocab, dtype, top_k) : 1;
  if (streamed) {
    if (lists * parts > K4_MAX_LISTS)
      return fail(TOME_ERR_UNSUPPORTED, "%d lists per row", lists * parts);
    if (ws_bytes < k4_workspace_bytes(rows, lists, list_cap, parts))
      return fail(TOME_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes, %zu needed", ws_bytes,
                  k4_workspace_bytes(rows, lists, list_cap, parts));
    if (!aligned16(workspace)) return fail(TOME_ERR_MISALIGNED, "workspace is not 16-byte aligned");
  }
  K4Params p = {};
  p.only_flagged = streamed ? 1 : 0;
  p.logits = logits;
  p.rows = rows;
  p.vocab = vocab;
  p.stride = row_stride;
  p.temperature = temperature;
  p.top_k = top_k;
  p.seed = seed;
  p.offset = offset;
  p.out_tokens = out_tokens;
  p.out_logprob = out_logprob;
  p.out_topk_idx = out_topk_idx;
  p.out_topk_val = out_topk_val;
  p.status = dev_status;
  if (streamed) {
    const K4Workspace w = k4_workspace(workspace, rows, lists, parts);
    p.marked = w.marked;
    p.marked_rows = w.marked_rows;
    bool in_kernel = (dtype == TOME_F32) && rows >= K4_FINISH_IN_KERNEL_MIN_ROWS;
    if (const char* e = getenv("TOME_K4_FINISH")) in_kernel = (e[0] == 'w');  // "warp" / "kernel"
    if (parts > 1) in_kernel = false;  // a row's parts meet in k4_finish_kernel
    // the count of rows left to the row kernel starts at zero: with the finisher inside the
    // streaming kernel (whose CTAs add to it at any time) by a memset before the launch,
    // otherwise the streaming kernel clears it itself (one stream operation fewer per call)
    if (in_kernel) {
      st = check_cuda(cudaMemsetAsync(w.marked, 0, sizeof(int32_t), s), "cudaMemsetAsync(marked rows)");
      if (st != TOME_OK) return st;
    }
    K1SampleArgs a;
    a.finish_in_kernel = in_kernel;
    a.parts = parts;
    a.part_ms = w.part_ms;
    a.temperature = temperature;
    a.top_k = top_k;
    a.seed = seed;
    a.offset = offset;
    a.out_tokens = out_tokens;
    a.out_logprob = out_logprob;
    a.out_topk_idx = out_topk_idx;
    a.out_topk_val = out_topk_val;
    a.row_thr = w.thr;
    a.lse = w.lse;
    a.cand_count = w.count;
    a.cand_entry = w.entry;
    a.marked = w.marked;
    a.marked_rows = w.marked_rows;
    st = k1_launch_sample(logits, dtype, rows, vocab, row_stride, a, dev_status, s);
    if (st != TOME_OK) return st;
    if (!in_kernel) {
      K4Lists lw;
      lw.lists = lists;
      lw.parts = parts;
      lw.part_ms = w.part_ms;
      lw.cap = list_cap;
      lw.vec_stride = k1_sample_vector_stride();
      lw.row_thr = w.thr;
      lw.lse = w.lse;
      lw.count = w.count;
      lw.entry = w.entry;
      const int grid_rows = static_cast<int>(std::min<int64_t>(
          (rows + K4_LIST_THREADS / 32 - 1) / (K4_LIST_THREADS / 32),
          static_cast<int64_t>(info.sm_count) * 16));
      void (*finish)(K4Params, K4Lists);
      if (lists * parts <= 8)
        finish = (dtype == TOME_F32) ? k4_finish_kernel<float, 8> : k4_finish_kernel<__nv_bfloat16, 8>;
      else
        finish = (dtype == TOME_F32) ? k4_finish_kernel<float, K4_MAX_LISTS>
                                     : k4_finish_kernel<__nv_bfloat16, K4_MAX_LISTS>;
      st = k4_launch_after(reinterpret_cast<const void*>(finish), grid_rows, K4_LIST_THREADS, 0, s,
                           p, lw);
      if (st != TOME_OK) return st;
    }
  }
  const int smem = static_cast<int>(sizeof(K4Smem));
  void (*split_kernel)(K4Params, int) = (dtype == TOME_F32)
                                            ? k4_sample_split_kernel<float>
                                            : k4_sample_split_kernel<__nv_bfloat16>;
  st = ensure_dynamic_smem(reinterpret_cast<const void*>(split_kernel), smem);
  if (st != TOME_OK) return st;
  const int split =
      streamed ? 0
               : k4_split_factor(reinterpret_cast<const void*>(split_kernel), smem, rows, vocab);
  if (split > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(rows * split), 1, 1);
    cfg.blockDim = dim3(K4_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = static_cast<unsigned>(split);
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, split_kernel, p, split), "k4 split launch");
  }
  // (redoing the rows a streamed batch left over: one CTA per SM; it usually finds none)
  const int grid = static_cast<int>(std::max<int64_t>(
      1, std::min<int64_t>(static_cast<int64_t>(info.sm_count) * (streamed ? 1 : 3), rows)));
  void (*row_kernel)(K4Params) =
      (dtype == TOME_F32) ? k4_sample_kernel<float> : k4_sample_kernel<__nv_bfloat16>;
  st = ensure_dynamic_smem(reinterpret_cast<const void*>(row_kernel), smem);
  if (st != TOME_OK) return st;
  if (streamed)
    return k4_launch_after(reinterpret_cast<const void*>(row_kernel), grid, K4_THREADS, smem, s, p);
  row_kernel<<<grid, K4_THREADS, smem, s>>>(p);
  return check_cuda(cudaGetLastError(), "k4 launch");
}

extern "C" int32_t tome_sample_topk_logprob(const void* logits, int32_t dtype, int64_t rows,
                                            int64_t vocab, int64_t row_stride, float temperature,
                                            int32_t top_k, uint64_t seed, uint64_t offset,
                                            int32_t* out_tokens, float* out_logprob,
                                            int32_t* out_topk_idx, float* out_topk_val,
                                            int32_t* dev_status, void* stream) {
  return k4_sample_impl(logits, dtype, rows, vocab, row_stride, temperature, top_k, seed, offset,
                        out_tokens, out_logprob, out_topk_idx, out_topk_val, nullptr, 0,
                        dev_status, stream);
}

extern "C" size_t tome_sample_workspace_bytes(int64_t rows, int64_t vocab) {
  // the size does not know the dtype: whatever either dtype would use
  if (rows <= 0 || vocab <= 0 ||
      !(k4_wants_stream(rows, vocab, TOME_F32) || k4_wants_stream(rows, vocab, TOME_BF16)))
    return 0;
  return k4_workspace_bytes(rows, k1_sample_lists_per_row(), k1_sample_list_capacity(),
                            k4_stream_parts_most(rows, vocab));
}

extern "C" int32_t tome_sample_topk_logprob_ws(const void* logits, int32_t dtype, int64_t rows,
                                               int64_t vocab, int64_t row_stride,
                                               float temperature, int32_t top_k, uint64_t seed,
                                               uint64_t offset, int32_t* out_tokens,
                                               float* out_logprob, int32_t* out_topk_idx,
                                               float* out_topk_val, void* workspace,
                                               size_t ws_bytes, int32_t* dev_status,
                                               void* stream) {
  return k4_sample_impl(logits, dtype, rows, vocab, row_stride, temperature, top_k, seed, offset,
                        out_tokens, out_logprob, out_topk_idx, out_topk_val, workspace, ws_bytes,
                        dev_status, stream);
}
