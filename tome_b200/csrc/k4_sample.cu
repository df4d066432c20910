// K4: top-k temperature sampling fused with the sampled token's full-vocabulary log-prob.
//
// One CTA per row.  A single sweep over the row keeps the online (max, sum-exp) of the full
// vocabulary AND collects the candidates for the top-k: a threshold derived from the first
// few thousand logits rejects almost everything with one compare, the survivors (a few
// hundred for ordinary data) go to a shared-memory list, and an all-pairs ranking picks the
// exact top-k ordered by (value descending, index ascending).  One thread then draws from the
// categorical distribution over the top-k with a counter-based generator and writes the
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

#include <algorithm>

#include "host_common.h"
#include "ptx.cuh"

namespace tome {

constexpr int K4_THREADS = 512;
constexpr int K4_WARPS = K4_THREADS / 32;
constexpr int K4_MAX_K = 64;
constexpr int K4_CAP = 8192;       // candidate list capacity
constexpr int K4_TRIGGER = 4096;   // compact when the list is longer than this at a block boundary
constexpr int K4_BLOCK_ELEMS = 4096;  // elements between two block boundaries (<= CAP - TRIGGER)
constexpr int K4_SAMPLE = 8192;    // leading logits used to derive the first threshold
constexpr int K4_RANK_MAX = 1024;  // above this many candidates, compact before ranking

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
  int32_t* status;
};

struct K4Smem {
  uint32_t cand_key[K4_CAP];
  int32_t cand_idx[K4_CAP];
  uint32_t top_key[K4_MAX_K];
  int32_t top_idx[K4_MAX_K];
  float red_f[2 * K4_WARPS];
  int32_t red_i[K4_WARPS];
  uint32_t sort_buf[K4_THREADS];
  int32_t count;
  int32_t bcast_i;
  uint32_t bcast_u;
};

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

// Exact k-th largest key among cand_key[0..n) by bisection on the bits (n >= k).
__device__ uint32_t k4_kth_key(K4Smem& sm, int32_t n, int32_t k) {
  uint32_t t = 0;
  for (int bit = 31; bit >= 0; --bit) {
    const uint32_t c = t | (1u << bit);
    int32_t cnt = 0;
    for (int32_t i = threadIdx.x; i < n; i += K4_THREADS) cnt += (sm.cand_key[i] >= c) ? 1 : 0;
    if (k4_block_sum(cnt, sm) >= k) t = c;
  }
  return t;
}

// Keeps exactly the k best candidates (value descending, index ascending) in cand[0..k).
// Returns the key of the k-th; ties at that key beyond the kept ones have larger indices.
__device__ uint32_t k4_compact(K4Smem& sm, int32_t n, int32_t k) {
  const uint32_t tkey = k4_kth_key(sm, n, k);
  int32_t c_gt = 0;
  for (int32_t i = threadIdx.x; i < n; i += K4_THREADS) c_gt += (sm.cand_key[i] > tkey) ? 1 : 0;
  const int32_t greater = k4_block_sum(c_gt, sm);
  const int32_t need_ties = k - greater;  // >= 1
  // the need_ties-th smallest index among the entries that tie at tkey, by bisection
  int32_t lo = 0;  // largest value with count(idx < lo) < need_ties ends the search
  for (int bit = 30; bit >= 0; --bit) {
    const int32_t c = lo | (1 << bit);
    int32_t cnt = 0;
    for (int32_t i = threadIdx.x; i < n; i += K4_THREADS)
      cnt += (sm.cand_key[i] == tkey && sm.cand_idx[i] < c) ? 1 : 0;
    if (k4_block_sum(cnt, sm) < need_ties) lo = c;
  }
  // keep (key > tkey) or (key == tkey and idx <= lo); each thread stages its survivors in
  // registers (at most n / THREADS + 1 entries), then the list is rewritten in place
  uint32_t my_key[K4_CAP / K4_THREADS];
  int32_t my_idx[K4_CAP / K4_THREADS];
  int32_t mine = 0;
  for (int32_t i = threadIdx.x; i < n; i += K4_THREADS) {
    const uint32_t key = sm.cand_key[i];
    const int32_t idx = sm.cand_idx[i];
    if (key > tkey || (key == tkey && idx <= lo)) {
      my_key[mine] = key;
      my_idx[mine] = idx;
      ++mine;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) sm.count = 0;
  __syncthreads();
  for (int32_t j = 0; j < mine; ++j) {
    const int32_t slot = atomicAdd(&sm.count, 1);
    sm.cand_key[slot] = my_key[j];
    sm.cand_idx[slot] = my_idx[j];
  }
  __syncthreads();
  return tkey;
}

// Philox-4x32-10: one 128-bit block for (counter, key); returns the first word.
__device__ uint32_t k4_philox(uint64_t ctr_lo, uint64_t ctr_hi, uint64_t key) {
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

template <typename T>
__global__ void __launch_bounds__(K4_THREADS) k4_sample_kernel(const K4Params p) {
  extern __shared__ __align__(16) uint8_t k4_smem_raw[];
  K4Smem& sm = *reinterpret_cast<K4Smem*>(k4_smem_raw);
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int32_t k = p.top_k;
  const bool greedy = !(p.temperature > 0.0f);
  const float temp = greedy ? 1.0f : p.temperature;  // temperature of the reported log-prob
  const float c = LOG2E / temp;

  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const T* src = reinterpret_cast<const T*>(p.logits) + row * p.stride;
    const int64_t V = p.vocab;
    const int32_t kk = static_cast<int32_t>(min(static_cast<int64_t>(k), V));

    // ---- first threshold: the kk-th largest of the per-thread maxima over the leading
    //      K4_SAMPLE logits; at least kk logits are >= it, so it bounds the answer from below
    const int64_t n_sample = min(static_cast<int64_t>(K4_SAMPLE), V);
    uint32_t local = 0u;
    for (int64_t i = tid; i < n_sample; i += K4_THREADS) local = max(local, k4_key(k4_load(src, i)));
    sm.sort_buf[tid] = local;
    if (tid == 0) sm.count = 0;
    __syncthreads();
    // rank of each per-thread maximum among the 512 (ties by thread id): all-pairs
    {
      int32_t rank = 0;
      for (int j = 0; j < K4_THREADS; ++j) {
        const uint32_t o = sm.sort_buf[j];
        rank += (o > local || (o == local && j < tid)) ? 1 : 0;
      }
      // with fewer than kk non-empty threads (tiny vocabularies) the threshold is 0: keep all
      const int32_t want =
          min(kk, static_cast<int32_t>(min(n_sample, static_cast<int64_t>(K4_THREADS)))) - 1;
      if (rank == want) sm.bcast_u = (n_sample >= kk && want == kk - 1) ? local : 0u;
    }
    __syncthreads();
    uint32_t thr = sm.bcast_u;   // candidates satisfy key >= thr (or > thr once strict)
    bool strict = false;
    __syncthreads();

    // ---- one sweep: online softmax of the whole row + candidate collection
    float m = -FLT_MAX, s = 0.0f;
    for (int64_t base = 0; base < V; base += K4_BLOCK_ELEMS) {
      const int64_t end = min(V, base + K4_BLOCK_ELEMS);
      for (int64_t i = base + tid; i < end; i += K4_THREADS) {
        const float x = k4_load(src, i);
        if (x > m) {
          s *= ex2f((m - x) * c);
          m = x;
        }
        s += ex2f((x - m) * c);
        const uint32_t key = k4_key(x);
        if (strict ? (key > thr) : (key >= thr)) {
          const int32_t slot = atomicAdd(&sm.count, 1);
          if (slot < K4_CAP) {
            sm.cand_key[slot] = key;
            sm.cand_idx[slot] = static_cast<int32_t>(i);
          }
        }
      }
      __syncthreads();
      const int32_t n = sm.count;   // <= TRIGGER + BLOCK_ELEMS <= CAP by construction
      __syncthreads();
      if (n > K4_TRIGGER) {
        thr = k4_compact(sm, n, kk);
        strict = true;  // later ties at thr have larger indices than the kept ones: they lose
      }
    }

    // ---- merge the online softmax across the block
    {
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
    const float lse = __fdiv_rn(row_m, temp) + logf(row_s);

    // ---- exact top-kk of the candidates, ordered (value desc, index asc)
    int32_t n = sm.count;
    __syncthreads();
    if (n > K4_RANK_MAX) {
      k4_compact(sm, n, kk);
      n = sm.count;
      __syncthreads();
    }
    for (int32_t i = tid; i < n; i += K4_THREADS) {
      const uint32_t key = sm.cand_key[i];
      const int32_t idx = sm.cand_idx[i];
      int32_t rank = 0;
      for (int32_t j = 0; j < n; ++j) {
        const uint32_t ok = sm.cand_key[j];
        rank += (ok > key || (ok == key && sm.cand_idx[j] < idx)) ? 1 : 0;
      }
      if (rank < kk) {
        sm.top_key[rank] = key;
        sm.top_idx[rank] = idx;
      }
    }
    __syncthreads();

    // ---- draw, score, write
    if (tid == 0) {
      int32_t pick = 0;
      if (!greedy && kk > 1) {
        // categorical over the top-kk of logits / temperature
        const float top = k4_unkey(sm.top_key[0]);
        float total = 0.0f;
        for (int32_t j = 0; j < kk; ++j) total += ex2f((k4_unkey(sm.top_key[j]) - top) * c);
        const uint32_t r = k4_philox(static_cast<uint64_t>(row), p.offset, p.seed);
        const float u = (static_cast<float>(r >> 8) + 0.5f) * (1.0f / 16777216.0f) * total;
        float acc = 0.0f;
        pick = kk - 1;
        for (int32_t j = 0; j < kk; ++j) {
          acc += ex2f((k4_unkey(sm.top_key[j]) - top) * c);
          if (u < acc) {
            pick = j;
            break;
          }
        }
      }
      const int32_t token = sm.top_idx[pick];
      p.out_tokens[row] = token;
      p.out_logprob[row] = __fdiv_rn(k4_unkey(sm.top_key[pick]), temp) - lse;
    }
    if (p.out_topk_idx != nullptr || p.out_topk_val != nullptr) {
      for (int32_t j = tid; j < k; j += K4_THREADS) {
        const bool have = j < kk;
        if (p.out_topk_idx != nullptr) p.out_topk_idx[row * k + j] = have ? sm.top_idx[j] : -1;
        if (p.out_topk_val != nullptr)
          p.out_topk_val[row * k + j] = have ? k4_unkey(sm.top_key[j]) : -INFINITY;
      }
    }
    __syncthreads();
  }
}

}  // namespace tome

using namespace tome;

extern "C" int32_t tome_sample_topk_logprob(const void* logits, int32_t dtype, int64_t rows,
                                            int64_t vocab, int64_t row_stride, float temperature,
                                            int32_t top_k, uint64_t seed, uint64_t offset,
                                            int32_t* out_tokens, float* out_logprob,
                                            int32_t* out_topk_idx, float* out_topk_val,
                                            int32_t* dev_status, void* stream) {
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
  K4Params p = {};
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
  const int smem = static_cast<int>(sizeof(K4Smem));
  const int grid = static_cast<int>(
      std::max<int64_t>(1, std::min<int64_t>(static_cast<int64_t>(info.sm_count) * 2, rows)));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == TOME_F32) {
    st = check_cuda(cudaFuncSetAttribute(k4_sample_kernel<float>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                    "cudaFuncSetAttribute(k4)");
    if (st != TOME_OK) return st;
    k4_sample_kernel<float><<<grid, K4_THREADS, smem, s>>>(p);
  } else {
    st = check_cuda(cudaFuncSetAttribute(k4_sample_kernel<__nv_bfloat16>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                    "cudaFuncSetAttribute(k4)");
    if (st != TOME_OK) return st;
    k4_sample_kernel<__nv_bfloat16><<<grid, K4_THREADS, smem, s>>>(p);
  }
  return check_cuda(cudaGetLastError(), "k4 launch");
}
