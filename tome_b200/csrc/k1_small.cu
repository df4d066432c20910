// K1, small batches: a cluster of CTAs shares each row (selective and full-matrix modes).
#include "k1_common.cuh"

namespace tome {

// ------------------------------------------------------------------ small batches
// With fewer rows than SMs a one-CTA-per-row launch leaves most of the GPU idle and the call
// takes as long as one CTA needs for a whole row.  Here a cluster of `split` CTAs shares a
// row: each streams 1/split of it with 128-bit loads, the per-CTA (m, s) pairs meet in the
// shared memory of the cluster's first CTA, which merges them and writes the row's result.
constexpr int K1_SPLIT_THREADS = 512;
constexpr int K1_SPLIT_MAX = 8;  // portable cluster size

template <typename T, int MODE>
__global__ void __launch_bounds__(K1_SPLIT_THREADS) k1_split_kernel(const K1Params p,
                                                                    const int split) {
  static_assert(MODE == K1_SELECTIVE || MODE == K1_FULL, "modes with one result set per row");
  __shared__ float2 part[K1_SPLIT_THREADS / 32];
  __shared__ __align__(8) float2 slot[K1_SPLIT_MAX];  // one pair per rank of the cluster
  __shared__ float2 result;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int64_t row = static_cast<int64_t>(blockIdx.x) / split;
  const T* src = reinterpret_cast<const T*>(p.src[0]) + row * p.stride;
  constexpr int64_t PER = 16 / static_cast<int64_t>(sizeof(T));
  const uintptr_t addr = reinterpret_cast<uintptr_t>(src);
  const int64_t head = min(p.vocab, static_cast<int64_t>(((16 - (addr & 15)) & 15) / sizeof(T)));
  const int64_t nvec = (p.vocab - head) / PER;
  const int64_t tail_begin = head + nvec * PER;
  const uint4* body = reinterpret_cast<const uint4*>(src + head);
  const int64_t v_begin = nvec * rank / split;
  const int64_t v_end = nvec * (rank + 1) / split;
  Fast fs;
  fast_init(fs, p.c);
  // four loads asked for before the first is used (the update's branch on a new maximum keeps
  // a `#pragma unroll`ed loop from hoisting them by itself)
  int64_t v = v_begin + threadIdx.x;
  for (; v + 3 * K1_SPLIT_THREADS < v_end; v += 4 * K1_SPLIT_THREADS) {
    const uint4 q0 = __ldg(body + v);
    const uint4 q1 = __ldg(body + v + K1_SPLIT_THREADS);
    const uint4 q2 = __ldg(body + v + 2 * K1_SPLIT_THREADS);
    const uint4 q3 = __ldg(body + v + 3 * K1_SPLIT_THREADS);
    fast_update<0>(fs, q0, p.c, T());
    fast_update<0>(fs, q1, p.c, T());
    fast_update<0>(fs, q2, p.c, T());
    fast_update<0>(fs, q3, p.c, T());
  }
  for (; v < v_end; v += K1_SPLIT_THREADS) fast_update<0>(fs, __ldg(body + v), p.c, T());
  Online st = fast_finish(fs, p.c);
  if (rank == 0) {  // the unaligned ends of the row
    for (int64_t j = threadIdx.x; j < head; j += K1_SPLIT_THREADS)
      online_update_scalar(st, to_float(src[j]), p.c);
    for (int64_t j = tail_begin + threadIdx.x; j < p.vocab; j += K1_SPLIT_THREADS)
      online_update_scalar(st, to_float(src[j]), p.c);
  }
  online_warp_reduce(st, p.c);
  if (lane == 0) part[warp] = make_float2(st.m, st.s);
  __syncthreads();
  if (warp == 0) {
    const float2 ms = (lane < K1_SPLIT_THREADS / 32) ? part[lane] : make_float2(-FLT_MAX, 0.0f);
    Online cta = {ms.x, ms.y};
    online_warp_reduce(cta, p.c);
    // SELECTIVE: only the first CTA finishes the row; FULL: every CTA needs the row's lse
    const int receivers = (MODE == K1_FULL) ? split : 1;
    if (lane < receivers) st_cluster_f32x2(mapa_shared(smem_u32(&slot[rank]), lane), cta.m, cta.s);
  }
  cluster_sync_all();  // release/acquire: the pairs are visible where they were sent
  if (MODE == K1_SELECTIVE && rank != 0) return;
  if (warp == 0) {
    const float2 ms = (lane < split) ? slot[lane] : make_float2(-FLT_MAX, 0.0f);
    Online all = {ms.x, ms.y};
    online_warp_reduce(all, p.c);
    float m = all.m, s = all.s;
    if (!(s >= 0.5f && s <= FLT_MAX)) exact_row(src, p.vocab, p.c, lane, m, s);
    if (lane == 0) {
      float x_t = 0.0f;
      bool target_ok = true;
      if (MODE == K1_SELECTIVE) {
        const int32_t t = p.targets[row];
        target_ok = (t >= 0) && (static_cast<int64_t>(t) < p.vocab);
        if (target_ok) x_t = to_float(src[t]);
        else raise_status(p.status, TOME_DEV_TARGET_OUT_OF_RANGE);
      }
      float carry = 0.0f;
      if (MODE == K1_SELECTIVE || rank == 0) emit_row<MODE>(p, row, 0, m, s, x_t, target_ok, carry);
      result = make_float2(m, s);
    }
  }
  if (MODE != K1_FULL) return;
  __syncthreads();
  // second pass over this CTA's part of the row (just read: it comes from L2)
  const float lse = finish_lse<MODE>(result.x, result.y, p);
  T* dst = reinterpret_cast<T*>(p.out_full) + row * p.out_stride;
  const bool dst_vec = ((reinterpret_cast<uintptr_t>(dst + head) & 15) == 0);
  if (dst_vec) {
    uint4* out = reinterpret_cast<uint4*>(dst + head);
#pragma unroll 4
    for (int64_t v = v_begin + threadIdx.x; v < v_end; v += K1_SPLIT_THREADS)
      out[v] = full_out_vec(__ldg(body + v), p.inv_temp, lse, T());
  } else {
    for (int64_t j = head + v_begin * PER + threadIdx.x; j < head + v_end * PER;
         j += K1_SPLIT_THREADS)
      dst[j] = full_out_scalar(src[j], p.inv_temp, lse);
  }
  if (rank == 0) {
    for (int64_t j = threadIdx.x; j < head; j += K1_SPLIT_THREADS)
      dst[j] = full_out_scalar(src[j], p.inv_temp, lse);
    for (int64_t j = tail_begin + threadIdx.x; j < p.vocab; j += K1_SPLIT_THREADS)
      dst[j] = full_out_scalar(src[j], p.inv_temp, lse);
  }
}

// Cluster size for a batch too small to fill the GPU with one CTA per row: the largest of 8
// and 4 whose clusters are all resident at once (measured on V = 151936: 4.7 vs 17 us for one
// fp32 row, 13 vs 19 us for 128 rows; clusters of 2 do not pay).  0: do not split.
// TOME_K1_SPLIT=0 switches the split off, 2/4/8 forces that size (read at every call: tests
// use it to reach the one-CTA-per-row kernels with few rows).
template <typename T, int MODE>
static int k1_split_factor(int64_t rows) {
  const char* e = getenv("TOME_K1_SPLIT");
  if (e != nullptr) {
    const int v = atoi(e);
    const bool valid = (v == 2 || v == 4 || v == 8) && rows * v <= 0x7fffffffLL;
    return valid ? v : 0;
  }
  const void* kernel = reinterpret_cast<const void*>(k1_split_kernel<T, MODE>);
  for (int split = K1_SPLIT_MAX; split >= 4; split >>= 1)
    if (rows <= max_active_clusters(kernel, K1_SPLIT_THREADS, 0, split)) return split;
  return 0;
}

template <typename T, int MODE>
static int32_t k1_launch_split(const K1Params& p, int split, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.n_rows * split), 1, 1);
  cfg.blockDim = dim3(K1_SPLIT_THREADS, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = static_cast<unsigned>(split);
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return check_cuda(cudaLaunchKernelEx(&cfg, k1_split_kernel<T, MODE>, p, split), "k1 split launch");
}

template <int MODE>
static int32_t small_batch_mode(const K1Params& p, int32_t dtype, cudaStream_t stream, bool* taken) {
  *taken = false;
  if (dtype == TOME_F32) {
    const int split = k1_split_factor<float, MODE>(p.n_rows);
    if (split <= 1) return TOME_OK;
    *taken = true;
    return k1_launch_split<float, MODE>(p, split, stream);
  }
  const int split = k1_split_factor<__nv_bfloat16, MODE>(p.n_rows);
  if (split <= 1) return TOME_OK;
  *taken = true;
  return k1_launch_split<__nv_bfloat16, MODE>(p, split, stream);
}

int32_t k1_small_batch_launch(const K1Params& p, int32_t dtype, int mode, cudaStream_t stream,
                              bool* taken) {
  if (mode == K1_FULL) return small_batch_mode<K1_FULL>(p, dtype, stream, taken);
  return small_batch_mode<K1_SELECTIVE>(p, dtype, stream, taken);
}

}  // namespace tome
