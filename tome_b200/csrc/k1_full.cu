// K1, full-matrix mode for rows of more than ~100 KB: a cluster of CTAs shares each row.
#include "k1_common.cuh"
#include "row_geom.cuh"

namespace tome {

// ------------------------------------------------------------------ full matrix, large batches
// The two-pass FULL mode of the pipeline kernel re-reads each row from L2, which holds only as
// long as the rows in flight (two per SM) fit there; fp32 rows of an LM vocabulary do not
// (measured DRAM traffic: 3 units per 2 algorithmic), bf16 rows barely.  Here a cluster of C
// CTAs shares a row, which divides the rows in flight by C:
//   pass 1: the consumers fold the chunks of their CTA's part into (m, s) as they land;
//   exchange: each CTA sends its pair to the others (st.shared::cluster + mbarrier arrive with
//             release.cluster), waits for theirs (acquire.cluster), every CTA computes the lse;
//   pass 2: the part is fetched again (from L2, marked as the last use) and the consumers turn
//           the chunks into outputs (streaming stores).
// Two CTAs per SM so that one computes while the other waits for its exchange.  Measured DRAM
// traffic of this form: 1.01 x the matrix read, 1.0 x written.
// Tried and dropped, 4096 x 151936 bf16 / 2048 x 151936 fp32, GB/s read + write, against 5430 /
// 5780 for this kernel at the time:
//   * keeping a CTA's part resident in shared memory between the passes (the row crosses the
//     memory system once), one CTA per SM with pass 1 of the next row run before pass 2 of the
//     current one: 4200 / 4500; the same with separate pass-1 and pass-2 warps: 4300 - 4700 /
//     4800 - 4900.  A slot stays occupied from its load to its write-out (~10 us) and 227 KB
//     per SM hold too few of them;
//   * one CTA per SM with separate rings, producers and warps for the two passes, pass 2
//     trailing pass 1 by a row so that nothing waits for the exchange: 4850 - 5100 / 5060 - 5300.
//   * this kernel with pass 1 of the cluster's next row run before pass 2 of the current one
//     (the exchange's answer is then a pass old when it is needed): 4540 / 4780 against 5770 /
//     5740; two rows per cluster between the passes no longer stay in L2.  It only wins with
//     clusters larger than the default (half as many rows in flight), and then stays behind
//     the default.
// What helped was cutting the instruction count of pass 2 (see full_out_vec); with it the
// kernel issues on 45 % of the cycles and keeps DRAM 67 % busy, the rest is the exchange.
#ifndef KF_CFG_WARPS
#define KF_CFG_WARPS 8
#endif
#ifndef KF_CFG_SLOTS
#define KF_CFG_SLOTS 4
#endif
#ifndef KF_CFG_CHUNK
#define KF_CFG_CHUNK 25600
#endif
#ifndef KF_CFG_CTAS_PER_SM
#define KF_CFG_CTAS_PER_SM 2
#endif
constexpr int KF_CONSUMER_WARPS = KF_CFG_WARPS;
constexpr int KF_CONSUMERS = KF_CONSUMER_WARPS * 32;
constexpr int KF_THREADS = KF_CONSUMERS + 32;
constexpr int KF_SLOTS = KF_CFG_SLOTS;
constexpr int KF_CHUNK_BYTES = KF_CFG_CHUNK;
constexpr int KF_MAX_CLUSTER = 8;
constexpr int KF_CTAS_PER_SM = KF_CFG_CTAS_PER_SM;

struct KFSmem {
  static constexpr int DATA = KF_SLOTS * KF_CHUNK_BYTES;
  static constexpr int FULL_BAR = DATA;                       // SLOTS mbarriers
  static constexpr int EMPTY_BAR = FULL_BAR + KF_SLOTS * 8;   // SLOTS mbarriers
  static constexpr int XCHG_BAR = EMPTY_BAR + KF_SLOTS * 8;   // 2 mbarriers (row parity)
  static constexpr int PART = XCHG_BAR + 16;                  // [2][WARPS] float2
  static constexpr int PAIRS = PART + 2 * KF_CONSUMER_WARPS * 8;   // [2][MAX_CLUSTER] float2
  static constexpr int LSE = PAIRS + 2 * KF_MAX_CLUSTER * 8;       // [2] float
  static constexpr int TOTAL = LSE + 8;
};

template <typename T>
__global__ void __launch_bounds__(KF_THREADS, KF_CTAS_PER_SM)
k1_full_cluster_kernel(const K1Params p, const int cluster, const int chunks_per_cta) {
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int ES = sizeof(T);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t full_bar = smem_base + KFSmem::FULL_BAR;
  const uint32_t empty_bar = smem_base + KFSmem::EMPTY_BAR;
  const uint32_t xchg_bar = smem_base + KFSmem::XCHG_BAR;
  float2* part = reinterpret_cast<float2*>(smem + KFSmem::PART);
  float2* pairs = reinterpret_cast<float2*>(smem + KFSmem::PAIRS);
  volatile float* lse_box = reinterpret_cast<volatile float*>(smem + KFSmem::LSE);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int64_t n_clusters = gridDim.x / cluster;
  const int64_t first_row = blockIdx.x / cluster;

  if (threadIdx.x == 0) {
    for (int i = 0; i < KF_SLOTS; ++i) {
      mbar_init(full_bar + i * 8, 1);
      mbar_init(empty_bar + i * 8, KF_CONSUMER_WARPS);
    }
    mbar_init(xchg_bar, cluster > 1 ? cluster - 1 : 1);
    mbar_init(xchg_bar + 8, cluster > 1 ? cluster - 1 : 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (cluster > 1) cluster_sync_all();  // nobody arrives on a barrier that is not there yet

  // this CTA's part of a row: chunks [rank * chunks_per_cta, (rank + 1) * chunks_per_cta) of
  // chunk_bytes each, counted from the row's first 16-byte boundary (the last chunks of a row
  // may be short or empty; a row that starts off the grid holds one vector fewer than the
  // aligned row the chunks are planned for)
  const int64_t bulk_most = (p.vocab * ES) & ~static_cast<int64_t>(15);
  const int64_t chunk_bytes = p.chunk_bytes;
  const int64_t part_begin = static_cast<int64_t>(rank) * chunks_per_cta * chunk_bytes;
  int my_chunks = 0;
  for (int k = 0; k < chunks_per_cta; ++k)
    if (part_begin + k * chunk_bytes < bulk_most) ++my_chunks;
  // the elements outside a row's 16-byte boundaries go with the last part
  const bool owns_ends = (rank == static_cast<uint32_t>(cluster) - 1);
  auto chunk_size = [&](int64_t bulk_bytes, int k) {
    return static_cast<uint32_t>(
        max(int64_t{0}, min(chunk_bytes, bulk_bytes - part_begin - k * chunk_bytes)));
  };

  if (warp == KF_CONSUMER_WARPS) {
    // ---------------- producer
    if (lane == 0) {
      const uint64_t policy = policy_evict_first();  // every byte is read once
      uint32_t it = 0;
      bool ok = true;
      for (int64_t row = first_row; row < p.n_rows && ok; row += n_clusters) {
        const T* row_src = reinterpret_cast<const T*>(p.src[0]) + row * p.stride;
        const K1RowGeom geom = k1_row_geom(row_src, p.vocab);
        const uint8_t* src = reinterpret_cast<const uint8_t*>(row_src + geom.head) + part_begin;
        // every chunk is fetched once per pass, the second time (served by L2) marked as the
        // last use
        for (int pass = 0; pass < 2 && ok; ++pass) {
          for (int k = 0; k < my_chunks; ++k, ++it) {
            const uint32_t slot = it % KF_SLOTS;
            const uint32_t phase = (it / KF_SLOTS) & 1u;
            if (!mbar_wait(empty_bar + slot * 8, phase ^ 1u)) {
              raise_status(p.status, TOME_DEV_TIMEOUT);
              ok = false;
              break;
            }
            const int64_t off = k * chunk_bytes;
            const uint32_t bytes = chunk_size(geom.bulk_bytes, k);
            mbar_arrive_expect_tx(full_bar + slot * 8, bytes);
            if (bytes == 0) continue;
            if (pass == 1)
              bulk_g2s_hint(smem_base + slot * KF_CHUNK_BYTES, src + off, bytes,
                            full_bar + slot * 8, policy);
            else
              bulk_g2s(smem_base + slot * KF_CHUNK_BYTES, src + off, bytes, full_bar + slot * 8);
          }
        }
      }
    }
    __syncwarp();
  } else {
  // ---------------- consumers
  // A consumer whose wait ran out stops touching data but stays in step with its cluster (the
  // peers keep storing into this CTA's shared memory until their last row).
  const int ctid = threadIdx.x;
  uint32_t it = 0;
  uint32_t row_it = 0;
  bool dead = false;
  for (int64_t row = first_row; row < p.n_rows; row += n_clusters, ++row_it) {
    const T* src = reinterpret_cast<const T*>(p.src[0]) + row * p.stride;
    T* dst = reinterpret_cast<T*>(p.out_full) + row * p.out_stride;
    const K1RowGeom geom = k1_row_geom(src, p.vocab);  // the output row sits on the grid alike
    const uint32_t par = row_it & 1u;
    // ---- pass 1: (m, s) of this CTA's part, chunks stay where they are
    Fast fs;
    fast_init(fs, p.c);
    for (int k = 0; k < my_chunks; ++k) {
      const uint32_t slot = (it + k) % KF_SLOTS;
      const uint32_t phase = ((it + k) / KF_SLOTS) & 1u;
      if (!dead && !mbar_wait(full_bar + slot * 8, phase)) {
        raise_status(p.status, TOME_DEV_TIMEOUT);
        dead = true;
      }
      if (dead) break;
      const uint32_t bytes = chunk_size(geom.bulk_bytes, k);
      const uint32_t nvec = bytes >> 4;
      const uint32_t sbase = smem_base + slot * KF_CHUNK_BYTES;
#pragma unroll 4
      for (uint32_t v = ctid; v < nvec; v += KF_CONSUMERS)
        fast_update<0>(fs, lds128(sbase + v * 16), p.c, T());
      __syncwarp();  // the slot is refilled for the second pass
      if (lane == 0) mbar_arrive(empty_bar + slot * 8);
    }
    it += static_cast<uint32_t>(my_chunks);  // the second pass has chunks of its own
    Online st = fast_finish(fs, p.c);
    if (owns_ends && ctid == 0) {
      for (int64_t j = 0; j < geom.head; ++j) online_update_scalar(st, to_float(src[j]), p.c);
      for (int64_t j = geom.tail_begin; j < p.vocab; ++j)
        online_update_scalar(st, to_float(src[j]), p.c);
    }
    online_warp_reduce(st, p.c);
    if (lane == 0) part[par * KF_CONSUMER_WARPS + warp] = make_float2(st.m, st.s);
    named_bar_sync(1, KF_CONSUMERS);
    if (warp == 0) {
      const float2 w = (lane < KF_CONSUMER_WARPS) ? part[par * KF_CONSUMER_WARPS + lane]
                                                  : make_float2(-FLT_MAX, 0.0f);
      Online cta = {w.x, w.y};
      online_warp_reduce(cta, p.c);
      // ---- exchange: lane q sends this CTA's pair to rank q, then all wait for the others
      if (lane < cluster) {
        if (static_cast<uint32_t>(lane) == rank) {
          pairs[par * KF_MAX_CLUSTER + rank] = make_float2(cta.m, cta.s);
        } else {
          st_cluster_f32x2(mapa_shared(smem_u32(&pairs[par * KF_MAX_CLUSTER + rank]), lane),
                           cta.m, cta.s);
          mbar_arrive_cluster(mapa_shared(xchg_bar + par * 8, lane));
        }
      }
      __syncwarp();
      bool ok = true;
      if (cluster > 1) ok = mbar_wait_cluster(xchg_bar + par * 8, (row_it >> 1) & 1u);
      const float2 o = (lane < cluster) ? pairs[par * KF_MAX_CLUSTER + lane]
                                        : make_float2(-FLT_MAX, 0.0f);
      Online all = {o.x, o.y};
      online_warp_reduce(all, p.c);
      float m = all.m, s = all.s;
      if (!(s >= 0.5f && s <= FLT_MAX)) exact_row(src, p.vocab, p.c, lane, m, s);
      float lse = finish_lse<K1_FULL>(m, s, p);
      if (!ok) {  // a peer never delivered: report, poison the row, keep the CTA in step
        raise_status(p.status, TOME_DEV_TIMEOUT);
        lse = __int_as_float(0x7fc00000);
      }
      if (lane == 0) {
        lse_box[par] = lse;
        if (rank == 0 && p.out0 != nullptr) p.out0[row] = lse;
      }
    }
    named_bar_sync(1, KF_CONSUMERS);
    const float lse = lse_box[par];
    // ---- pass 2: outputs; a slot is released once it is written out
    for (int k = 0; k < my_chunks; ++k, ++it) {
      const uint32_t slot = it % KF_SLOTS;
      if (!dead && !mbar_wait(full_bar + slot * 8, (it / KF_SLOTS) & 1u)) {
        raise_status(p.status, TOME_DEV_TIMEOUT);
        dead = true;
      }
      const int64_t off = part_begin + k * chunk_bytes;
      const uint32_t bytes = chunk_size(geom.bulk_bytes, k);
      const uint32_t nvec = dead ? 0u : (bytes >> 4);
      const uint32_t sbase = smem_base + slot * KF_CHUNK_BYTES;
      uint8_t* drow = reinterpret_cast<uint8_t*>(dst + geom.head) + off;
#pragma unroll 4
      for (uint32_t v = ctid; v < nvec; v += KF_CONSUMERS)
        stg128_streaming(drow + static_cast<size_t>(v) * 16,
                         full_out_vec(lds128(sbase + v * 16), p.inv_temp, lse, T()));
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar + slot * 8);
    }
    if (owns_ends && ctid == 0) {
      for (int64_t j = 0; j < geom.head; ++j) dst[j] = full_out_scalar(src[j], p.inv_temp, lse);
      for (int64_t j = geom.tail_begin; j < p.vocab; ++j)
        dst[j] = full_out_scalar(src[j], p.inv_temp, lse);
    }
  }
  }
  // no CTA leaves while a peer may still store into its shared memory or arrive on its barriers
  if (cluster > 1) cluster_sync_all();
}

// Chunking for a cluster of `cluster` CTAs.
static void kf_plan_streamed(int64_t bulk_bytes, int cluster, int* chunks_per_cta,
                             int32_t* chunk_bytes) {
  const int64_t per_cta = (bulk_bytes + cluster - 1) / cluster;
  const int64_t n = std::max<int64_t>(1, (per_cta + KF_CHUNK_BYTES - 1) / KF_CHUNK_BYTES);
  const int64_t total = n * cluster;
  const int64_t al = K1_CHUNK_ALIGN;
  int64_t cb = std::max<int64_t>(al, ((bulk_bytes + total - 1) / total + al - 1) / al * al);
  int64_t chunks = n;
  if (cb > KF_CHUNK_BYTES) {  // rounding pushed a chunk over the slot size: one more chunk
    chunks = n + 1;
    cb = std::max<int64_t>(al, ((bulk_bytes + chunks * cluster - 1) / (chunks * cluster) + al - 1) / al * al);
  }
  *chunks_per_cta = static_cast<int>(chunks);
  *chunk_bytes = static_cast<int32_t>(std::min<int64_t>(cb, KF_CHUNK_BYTES));
}

template <typename T>
static int32_t k1_launch_full_cluster(const K1Params& p_in, int cluster, int chunks_per_cta,
                                      int32_t chunk_bytes, int sm_count, cudaStream_t stream) {
  K1Params p = p_in;
  p.chunk_bytes = chunk_bytes;
  void (*kernel)(K1Params, int, int) = k1_full_cluster_kernel<T>;
  int32_t st = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), KFSmem::TOTAL);
  if (st != TOME_OK) return st;
  // persistent clusters: as many as the device holds at once
  int fit = max_active_clusters(reinterpret_cast<const void*>(kernel), KF_THREADS, KFSmem::TOTAL,
                                cluster);
  if (fit <= 0) fit = std::max(1, sm_count * KF_CTAS_PER_SM / cluster);
  const int64_t n_clusters = std::max<int64_t>(1, std::min<int64_t>(fit, p.n_rows));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(n_clusters * cluster), 1, 1);
  cfg.blockDim = dim3(KF_THREADS, 1, 1);
  cfg.dynamicSmemBytes = KFSmem::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = static_cast<unsigned>(cluster);
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return check_cuda(cudaLaunchKernelEx(&cfg, kernel, p, cluster, chunks_per_cta),
                    "k1 full cluster launch");
}

int32_t k1_full_cluster_launch(const K1Params& p, int32_t dtype, bool bulk_ok, int sm_count,
                               cudaStream_t stream, bool* taken) {
  *taken = false;
  // Rows of up to 80 KB stay with the pipeline kernel (two rows per SM in flight fit L2).
  // Beyond that the cluster kernel, with the smallest cluster whose CTAs get at most 160 KB of
  // a row.  TOME_K1_FULL_CLUSTER forces a form (the tests reach all of them): 0 = pipeline
  // kernel, 1 = the cluster kernel with its default cluster, s1 / s2 / s4 / s8 = clusters of
  // that size.
  const int64_t es = (dtype == TOME_F32) ? 4 : 2;
  const char* e = getenv("TOME_K1_FULL_CLUSTER");
  int cluster = 0, chunks_per_cta = 0;
  int32_t chunk_bytes = 0;
  const int64_t bulk_bytes = (p.vocab * es) & ~15ll;
  if (!bulk_ok || bulk_bytes < 16) return TOME_OK;
  if (e != nullptr && e[0] == 's') {
    cluster = atoi(e + 1);
    if (cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8) return TOME_OK;
  } else {
    if (e != nullptr ? atoi(e) == 0 : bulk_bytes <= 80 * 1024) return TOME_OK;
    const int64_t per_cta = 160 * 1024;
    cluster = 1;
    while (cluster < KF_MAX_CLUSTER && bulk_bytes > per_cta * cluster) cluster <<= 1;
  }
  kf_plan_streamed(bulk_bytes, cluster, &chunks_per_cta, &chunk_bytes);
  *taken = true;
  if (dtype == TOME_F32)
    return k1_launch_full_cluster<float>(p, cluster, chunks_per_cta, chunk_bytes, sm_count, stream);
  return k1_launch_full_cluster<__nv_bfloat16>(p, cluster, chunks_per_cta, chunk_bytes, sm_count,
                                               stream);
}

}  // namespace tome
