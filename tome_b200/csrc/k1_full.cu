// K1, full-matrix mode for rows of more than ~100 KB: a cluster of CTAs shares each row.
#include "k1_common.cuh"

namespace tome {

// ------------------------------------------------------------------ full matrix, large batches
// The two-pass FULL mode of the pipeline kernel re-reads each row from L2, which holds only as
// long as the rows in flight (two per SM) fit there; fp32 rows of an LM vocabulary do not
// (measured DRAM traffic: 3 units per 2 algorithmic), bf16 rows barely.  Here a cluster of C
// CTAs shares a row, which divides the rows in flight by C:
//   pass 1: the consumers fold the chunks of their CTA's part into (m, s) as they land;
//   exchange: each CTA sends its pair to the others (st.shared::cluster + mbarrier arrive with
//             release.cluster), waits for theirs (acquire.cluster), every CTA computes the lse;
//   pass 2: the consumers turn the chunks into outputs and store them (streaming stores).
// Two kernels:
//   k1_full_resident_kernel (default where a row fits the rings of <= 8 CTAs): one CTA per SM
//     with a ring that holds its whole part of a row and a few chunks more.  A chunk stays in
//     its slot from pass 1 to pass 2, so the row crosses the memory system exactly once; pass 1
//     of the next row runs on the spare slots BEFORE pass 2 of the current one, which hides the
//     exchange behind work.
//   k1_full_cluster_kernel (longer rows, or on request): the ring is an ordinary pipeline, the
//     producer fetches every chunk once per pass and the second fetch comes from L2; two CTAs
//     per SM so that one computes while the other waits for its exchange.
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
#ifndef KF_CFG_WANT_SPARE
#define KF_CFG_WANT_SPARE 1
#endif
constexpr int KF_CONSUMER_WARPS = KF_CFG_WARPS;
constexpr int KF_CONSUMERS = KF_CONSUMER_WARPS * 32;
constexpr int KF_THREADS = KF_CONSUMERS + 32;
constexpr int KF_SLOTS = KF_CFG_SLOTS;
constexpr int KF_CHUNK_BYTES = KF_CFG_CHUNK;
constexpr int KF_MAX_CLUSTER = 8;
constexpr int KF_CTAS_PER_SM = KF_CFG_CTAS_PER_SM;
constexpr int KF_WANT_SPARE = KF_CFG_WANT_SPARE;  // free slots preferred (at least one is required)

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
  // chunk_bytes each (the last chunks of a row may be short or empty)
  const int64_t bulk_bytes = (p.vocab * ES) & ~static_cast<int64_t>(15);
  const int64_t chunk_bytes = p.chunk_bytes;
  const int64_t part_begin = static_cast<int64_t>(rank) * chunks_per_cta * chunk_bytes;
  int my_chunks = 0;
  for (int k = 0; k < chunks_per_cta; ++k)
    if (part_begin + k * chunk_bytes < bulk_bytes) ++my_chunks;
  const int64_t tail_begin = bulk_bytes / ES;  // elements past the last 16-byte boundary
  const bool owns_tail = (rank == static_cast<uint32_t>(cluster) - 1);

  if (warp == KF_CONSUMER_WARPS) {
    // ---------------- producer
    if (lane == 0) {
      const uint64_t policy = policy_evict_first();  // every byte is read once
      uint32_t it = 0;
      bool ok = true;
      for (int64_t row = first_row; row < p.n_rows && ok; row += n_clusters) {
        const uint8_t* src = reinterpret_cast<const uint8_t*>(p.src[0]) + row * p.stride * ES +
                             part_begin;
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
            const uint32_t bytes =
                static_cast<uint32_t>(min(chunk_bytes, bulk_bytes - part_begin - off));
            mbar_arrive_expect_tx(full_bar + slot * 8, bytes);
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
      const uint32_t bytes = static_cast<uint32_t>(
          min(chunk_bytes, bulk_bytes - part_begin - k * chunk_bytes));
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
    if (owns_tail && ctid == 0)
      for (int64_t j = tail_begin; j < p.vocab; ++j) online_update_scalar(st, to_float(src[j]), p.c);
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
      const uint32_t bytes = static_cast<uint32_t>(min(chunk_bytes, bulk_bytes - off));
      const uint32_t nvec = dead ? 0u : (bytes >> 4);
      const uint32_t sbase = smem_base + slot * KF_CHUNK_BYTES;
      uint8_t* drow = reinterpret_cast<uint8_t*>(dst) + off;
#pragma unroll 4
      for (uint32_t v = ctid; v < nvec; v += KF_CONSUMERS)
        stg128_streaming(drow + static_cast<size_t>(v) * 16,
                         full_out_vec(lds128(sbase + v * 16), p.inv_temp, lse, T()));
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar + slot * 8);
    }
    if (owns_tail && ctid == 0)
      for (int64_t j = tail_begin; j < p.vocab; ++j)
        dst[j] = full_out_scalar(src[j], p.inv_temp, lse);
  }
  }
  // no CTA leaves while a peer may still store into its shared memory or arrive on its barriers
  if (cluster > 1) cluster_sync_all();
}

// ------------------------------------------------------------------ resident form
#ifndef KR_CFG_WARPS
#define KR_CFG_WARPS 8
#endif
#ifndef KR_CFG_SLOTS
#define KR_CFG_SLOTS 9
#endif
#ifndef KR_CFG_CHUNK
#define KR_CFG_CHUNK 25600
#endif
constexpr int KR_CONSUMER_WARPS = KR_CFG_WARPS;
constexpr int KR_CONSUMERS = KR_CONSUMER_WARPS * 32;
constexpr int KR_THREADS = KR_CONSUMERS + 32;
constexpr int KR_SLOTS = KR_CFG_SLOTS;
constexpr int KR_CHUNK_BYTES = KR_CFG_CHUNK;
static_assert(KR_CHUNK_BYTES % K1_CHUNK_ALIGN == 0, "slots keep the chunk alignment");
static_assert(KR_CONSUMER_WARPS <= 32, "row-end merge reads one partial per lane");

struct KRSmem {
  static constexpr int DATA = KR_SLOTS * KR_CHUNK_BYTES;
  static constexpr int FULL_BAR = DATA;                       // SLOTS mbarriers
  static constexpr int EMPTY_BAR = FULL_BAR + KR_SLOTS * 8;   // SLOTS mbarriers
  static constexpr int XCHG_BAR = EMPTY_BAR + KR_SLOTS * 8;   // 2 mbarriers (row parity)
  static constexpr int PART = XCHG_BAR + 16;                  // [2][WARPS] float2
  static constexpr int PAIRS = PART + 2 * KR_CONSUMER_WARPS * 8;   // [2][MAX_CLUSTER] float2
  static constexpr int LSE = PAIRS + 2 * KF_MAX_CLUSTER * 8;       // [2] float
  static constexpr int TOTAL = LSE + 8;
};

// One CTA per SM; the ring of KR_SLOTS slots holds the CTA's whole part of a row (n chunks)
// plus KR_SLOTS - n spare ones.  The consumers work through the chunks in one fixed order,
// per row i of this cluster (lead = min(n, KR_SLOTS - n)):
//   1. pass 1 of the first `lead` chunks of row i (they were loaded while row i-1 was written);
//   2. the lse of row i-1: wait for the peers' pairs (sent a whole step ago), merge;
//      then pass 2 of row i-1, which frees its slots for the loads of rows i and i+1;
//   3. pass 1 of the remaining chunks of row i; this CTA's (m, s) goes to the peers.
// When two parts fit (lead = n) step 3 is empty and the pair is sent in step 2, after the
// wait.  Every CTA reads the pairs of row i-1 before it sends its pair of row i, and a peer
// can send its pair of row i+1 (which lands in the same slot as that of row i-1) only after
// it has received this CTA's pair of row i: two slots per CTA are enough.
template <typename T>
__global__ void __launch_bounds__(KR_THREADS, 1)
k1_full_resident_kernel(const K1Params p, const int cluster, const int chunks_per_cta) {
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int ES = sizeof(T);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t full_bar = smem_base + KRSmem::FULL_BAR;
  const uint32_t empty_bar = smem_base + KRSmem::EMPTY_BAR;
  const uint32_t xchg_bar = smem_base + KRSmem::XCHG_BAR;
  float2* part = reinterpret_cast<float2*>(smem + KRSmem::PART);
  float2* pairs = reinterpret_cast<float2*>(smem + KRSmem::PAIRS);
  volatile float* lse_box = reinterpret_cast<volatile float*>(smem + KRSmem::LSE);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int64_t n_clusters = gridDim.x / cluster;
  const int64_t first_row = blockIdx.x / cluster;

  if (threadIdx.x == 0) {
    for (int i = 0; i < KR_SLOTS; ++i) {
      mbar_init(full_bar + i * 8, 1);
      mbar_init(empty_bar + i * 8, KR_CONSUMER_WARPS);
    }
    mbar_init(xchg_bar, cluster > 1 ? cluster - 1 : 1);
    mbar_init(xchg_bar + 8, cluster > 1 ? cluster - 1 : 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (cluster > 1) cluster_sync_all();  // nobody arrives on a barrier that is not there yet

  // this CTA's part of a row: chunks [rank * chunks_per_cta, (rank + 1) * chunks_per_cta) of
  // chunk_bytes each (the last chunks of a row may be short or missing)
  const int64_t bulk_bytes = (p.vocab * ES) & ~static_cast<int64_t>(15);
  const int64_t chunk_bytes = p.chunk_bytes;
  const int64_t part_begin = static_cast<int64_t>(rank) * chunks_per_cta * chunk_bytes;
  int my_chunks = 0;
  for (int k = 0; k < chunks_per_cta; ++k)
    if (part_begin + k * chunk_bytes < bulk_bytes) ++my_chunks;
  const int64_t tail_begin = bulk_bytes / ES;  // elements past the last 16-byte boundary
  const bool owns_tail = (rank == static_cast<uint32_t>(cluster) - 1);

  if (warp == KR_CONSUMER_WARPS) {
    // ---------------- producer: every chunk is fetched once, in ring order
    if (lane == 0) {
      const uint64_t policy = policy_evict_first();
      uint32_t it = 0;
      bool ok = true;
      for (int64_t row = first_row; row < p.n_rows && ok; row += n_clusters) {
        const uint8_t* src = reinterpret_cast<const uint8_t*>(p.src[0]) + row * p.stride * ES +
                             part_begin;
        for (int k = 0; k < my_chunks; ++k, ++it) {
          const uint32_t slot = it % KR_SLOTS;
          const uint32_t phase = (it / KR_SLOTS) & 1u;
          if (!mbar_wait(empty_bar + slot * 8, phase ^ 1u)) {
            raise_status(p.status, TOME_DEV_TIMEOUT);
            ok = false;
            break;
          }
          const int64_t off = k * chunk_bytes;
          const uint32_t bytes =
              static_cast<uint32_t>(min(chunk_bytes, bulk_bytes - part_begin - off));
          mbar_arrive_expect_tx(full_bar + slot * 8, bytes);
          bulk_g2s_hint(smem_base + slot * KR_CHUNK_BYTES, src + off, bytes, full_bar + slot * 8,
                        policy);
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- consumers
    // A consumer whose wait ran out (`dead`) stops touching data but stays in step with its
    // CTA and its cluster: it keeps passing the barriers and releasing the slots.
    const int ctid = threadIdx.x;
    const int lead = min(my_chunks, KR_SLOTS - my_chunks);
    uint32_t head = 0;  // ring position of the next chunk of pass 1
    uint32_t tail = 0;  // ring position of the next chunk of pass 2
    bool dead = false;
    Fast fs;
    fast_init(fs, p.c);
    Online cta = {-FLT_MAX, 0.0f};  // warp 0: this CTA's pair of the row in pass 1
    int64_t prev_row = -1;

    // pass 1 of chunks [k0, k1) of the current row
    auto pass1 = [&](int k0, int k1) {
      for (int k = k0; k < k1; ++k, ++head) {
        const uint32_t slot = head % KR_SLOTS;
        if (!dead && !mbar_wait(full_bar + slot * 8, (head / KR_SLOTS) & 1u)) {
          raise_status(p.status, TOME_DEV_TIMEOUT);
          dead = true;
        }
        const uint32_t bytes = static_cast<uint32_t>(
            min(chunk_bytes, bulk_bytes - part_begin - k * chunk_bytes));
        const uint32_t nvec = dead ? 0u : (bytes >> 4);
        const uint32_t sbase = smem_base + slot * KR_CHUNK_BYTES;
#pragma unroll 4
        for (uint32_t v = ctid; v < nvec; v += KR_CONSUMERS)
          fast_update<0>(fs, lds128(sbase + v * 16), p.c, T());
      }
    };
    // end of pass 1 of a row: the CTA's (m, s), in warp 0
    auto reduce_row = [&](const T* src, uint32_t par) {
      Online st = fast_finish(fs, p.c);
      if (dead) st.s = __int_as_float(0x7fc00000);
      if (owns_tail && ctid == 0)
        for (int64_t j = tail_begin; j < p.vocab; ++j)
          online_update_scalar(st, to_float(src[j]), p.c);
      online_warp_reduce(st, p.c);
      if (lane == 0) part[par * KR_CONSUMER_WARPS + warp] = make_float2(st.m, st.s);
      named_bar_sync(1, KR_CONSUMERS);
      if (warp == 0) {
        const float2 w = (lane < KR_CONSUMER_WARPS) ? part[par * KR_CONSUMER_WARPS + lane]
                                                    : make_float2(-FLT_MAX, 0.0f);
        cta.m = w.x;
        cta.s = w.y;
        online_warp_reduce(cta, p.c);
      }
      fast_init(fs, p.c);
    };
    // warp 0: lane q sends this CTA's pair to rank q
    auto send_pair = [&](uint32_t par) {
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
    };
    // warp 0: the lse of a row whose pairs were sent a step ago
    auto finish_row = [&](int64_t row, uint32_t row_it) {
      const uint32_t par = row_it & 1u;
      bool ok = true;
      if (cluster > 1) ok = mbar_wait_cluster(xchg_bar + par * 8, (row_it >> 1) & 1u);
      const float2 o = (lane < cluster) ? pairs[par * KF_MAX_CLUSTER + lane]
                                        : make_float2(-FLT_MAX, 0.0f);
      Online all = {o.x, o.y};
      online_warp_reduce(all, p.c);
      float m = all.m, s = all.s;
      if (!(s >= 0.5f && s <= FLT_MAX))
        exact_row(reinterpret_cast<const T*>(p.src[0]) + row * p.stride, p.vocab, p.c, lane, m, s);
      float lse = finish_lse<K1_FULL>(m, s, p);
      if (!ok) {  // a peer never delivered: report, poison the row, keep the CTA in step
        raise_status(p.status, TOME_DEV_TIMEOUT);
        lse = __int_as_float(0x7fc00000);
      }
      if (lane == 0) {
        lse_box[par] = lse;
        if (rank == 0 && p.out0 != nullptr) p.out0[row] = lse;
      }
    };
    // pass 2 of every chunk of a row; a slot is released once it is written out
    auto pass2 = [&](int64_t row, float lse) {
      const T* src = reinterpret_cast<const T*>(p.src[0]) + row * p.stride;
      T* dst = reinterpret_cast<T*>(p.out_full) + row * p.out_stride;
      for (int k = 0; k < my_chunks; ++k, ++tail) {
        const uint32_t slot = tail % KR_SLOTS;
        const int64_t off = part_begin + k * chunk_bytes;
        const uint32_t bytes = static_cast<uint32_t>(min(chunk_bytes, bulk_bytes - off));
        const uint32_t nvec = dead ? 0u : (bytes >> 4);
        const uint32_t sbase = smem_base + slot * KR_CHUNK_BYTES;
        uint8_t* drow = reinterpret_cast<uint8_t*>(dst) + off;
#pragma unroll 4
        for (uint32_t v = ctid; v < nvec; v += KR_CONSUMERS)
          stg128_streaming(drow + static_cast<size_t>(v) * 16,
                           full_out_vec(lds128(sbase + v * 16), p.inv_temp, lse, T()));
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar + slot * 8);
      }
      if (owns_tail && ctid == 0)
        for (int64_t j = tail_begin; j < p.vocab; ++j)
          dst[j] = full_out_scalar(src[j], p.inv_temp, lse);
    };

    uint32_t row_it = 0;
    for (int64_t row = first_row;; row += n_clusters, ++row_it) {
      const bool have = row < p.n_rows;
      const bool have_prev = prev_row >= 0;
      if (!have && !have_prev) break;
      const T* src = reinterpret_cast<const T*>(p.src[0]) + row * p.stride;
      const uint32_t par = row_it & 1u;
      const bool whole = (lead == my_chunks);  // the whole part is reduced in step 1
      if (have) {
        pass1(0, lead);
        if (whole) reduce_row(src, par);
      }
      if (warp == 0) {
        if (have_prev) finish_row(prev_row, row_it - 1);
        if (have && whole) send_pair(par);
      }
      if (have_prev) {
        named_bar_sync(1, KR_CONSUMERS);
        pass2(prev_row, lse_box[(row_it - 1) & 1u]);
      }
      if (have && !whole) {
        pass1(lead, my_chunks);
        reduce_row(src, par);
        if (warp == 0) send_pair(par);
      }
      if (!have) break;
      prev_row = row;
    }
  }
  // no CTA leaves while a peer may still store into its shared memory or arrive on its barriers
  if (cluster > 1) cluster_sync_all();
}

// Chunking of the resident form for a cluster of `cluster` CTAs: false if a CTA's part does not
// leave at least one slot of its ring spare.
static bool kr_plan(int64_t bulk_bytes, int cluster, int* chunks_per_cta, int32_t* chunk_bytes) {
  const int64_t per_cta = (bulk_bytes + cluster - 1) / cluster;
  int64_t n = std::max<int64_t>(1, (per_cta + KR_CHUNK_BYTES - 1) / KR_CHUNK_BYTES);
  const int64_t al = K1_CHUNK_ALIGN;
  for (; n <= KR_SLOTS - 1; ++n) {  // rounding a chunk up to the alignment may cost one more
    const int64_t total = n * cluster;
    const int64_t cb = std::max<int64_t>(al, ((bulk_bytes + total - 1) / total + al - 1) / al * al);
    if (cb > KR_CHUNK_BYTES) continue;
    *chunks_per_cta = static_cast<int>(n);
    *chunk_bytes = static_cast<int32_t>(cb);
    return true;
  }
  return false;
}

// Chunking for a cluster of `cluster` CTAs that streams its parts twice (no residency limit).
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
                                      int32_t chunk_bytes, bool resident, int sm_count,
                                      cudaStream_t stream) {
  K1Params p = p_in;
  p.chunk_bytes = chunk_bytes;
  void (*kernel)(K1Params, int, int) =
      resident ? k1_full_resident_kernel<T> : k1_full_cluster_kernel<T>;
  const int smem = resident ? KRSmem::TOTAL : KFSmem::TOTAL;
  const int threads = resident ? KR_THREADS : KF_THREADS;
  int32_t st = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
  if (st != TOME_OK) return st;
  // persistent clusters: as many as the device holds at once
  int fit = max_active_clusters(reinterpret_cast<const void*>(kernel), threads, smem, cluster);
  if (fit <= 0) fit = std::max(1, sm_count * (resident ? 1 : KF_CTAS_PER_SM) / cluster);
  const int64_t n_clusters = std::max<int64_t>(1, std::min<int64_t>(fit, p.n_rows));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(n_clusters * cluster), 1, 1);
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
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
  // Beyond that: the resident form with the smallest cluster whose CTAs can hold their part,
  // or, for rows too long for eight rings, the streamed form with CTAs of at most 160 KB.
  // TOME_K1_FULL_CLUSTER forces a form (the tests reach all of them): 0 = pipeline kernel,
  // 1 = resident with the default cluster, r1 / r2 / r4 / r8 = resident, s1 / s2 / s4 / s8 =
  // streamed, by clusters of that size.
  const int64_t es = (dtype == TOME_F32) ? 4 : 2;
  const char* e = getenv("TOME_K1_FULL_CLUSTER");
  int cluster = 0, chunks_per_cta = 0;
  int32_t chunk_bytes = 0;
  const int64_t bulk_bytes = (p.vocab * es) & ~15ll;
  if (!bulk_ok || bulk_bytes < 16) return TOME_OK;
  bool resident = false;
  auto plan_resident = [&]() {
    for (int c = 1; c <= KF_MAX_CLUSTER; c <<= 1)
      if (kr_plan(bulk_bytes, c, &chunks_per_cta, &chunk_bytes)) {
        cluster = c;
        return true;
      }
    return false;
  };
  if (e != nullptr && (e[0] == 's' || e[0] == 'r')) {
    cluster = atoi(e + 1);
    if (cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8) return TOME_OK;
    if (e[0] == 'r') {
      if (!kr_plan(bulk_bytes, cluster, &chunks_per_cta, &chunk_bytes)) return TOME_OK;
      resident = true;
    }
  } else if (e != nullptr) {
    if (atoi(e) == 0 || !plan_resident()) return TOME_OK;
    resident = true;
  } else {
    if (bulk_bytes <= 80 * 1024) return TOME_OK;
    resident = plan_resident();
    if (!resident) {
      const int64_t per_cta = 160 * 1024;
      cluster = 1;
      while (cluster < KF_MAX_CLUSTER && bulk_bytes > per_cta * cluster) cluster <<= 1;
    }
  }
  if (!resident) kf_plan_streamed(bulk_bytes, cluster, &chunks_per_cta, &chunk_bytes);
  *taken = true;
  if (dtype == TOME_F32)
    return k1_launch_full_cluster<float>(p, cluster, chunks_per_cta, chunk_bytes, resident,
                                         sm_count, stream);
  return k1_launch_full_cluster<__nv_bfloat16>(p, cluster, chunks_per_cta, chunk_bytes, resident,
                                               sm_count, stream);
}

}  // namespace tome
