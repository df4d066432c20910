// K1: streaming log-softmax kernels over materialised logits (HBM-bound).
//
// Four small persistent CTAs per SM, each working on its own rows.  In every CTA a producer
// thread streams the row through a two-stage shared-memory ring with 1-D bulk (TMA) copies
// that complete on mbarriers, in equal chunks of about 25 KB that start on 1 KB boundaries;
// four consumer warps read the stages with 128-bit shared loads and keep a per-thread online
// (max, sum-exp) pair in fp32, so every logit is read from HBM exactly once.  The ring runs
// across row boundaries, so the loads of the next row are in flight while a row is being
// reduced, and the four CTAs of an SM are never in the same phase, which keeps the exp unit
// and the memory pipe busy while one of them merges a row.  (Measured: one CTA of 16 warps
// per SM reached 6.0 TB/s, two of 8 warps 6.6, four of 4 warps 6.85 on 20480 x 151936 bf16.)
//
// These modes share the pipeline:
//   SELECTIVE  logprob of one target per row             (mlx-impl/node.py:400-404)
//   DUAL       policy + reference rows of a ragged window, plus the k3 KL estimate
//              (window = completion slice, mlx-impl/node.py:446-451)
//   FULL       full-matrix log-softmax in the input dtype, with the order of operations of
//              the reference's Metal kernel (mlx-impl/model.py:16-66); the row is streamed
//              twice (the second pass is served mostly by L2)
//
//   SAMPLE     top-k sampling + log-prob of the drawn token for large batches (see below)
//
// Rows may start anywhere on the element grid (odd vocabulary sizes, views): a row is copied
// from its first 16-byte boundary to its last and one thread reads the few elements outside
// with ordinary loads (row_geom.cuh).  The FULL mode's 128-bit stores need every output row to
// sit on the grid like its input row; where they do not, a plain-load kernel with the same
// arithmetic takes the call.
// Small batches and long rows of the FULL mode have kernels of their own (k1_small.cu,
// k1_full.cu).
#include "k1_common.cuh"
#include "k1_sample.h"
#include "row_geom.cuh"
#include "sampling.cuh"

namespace tome {

// ------------------------------------------------------------------ bulk-copy pipeline kernel
// FULL mode runs two CTAs per SM (see the launch code), so each can afford a deeper ring.
#ifndef K1_CFG_FULL_STAGES
#define K1_CFG_FULL_STAGES 2
#endif
#ifndef K1_CFG_FULL_KEEP
#define K1_CFG_FULL_KEEP 0
#endif
constexpr int K1_FULL_STAGES = K1_CFG_FULL_STAGES;
__host__ __device__ constexpr int k1_stages(int mode) { return mode == K1_FULL ? K1_FULL_STAGES : K1_STAGES; }

// SAMPLE mode: where a logit reaches the row's current threshold, the place is noted: one
// entry per thread and loop step, two words: (index of the step's first 16-byte vector << 4) |
// mask of the step's four vectors (K1_CONSUMERS apart) that hold such a logit, and the largest
// logit of those four vectors (with which the next kernel drops, unread, the entries that the
// row's final threshold has left behind).  Each consumer warp
// keeps a list of its own; its lanes take their slots with one ballot and a register counter
// (no atomic, no memory round trip), and the warp copies the list out once per row.  The
// kernel that follows fetches the vectors again (about 1 % of the row).  Earlier forms:
// unpacking the vectors here cost ~600 warp-cycles each; one list per CTA filled through a
// shared-memory atomic stalled a warp for the atomic's round trip at every second step;
// copying the vectors themselves, with a ballot per vector, cost 45 instructions per hit step.
constexpr int K1_SAMPLE_WARP_LIST = 112;
#ifndef K1_CFG_POLL_NS
#define K1_CFG_POLL_NS 100
#endif
constexpr int K1_FINISH_CAP = 128;     // surviving entries, vectors and codes the finisher handles per row
constexpr int K1_FINISH_TRIPS = 5;     // entries of a row it reads: at most 32 per trip
constexpr int K1_SAMPLE_TOP = 32 / K1_CONSUMER_WARPS;  // lane maxima each warp puts forward
static_assert(32 % K1_CONSUMER_WARPS == 0 && K1_CONSUMERS <= 128, "threshold keys: 7 id bits");
struct K1SampleSmem {
  uint2 entry[K1_CONSUMER_WARPS][K1_SAMPLE_WARP_LIST];
  uint32_t pub[2][32];  // threshold refinement: what the warps put forward (by parity)
  // the producer warp's scratch for finishing rows (see K1Finisher)
  unsigned long long codes[K1_FINISH_CAP];  // first the surviving entries / vector numbers (32-bit)
  unsigned long long top[K4_MAX_K];
  int32_t lists_done;  // lists written out so far by the consumer warps, all rows together
  int32_t n_codes;
};

// SPLIT: with a few rows per CTA the last round leaves most CTAs idle (1024 rows on 592 CTAs:
// 432 do two rows, 160 one).  The kernel is then launched in clusters of K1_SPLIT CTAs: the
// rows that fill whole rounds are dealt one per CTA as usual, the remaining ones one per
// cluster, each CTA taking a quarter of the row's chunks; the quarters' (m, s) pairs meet in
// the first CTA's shared memory (st.shared::cluster + mbarrier), which merges them and writes
// the row.  A cluster shares fewer than K1_SPLIT_ITEMS + 1 rows (the remainder is smaller
// than the grid), so every pair slot and barrier is used once.
constexpr int K1_SPLIT = 4;
constexpr int K1_SPLIT_ITEMS = 4;

template <int STAGES>
struct K1SmemT {
  static constexpr int DATA = STAGES * K1_CHUNK_BYTES;
  static constexpr int BAR_OFF = DATA;                                   // 2 * STAGES mbarriers
  static constexpr int PART_OFF = BAR_OFF + 2 * STAGES * 8;              // [2][WARPS] float2
  static constexpr int CUM_OFF = PART_OFF + 2 * K1_CONSUMER_WARPS * 8;   // DUAL: prefix sums
  static constexpr int SCRATCH_OFF = CUM_OFF + (K1_MAX_SEQ + 1) * 4 + 12;
  static constexpr int TOTAL_DUAL = SCRATCH_OFF + K1_THREADS * 4;
  static constexpr int TOTAL_PLAIN = CUM_OFF;
  static constexpr int SAMPLE_OFF = (CUM_OFF + 15) & ~15;                // SAMPLE: K1SampleSmem
  // SPLIT (selective mode, rows shared by a cluster): pairs [K1_SPLIT_ITEMS][K1_SPLIT] float2,
  // then one mbarrier per shared row
  static constexpr int SPLIT_OFF = (CUM_OFF + 15) & ~15;
  static constexpr int SPLIT_BAR_OFF = SPLIT_OFF + K1_SPLIT_ITEMS * K1_SPLIT * 8;
  static constexpr int TOTAL_SPLIT = SPLIT_BAR_OFF + K1_SPLIT_ITEMS * 8;
};


// SAMPLE mode: finishes a row once the consumers have streamed it, in the producer warp.  The
// consumers leave, per row and in global memory, a threshold (a value that at least top_k
// logits reach), the logsumexp and one list of entries per consumer warp.  The finisher drops
// the entries whose largest logit stays below the threshold, fetches the vectors the others
// name, keeps the logits that reach the threshold as (value, index) codes, ranks them (exact
// top-k), draws a token and writes it with its log-prob.  A row it cannot hold (a list that ran
// over, more than K1_FINISH_CAP survivors, fewer than top_k numbers) goes on the list of rows
// for k4_sample_kernel.  The work is cut into steps of one global round trip or a few hundred
// instructions, so that the copies the warp is there to issue are never kept waiting long;
// what a step loads is used by the next one.
template <typename T>
struct K1Finisher {
  static constexpr int PER = 16 / static_cast<int>(sizeof(T));
  const K1Params& p;
  K1SampleSmem& smp;
  const int lane;
  int32_t done = 0;   // rows finished
  int phase = 0;
  int64_t row = 0;
  float thr = 0.0f;
  bool spoilt = false;                 // the row goes to the row kernel
  uint2 ent[K1_FINISH_TRIPS];          // phase 1: the entries this lane looks at
  int32_t begin[K1_CONSUMER_WARPS];    // where each list begins when they are put end to end
  int32_t trip0 = 0;                   // first of the trips held in ent[]
  int32_t n_kept = 0;                  // entries that survived so far
  int32_t total = 0;                   // entries of the row
  uint4 vec[K1_FINISH_CAP / 32];       // phase 2: the vectors this lane unpacks
  int32_t vec_at[K1_FINISH_CAP / 32];  // their numbers within the row (-1: none)
  int32_t n_vec = 0;

  __device__ K1Finisher(const K1Params& params, K1SampleSmem& s, int l) : p(params), smp(s), lane(l) {}
  __device__ int64_t rows_finished() const { return done; }

  __device__ __forceinline__ void give_up_row() {  // left to the row kernel
    if (lane == 0) p.marked_rows[atomicAdd(p.marked, 1)] = static_cast<int32_t>(row);
    ++done;
    phase = 0;
  }

  // Asks for the entries of trips [trip0, trip0 + K1_FINISH_TRIPS).
  __device__ __forceinline__ void load_entries() {
#pragma unroll
    for (int t = 0; t < K1_FINISH_TRIPS; ++t) {
      const int32_t g = (trip0 + t) * 32 + lane;
      int32_t l = 0, at = g;  // the last list that begins at or before g, and the place in it
#pragma unroll
      for (int q = 1; q < K1_CONSUMER_WARPS; ++q)
        if (g >= begin[q]) {
          l = q;
          at = g - begin[q];
        }
      ent[t] = (g < total && !spoilt)
                   ? p.cand_entry[(row * K1_CONSUMER_WARPS + l) * p.cand_cap + at]
                   : make_uint2(0u, 0u);
    }
  }

  // One step; false if there was nothing to do.
  __device__ __forceinline__ bool step() {
    const uint32_t below = (1u << lane) - 1u;
    if (phase == 0) {
      // a row is ready when every consumer warp has written its list out
      const int32_t lists = *reinterpret_cast<volatile int32_t*>(&smp.lists_done);
      if (lists < (done + 1) * K1_CONSUMER_WARPS) return false;
      __threadfence_block();
      row = static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(done) * gridDim.x;
      thr = p.row_thr[row];
      spoilt = false;
      total = 0;
#pragma unroll
      for (int l = 0; l < K1_CONSUMER_WARPS; ++l) {
        const int32_t n = p.cand_count[row * K1_CONSUMER_WARPS + l];
        spoilt |= (n > p.cand_cap);
        begin[l] = total;
        total += min(n, p.cand_cap);
      }
      trip0 = 0;
      n_kept = 0;
      load_entries();
      phase = 1;
      return true;
    }
    if (phase == 1) {
      if (spoilt) {
        give_up_row();
        return true;
      }
      // surviving entries, gathered (their first words) in shared memory ...
      uint32_t* kept = reinterpret_cast<uint32_t*>(smp.codes);
#pragma unroll
      for (int t = 0; t < K1_FINISH_TRIPS; ++t) {
        const bool keep =
            ((trip0 + t) * 32 + lane < total) && !(__uint_as_float(ent[t].y) < thr);
        const uint32_t bal = __ballot_sync(0xffffffffu, keep);
        const int32_t to = n_kept + __popc(bal & below);
        if (keep && to < K1_FINISH_CAP) kept[to] = ent[t].x;
        n_kept += __popc(bal);
      }
      __syncwarp();
      if (n_kept > K1_FINISH_CAP) {
        give_up_row();
        return true;
      }
      trip0 += K1_FINISH_TRIPS;
      if (trip0 * 32 < total) {  // a long row: the next entries, same step again
        load_entries();
        return true;
      }
      // ... taken into registers, then expanded in place into vector numbers
      uint32_t mine[K1_FINISH_CAP / 32];
#pragma unroll
      for (int t = 0; t < K1_FINISH_CAP / 32; ++t)
        mine[t] = (t * 32 + lane < n_kept) ? kept[t * 32 + lane] : 0u;
      __syncwarp();
      n_vec = 0;
#pragma unroll
      for (int t = 0; t < K1_FINISH_CAP / 32; ++t) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const bool bit = (mine[t] >> j) & 1u;
          const uint32_t bal = __ballot_sync(0xffffffffu, bit);
          const int32_t to = n_vec + __popc(bal & below);
          if (bit && to < K1_FINISH_CAP)
            kept[to] = (mine[t] >> 4) + static_cast<uint32_t>(j * K1_CONSUMERS);
          n_vec += __popc(bal);
        }
      }
      __syncwarp();
      if (n_vec > K1_FINISH_CAP) {
        give_up_row();
        return true;
      }
      // the vectors are asked for now and unpacked in the next step
      const T* src = reinterpret_cast<const T*>(p.src[0]) + row * p.stride;
      const K1RowGeom geom = k1_row_geom(src, p.vocab);
      const uint4* body = reinterpret_cast<const uint4*>(src + geom.head);
#pragma unroll
      for (int t = 0; t < K1_FINISH_CAP / 32; ++t) {
        const int32_t i = t * 32 + lane;
        vec_at[t] = (i < n_vec) ? static_cast<int32_t>(kept[i]) : -1;
        vec[t] = make_uint4(0u, 0u, 0u, 0u);
        if (vec_at[t] >= 0 && static_cast<int64_t>(vec_at[t]) * 16 < geom.bulk_bytes)
          vec[t] = __ldg(body + vec_at[t]);
      }
      if (lane == 0) smp.n_codes = 0;
      __syncwarp();
      phase = 2;
      return true;
    }
    if (phase == 2) {
      const T* src = reinterpret_cast<const T*>(p.src[0]) + row * p.stride;
      const K1RowGeom geom = k1_row_geom(src, p.vocab);
      const int32_t kk = p.sample_kk;
#pragma unroll
      for (int t = 0; t < K1_FINISH_CAP / 32; ++t) {
        if (vec_at[t] < 0) continue;
        const int64_t e0 = geom.head + static_cast<int64_t>(vec_at[t]) * PER;
        if (static_cast<int64_t>(vec_at[t]) * 16 < geom.bulk_bytes) {
          const uint32_t u[4] = {vec[t].x, vec[t].y, vec[t].z, vec[t].w};
#pragma unroll
          for (int q = 0; q < PER; ++q) {
            const float x = (sizeof(T) == 4)
                                ? __uint_as_float(u[q])
                                : __uint_as_float((q & 1) ? (u[q >> 1] & 0xffff0000u) : (u[q >> 1] << 16));
            if (x >= thr) {
              const int32_t at = atomicAdd(&smp.n_codes, 1);
              if (at < K1_FINISH_CAP) smp.codes[at] = k4_pack(x, e0 + q);
            }
          }
        } else {  // the short vector: the elements outside the row's 16-byte boundaries
          const int64_t n_ends = geom.head + (p.vocab - geom.tail_begin);
          for (int64_t i = 0; i < n_ends; ++i) {
            const int64_t q = (i < geom.head) ? i : geom.tail_begin + (i - geom.head);
            const float x = to_float(src[q]);
            if (x >= thr) {
              const int32_t at = atomicAdd(&smp.n_codes, 1);
              if (at < K1_FINISH_CAP) smp.codes[at] = k4_pack(x, q);
            }
          }
        }
      }
      __syncwarp();
      const int32_t n = smp.n_codes;
      if (n > K1_FINISH_CAP || n < kk) {
        give_up_row();
        return true;
      }
      // exact top-kk by ranking every code against all (codes are distinct), two per lane and trip
      for (int32_t i0 = 0; i0 < n; i0 += 64) {
        const int32_t ia = i0 + lane, ib = i0 + 32 + lane;
        const unsigned long long a = (ia < n) ? smp.codes[ia] : ~0ull;
        const unsigned long long b = (ib < n) ? smp.codes[ib] : ~0ull;
        int32_t rank_a = 0, rank_b = 0;
#pragma unroll 4
        for (int32_t j = 0; j < n; ++j) {
          const unsigned long long o = smp.codes[j];
          rank_a += (o > a) ? 1 : 0;
          rank_b += (o > b) ? 1 : 0;
        }
        if (ia < n && rank_a < kk) smp.top[rank_a] = a;
        if (ib < n && rank_b < kk) smp.top[rank_b] = b;
      }
      __syncwarp();
      phase = 3;
      return true;
    }
    // phase 3: draw, score, write
    const int32_t kk = p.sample_kk;
    const bool greedy = !(p.sample_temperature > 0.0f);
    const int32_t pick =
        greedy ? 0 : k4_draw_warp(smp.top, kk, p.c, row, p.sample_seed, p.sample_offset);
    if (lane == 0) {
      p.out_tokens[row] = k4_index(smp.top[pick]);
      p.out0[row] = __fdiv_rn(k4_value(smp.top[pick]), p.temp) - p.out1[row];
    }
    const int32_t k = p.sample_top_k;
    if (p.out_topk_idx != nullptr || p.out_topk_val != nullptr) {
      for (int32_t j = lane; j < k; j += 32) {
        const bool have = j < kk;
        if (p.out_topk_idx != nullptr)
          p.out_topk_idx[row * k + j] = have ? k4_index(smp.top[j]) : -1;
        if (p.out_topk_val != nullptr)
          p.out_topk_val[row * k + j] = have ? k4_value(smp.top[j]) : -INFINITY;
      }
    }
    __syncwarp();
    ++done;
    phase = 0;
    return true;
  }
};

// One unit of work of a CTA: chunks [k_begin, k_end) of row / window position `item`.
struct K1Item {
  int64_t item;
  int64_t k_begin, k_end;
  bool shared;  // SPLIT: the row is shared by the cluster (this CTA has a quarter of it)
};

// The round-th unit of this CTA; false when there is none.  Without SPLIT: rows blockIdx.x,
// blockIdx.x + gridDim.x, ...  With SPLIT: `whole_rounds` such rows, then the cluster's share
// of the remaining rows, a quarter of the chunks each.
template <bool SPLIT>
__device__ __forceinline__ bool k1_next_item(int64_t round, int64_t n_items, int64_t whole_rounds,
                                             int64_t split_rows, int64_t n_clusters,
                                             int64_t cluster_id, uint32_t crank, int64_t n_chunks,
                                             K1Item& w) {
  w.k_begin = 0;
  w.k_end = n_chunks;
  w.shared = false;
  if (!SPLIT || round < whole_rounds) {
    w.item = static_cast<int64_t>(blockIdx.x) + round * gridDim.x;
    return SPLIT || w.item < n_items;
  }
  const int64_t j = cluster_id + (round - whole_rounds) * n_clusters;
  if (j >= split_rows) return false;
  w.item = whole_rounds * gridDim.x + j;
  w.k_begin = n_chunks * crank / K1_SPLIT;
  w.k_end = n_chunks * (crank + 1) / K1_SPLIT;
  w.shared = true;
  return true;
}

// Size of the k-th bulk copy of a row: chunk_bytes, less for the last one, which is empty for a
// row that starts off the grid and so holds one vector fewer than the launch planned for.
__device__ __forceinline__ uint32_t k1_chunk_size(int64_t k, int64_t chunk_bytes,
                                                  int64_t bulk_bytes) {
  return static_cast<uint32_t>(max(int64_t{0}, min(chunk_bytes, bulk_bytes - k * chunk_bytes)));
}

// SAMPLE mode with rows cut into parts: neighbouring items are the parts of one row, each with an
// equal share of the row's chunks.  Returns the row and sets the item's chunk range.
__device__ __forceinline__ int64_t k1_sample_part(const K1Params& p, int64_t n_chunks, K1Item& w) {
  const int lg = p.sample_parts_log2;
  const int64_t part = w.item & ((int64_t{1} << lg) - 1);
  w.k_begin = (n_chunks * part) >> lg;
  w.k_end = (n_chunks * (part + 1)) >> lg;
  return w.item >> lg;
}

template <typename T, int MODE, int POLY, bool SPLIT = false, bool FINISH = false>
__global__ void __launch_bounds__(K1_THREADS, K1_CTAS_PER_SM) k1_stream_kernel(const K1Params p) {
  static_assert(!SPLIT || MODE == K1_SELECTIVE, "rows are shared by clusters in selective mode only");
  static_assert(!FINISH || MODE == K1_SAMPLE, "rows are finished in the kernel in sampling mode only");
  constexpr int STAGES = k1_stages(MODE);
  using Smem = K1SmemT<STAGES>;
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int NSUB = (MODE == K1_DUAL || MODE == K1_FULL) ? 2 : 1;
  constexpr bool WINDOWED = k1_windowed(MODE);
  constexpr int ES = sizeof(T);
  constexpr int PER_VEC = 16 / ES;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t full_bar = smem_base + Smem::BAR_OFF;
  const uint32_t empty_bar = full_bar + STAGES * 8;
  float2* part = reinterpret_cast<float2*>(smem + Smem::PART_OFF);
  int32_t* cum = reinterpret_cast<int32_t*>(smem + Smem::CUM_OFF);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(full_bar + i * 8, 1);
      mbar_init(empty_bar + i * 8, K1_CONSUMER_WARPS);
    }
    if (SPLIT)
      for (int i = 0; i < K1_SPLIT_ITEMS; ++i)
        mbar_init(smem_base + Smem::SPLIT_BAR_OFF + i * 8, K1_SPLIT - 1);
    fence_mbar_init();
    if (MODE == K1_SAMPLE)
      reinterpret_cast<K1SampleSmem*>(smem + Smem::SAMPLE_OFF)->lists_done = 0;
    // SAMPLE without the finisher: this kernel never touches the count of rows left to the row
    // kernel (the kernels after it do, once it has completed), so it can clear it for them
    if (MODE == K1_SAMPLE && !FINISH && blockIdx.x == 0 && p.marked != nullptr) *p.marked = 0;
  }
  // SPLIT: every CTA does `whole_rounds` rows of its own, then a quarter of each row of its
  // cluster's share of the remainder
  const uint32_t crank = SPLIT ? cluster_ctarank() : 0u;
  const int64_t whole_rounds = SPLIT ? p.n_rows / gridDim.x : 0;
  const int64_t whole_rows = whole_rounds * gridDim.x;
  const int64_t split_rows = SPLIT ? p.n_rows - whole_rows : 0;
  const int64_t n_clusters = SPLIT ? gridDim.x / K1_SPLIT : 1;
  const int64_t cluster_id = SPLIT ? blockIdx.x / K1_SPLIT : 0;
  int64_t n_items = p.n_rows;
  if (MODE == K1_SAMPLE) n_items <<= p.sample_parts_log2;
  if (WINDOWED) {
    n_items = dual_build_prefix(p, cum, reinterpret_cast<int32_t*>(smem + Smem::SCRATCH_OFF));
    if (MODE == K1_DUAL) dual_zero_masked(p);
    if (MODE == K1_RAGGED && blockIdx.x == 0 && p.out_offsets != nullptr)
      for (int i = threadIdx.x; i <= p.n_seq; i += blockDim.x) p.out_offsets[i] = cum[i];
    if (MODE == K1_RAGGED && n_items > p.packed_capacity) {
      // the windows cover more positions than the packed arrays hold: score what fits
      if (threadIdx.x == 0) raise_status(p.status, TOME_DEV_RAGGED_OVERFLOW);
      n_items = p.packed_capacity;
    }
  }
  __syncthreads();
  if (SPLIT) cluster_sync_all();  // the peers' barriers exist before anything arrives on them
  // SAMPLE: the kernels that follow (k4_sample.cu) may be set up while this one runs; they wait
  // for its completion before they read anything
  if (MODE == K1_SAMPLE) griddep_launch_dependents();

  const int64_t n_chunks = p.n_chunks;
  const int64_t chunk_bytes = p.chunk_bytes;

  if (FINISH && warp == K1_CONSUMER_WARPS) {
    // ---------------- producer of the sampling mode: lane 0 issues the bulk copies, and while
    // it waits for a stage to come free the whole warp finishes the rows the consumers have
    // handed over (K1Finisher), one short step at a time
    K1SampleSmem& smp = *reinterpret_cast<K1SampleSmem*>(smem + Smem::SAMPLE_OFF);
    K1Finisher<T> fin(p, smp, lane);
    const uint64_t policy = policy_evict_first();
    uint32_t it = 0;
    bool ok = true;
    int64_t my_rows = 0;
    for (int64_t row = blockIdx.x; row < n_items && ok; row += gridDim.x, ++my_rows) {
      const T* row_src = reinterpret_cast<const T*>(p.src[0]) + row * p.stride;
      const K1RowGeom geom = k1_row_geom(row_src, p.vocab);
      const uint8_t* src = reinterpret_cast<const uint8_t*>(row_src + geom.head);
      for (int64_t k = 0; k < n_chunks && ok; ++k, ++it) {
        const uint32_t stage = it % STAGES;
        const uint32_t parity = ((it / STAGES) & 1u) ^ 1u;
        const long long t0 = clock64();
        for (;;) {
          const bool ready = __shfl_sync(
              0xffffffffu, (lane == 0) && mbar_try_wait(empty_bar + stage * 8, parity), 0);
          if (ready) break;
          if (!fin.step()) {
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
              if (lane == 0) raise_status(p.status, TOME_DEV_TIMEOUT);
              ok = false;
              break;
            }
            __nanosleep(K1_CFG_POLL_NS);  // nothing to do: leave the issue slots to the consumers
          }
        }
        if (ok && lane == 0) {
          const int64_t off = k * chunk_bytes;
          const uint32_t bytes = k1_chunk_size(k, chunk_bytes, geom.bulk_bytes);
          mbar_arrive_expect_tx(full_bar + stage * 8, bytes);
          if (bytes != 0)
            bulk_g2s_hint(smem_base + stage * K1_CHUNK_BYTES, src + off, bytes,
                          full_bar + stage * 8, policy);
        }
      }
    }
    // the rows still to be finished once every copy is on its way
    const long long t0 = clock64();
    while (ok && fin.rows_finished() < my_rows) {
      if (!fin.step()) {
        if (clock64() - t0 > 4 * WAIT_LIMIT_CYCLES) {
          if (lane == 0) raise_status(p.status, TOME_DEV_TIMEOUT);
          break;
        }
        __nanosleep(K1_CFG_POLL_NS);
      }
    }
    return;
  }
  if (warp == K1_CONSUMER_WARPS) {
    // ---------------- producer: one thread issues every bulk copy of this CTA
    if (lane == 0) {
      const uint64_t policy = policy_evict_first();
      const uint64_t keep = policy_evict_last();
      uint32_t it = 0;
      bool ok = true;
      for (int64_t round = 0; ok; ++round) {
        K1Item w;
        if (!k1_next_item<SPLIT>(round, n_items, whole_rounds, split_rows, n_clusters, cluster_id,
                                 crank, n_chunks, w))
          break;
        const int64_t row = WINDOWED               ? dual_row_of_item(p, cum, w.item)
                            : (MODE == K1_SAMPLE) ? k1_sample_part(p, n_chunks, w)
                                                  : w.item;
        for (int sub = 0; sub < NSUB && ok; ++sub) {
          const T* row_src =
              reinterpret_cast<const T*>(p.src[(MODE == K1_DUAL) ? sub : 0]) + row * p.stride;
          const K1RowGeom geom = k1_row_geom(row_src, p.vocab);
          const uint8_t* src = reinterpret_cast<const uint8_t*>(row_src + geom.head);
          for (int64_t k = w.k_begin; k < w.k_end; ++k, ++it) {
            const uint32_t stage = it % STAGES;
            const uint32_t phase = (it / STAGES) & 1u;
            if (!mbar_wait(empty_bar + stage * 8, phase ^ 1u)) {
              raise_status(p.status, TOME_DEV_TIMEOUT);
              ok = false;
              break;
            }
            const int64_t off = k * chunk_bytes;
            const uint32_t bytes = k1_chunk_size(k, chunk_bytes, geom.bulk_bytes);
            mbar_arrive_expect_tx(full_bar + stage * 8, bytes);
            if (bytes == 0) continue;  // (a row off the 16-byte grid may lack the last copy)
            // FULL re-reads the row in its second pass: keep it in L2 after the first.
            if (K1_CFG_FULL_KEEP && MODE == K1_FULL && sub == 0)
              bulk_g2s_hint(smem_base + stage * K1_CHUNK_BYTES, src + off, bytes,
                            full_bar + stage * 8, keep);
            else if (!K1_CFG_L2_HINT || (MODE == K1_FULL && sub == 0))
              bulk_g2s(smem_base + stage * K1_CHUNK_BYTES, src + off, bytes, full_bar + stage * 8);
            else
              bulk_g2s_hint(smem_base + stage * K1_CHUNK_BYTES, src + off, bytes,
                            full_bar + stage * 8, policy);
          }
        }
      }
    }
    if (SPLIT) {  // nobody leaves while a peer may still address its shared memory
      __syncwarp();
      cluster_sync_all();
    }
    return;
  }

  // ---------------- consumers
  // A consumer whose wait ran out (`dead`) stops touching the ring's data but stays in step
  // with the others: it keeps arriving on the empty barriers and on the named barriers, so
  // that nobody is left waiting for it; its rows are redone by exact_row() or come out NaN.
  const int ctid = threadIdx.x;  // 0 .. K1_CONSUMERS-1
  uint32_t it = 0;
  uint32_t red_it = 0;
  float carry = 0.0f;
  bool dead = false;
  uint32_t refinements = 0;  // SAMPLE: threshold updates so far (their parity picks the buffer)
  uint32_t split_it = 0;     // SPLIT: shared rows this cluster has finished
  for (int64_t round = 0;; ++round) {
    K1Item w;
    if (!k1_next_item<SPLIT>(round, n_items, whole_rounds, split_rows, n_clusters, cluster_id, crank,
                             n_chunks, w))
      break;
    const int64_t item = w.item;  // SAMPLE: also where the item's threshold and lists go
    const int64_t row = WINDOWED               ? dual_row_of_item(p, cum, item)
                        : (MODE == K1_SAMPLE) ? k1_sample_part(p, n_chunks, w)
                                              : item;
    const int64_t oidx = (MODE == K1_RAGGED) ? item : row;  // where targets/outputs live
    float lse_row = 0.0f;
    for (int sub = 0; sub < NSUB; ++sub) {
      const T* src = reinterpret_cast<const T*>(p.src[(MODE == K1_DUAL) ? sub : 0]) +
                     row * p.stride;
      const K1RowGeom geom = k1_row_geom(src, p.vocab);
      const bool reduce_pass = (MODE != K1_FULL) || (sub == 0);

      // the one thread that finishes the row fetches the target logit early
      float x_t = 0.0f;
      bool target_ok = true;
      if (MODE != K1_FULL && MODE != K1_SAMPLE && ctid == 0 && !(w.shared && crank != 0)) {
        const int32_t t = p.targets[oidx];
        target_ok = (t >= 0) && (static_cast<int64_t>(t) < p.vocab);
        if (target_ok) x_t = to_float(src[t]);
        else raise_status(p.status, TOME_DEV_TARGET_OUT_OF_RANGE);
      }

      Fast fs;
      fast_init(fs, p.c);
      T* dst = nullptr;
      if (MODE == K1_FULL) dst = reinterpret_cast<T*>(p.out_full) + row * p.out_stride;

      // SAMPLE: the row's threshold is a value that at least top_k of its logits reach.  Every
      // consumer keeps the maximum of the logits it has seen (128 disjoint groups).  Each warp
      // puts its 8 largest lane maxima forward and the top_k-th largest of the 32 values put
      // forward becomes the threshold: at least top_k groups, hence logits, reach it, and it is
      // the exact top_k-th largest group maximum unless one warp holds more than 8 of the best.
      // (top_k > 32: each warp certifies its ceil(top_k / warps)-th largest lane maximum and the
      // smallest of those is taken.)  The first chunk is looked at twice (maxima first), later
      // the threshold is raised after chunks 3, 15, 63, ... (each time the sample has grown
      // fourfold), which keeps the noted places near 130 per row, and after the last chunk.  A
      // later kernel fetches them, keeps what reaches the final threshold, ranks and draws.
      K1SampleSmem& smp = *reinterpret_cast<K1SampleSmem*>(smem + Smem::SAMPLE_OFF);
      float thr_val = __int_as_float(0x7f800000);  // +inf: nothing qualifies
      float tmax = __int_as_float(0xff800000);     // largest logit this thread has seen
      int32_t wcount = 0;                          // entries in this warp's list (same in every lane)
      auto note = [&](uint32_t mask, int64_t vec_index, float largest) {
        const uint32_t bal = __ballot_sync(0xffffffffu, mask != 0u);
        if (mask != 0u) {
          const int32_t slot = wcount + __popc(bal & ((1u << lane) - 1u));
          if (slot < K1_SAMPLE_WARP_LIST)
            smp.entry[warp][slot] =
                make_uint2((static_cast<uint32_t>(vec_index) << 4) | mask, __float_as_uint(largest));
        }
        wcount += __popc(bal);
      };
      auto refine = [&]() {
        // order-preserving key of the lane maximum; its low 7 bits carry the thread's number,
        // which makes the keys distinct and lowers the value by at most 127 ulps (still a
        // value that the group reaches).  Selection is by warp-wide max / min reductions
        // (redux.sync), one instruction each.
        uint32_t key = (k4_key(tmax) & ~127u) | static_cast<uint32_t>(127 - ctid);
        uint32_t* pub = smp.pub[refinements & 1u];
        const bool union_form = p.sample_kk <= 32;
        if (union_form) {
#pragma unroll
          for (int r = 0; r < K1_SAMPLE_TOP; ++r) {  // the warp's largest keys, one by one
            const uint32_t best = __reduce_max_sync(0xffffffffu, key);
            if (key == best) {
              pub[warp * K1_SAMPLE_TOP + r] = best;
              key = 0u;
            }
          }
        } else {
          uint32_t best = 0u;
          for (int r = 0; r < p.sample_q; ++r) {
            best = __reduce_max_sync(0xffffffffu, key);
            if (key == best) key = 0u;
          }
          if (lane == 0) pub[warp] = best;
        }
        named_bar_sync(2, K1_CONSUMERS);
        uint32_t best = 0u;
        if (union_form) {
          // the kk-th largest of the 32 keys put forward is the (33 - kk)-th smallest: take it
          // from the nearer end
          uint32_t mine = pub[lane];
          const int32_t kk = p.sample_kk;
          if (2 * kk <= 33) {
            for (int32_t r = 0; r < kk; ++r) {
              best = __reduce_max_sync(0xffffffffu, mine);
              if (mine == best) mine = 0u;
            }
          } else {
            for (int32_t r = 0; r < 33 - kk; ++r) {
              best = __reduce_min_sync(0xffffffffu, mine);
              if (mine == best) mine = 0xffffffffu;
            }
          }
        } else {
          best = pub[0];
#pragma unroll
          for (int w = 1; w < K1_CONSUMER_WARPS; ++w) best = min(best, pub[w]);
        }
        ++refinements;
        const float t = k4_unkey(best & ~127u);
        thr_val = (t != t) ? __int_as_float(0xff800000) : t;  // -inf with its low bits cleared
      };

      // (running values instead of products per chunk: this loop's overhead is paid 12 - 24 times
      // per row)
      int64_t off = w.k_begin * chunk_bytes;        // of the chunk within the row's bulk range
      int64_t left = geom.bulk_bytes - off;         // bytes of that range from this chunk on
      int32_t kr = 0;                               // chunks of this item done
      for (int64_t k = w.k_begin; k < w.k_end; ++k, ++it, off += chunk_bytes, left -= chunk_bytes) {
        const uint32_t stage = it % STAGES;
        const uint32_t phase = (it / STAGES) & 1u;
        if (!dead && !mbar_wait(full_bar + stage * 8, phase)) {
          raise_status(p.status, TOME_DEV_TIMEOUT);
          dead = true;
        }
        const uint32_t bytes = static_cast<uint32_t>(max(int64_t{0}, min(chunk_bytes, left)));
        const uint32_t nvec = dead ? 0u : (bytes >> 4);
        const uint32_t sbase = smem_base + stage * K1_CHUNK_BYTES;
        if (MODE == K1_SAMPLE && k == w.k_begin) {
          for (uint32_t v = ctid; v < nvec; v += K1_CONSUMERS)
            tmax = fmaxf(tmax, vec_max(lds128(sbase + v * 16), T()));
          refine();
        }
        // the loops run on the warp's first vector so that every lane makes the same trips
        uint32_t vb = warp * 32;
        if (reduce_pass) {
          for (; vb + 3 * K1_CONSUMERS + 32 <= nvec; vb += 4 * K1_CONSUMERS) {
            const uint32_t v = vb + lane;
            const uint4 a = lds128(sbase + v * 16);
            const uint4 b = lds128(sbase + (v + K1_CONSUMERS) * 16);
            const uint4 cc = lds128(sbase + (v + 2 * K1_CONSUMERS) * 16);
            const uint4 d = lds128(sbase + (v + 3 * K1_CONSUMERS) * 16);
            const float ma = fast_update<POLY>(fs, a, p.c, T());
            const float mb = fast_update<POLY>(fs, b, p.c, T());
            const float mc = fast_update<POLY>(fs, cc, p.c, T());
            const float md = fast_update<POLY>(fs, d, p.c, T());
            if (MODE == K1_SAMPLE) {
              // a NaN maximum (a bf16 vector holding a NaN) counts as a hit: the vector's other
              // logits are looked at later; the running maximum ignores it
              const float m4 = fmax3_nan(fmax_nan(ma, mb), mc, md);
              tmax = fmaxf(tmax, m4);
              if (__any_sync(0xffffffffu, !(m4 < thr_val))) {
                const uint32_t mask = (!(ma < thr_val) ? 1u : 0u) | (!(mb < thr_val) ? 2u : 0u) |
                                      (!(mc < thr_val) ? 4u : 0u) | (!(md < thr_val) ? 8u : 0u);
                note(mask, (off >> 4) + v, m4);  // v: this thread's first vector of the step
              }
            }
          }
          for (; vb < nvec; vb += K1_CONSUMERS) {
            const uint32_t v = vb + lane;
            bool hit = false;
            float ma = 0.0f;
            if (v < nvec) {
              ma = fast_update<POLY>(fs, lds128(sbase + v * 16), p.c, T());
              if (MODE == K1_SAMPLE) {
                hit = !(ma < thr_val);
                tmax = fmaxf(tmax, ma);
              }
            }
            if (MODE == K1_SAMPLE && __any_sync(0xffffffffu, hit))
              note(hit ? 1u : 0u, (off >> 4) + v, ma);
          }
        } else {
          uint8_t* drow = reinterpret_cast<uint8_t*>(dst + geom.head) + off;
          for (uint32_t v = ctid; v < nvec; v += K1_CONSUMERS) {
            const uint4 a = lds128(sbase + v * 16);
            stg128_streaming(drow + static_cast<size_t>(v) * 16,
                             full_out_vec(a, p.inv_temp, lse_row, T()));
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar + stage * 8);
        // the sample has grown fourfold: raise the threshold.  Once more after the row's last
        // chunk: nothing is noted any more, but the kernel that follows has a third of the
        // logits to rank.
        ++kr;
        if (MODE == K1_SAMPLE &&
            ((kr >= 4 && (kr & (kr - 1)) == 0 && (kr & 0x55555555) != 0) || k + 1 == w.k_end))
          refine();
      }

      Online st = fast_finish(fs, p.c);
      if (dead) st.s = __int_as_float(0x7fc00000);  // the row takes the exact path below
      // elements before the first and past the last 16-byte boundary of the row (at most
      // PER_VEC - 1 each)
      if (ctid == 0 && w.k_end == n_chunks) {
        auto end_element = [&](int64_t j) {
          if (reduce_pass) online_update_scalar(st, to_float(src[j]), p.c);
          else dst[j] = full_out_scalar(src[j], p.inv_temp, lse_row);
        };
        for (int64_t j = 0; j < geom.head; ++j) end_element(j);
        for (int64_t j = geom.tail_begin; j < p.vocab; ++j) end_element(j);
      }
      if (MODE == K1_SAMPLE && warp == 0 && w.k_end == n_chunks &&
          (geom.head > 0 || geom.tail_begin < p.vocab)) {
        // those elements count as one more (short) vector, numbered after the whole ones
        float ends_max = __int_as_float(0xff800000);
        for (int64_t j = 0; j < geom.head; ++j) ends_max = fmax_nan(ends_max, to_float(src[j]));
        for (int64_t j = geom.tail_begin; j < p.vocab; ++j)
          ends_max = fmax_nan(ends_max, to_float(src[j]));
        note((lane == 0 && !(ends_max < thr_val)) ? 1u : 0u, geom.bulk_bytes >> 4, ends_max);
      }

      if (reduce_pass) {
        online_warp_reduce(st, p.c);
        float2* slot = part + (red_it & 1u) * K1_CONSUMER_WARPS;
        if (lane == 0) slot[warp] = make_float2(st.m, st.s);
        named_bar_sync(1, K1_CONSUMERS);
        if (warp == 0 || MODE == K1_FULL) {
          float2 ms = (lane < K1_CONSUMER_WARPS) ? slot[lane] : make_float2(-FLT_MAX, 0.0f);
          float m = ms.x;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
          float s = ms.y * ex2f((ms.x - m) * p.c);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
          bool writes_row = true;
          if (SPLIT && w.shared) {
            // the quarters meet in the cluster's first CTA; slot and barrier of this shared row
            // are used this once
            float2* pairs = reinterpret_cast<float2*>(smem + Smem::SPLIT_OFF) + split_it * K1_SPLIT;
            const uint32_t bar = smem_base + Smem::SPLIT_BAR_OFF + split_it * 8;
            if (crank != 0) {
              if (lane == 0) {
                st_cluster_f32x2(mapa_shared(smem_u32(&pairs[crank]), 0), m, s);
                mbar_arrive_cluster(mapa_shared(bar, 0));
              }
              writes_row = false;
            } else {
              if (!mbar_wait_cluster(bar, 0)) {
                raise_status(p.status, TOME_DEV_TIMEOUT);
                s = __int_as_float(0x7fc00000);
              }
              const float2 o = (lane >= 1 && lane < K1_SPLIT) ? pairs[lane]
                               : (lane == 0)                  ? make_float2(m, s)
                                                              : make_float2(-FLT_MAX, 0.0f);
              Online all = {o.x, o.y};
              online_warp_reduce(all, p.c);
              m = all.m;
              s = all.s;
            }
          }
          // the true maximum contributes 2^0, so a healthy row has s >= ~1
          // (a part of a row keeps its pair as it is: the kernel that merges the parts leaves a row
          // with an unhealthy sum to the row kernel)
          const bool in_parts = (MODE == K1_SAMPLE) && p.sample_parts_log2 != 0;
          if (writes_row && !in_parts && !(s >= 0.5f && s <= FLT_MAX))
            exact_row(src, p.vocab, p.c, lane, m, s);
          if (MODE == K1_FULL) lse_row = finish_lse<MODE>(m, s, p);
          if (MODE == K1_SAMPLE && ctid == 0) {
            if (in_parts) p.part_ms[item] = make_float2(m, s);
            else p.out1[row] = finish_lse<MODE>(m, s, p);
          }
          if (MODE != K1_SAMPLE && ctid == 0 && writes_row)
            emit_row<MODE>(p, oidx, sub, m, s, x_t, target_ok, carry);
        }
        if (SPLIT && w.shared) ++split_it;
        if (MODE == K1_SAMPLE) {
          // each warp copies its own list out; nothing here waits for another warp.  Entries
          // that the final threshold has left behind (most: the threshold rose while the row
          // passed) stay here, which shortens what the finishing step has to read.
          const int32_t keep = min(wcount, min(K1_SAMPLE_WARP_LIST, p.cand_cap));
          const int64_t base = (item * K1_CONSUMER_WARPS + warp) * p.cand_cap;
          int32_t alive = 0;
          for (int32_t i0 = 0; i0 < keep; i0 += 32) {
            const int32_t i = i0 + lane;
            const uint2 e = (i < keep) ? smp.entry[warp][i] : make_uint2(0u, 0u);
            const bool stays = (i < keep) && !(__uint_as_float(e.y) < thr_val);  // a NaN stays
            const uint32_t bal = __ballot_sync(0xffffffffu, stays);
            if (stays) p.cand_entry[base + alive + __popc(bal & ((1u << lane) - 1u))] = e;
            alive += __popc(bal);
          }
          if (lane == 0)  // more than kept: overflow
            p.cand_count[item * K1_CONSUMER_WARPS + warp] = (wcount > keep) ? p.cand_cap + 1 : alive;
          if (ctid == 0) p.row_thr[item] = thr_val;
          // FINISH: hand the row to the producer warp, which finishes it between its copies: the
          // list (and, in warp 0, the threshold and the lse) is written before the count moves
          if (FINISH) __threadfence_block();
          __syncwarp();  // also: the list is reused by the next row
          if (FINISH && lane == 0) atomicAdd(&smp.lists_done, 1);
        }
        ++red_it;
      }
    }
  }
  (void)PER_VEC;
  if (SPLIT) {  // nobody leaves while a peer may still address its shared memory
    __syncwarp();
    cluster_sync_all();
  }
}

// ------------------------------------------------------------------ plain-load kernel
// Same arithmetic with ordinary loads; any alignment, any pitch.  One CTA per row at a time;
// each row is read with 128-bit loads from its first 16-byte boundary on.
constexpr int K1_PLAIN_THREADS = 256;

template <typename T, int MODE>
__global__ void __launch_bounds__(K1_PLAIN_THREADS) k1_plain_kernel(const K1Params p) {
  __shared__ float2 part[K1_PLAIN_THREADS / 32];
  __shared__ float2 result;
  constexpr bool WINDOWED = k1_windowed(MODE);
  __shared__ int32_t cum[WINDOWED ? (K1_MAX_SEQ + 1) : 1];
  __shared__ int32_t scratch[WINDOWED ? K1_PLAIN_THREADS : 1];
  constexpr int NSUB = (MODE == K1_DUAL) ? 2 : 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  int64_t n_items = p.n_rows;
  if (WINDOWED) {
    n_items = dual_build_prefix(p, cum, scratch);
    if (MODE == K1_DUAL) dual_zero_masked(p);
    if (MODE == K1_RAGGED && blockIdx.x == 0 && p.out_offsets != nullptr)
      for (int i = threadIdx.x; i <= p.n_seq; i += blockDim.x) p.out_offsets[i] = cum[i];
    if (MODE == K1_RAGGED && n_items > p.packed_capacity) {
      if (threadIdx.x == 0) raise_status(p.status, TOME_DEV_RAGGED_OVERFLOW);
      n_items = p.packed_capacity;
    }
    __syncthreads();
  }
  float carry = 0.0f;
  for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int64_t row = WINDOWED ? dual_row_of_item(p, cum, item) : item;
    const int64_t oidx = (MODE == K1_RAGGED) ? item : row;
    for (int sub = 0; sub < NSUB; ++sub) {
      const T* src = reinterpret_cast<const T*>(p.src[(MODE == K1_DUAL) ? sub : 0]) +
                     row * p.stride;
      // a row may start anywhere: scalar loads up to the first 16-byte boundary, 128-bit
      // loads for the aligned body (packed fast path), scalar loads for what is left
      constexpr int64_t PER = 16 / static_cast<int64_t>(sizeof(T));
      const uintptr_t addr = reinterpret_cast<uintptr_t>(src);
      const int64_t head = min(p.vocab, static_cast<int64_t>(((16 - (addr & 15)) & 15) / sizeof(T)));
      const int64_t nvec = (p.vocab - head) / PER;
      const int64_t tail_begin = head + nvec * PER;
      const uint4* body = reinterpret_cast<const uint4*>(src + head);
      Fast fs;
      fast_init(fs, p.c);
#pragma unroll 4
      for (int64_t v = threadIdx.x; v < nvec; v += K1_PLAIN_THREADS)
        fast_update<0>(fs, __ldg(body + v), p.c, T());
      Online st = fast_finish(fs, p.c);
      for (int64_t j = threadIdx.x; j < head; j += K1_PLAIN_THREADS)
        online_update_scalar(st, to_float(src[j]), p.c);
      for (int64_t j = tail_begin + threadIdx.x; j < p.vocab; j += K1_PLAIN_THREADS)
        online_update_scalar(st, to_float(src[j]), p.c);
      online_warp_reduce(st, p.c);
      if (lane == 0) part[warp] = make_float2(st.m, st.s);
      __syncthreads();
      if (warp == 0) {
        float2 ms = (lane < K1_PLAIN_THREADS / 32) ? part[lane] : make_float2(-FLT_MAX, 0.0f);
        float m = ms.x;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float s = ms.y * ex2f((ms.x - m) * p.c);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        // the true maximum contributes 2^0, so a healthy row has s >= ~1 (see online.cuh)
        if (!(s >= 0.5f && s <= FLT_MAX)) exact_row(src, p.vocab, p.c, lane, m, s);
        if (lane == 0) {
          float x_t = 0.0f;
          bool target_ok = true;
          if (MODE != K1_FULL) {
            const int32_t t = p.targets[oidx];
            target_ok = (t >= 0) && (static_cast<int64_t>(t) < p.vocab);
            if (target_ok) x_t = to_float(src[t]);
            else raise_status(p.status, TOME_DEV_TARGET_OUT_OF_RANGE);
          }
          emit_row<MODE>(p, oidx, sub, m, s, x_t, target_ok, carry);
          result = make_float2(m, s);
        }
      }
      __syncthreads();
      if (MODE == K1_FULL) {
        const float lse = finish_lse<MODE>(result.x, result.y, p);
        T* dst = reinterpret_cast<T*>(p.out_full) + row * p.out_stride;
        // second pass (the row was just read: it comes from L2).  Where the output row sits
        // on the 16-byte grid like the input row, the aligned body is written with 128-bit
        // stores and only the ends element by element.
        if ((reinterpret_cast<uintptr_t>(dst + head) & 15) == 0) {
          uint4* out = reinterpret_cast<uint4*>(dst + head);
#pragma unroll 4
          for (int64_t v = threadIdx.x; v < nvec; v += K1_PLAIN_THREADS)
            out[v] = full_out_vec(__ldg(body + v), p.inv_temp, lse, T());
          for (int64_t j = threadIdx.x; j < head; j += K1_PLAIN_THREADS)
            dst[j] = full_out_scalar(src[j], p.inv_temp, lse);
          for (int64_t j = tail_begin + threadIdx.x; j < p.vocab; j += K1_PLAIN_THREADS)
            dst[j] = full_out_scalar(src[j], p.inv_temp, lse);
        } else {
          for (int64_t j = threadIdx.x; j < p.vocab; j += K1_PLAIN_THREADS)
            dst[j] = full_out_scalar(src[j], p.inv_temp, lse);
        }
        __syncthreads();
      }
    }
  }
}

// ------------------------------------------------------------------ host side
// Tuning knob TOME_K1_POLY = 0 .. 4: how many of the 8 logits of a bf16 vector take the
// polynomial exp2 (FMA pipe) instead of ex2.approx (exp unit).  Read once per process.
static int k1_poly_setting() {
  static const int value = [] {
    const char* e = getenv("TOME_K1_POLY");
    const int v = (e != nullptr) ? atoi(e) : K1_POLY_DEFAULT;
    return v < 0 ? 0 : (v > 4 ? 4 : v);
  }();
  return value;
}

template <typename T, int MODE>
static void (*pick_stream_kernel())(K1Params) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value && MODE != K1_FULL) {
    const int poly = k1_poly_setting();
    if (poly == 1) return k1_stream_kernel<T, MODE, 1>;
    if (poly == 2) return k1_stream_kernel<T, MODE, 2>;
    if (poly == 3) return k1_stream_kernel<T, MODE, 3>;
    if (poly == 4) return k1_stream_kernel<T, MODE, 4>;
  }
  return k1_stream_kernel<T, MODE, 0>;
}

// Selective mode with the rows of the last, partial round shared by clusters of K1_SPLIT CTAs.
// Taken when that round is thin: at most one shared row per cluster after at least one whole
// round, with fewer than 8 rows per CTA in all.  Then the few CTAs of the last round cannot
// fill the memory system on their own (600 bf16 rows: 44.7 -> 38.3 us).  A fuller last round
// keeps HBM busy as it is and sharing its rows gains nothing (1024 fp32 rows: 104.1 us plain,
// 105.7 shared; 300 rows, all shared: 37.0 -> 41.1), so those stay with the plain launch.
// Further conditions: a row has a chunk for every CTA of a cluster and the exponential variant
// is the default one.  TOME_K1_TAIL=0 switches the sharing off, 2 takes it whenever the row
// count allows (read at every call; tests).
template <typename T>
static int32_t k1_launch_split_tail(const K1Params& p, const DeviceInfo& info, cudaStream_t stream,
                                    bool* taken) {
  *taken = false;
  constexpr bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr int POLY = bf16 ? K1_POLY_DEFAULT : 0;
  if (bf16 && k1_poly_setting() != K1_POLY_DEFAULT) return TOME_OK;
  if (p.n_chunks < K1_SPLIT) return TOME_OK;
  const char* e = getenv("TOME_K1_TAIL");
  const int knob = (e != nullptr) ? atoi(e) : 1;
  if (knob == 0) return TOME_OK;
  using Smem = K1SmemT<K1_STAGES>;
  constexpr int smem = Smem::TOTAL_SPLIT;
  void (*kernel)(K1Params) = k1_stream_kernel<T, K1_SELECTIVE, POLY, true>;
  int32_t st = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
  if (st != TOME_OK) return st;
  const int fit = max_active_clusters(reinterpret_cast<const void*>(kernel), K1_THREADS, smem, K1_SPLIT);
  if (fit <= 0) return TOME_OK;
  const int64_t grid_full = static_cast<int64_t>(fit) * K1_SPLIT;
  const int64_t last_round = p.n_rows % grid_full;
  if (last_round == 0) return TOME_OK;
  if (knob != 2 && (p.n_rows < grid_full || p.n_rows >= 8 * grid_full || last_round > fit))
    return TOME_OK;
  // fewer rows than CTAs: every row is shared, by as many clusters as there are rows at most
  const int64_t n_clusters = (p.n_rows >= grid_full) ? fit : std::min<int64_t>(fit, p.n_rows);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(n_clusters * K1_SPLIT), 1, 1);
  cfg.blockDim = dim3(K1_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = K1_SPLIT;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  *taken = true;
  return check_cuda(cudaLaunchKernelEx(&cfg, kernel, p), "k1 split-tail launch");
}

template <typename T, int MODE>
static int32_t k1_launch_typed(const K1Params& p_in, bool bulk_ok, int64_t max_items,
                               cudaStream_t stream) {
  DeviceInfo info;
  int32_t st = current_device_info(&info);
  if (st != TOME_OK) return st;
  constexpr int32_t dtype = std::is_same<T, float>::value ? TOME_F32 : TOME_BF16;
  if constexpr (MODE == K1_SELECTIVE || MODE == K1_FULL) {
    // few rows: a cluster of CTAs shares each row (k1_small.cu)
    bool taken = false;
    st = k1_small_batch_launch(p_in, dtype, MODE, stream, &taken);
    if (taken || st != TOME_OK) return st;
  }
  if constexpr (MODE == K1_FULL) {
    // rows of more than ~100 KB: a cluster of CTAs shares each row (k1_full.cu)
    bool taken = false;
    st = k1_full_cluster_launch(p_in, dtype, bulk_ok, info.sm_count, stream, &taken);
    if (taken || st != TOME_OK) return st;
  }
  if (bulk_ok) {
    // equal-sized bulk copies: a row is cut into the fewest chunks that fit a stage
    K1Params p = p_in;
    constexpr int64_t es = sizeof(T);
    const int64_t bulk_bytes = (p.vocab * es) & ~static_cast<int64_t>(15);
    const int64_t n = (bulk_bytes + K1_CHUNK_BYTES - 1) / K1_CHUNK_BYTES;
    p.n_chunks = static_cast<int32_t>(n);
    const int64_t al = K1_CHUNK_ALIGN;
    p.chunk_bytes = (n > 0) ? static_cast<int32_t>(((bulk_bytes + n - 1) / n + al - 1) / al * al)
                            : K1_CHUNK_ALIGN;
    using Smem = K1SmemT<k1_stages(MODE)>;
    const int smem = k1_windowed(MODE) ? Smem::TOTAL_DUAL
                     : (MODE == K1_SAMPLE)
                         ? Smem::SAMPLE_OFF + static_cast<int>(sizeof(K1SampleSmem))
                         : Smem::TOTAL_PLAIN;
    if (smem > info.max_smem_optin)
      return fail(TOME_ERR_UNSUPPORTED, "device offers %d bytes of shared memory, need %d",
                  info.max_smem_optin, smem);
    if constexpr (MODE == K1_SELECTIVE) {
      // few rows per CTA: the last round's rows are shared by clusters (see K1_SPLIT)
      bool taken = false;
      st = k1_launch_split_tail<T>(p, info, stream, &taken);
      if (taken || st != TOME_OK) return st;
    }
    void (*kernel)(K1Params) = pick_stream_kernel<T, MODE>();
    if constexpr (MODE == K1_SAMPLE) {
      // the form whose producer warp also finishes the rows (default exponential variant only)
      constexpr int POLY = std::is_same<T, __nv_bfloat16>::value ? K1_POLY_DEFAULT : 0;
      if (p.finish_in_kernel) kernel = k1_stream_kernel<T, K1_SAMPLE, POLY, false, true>;
    }
    st = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
    if (st != TOME_OK) return st;
    int64_t ctas_per_sm = K1_CTAS_PER_SM;
    if (MODE == K1_FULL) {
      // the second pass over a row should find it in L2: keep the rows in flight (one per CTA)
      // under ~100 MB, but never fewer than two CTAs per SM (measured: 4.2 -> 4.9 TB/s on bf16)
      const int64_t row_bytes = std::max<int64_t>(1, p.vocab * es);
      const int64_t fit = std::max<int64_t>(1, info.max_smem_optin / (smem + 1024));
      ctas_per_sm = std::min<int64_t>(fit, std::max<int64_t>(
          2, std::min<int64_t>(K1_CTAS_PER_SM, (100ll << 20) / (row_bytes * info.sm_count))));
    }
    const int grid = static_cast<int>(
        std::max<int64_t>(1, std::min<int64_t>(info.sm_count * ctas_per_sm, max_items)));
    kernel<<<grid, K1_THREADS, smem, stream>>>(p);
  } else {
    const int grid = static_cast<int>(std::max<int64_t>(
        1, std::min<int64_t>(static_cast<int64_t>(info.sm_count) * 8, max_items)));
    k1_plain_kernel<T, MODE><<<grid, K1_PLAIN_THREADS, 0, stream>>>(p_in);
  }
  return check_cuda(cudaGetLastError(), "k1 launch");
}

template <int MODE>
static int32_t k1_launch(const K1Params& p, int32_t dtype, bool bulk_ok, int64_t max_items,
                         cudaStream_t stream) {
  if (dtype == TOME_F32) return k1_launch_typed<float, MODE>(p, bulk_ok, max_items, stream);
  return k1_launch_typed<__nv_bfloat16, MODE>(p, bulk_ok, max_items, stream);
}

static int32_t k1_check_common(const void* logits, int32_t dtype, int64_t rows, int64_t vocab,
                               int64_t row_stride, float temperature) {
  if (dtype != TOME_F32 && dtype != TOME_BF16)
    return fail(TOME_ERR_BAD_DTYPE, "dtype %d is neither TOME_F32 nor TOME_BF16", dtype);
  if (rows < 0 || vocab <= 0)
    return fail(TOME_ERR_BAD_SHAPE, "rows=%lld vocab=%lld", (long long)rows, (long long)vocab);
  if (vocab > 0x7fffffffLL)
    return fail(TOME_ERR_BAD_SHAPE, "vocab=%lld does not fit int32 targets", (long long)vocab);
  if (row_stride < vocab)
    return fail(TOME_ERR_BAD_STRIDE, "row_stride=%lld < vocab=%lld", (long long)row_stride,
                (long long)vocab);
  if (!temperature_ok(temperature))
    return fail(TOME_ERR_BAD_TEMPERATURE, "temperature=%g must be > 0 and finite", temperature);
  if (rows > 0 && logits == nullptr) return fail(TOME_ERR_NULL_POINTER, "logits is NULL");
  const size_t es = (dtype == TOME_F32) ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(logits) % es) != 0)
    return fail(TOME_ERR_MISALIGNED, "logits is not aligned to its element size");
  return TOME_OK;
}

// The reading modes take the bulk-copy pipeline for any element-aligned rows (each row is copied
// from its first 16-byte boundary, see row_geom.cuh).  TOME_K1_BULK=0 sends them to the
// plain-load kernel instead (read at every call; tests).
static bool bulk_wanted() {
  const char* e = getenv("TOME_K1_BULK");
  return e == nullptr || atoi(e) != 0;
}

}  // namespace tome

using namespace tome;

extern "C" int32_t tome_selective_logprob(const void* logits, int32_t dtype, int64_t rows,
                                          int64_t vocab, int64_t row_stride,
                                          const int32_t* targets, float temperature,
                                          float* out_logprob, float* out_lse,
                                          float* out_target_raw, int32_t* dev_status,
                                          void* stream) {
  int32_t st = k1_check_common(logits, dtype, rows, vocab, row_stride, temperature);
  if (st != TOME_OK) return st;
  if (rows == 0) return TOME_OK;
  if (targets == nullptr || out_logprob == nullptr)
    return fail(TOME_ERR_NULL_POINTER, "targets or out_logprob is NULL");
  K1Params p = {};
  p.src[0] = logits;
  p.n_rows = rows;
  p.vocab = vocab;
  p.stride = row_stride;
  p.targets = targets;
  p.c = LOG2E / temperature;
  p.temp = temperature;
  p.inv_temp = 1.0f / temperature;
  p.out0 = out_logprob;
  p.out1 = out_lse;
  p.out2 = out_target_raw;
  p.status = dev_status;
  return k1_launch<K1_SELECTIVE>(p, dtype, bulk_wanted(), rows,
                                 static_cast<cudaStream_t>(stream));
}

extern "C" int32_t tome_log_softmax_full(const void* logits, int32_t dtype, int64_t rows,
                                         int64_t vocab, int64_t row_stride, float temperature,
                                         void* out, int64_t out_row_stride, float* out_lse,
                                         int32_t* dev_status, void* stream) {
  int32_t st = k1_check_common(logits, dtype, rows, vocab, row_stride, temperature);
  if (st != TOME_OK) return st;
  if (out_row_stride < vocab)
    return fail(TOME_ERR_BAD_STRIDE, "out_row_stride=%lld < vocab=%lld",
                (long long)out_row_stride, (long long)vocab);
  if (rows == 0) return TOME_OK;
  if (out == nullptr) return fail(TOME_ERR_NULL_POINTER, "out is NULL");
  const size_t es = (dtype == TOME_F32) ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(out) % es) != 0)
    return fail(TOME_ERR_MISALIGNED, "out is not aligned to its element size");
  K1Params p = {};
  p.src[0] = logits;
  p.n_rows = rows;
  p.vocab = vocab;
  p.stride = row_stride;
  p.c = LOG2E / temperature;
  p.temp = temperature;
  p.inv_temp = 1.0f / temperature;
  p.out0 = out_lse;
  p.out_full = out;
  p.out_stride = out_row_stride;
  p.status = dev_status;
  // the 128-bit stores of the bulk-copy kernels need every output row to sit on the 16-byte
  // grid like its input row (e.g. two contiguous tensors of any row length)
  const uintptr_t apart = reinterpret_cast<uintptr_t>(out) - reinterpret_cast<uintptr_t>(logits);
  const bool alike =
      (apart % 16 == 0) && (((out_row_stride - row_stride) * static_cast<int64_t>(es)) % 16 == 0);
  return k1_launch<K1_FULL>(p, dtype, alike && bulk_wanted(), rows,
                            static_cast<cudaStream_t>(stream));
}

extern "C" int32_t tome_dual_logprob_kl(const void* policy_logits, const void* ref_logits,
                                        int32_t dtype, int64_t n_seq, int64_t seq_len,
                                        int64_t vocab, int64_t row_stride,
                                        const int32_t* targets, const int32_t* lengths,
                                        const int32_t* starts, float temperature,
                                        float* out_lp_policy, float* out_lp_ref, float* out_kl,
                                        int32_t* dev_status, void* stream) {
  if (n_seq < 0 || seq_len < 0)
    return fail(TOME_ERR_BAD_SHAPE, "n_seq=%lld seq_len=%lld", (long long)n_seq,
                (long long)seq_len);
  if (n_seq > K1_MAX_SEQ)
    return fail(TOME_ERR_TOO_LARGE, "n_seq=%lld exceeds the limit of %d sequences per call",
                (long long)n_seq, K1_MAX_SEQ);
  if (seq_len > 0x7fffffffLL / (n_seq > 0 ? n_seq : 1))
    return fail(TOME_ERR_TOO_LARGE, "n_seq * seq_len does not fit int32");
  const int64_t rows = n_seq * seq_len;
  int32_t st = k1_check_common(policy_logits, dtype, rows, vocab, row_stride, temperature);
  if (st != TOME_OK) return st;
  if (rows == 0) return TOME_OK;
  if (ref_logits == nullptr || targets == nullptr || lengths == nullptr ||
      out_lp_policy == nullptr || out_lp_ref == nullptr || out_kl == nullptr)
    return fail(TOME_ERR_NULL_POINTER, "a required pointer is NULL");
  const size_t es = (dtype == TOME_F32) ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(ref_logits) % es) != 0)
    return fail(TOME_ERR_MISALIGNED, "ref_logits is not aligned to its element size");
  K1Params p = {};
  p.src[0] = policy_logits;
  p.src[1] = ref_logits;
  p.n_rows = rows;
  p.vocab = vocab;
  p.stride = row_stride;
  p.targets = targets;
  p.c = LOG2E / temperature;
  p.temp = temperature;
  p.inv_temp = 1.0f / temperature;
  p.out0 = out_lp_policy;
  p.out1 = out_lp_ref;
  p.out2 = out_kl;
  p.lengths = lengths;
  p.starts = starts;
  p.n_seq = static_cast<int32_t>(n_seq);
  p.seq_len = static_cast<int32_t>(seq_len);
  p.status = dev_status;
  const bool bulk = bulk_wanted();
  return k1_launch<K1_DUAL>(p, dtype, bulk, rows, static_cast<cudaStream_t>(stream));
}

extern "C" int32_t tome_ragged_logprob(const void* logits, int32_t dtype, int64_t n_seq,
                                       int64_t seq_len, int64_t vocab, int64_t row_stride,
                                       const int32_t* targets_packed, int64_t packed_capacity,
                                       const int32_t* lengths, const int32_t* starts,
                                       float temperature,
                                       float* out_logprob_packed, float* out_lse_packed,
                                       int32_t* out_offsets, int32_t* dev_status, void* stream) {
  if (n_seq < 0 || seq_len < 0)
    return fail(TOME_ERR_BAD_SHAPE, "n_seq=%lld seq_len=%lld", (long long)n_seq,
                (long long)seq_len);
  if (n_seq > K1_MAX_SEQ)
    return fail(TOME_ERR_TOO_LARGE, "n_seq=%lld exceeds the limit of %d sequences per call",
                (long long)n_seq, K1_MAX_SEQ);
  if (seq_len > 0x7fffffffLL / (n_seq > 0 ? n_seq : 1))
    return fail(TOME_ERR_TOO_LARGE, "n_seq * seq_len does not fit int32");
  const int64_t rows = n_seq * seq_len;
  int32_t st = k1_check_common(logits, dtype, rows, vocab, row_stride, temperature);
  if (st != TOME_OK) return st;
  if (packed_capacity < 0)
    return fail(TOME_ERR_BAD_SHAPE, "packed_capacity=%lld", (long long)packed_capacity);
  if (rows == 0) return TOME_OK;
  if (lengths == nullptr ||
      (packed_capacity > 0 && (targets_packed == nullptr || out_logprob_packed == nullptr)))
    return fail(TOME_ERR_NULL_POINTER, "a required pointer is NULL");
  K1Params p = {};
  p.src[0] = logits;
  p.n_rows = rows;
  p.vocab = vocab;
  p.stride = row_stride;
  p.targets = targets_packed;
  p.c = LOG2E / temperature;
  p.temp = temperature;
  p.inv_temp = 1.0f / temperature;
  p.out0 = out_logprob_packed;
  p.out1 = out_lse_packed;
  p.lengths = lengths;
  p.starts = starts;
  p.n_seq = static_cast<int32_t>(n_seq);
  p.seq_len = static_cast<int32_t>(seq_len);
  p.out_offsets = out_offsets;
  p.packed_capacity = packed_capacity;
  p.status = dev_status;
  return k1_launch<K1_RAGGED>(p, dtype, bulk_wanted(), rows,
                              static_cast<cudaStream_t>(stream));
}

namespace tome {

bool k1_sample_eligible(const void* logits, int32_t dtype, int64_t vocab, int64_t row_stride) {
  const int64_t es = (dtype == TOME_F32) ? 4 : 2;
  // (any element-aligned rows) a row holds 16-byte vectors, few enough for the entries' 28
  // index bits
  (void)logits;
  (void)row_stride;
  return vocab * es >= 32 && vocab * es / 16 < (int64_t{1} << 27);
}

int32_t k1_launch_sample(const void* logits, int32_t dtype, int64_t rows, int64_t vocab,
                         int64_t row_stride, const K1SampleArgs& a, int32_t* dev_status,
                         cudaStream_t stream) {
  K1Params p = {};
  p.src[0] = logits;
  p.n_rows = rows;
  p.vocab = vocab;
  p.stride = row_stride;
  const float temp = (a.temperature > 0.0f) ? a.temperature : 1.0f;  // greedy: scored at 1
  p.c = LOG2E / temp;
  p.temp = temp;
  p.inv_temp = 1.0f / temp;
  p.finish_in_kernel = a.finish_in_kernel ? 1 : 0;
  if ((a.parts != 1 && a.parts != 2 && a.parts != 4) ||
      a.parts > k1_sample_max_parts(vocab, dtype) ||
      (a.parts > 1 && (a.finish_in_kernel || a.part_ms == nullptr)))
    return fail(TOME_ERR_UNSUPPORTED, "sampling pass: %d parts per row", a.parts);
  p.sample_parts_log2 = (a.parts == 4) ? 2 : (a.parts == 2) ? 1 : 0;
  p.part_ms = a.part_ms;
  p.out0 = a.out_logprob;
  p.out1 = a.lse;
  p.row_thr = a.row_thr;
  p.cand_count = a.cand_count;
  p.cand_entry = a.cand_entry;
  p.cand_cap = K1_SAMPLE_WARP_LIST;
  const int64_t kk = std::max<int64_t>(1, std::min<int64_t>(a.top_k, vocab));
  p.sample_kk = static_cast<int32_t>(kk);
  p.sample_q = static_cast<int32_t>((kk + K1_CONSUMER_WARPS - 1) / K1_CONSUMER_WARPS);
  p.sample_top_k = a.top_k;
  p.sample_temperature = a.temperature;
  p.sample_seed = a.seed;
  p.sample_offset = a.offset;
  p.out_tokens = a.out_tokens;
  p.out_topk_idx = a.out_topk_idx;
  p.out_topk_val = a.out_topk_val;
  p.marked = a.marked;
  p.marked_rows = a.marked_rows;
  p.status = dev_status;
  return k1_launch<K1_SAMPLE>(p, dtype, true, rows * a.parts, stream);
}

int k1_sample_max_parts(int64_t vocab, int32_t dtype) {
  const int64_t es = (dtype == TOME_F32) ? 4 : 2;
  const int64_t bulk_bytes = (vocab * es) & ~static_cast<int64_t>(15);
  const int64_t chunks = (bulk_bytes + K1_CHUNK_BYTES - 1) / K1_CHUNK_BYTES;  // as k1_launch_typed
  return chunks >= 4 ? 4 : chunks >= 2 ? 2 : 1;
}

int k1_sample_lists_per_row() { return K1_CONSUMER_WARPS; }
int k1_sample_list_capacity() { return K1_SAMPLE_WARP_LIST; }
int k1_sample_vector_stride() { return K1_CONSUMERS; }

}  // namespace tome
