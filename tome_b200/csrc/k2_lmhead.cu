// K2: fused LM head + selective log-prob on the 5th-generation tensor cores (tensor-bound).
//
// logits = hidden[rows, K] @ weight[V, K]^T are produced 128 x 256 tiles at a time by
// tcgen05.mma (bf16 in, fp32 accumulate in TMEM) and consumed straight out of TMEM by the
// epilogue warps, which keep a running (max, sum-exp, target-logit) per row in registers.
// No logits are ever written to memory.  Replaces "x @ embed_tokens.weight.T"
// (mlx-impl/model.py:538) followed by local_compute_logprobs (mlx-impl/node.py:400-404).
//
// Structure of one persistent CTA (192 threads, one per SM):
//   warp 0      producer: 2-D tiled TMA loads of the hidden tile (128 x 64) and the weight
//               tile (256 x 64) into a ring of 128B-swizzled shared-memory stages
//   warp 1      one thread issues tcgen05.mma into one of two 256-column TMEM accumulators
//   warps 2-5   epilogue: thread i owns row i of the tile (tcgen05.ld 32x32b), reduces the
//               256 columns into its running triple while the next tile is being multiplied
//
// Work decomposition.  The vocabulary is cut into bands of NB column tiles.  A work item is
// (row tile, band): the CTA sweeps the band's column tiles with the running triple in
// registers and writes one partial triple per row to the workspace; a merge kernel folds
// the bands.  Items are ordered so that the CTAs running at the same time share a small set
// of hidden tiles (GM row tiles, sized to stay in L2) and stream the same few weight bands,
// so the weight matrix is read from HBM about once per GM row tiles.
#include <cuda.h>
#include <cuda_bf16.h>
#include <float.h>
#include <stdint.h>
#include <stdlib.h>

#include <algorithm>
#include <mutex>

#include "combine.h"
#include "host_common.h"
#include "ptx.cuh"

namespace tome {

constexpr int K2_BM = 128;   // rows of the tile held by one CTA (TMEM lanes)
constexpr int K2_BN = 256;   // columns of a tile
constexpr int K2_BK = 64;    // 64 bf16 = 128 bytes = one swizzle row
constexpr int K2_A_BYTES = K2_BM * K2_BK * 2;
constexpr int K2_THREADS = 192;
constexpr int K2_EPI_WARPS = 4;
constexpr int K2_TMEM_COLS = 512;

// PAIR = false: one CTA computes a 128 x 256 tile (tcgen05 cta_group::1).
// PAIR = true : a cluster of two CTAs computes a 256 x 256 tile (cta_group::2); each CTA
//               loads its own 128 hidden rows and HALF of the weight rows of the tile, the
//               leader CTA issues the MMAs for both, and each CTA reduces the 128 rows that
//               land in its own TMEM.  Per CTA that is one third less shared-memory fill
//               per FLOP, so six stages fit where the single-CTA form has four.
template <bool PAIR>
struct K2Cfg {
  static constexpr int B_ROWS = PAIR ? 128 : 256;  // weight rows this CTA loads per tile
  static constexpr int B_BYTES = B_ROWS * K2_BK * 2;
  static constexpr int STAGE_BYTES = K2_A_BYTES + B_BYTES;
  static constexpr int STAGES = PAIR ? 6 : 4;
  static constexpr int ITEM_ROWS = PAIR ? 256 : 128;  // rows of a work item's row tile
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256;
};

struct K2Params {
  int64_t rows;
  int64_t k_dim;
  int64_t vocab_local;
  int64_t vocab_offset;
  int64_t vocab_check;     // > 0: targets must lie in [0, vocab_check)
  const int32_t* targets;
  float c;                 // log2(e) / temperature
  float temp;
  float* part_m;           // [n_bands][rows]
  float* part_s;
  float* part_t;
  int32_t m_tiles;         // row tiles of ITEM_ROWS rows
  int32_t n_tiles, k_blocks;
  int32_t nb;              // column tiles per band
  int32_t n_bands;
  int32_t gm;              // row tiles per group
  int64_t n_items;
  int32_t round_bf16;      // round every logit to bf16 before the reduction
  int32_t* status;
};

struct K2Item {
  int32_t mt;     // row tile
  int32_t band;
  int32_t n_begin, n_end;  // column tiles
};

// Item order: row-tile groups outermost, then bands, then the row tiles of the group.
__device__ __forceinline__ K2Item k2_decode(const K2Params& p, int64_t i) {
  const int32_t full_groups = p.m_tiles / p.gm;
  const int64_t per_group = static_cast<int64_t>(p.n_bands) * p.gm;
  int32_t g, gm_here;
  int64_t r;
  if (i < full_groups * per_group) {
    g = static_cast<int32_t>(i / per_group);
    r = i - g * per_group;
    gm_here = p.gm;
  } else {
    g = full_groups;
    r = i - full_groups * per_group;
    gm_here = p.m_tiles - full_groups * p.gm;
  }
  K2Item it;
  it.band = static_cast<int32_t>(r / gm_here);
  it.mt = g * p.gm + static_cast<int32_t>(r - static_cast<int64_t>(it.band) * gm_here);
  it.n_begin = it.band * p.nb;
  it.n_end = min(p.n_tiles, it.n_begin + p.nb);
  return it;
}

// K-major, 128B-swizzled operand tile whose rows are 128 bytes: 8-row groups are 1024 bytes
// apart (stride byte offset), the leading byte offset is unused (1), descriptor version 1.
__device__ __forceinline__ uint64_t k2_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// kind::f16 instruction descriptor: fp32 accumulator, bf16 A and B, both K-major.
__host__ __device__ constexpr uint32_t k2_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void k2_raise(int32_t* status, int32_t bit) {
  if (status != nullptr) atomicOr(status, bit);
}

template <bool PAIR>
__global__ void __launch_bounds__(K2_THREADS, 1)
k2_lmhead_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b, const K2Params p) {
  using Cfg = K2Cfg<PAIR>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int STAGE_BYTES = Cfg::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // swizzled tiles want 1024-byte alignment
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t bars = base + STAGES * STAGE_BYTES;
  const uint32_t full_bar = bars;
  const uint32_t empty_bar = bars + STAGES * 8;
  const uint32_t tfull_bar = bars + 2 * STAGES * 8;
  const uint32_t tempty_bar = tfull_bar + 16;
  const uint32_t tmem_slot = tempty_bar + 16;
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem + STAGES * STAGE_BYTES + 2 * STAGES * 8 + 32);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // the identical smem layout in both CTAs of a pair makes every offset valid in the peer
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = (rank == 0u);
  const int64_t worker = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
  const int64_t n_workers = PAIR ? (gridDim.x >> 1) : gridDim.x;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(full_bar + i * 8, 1);
      mbar_init(empty_bar + i * 8, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull_bar + i * 8, 1);
      mbar_init(tempty_bar + i * 8, PAIR ? 2 * K2_EPI_WARPS : K2_EPI_WARPS);
    }
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(tmem_slot, K2_TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, K2_TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // data of both CTAs of a pair is counted on the LEADER's full barrier
      const uint32_t full_signal = PAIR ? mapa_shared(full_bar, 0) : full_bar;
      uint32_t it = 0;
      bool ok = true;
      for (int64_t i = worker; i < p.n_items && ok; i += n_workers) {
        const K2Item item = k2_decode(p, i);
        const int32_t row0 = item.mt * Cfg::ITEM_ROWS + static_cast<int32_t>(rank) * K2_BM;
        for (int32_t n = item.n_begin; n < item.n_end && ok; ++n) {
          const int32_t wrow0 = n * K2_BN + static_cast<int32_t>(rank) * Cfg::B_ROWS;
          for (int32_t kb = 0; kb < p.k_blocks; ++kb, ++it) {
            const uint32_t stage = it % STAGES;
            const uint32_t phase = (it / STAGES) & 1u;
            if (!mbar_wait(empty_bar + stage * 8, phase ^ 1u)) {
              k2_raise(p.status, TOME_DEV_TIMEOUT);
              ok = false;
              break;
            }
            const uint32_t sa = base + stage * STAGE_BYTES;
            if (PAIR) {
              if (leader) mbar_arrive_expect_tx(full_bar + stage * 8, 2 * STAGE_BYTES);
              tma_load_2d_pair(sa, &tmap_a, kb * K2_BK, row0, full_signal + stage * 8);
              tma_load_2d_pair(sa + K2_A_BYTES, &tmap_b, kb * K2_BK, wrow0,
                               full_signal + stage * 8);
            } else {
              mbar_arrive_expect_tx(full_bar + stage * 8, STAGE_BYTES);
              tma_load_2d(sa, &tmap_a, kb * K2_BK, row0, full_bar + stage * 8);
              tma_load_2d(sa + K2_A_BYTES, &tmap_b, kb * K2_BK, wrow0, full_bar + stage * 8);
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = k2_idesc(PAIR ? 256 : 128, K2_BN);
      // completion is signalled to the same barrier in both CTAs of a pair
      const uint32_t empty_own = PAIR ? mapa_shared(empty_bar, 0) : empty_bar;
      const uint32_t empty_peer = PAIR ? mapa_shared(empty_bar, 1) : 0u;
      const uint32_t tfull_own = PAIR ? mapa_shared(tfull_bar, 0) : tfull_bar;
      const uint32_t tfull_peer = PAIR ? mapa_shared(tfull_bar, 1) : 0u;
      uint32_t it = 0, tc = 0;
      bool ok = true;
      for (int64_t i = worker; i < p.n_items && ok; i += n_workers) {
        const K2Item item = k2_decode(p, i);
        for (int32_t n = item.n_begin; n < item.n_end && ok; ++n, ++tc) {
          const uint32_t acc = tc & 1u;
          const uint32_t aphase = (tc >> 1) & 1u;
          if (!mbar_wait(tempty_bar + acc * 8, aphase ^ 1u)) {
            k2_raise(p.status, TOME_DEV_TIMEOUT);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + acc * K2_BN;
          for (int32_t kb = 0; kb < p.k_blocks; ++kb, ++it) {
            const uint32_t stage = it % STAGES;
            const uint32_t phase = (it / STAGES) & 1u;
            if (!mbar_wait(full_bar + stage * 8, phase)) {
              k2_raise(p.status, TOME_DEV_TIMEOUT);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t sa = base + stage * STAGE_BYTES;
            const uint64_t da = k2_smem_desc(sa);
            const uint64_t db = k2_smem_desc(sa + K2_A_BYTES);
#pragma unroll
            for (int k = 0; k < K2_BK / 16; ++k) {
              // 16 bf16 = 32 bytes further along K inside the swizzle row: +2 in 16-byte units
              const uint32_t accumulate = (kb | k) != 0 ? 1u : 0u;
              if (PAIR)
                umma_bf16_ss_pair(d_tmem, da + static_cast<uint64_t>(k * 2),
                                  db + static_cast<uint64_t>(k * 2), idesc, accumulate);
              else
                umma_bf16_ss(d_tmem, da + static_cast<uint64_t>(k * 2),
                             db + static_cast<uint64_t>(k * 2), idesc, accumulate);
            }
            // frees the stage (in both CTAs) once these MMAs have read it
            if (PAIR) {
              umma_commit_pair(empty_own + stage * 8);
              umma_commit_pair(empty_peer + stage * 8);
            } else {
              umma_commit(empty_bar + stage * 8);
            }
          }
          if (ok) {  // accumulator complete
            if (PAIR) {
              umma_commit_pair(tfull_own + acc * 8);
              umma_commit_pair(tfull_peer + acc * 8);
            } else {
              umma_commit(tfull_bar + acc * 8);
            }
          }
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    // accumulators are handed back to the leader's MMA warp
    const uint32_t tempty_signal = PAIR ? mapa_shared(tempty_bar, 0) : tempty_bar;
    uint32_t tc = 0;
    bool ok = true;
    const float c = p.c;
    for (int64_t i = worker; i < p.n_items && ok; i += n_workers) {
      const K2Item item = k2_decode(p, i);
      const int64_t row = static_cast<int64_t>(item.mt) * Cfg::ITEM_ROWS + rank * K2_BM + q * 32 + lane;
      const bool row_ok = row < p.rows;
      int64_t tloc = -1;  // target column local to this shard, -1 if not owned
      if (row_ok) {
        const int64_t t = p.targets[row];
        if (p.vocab_check > 0 && (t < 0 || t >= p.vocab_check) && item.band == 0)
          k2_raise(p.status, TOME_DEV_TARGET_OUT_OF_RANGE);
        const int64_t l = t - p.vocab_offset;
        if (l >= 0 && l < p.vocab_local) tloc = l;
      }
      float m = -FLT_MAX, mc = -FLT_MAX, s = 0.0f, xt = 0.0f;
      for (int32_t n = item.n_begin; n < item.n_end && ok; ++n, ++tc) {
        const uint32_t acc = tc & 1u;
        const uint32_t aphase = (tc >> 1) & 1u;
        if (!mbar_wait(tfull_bar + acc * 8, aphase)) {
          k2_raise(p.status, TOME_DEV_TIMEOUT);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const int64_t col0 = static_cast<int64_t>(n) * K2_BN;
        const int32_t n_valid =
            static_cast<int32_t>(min(static_cast<int64_t>(K2_BN), p.vocab_local - col0));
        const int32_t n_chunks = (n_valid + 31) >> 5;
        const uint32_t taddr = tmem_base + lane_base + acc * K2_BN;
        const int64_t trel = tloc - col0;  // target column relative to this tile

        uint32_t buf[2][32];
        tmem_ld32(taddr, buf[0]);
#pragma unroll
        for (int ch = 0; ch < K2_BN / 32; ++ch) {
          if (ch < n_chunks) {
            tmem_ld_wait_dep(buf[ch & 1]);
            if (ch + 1 < n_chunks) tmem_ld32(taddr + (ch + 1) * 32, buf[(ch + 1) & 1]);
            uint32_t(&v)[32] = buf[ch & 1];
            if (p.round_bf16) {
              // what the reference reduces are logits already rounded to bf16 (model.py:538)
#pragma unroll
              for (int j = 0; j < 32; ++j)
                v[j] = __float_as_uint(
                    __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[j]))));
            }
            const int32_t valid = n_valid - ch * 32;
            if (valid < 32) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j >= valid) v[j] = 0xff800000u;  // -inf: columns past the vocabulary
            }
            // target pick (rare: only when some row of the warp has its target in this chunk)
            const int64_t tj = trel - ch * 32;
            const bool mine = (tj >= 0) && (tj < 32);
            if (__any_sync(0xffffffffu, mine)) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (mine && tj == j) xt = __uint_as_float(v[j]);
            }
            float cmax = fmax3(__uint_as_float(v[0]), __uint_as_float(v[1]), __uint_as_float(v[2]));
#pragma unroll
            for (int j = 3; j + 1 < 32; j += 2)
              cmax = fmax3(cmax, __uint_as_float(v[j]), __uint_as_float(v[j + 1]));
            cmax = fmaxf(cmax, __uint_as_float(v[31]));
            if (cmax > m) {
              // s always equals sum 2^(x*c - mc) for the CURRENT rounded mc, so the rescale
              // uses the difference of the two rounded products
              const float mc_new = cmax * c;
              s *= ex2f(mc - mc_new);
              m = cmax;
              mc = mc_new;
            }
            const float2 c2 = make_float2(c, c);
            const float2 n2 = make_float2(-mc, -mc);
            float2 a0 = make_float2(0.0f, 0.0f), a1 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float2 t0 = __ffma2_rn(
                  make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1])), c2, n2);
              const float2 t1 = __ffma2_rn(
                  make_float2(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])), c2, n2);
              a0 = __fadd2_rn(a0, make_float2(ex2f(t0.x), ex2f(t0.y)));
              a1 = __fadd2_rn(a1, make_float2(ex2f(t1.x), ex2f(t1.y)));
            }
            s += (a0.x + a0.y) + (a1.x + a1.y);
          }
        }
        // accumulator drained: hand it back to the MMA warp
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (PAIR) mbar_arrive_cluster(tempty_signal + acc * 8);
          else mbar_arrive(tempty_bar + acc * 8);
        }
      }
      if (row_ok && ok) {
        const int64_t o = static_cast<int64_t>(item.band) * p.rows + row;
        // exponents were formed as x*c - fl(m*c); fold the rounding residual of m*c back in
        const float delta = fmaf(m, c, -mc);
        p.part_m[o] = __fdiv_rn(m, p.temp);
        p.part_s[o] = s * ex2f(-delta);
        p.part_t[o] = (tloc >= 0) ? __fdiv_rn(xt, p.temp) : 0.0f;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  // nobody leaves while the peer may still signal this CTA's barriers or read its smem
  if (PAIR) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    if (PAIR) tmem_dealloc_pair(tmem_base, K2_TMEM_COLS);
    else tmem_dealloc(tmem_base, K2_TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime so that the library has no
// link-time dependency on libcuda (it must load on machines without a driver).
static int32_t get_encoder(EncodeTiledFn* out) {
  static std::mutex mu;
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    int32_t st = check_cuda(
        cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres),
        "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
    if (st != TOME_OK) return st;
    if (sym == nullptr || qres != cudaDriverEntryPointSuccess)
      return fail(TOME_ERR_CUDA, "cuTensorMapEncodeTiled is not available in this driver");
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  *out = fn;
  return TOME_OK;
}

// Row-major bf16 matrix [n_rows, k] with k contiguous; box = 64 columns x box_rows rows.
static int32_t make_tmap(CUtensorMap* map, const void* ptr, int64_t n_rows, int64_t k,
                         int box_rows) {
  EncodeTiledFn enc;
  int32_t st = get_encoder(&enc);
  if (st != TOME_OK) return st;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(n_rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(K2_BK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims,
                         strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(TOME_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return TOME_OK;
}

struct K2Plan {
  int32_t m_tiles, n_tiles, k_blocks, nb, n_bands, gm;
  int64_t n_items;
};

// Row tiles per group: the hidden tiles of a group (about 40 MB) stay L2-resident while the
// group sweeps the vocabulary.
static int32_t k2_group_size(int32_t m_tiles, int64_t k, int item_rows) {
  const int64_t a_bytes = static_cast<int64_t>(item_rows) * k * 2;
  int64_t gm = std::max<int64_t>(1, (40ll << 20) / std::max<int64_t>(a_bytes, 1));
  if (gm >= m_tiles) return m_tiles;
  // a divisor of the number of concurrent workers keeps a wave on whole bands
  if (gm >= 148 && item_rows == K2_BM) return 148;
  if (gm >= 74) return 74;
  if (gm >= 37) return 37;
  return static_cast<int32_t>(gm);
}

// Largest per-worker load (in column tiles) when the items, in launch order, are dealt
// round-robin to `workers` persistent workers.
static int64_t k2_makespan(int32_t m_tiles, int32_t n_tiles, int32_t nb, int32_t gm,
                           int32_t workers) {
  const int32_t n_bands = (n_tiles + nb - 1) / nb;
  const int32_t tail = n_tiles - (n_bands - 1) * nb;
  int64_t loads[256] = {0};
  const int32_t W = std::min<int32_t>(workers, 256);
  int64_t idx = 0;
  auto deal = [&](int64_t len, int64_t size) {
    if (len <= 0) return;
    for (int32_t w = 0; w < W; ++w) {
      const int64_t first = idx + ((w - idx % W) + W) % W;
      if (first < idx + len) loads[w] += ((idx + len - 1 - first) / W + 1) * size;
    }
    idx += len;
  };
  for (int32_t g0 = 0; g0 < m_tiles; g0 += gm) {
    const int64_t gm_here = std::min<int32_t>(gm, m_tiles - g0);
    deal(static_cast<int64_t>(n_bands - 1) * gm_here, nb);
    deal(gm_here, tail);
  }
  int64_t worst = 0;
  for (int32_t w = 0; w < W; ++w) worst = std::max(worst, loads[w]);
  return worst;
}

// Work decomposition for one problem size.  item_rows: rows of a work item's row tile (128
// single-CTA, 256 CTA pair).  The number of bands, hence the workspace size, must not depend
// on the device or on item_rows, so it is planned for 148 workers of 128-row tiles.
static K2Plan k2_plan_uncached(int64_t rows, int64_t k, int64_t vocab_local, int item_rows);

// The band search costs tens of microseconds of host time; callers come back with the same
// few shapes, so the last plans are kept (thread-safe, a handful of entries).
static K2Plan k2_plan(int64_t rows, int64_t k, int64_t vocab_local, int item_rows = K2_BM) {
  struct Entry {
    int64_t rows, k, vocab;
    int item_rows;
    K2Plan plan;
  };
  constexpr int SLOTS = 16;
  static std::mutex mu;
  static Entry cache[SLOTS];
  static int used = 0, next = 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; ++i)
      if (cache[i].rows == rows && cache[i].k == k && cache[i].vocab == vocab_local &&
          cache[i].item_rows == item_rows)
        return cache[i].plan;
  }
  const K2Plan pl = k2_plan_uncached(rows, k, vocab_local, item_rows);
  std::lock_guard<std::mutex> lock(mu);
  cache[next] = Entry{rows, k, vocab_local, item_rows, pl};
  next = (next + 1) % SLOTS;
  used = std::min(used + 1, SLOTS);
  return pl;
}

static K2Plan k2_plan_uncached(int64_t rows, int64_t k, int64_t vocab_local, int item_rows) {
  K2Plan pl;
  pl.n_tiles = static_cast<int32_t>((vocab_local + K2_BN - 1) / K2_BN);
  pl.k_blocks = static_cast<int32_t>((k + K2_BK - 1) / K2_BK);
  // band length: at most about 16 MB of weight rows (2..32 column tiles); among those the
  // longest one whose round-robin schedule is within 0.2 % of the best balanced
  const int64_t tile_bytes = static_cast<int64_t>(K2_BN) * k * 2;
  int64_t nb_max = (16ll << 20) / std::max<int64_t>(tile_bytes, 1);
  nb_max = std::max<int64_t>(2, std::min<int64_t>(32, nb_max));
  nb_max = std::min<int64_t>(nb_max, pl.n_tiles);
  const int32_t plan_tiles = static_cast<int32_t>((rows + K2_BM - 1) / K2_BM);
  const int32_t plan_gm = k2_group_size(plan_tiles, k, K2_BM);
  int64_t best = INT64_MAX;
  const int32_t nb_min = static_cast<int32_t>(std::min<int64_t>(2, nb_max));
  for (int32_t nb = static_cast<int32_t>(nb_max); nb >= nb_min; --nb)
    best = std::min(best, k2_makespan(plan_tiles, pl.n_tiles, nb, plan_gm, 148));
  pl.nb = nb_min;
  for (int32_t nb = static_cast<int32_t>(nb_max); nb >= nb_min; --nb) {
    if (k2_makespan(plan_tiles, pl.n_tiles, nb, plan_gm, 148) * 500 <= best * 501) {
      pl.nb = nb;
      break;
    }
  }
  pl.n_bands = (pl.n_tiles + pl.nb - 1) / pl.nb;
  pl.m_tiles = static_cast<int32_t>((rows + item_rows - 1) / item_rows);
  pl.gm = k2_group_size(pl.m_tiles, k, item_rows);
  pl.n_items = static_cast<int64_t>(pl.m_tiles) * pl.n_bands;
  return pl;
}

static int32_t k2_check(const void* hidden, const void* weight, int64_t rows, int64_t k,
                        int64_t vocab_local, int64_t vocab_offset, const int32_t* targets,
                        float temperature, const void* workspace, size_t ws_bytes) {
  if (rows < 0 || k <= 0 || vocab_local <= 0 || vocab_offset < 0)
    return fail(TOME_ERR_BAD_SHAPE, "rows=%lld hidden_dim=%lld vocab_local=%lld vocab_offset=%lld",
                (long long)rows, (long long)k, (long long)vocab_local, (long long)vocab_offset);
  if (k % 8 != 0)
    return fail(TOME_ERR_UNSUPPORTED, "hidden_dim=%lld must be a multiple of 8 (16-byte rows)",
                (long long)k);
  if (rows > 0x7fffffffLL || vocab_local > 0x7fffffffLL || k > 0x7fffffffLL)
    return fail(TOME_ERR_TOO_LARGE, "a dimension exceeds int32");
  if (!temperature_ok(temperature))
    return fail(TOME_ERR_BAD_TEMPERATURE, "temperature=%g must be > 0 and finite", temperature);
  if (rows == 0) return TOME_OK;
  if (hidden == nullptr || weight == nullptr || targets == nullptr || workspace == nullptr)
    return fail(TOME_ERR_NULL_POINTER, "a required pointer is NULL");
  if (!aligned16(hidden) || !aligned16(weight) || !aligned16(workspace))
    return fail(TOME_ERR_MISALIGNED, "hidden, weight and workspace must be 16-byte aligned");
  const size_t need = tome_lmhead_workspace_bytes(rows, k, vocab_local);
  if (ws_bytes < need)
    return fail(TOME_ERR_WORKSPACE_TOO_SMALL, "workspace has %zu bytes, need %zu", ws_bytes, need);
  return TOME_OK;
}

// Tuning knob TOME_K2_PAIR = 0 | 1: single-CTA tiles (cta_group::1, the default) or CTA-pair
// tiles (cta_group::2).  Under the board power cap the single-CTA form measured 1-9 % faster
// on both head shapes, so it is the default.  Read once per process.
static bool k2_pair_setting() {
  static const bool value = [] {
    const char* e = getenv("TOME_K2_PAIR");
    return (e != nullptr) ? (atoi(e) != 0) : false;
  }();
  return value;
}

// Launches the GEMM+reduce kernel; partial triples land in the workspace.
static int32_t k2_launch(const void* hidden, const void* weight, int64_t rows, int64_t k,
                         int64_t vocab_local, int64_t vocab_offset, int64_t vocab_check,
                         const int32_t* targets, float temperature, int32_t flags,
                         void* workspace, int32_t* dev_status, cudaStream_t stream,
                         K2Plan* plan_out) {
  DeviceInfo info;
  int32_t st = current_device_info(&info);
  if (st != TOME_OK) return st;
  if (info.cc_major != 10)
    return fail(TOME_ERR_UNSUPPORTED, "the fused LM head needs an sm_100 device (found sm_%d*)",
                info.cc_major * 10);
  const bool pair = k2_pair_setting();
  const K2Plan pl = k2_plan(rows, k, vocab_local, pair ? 256 : 128);
  *plan_out = pl;
  CUtensorMap ta, tb;
  st = make_tmap(&ta, hidden, rows, k, K2_BM);
  if (st != TOME_OK) return st;
  st = make_tmap(&tb, weight, vocab_local, k, pair ? K2Cfg<true>::B_ROWS : K2Cfg<false>::B_ROWS);
  if (st != TOME_OK) return st;
  K2Params p = {};
  p.rows = rows;
  p.k_dim = k;
  p.vocab_local = vocab_local;
  p.vocab_offset = vocab_offset;
  p.vocab_check = vocab_check;
  p.targets = targets;
  p.c = LOG2E / temperature;
  p.temp = temperature;
  float* ws = static_cast<float*>(workspace);
  const int64_t plane = static_cast<int64_t>(pl.n_bands) * rows;
  p.part_m = ws;
  p.part_s = ws + plane;
  p.part_t = ws + 2 * plane;
  p.m_tiles = pl.m_tiles;
  p.n_tiles = pl.n_tiles;
  p.k_blocks = pl.k_blocks;
  p.nb = pl.nb;
  p.n_bands = pl.n_bands;
  p.gm = pl.gm;
  p.n_items = pl.n_items;
  p.round_bf16 = (flags & TOME_LMHEAD_ROUND_LOGITS_BF16) ? 1 : 0;
  p.status = dev_status;
  if (pair) {
    constexpr int smem = K2Cfg<true>::SMEM_BYTES;
    st = ensure_dynamic_smem(reinterpret_cast<const void*>(k2_lmhead_kernel<true>), smem);
    if (st != TOME_OK) return st;
    const int pairs = static_cast<int>(
        std::max<int64_t>(1, std::min<int64_t>(info.sm_count / 2, pl.n_items)));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(K2_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, k2_lmhead_kernel<true>, ta, tb, p),
                      "k2 pair launch");
  }
  constexpr int smem = K2Cfg<false>::SMEM_BYTES;
  st = ensure_dynamic_smem(reinterpret_cast<const void*>(k2_lmhead_kernel<false>), smem);
  if (st != TOME_OK) return st;
  const int grid =
      static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(info.sm_count, pl.n_items)));
  k2_lmhead_kernel<false><<<grid, K2_THREADS, smem, stream>>>(ta, tb, p);
  return check_cuda(cudaGetLastError(), "k2 launch");
}

}  // namespace tome

using namespace tome;

extern "C" size_t tome_lmhead_workspace_bytes(int64_t rows, int64_t hidden_dim,
                                              int64_t vocab_local) {
  if (rows <= 0 || hidden_dim <= 0 || vocab_local <= 0) return 0;
  const K2Plan pl = k2_plan(rows, hidden_dim, vocab_local);
  return static_cast<size_t>(3) * pl.n_bands * rows * sizeof(float);
}

extern "C" int32_t tome_lmhead_partials(const void* hidden, const void* weight, int64_t rows,
                                        int64_t hidden_dim, int64_t vocab_local,
                                        int64_t vocab_offset, const int32_t* targets,
                                        float temperature, int32_t flags, float* out_m,
                                        float* out_s, float* out_t, void* workspace,
                                        size_t workspace_bytes, int32_t* dev_status,
                                        void* stream) {
  int32_t st = k2_check(hidden, weight, rows, hidden_dim, vocab_local, vocab_offset, targets,
                        temperature, workspace, workspace_bytes);
  if (st != TOME_OK || rows == 0) return st;
  if (out_m == nullptr || out_s == nullptr || out_t == nullptr)
    return fail(TOME_ERR_NULL_POINTER, "an output pointer is NULL");
  K2Plan pl;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  st = k2_launch(hidden, weight, rows, hidden_dim, vocab_local, vocab_offset, 0, targets,
                 temperature, flags, workspace, dev_status, s, &pl);
  if (st != TOME_OK) return st;
  const float* ws = static_cast<const float*>(workspace);
  const int64_t plane = static_cast<int64_t>(pl.n_bands) * rows;
  return launch_combine(false, ws, ws + plane, rows, pl.n_bands, ws + 2 * plane, rows, pl.n_bands,
                        rows, out_m, out_s, out_t, s);
}

extern "C" int32_t tome_lmhead_logprob(const void* hidden, const void* weight, int64_t rows,
                                       int64_t hidden_dim, int64_t vocab, const int32_t* targets,
                                       float temperature, int32_t flags, float* out_logprob,
                                       float* out_lse, void* workspace, size_t workspace_bytes,
                                       int32_t* dev_status, void* stream) {
  int32_t st = k2_check(hidden, weight, rows, hidden_dim, vocab, 0, targets, temperature,
                        workspace, workspace_bytes);
  if (st != TOME_OK || rows == 0) return st;
  if (out_logprob == nullptr) return fail(TOME_ERR_NULL_POINTER, "out_logprob is NULL");
  K2Plan pl;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  st = k2_launch(hidden, weight, rows, hidden_dim, vocab, 0, vocab, targets, temperature, flags,
                 workspace, dev_status, s, &pl);
  if (st != TOME_OK) return st;
  const float* ws = static_cast<const float*>(workspace);
  const int64_t plane = static_cast<int64_t>(pl.n_bands) * rows;
  return launch_combine(true, ws, ws + plane, rows, pl.n_bands, ws + 2 * plane, rows, pl.n_bands,
                        rows, out_logprob, out_lse, nullptr, s);
}

// ------------------------------------------------------------------ final RMSNorm
// y = bf16(float(x) * rsqrt(mean(x^2) + eps) * float(w)), one warp per row, fp32 arithmetic:
// the model's last step before the head (mlx-impl/model.py:336-343, 536), so that the fused
// head can be fed from the un-normalised hidden states.
__global__ void __launch_bounds__(256) k2_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x,
                                                         const __nv_bfloat16* __restrict__ w,
                                                         int64_t rows, int64_t dim, float eps,
                                                         __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t nvec = dim >> 3;  // dim is a multiple of 8
  for (int64_t row = warp_global; row < rows; row += n_warps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
    float ss = 0.0f;
    for (int64_t v = lane; v < nvec; v += 32) {
      const uint4 q = xr[v];
      const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = __uint_as_float(ws[j] << 16), b = __uint_as_float(ws[j] & 0xffff0000u);
        ss = fmaf(a, a, ss);
        ss = fmaf(b, b, ss);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss / static_cast<float>(dim) + eps);
    uint4* orow = reinterpret_cast<uint4*>(out + row * dim);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    for (int64_t v = lane; v < nvec; v += 32) {
      const uint4 q = xr[v];
      const uint4 g = wr[v];
      const uint32_t xs[4] = {q.x, q.y, q.z, q.w};
      const uint32_t gs[4] = {g.x, g.y, g.z, g.w};
      uint32_t os[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = __uint_as_float(xs[j] << 16) * inv * __uint_as_float(gs[j] << 16);
        const float b =
            __uint_as_float(xs[j] & 0xffff0000u) * inv * __uint_as_float(gs[j] & 0xffff0000u);
        os[j] = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(a))) |
                (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(b))) << 16);
      }
      orow[v] = make_uint4(os[0], os[1], os[2], os[3]);
    }
  }
}

extern "C" int32_t tome_rmsnorm_bf16(const void* x, const void* weight, int64_t rows, int64_t dim,
                                     float eps, void* out, void* stream) {
  if (rows < 0 || dim <= 0)
    return fail(TOME_ERR_BAD_SHAPE, "rows=%lld dim=%lld", (long long)rows, (long long)dim);
  if (dim % 8 != 0)
    return fail(TOME_ERR_UNSUPPORTED, "dim=%lld must be a multiple of 8", (long long)dim);
  if (!(eps >= 0.0f)) return fail(TOME_ERR_BAD_SHAPE, "eps=%g must be >= 0", eps);
  if (rows == 0) return TOME_OK;
  if (x == nullptr || weight == nullptr || out == nullptr)
    return fail(TOME_ERR_NULL_POINTER, "a required pointer is NULL");
  if (!aligned16(x) || !aligned16(weight) || !aligned16(out))
    return fail(TOME_ERR_MISALIGNED, "x, weight and out must be 16-byte aligned");
  const int64_t want = (rows + 7) / 8;  // 8 warps (rows) per CTA
  const int grid = static_cast<int>(std::min<int64_t>(want, 148 * 16));
  k2_rmsnorm_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(weight), rows, dim,
      eps, static_cast<__nv_bfloat16*>(out));
  return check_cuda(cudaGetLastError(), "rmsnorm launch");
}

// ------------------------------------------------------------------ no-allocation variant
// Scratch for tome_lmhead_logprob_static: one fixed array in the library's device image.
// Every GPU that loads the library holds these 8 MiB until the process exits.
constexpr size_t K2_STATIC_SCRATCH_BYTES = static_cast<size_t>(8) << 20;
static __device__ __align__(256) unsigned char k2_static_scratch[K2_STATIC_SCRATCH_BYTES];

// Device address of the static scratch on the CURRENT device.  In host code the array's name
// is only a handle, not a device pointer, so the address is asked for once per device (with
// that device current) through cudaGetSymbolAddress and remembered.
static int32_t k2_static_scratch_address(void** out) {
  constexpr int MAX_DEV = 64;
  static std::mutex mu;
  static void* cached[MAX_DEV] = {nullptr};
  int dev = 0;
  int32_t st = tome::check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
  if (st != TOME_OK) return st;
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && dev < MAX_DEV && cached[dev] != nullptr) {
    *out = cached[dev];
    return TOME_OK;
  }
  void* ptr = nullptr;
  st = tome::check_cuda(cudaGetSymbolAddress(&ptr, k2_static_scratch),
                        "cudaGetSymbolAddress(k2_static_scratch)");
  if (st != TOME_OK) return st;
  if (ptr == nullptr) return tome::fail(TOME_ERR_CUDA, "static scratch has no device address");
  if (dev >= 0 && dev < MAX_DEV) cached[dev] = ptr;
  *out = ptr;
  return TOME_OK;
}

extern "C" size_t tome_lmhead_static_scratch_bytes(void) { return K2_STATIC_SCRATCH_BYTES; }

extern "C" int32_t tome_lmhead_logprob_static(const void* hidden, const void* weight,
                                              int64_t rows, int64_t hidden_dim, int64_t vocab,
                                              const int32_t* targets, float temperature,
                                              float* out_logprob, float* out_lse,
                                              int32_t* dev_status, void* stream) {
  if (rows > 0 && hidden_dim > 0 && vocab > 0) {
    const size_t need = tome_lmhead_workspace_bytes(rows, hidden_dim, vocab);
    if (need > K2_STATIC_SCRATCH_BYTES)
      return fail(TOME_ERR_TOO_LARGE,
                  "this problem needs %zu bytes of scratch but the built-in scratch holds %zu; "
                  "use tome_lmhead_logprob with a caller-provided workspace, or fewer rows per call",
                  need, K2_STATIC_SCRATCH_BYTES);
  }
  void* scratch = nullptr;
  if (rows > 0) {
    const int32_t st = k2_static_scratch_address(&scratch);
    if (st != TOME_OK) return st;
  } else {
    scratch = reinterpret_cast<void*>(static_cast<uintptr_t>(256));  // never used when rows == 0
  }
  return tome_lmhead_logprob(hidden, weight, rows, hidden_dim, vocab, targets, temperature, 0,
                             out_logprob, out_lse, scratch, K2_STATIC_SCRATCH_BYTES, dev_status,
                             stream);
}
