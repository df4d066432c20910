// K5: paged KV-cache gather and update (pure data movement, HBM-bound, byte-exact).
//
// The pool holds fixed-size blocks, [num_blocks, H, block_size, D]; a block table per
// sequence maps logical block i to a physical block.  gather copies the first offsets[b]
// tokens of every sequence into a dense [B, H, max_seq_len, D] tensor and zero-fills the
// rest (mlx-impl/paged_kv.py:57-116, the reference's Metal kernel); update scatters new
// tokens into the pool block by block (mlx-impl/paged_kv.py:6-54, a host loop of
// slice_update calls in the reference).  One thread moves 16 bytes; a (b, h, s) row of D
// elements is contiguous on both sides, so loads and stores are fully coalesced.
#include <algorithm>

#include "host_common.h"

namespace tome {

struct K5Params {
  const int32_t* block_tables;  // [B, max_blocks]
  const int32_t* offsets;       // [B]
  const int32_t* lengths;       // update: [B] or null (= S)
  const uint4* k_src;
  const uint4* v_src;
  uint4* k_dst;
  uint4* v_dst;
  int64_t B, H, S, vec_per_row;  // S = max_seq_len (gather) or S_new (update); row = D elements
  int32_t block_size, max_blocks, num_blocks;
  int32_t* status;
};

__device__ __forceinline__ void k5_raise(int32_t* status, int32_t bit) {
  if (status != nullptr) atomicOr(status, bit);
}

// out[b, h, s, :] = s < offsets[b] ? pool[table[b, s / bs], h, s % bs, :] : 0
__global__ void __launch_bounds__(256) k5_gather_kernel(const K5Params p) {
  const int64_t total = p.B * p.H * p.S * p.vec_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t dv = i % p.vec_per_row;
    const int64_t row = i / p.vec_per_row;  // (b * H + h) * S + s
    const int64_t s = row % p.S;
    const int64_t bh = row / p.S;
    const int64_t h = bh % p.H;
    const int64_t b = bh / p.H;
    uint4 kq = make_uint4(0, 0, 0, 0), vq = make_uint4(0, 0, 0, 0);
    if (s < p.offsets[b]) {
      const int64_t blk = s / p.block_size;
      const int64_t in_blk = s - blk * p.block_size;
      int32_t phys = -1;
      if (blk < p.max_blocks) phys = p.block_tables[b * p.max_blocks + blk];
      if (phys >= 0 && phys < p.num_blocks) {
        const int64_t src = ((static_cast<int64_t>(phys) * p.H + h) * p.block_size + in_blk) *
                                p.vec_per_row + dv;
        kq = __ldcs(p.k_src + src);  // every byte is touched once: stream through the caches
        vq = __ldcs(p.v_src + src);
      } else {
        k5_raise(p.status, TOME_DEV_BLOCK_OUT_OF_RANGE);
      }
    }
    __stcs(p.k_dst + i, kq);
    __stcs(p.v_dst + i, vq);
  }
}

// for t < lengths[b]: i = t / bs; logical block = (offsets[b] + i * bs) / bs; if it is inside
// the table: pool[table[b, logical], h, t % bs, :] = new[b, h, t, :]
// (the reference writes every piece at the START of its block: paged_kv.py:42-49)
__global__ void __launch_bounds__(256) k5_update_kernel(const K5Params p) {
  const int64_t total = p.B * p.H * p.S * p.vec_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t dv = i % p.vec_per_row;
    const int64_t row = i / p.vec_per_row;
    const int64_t t = row % p.S;
    const int64_t bh = row / p.S;
    const int64_t h = bh % p.H;
    const int64_t b = bh / p.H;
    const int64_t len = (p.lengths != nullptr) ? min(static_cast<int64_t>(p.lengths[b]), p.S) : p.S;
    if (t >= len) continue;
    const int64_t piece = t / p.block_size;
    const int64_t in_blk = t - piece * p.block_size;
    const int64_t logical = (static_cast<int64_t>(p.offsets[b]) + piece * p.block_size) / p.block_size;
    if (logical < 0 || logical >= p.max_blocks) continue;  // the reference stops at the table's end
    const int32_t phys = p.block_tables[b * p.max_blocks + logical];
    if (phys < 0 || phys >= p.num_blocks) {
      k5_raise(p.status, TOME_DEV_BLOCK_OUT_OF_RANGE);
      continue;
    }
    const int64_t dst = ((static_cast<int64_t>(phys) * p.H + h) * p.block_size + in_blk) *
                            p.vec_per_row + dv;
    __stcs(p.k_dst + dst, __ldcs(p.k_src + i));
    __stcs(p.v_dst + dst, __ldcs(p.v_src + i));
  }
}

static int32_t k5_check(const void* a, const void* b, const void* c, const void* d,
                        const int32_t* tables, const int32_t* offsets, int32_t elem_bytes,
                        int64_t B, int64_t H, int64_t S, int64_t D, int32_t block_size,
                        int32_t max_blocks, int32_t num_blocks, int64_t* vec_per_row) {
  if (elem_bytes != 2 && elem_bytes != 4)
    return fail(TOME_ERR_BAD_DTYPE, "elem_bytes=%d must be 2 or 4", elem_bytes);
  if (B < 0 || H <= 0 || S < 0 || D <= 0 || block_size <= 0 || max_blocks < 0 || num_blocks < 0)
    return fail(TOME_ERR_BAD_SHAPE, "B=%lld H=%lld S=%lld D=%lld block_size=%d max_blocks=%d",
                (long long)B, (long long)H, (long long)S, (long long)D, block_size, max_blocks);
  if ((D * elem_bytes) % 16 != 0)
    return fail(TOME_ERR_UNSUPPORTED, "head_dim * elem_bytes = %lld must be a multiple of 16",
                (long long)(D * elem_bytes));
  *vec_per_row = D * elem_bytes / 16;
  if (B == 0 || S == 0) return TOME_OK;
  if (a == nullptr || b == nullptr || c == nullptr || d == nullptr || tables == nullptr ||
      offsets == nullptr)
    return fail(TOME_ERR_NULL_POINTER, "a required pointer is NULL");
  if (!aligned16(a) || !aligned16(b) || !aligned16(c) || !aligned16(d))
    return fail(TOME_ERR_MISALIGNED, "pool and dense tensors must be 16-byte aligned");
  return TOME_OK;
}

static int k5_grid(int64_t total_vecs) {
  DeviceInfo info;
  const int sms = (current_device_info(&info) == TOME_OK) ? info.sm_count : 148;
  const int64_t want = (total_vecs + 255) / 256;
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(want, static_cast<int64_t>(sms) * 16)));
}

}  // namespace tome

using namespace tome;

extern "C" int32_t tome_gather_paged_kv(const int32_t* block_tables, const int32_t* offsets,
                                        const void* k_pool, const void* v_pool,
                                        int32_t elem_bytes, int64_t batch, int64_t heads,
                                        int64_t head_dim, int32_t block_size, int32_t max_blocks,
                                        int32_t num_blocks, int64_t max_seq_len, void* k_out,
                                        void* v_out, int32_t* dev_status, void* stream) {
  int64_t vpr = 0;
  int32_t st = k5_check(k_pool, v_pool, k_out, v_out, block_tables, offsets, elem_bytes, batch,
                        heads, max_seq_len, head_dim, block_size, max_blocks, num_blocks, &vpr);
  if (st != TOME_OK || batch == 0 || max_seq_len == 0) return st;
  K5Params p = {};
  p.block_tables = block_tables;
  p.offsets = offsets;
  p.k_src = static_cast<const uint4*>(k_pool);
  p.v_src = static_cast<const uint4*>(v_pool);
  p.k_dst = static_cast<uint4*>(k_out);
  p.v_dst = static_cast<uint4*>(v_out);
  p.B = batch;
  p.H = heads;
  p.S = max_seq_len;
  p.vec_per_row = vpr;
  p.block_size = block_size;
  p.max_blocks = max_blocks;
  p.num_blocks = num_blocks;
  p.status = dev_status;
  k5_gather_kernel<<<k5_grid(batch * heads * max_seq_len * vpr), 256, 0,
                     static_cast<cudaStream_t>(stream)>>>(p);
  return check_cuda(cudaGetLastError(), "paged gather launch");
}

extern "C" int32_t tome_update_paged_kv(const void* k_new, const void* v_new,
                                        const int32_t* block_tables, const int32_t* offsets,
                                        const int32_t* lengths, void* k_pool, void* v_pool,
                                        int32_t elem_bytes, int64_t batch, int64_t heads,
                                        int64_t new_len, int64_t head_dim, int32_t block_size,
                                        int32_t max_blocks, int32_t num_blocks,
                                        int32_t* dev_status, void* stream) {
  int64_t vpr = 0;
  int32_t st = k5_check(k_new, v_new, k_pool, v_pool, block_tables, offsets, elem_bytes, batch,
                        heads, new_len, head_dim, block_size, max_blocks, num_blocks, &vpr);
  if (st != TOME_OK || batch == 0 || new_len == 0) return st;
  K5Params p = {};
  p.block_tables = block_tables;
  p.offsets = offsets;
  p.lengths = lengths;
  p.k_src = static_cast<const uint4*>(k_new);
  p.v_src = static_cast<const uint4*>(v_new);
  p.k_dst = static_cast<uint4*>(k_pool);
  p.v_dst = static_cast<uint4*>(v_pool);
  p.B = batch;
  p.H = heads;
  p.S = new_len;
  p.vec_per_row = vpr;
  p.block_size = block_size;
  p.max_blocks = max_blocks;
  p.num_blocks = num_blocks;
  p.status = dev_status;
  k5_update_kernel<<<k5_grid(batch * heads * new_len * vpr), 256, 0,
                     static_cast<cudaStream_t>(stream)>>>(p);
  return check_cuda(cudaGetLastError(), "paged update launch");
}
