// TEST INFRASTRUCTURE ONLY: runs the reference's Metal kernel body on the CPU.
//
// The reference's full-matrix log-softmax is a Metal Shading Language kernel body kept as a
// Python string (mlx-impl/model.py:14-66) and launched with 1024 threads per row
// (model.py:77-89).  The body uses a small subset of MSL that is also valid C++ once the
// names it relies on exist.  This file provides those names and the execution model
// (threadgroups of 1024 threads in 32 simdgroups, threadgroup barriers, simdgroup
// reductions), and includes the body VERBATIM from a file that oracle/build_ref.py extracts
// from the reference checkout at build time (nothing of the reference is stored in this
// repository).  Only tests and fixture generators load the resulting library.
//
// Execution model: every GPU thread is a cooperative fiber (ucontext).  A fiber runs until
// it needs the others (a barrier or a simdgroup reduction), then yields; the scheduler
// resumes the fibers round robin.  Differences from a real Apple GPU, none of which change
// the arithmetic the kernel specifies:
//   * metal::fast::exp / fast::log are the libm expf / logf here (the GPU's are
//     approximations of them);
//   * simd_sum / simd_max reduce in butterfly (xor-shuffle) order;
//   * bfloat arithmetic is done in float and rounded to nearest even, as MSL specifies.
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <ucontext.h>

#include <vector>

namespace {

constexpr int kThreads = 1024;  // threadgroup=(1024, 1, 1), model.py:87
constexpr int kSimdWidth = 32;
constexpr int kSimdGroups = kThreads / kSimdWidth;
constexpr size_t kStackBytes = 64 * 1024;

// ---------------------------------------------------------------- MSL names the body uses
typedef unsigned int uint;

struct uint3 {
  uint x, y, z;
};

namespace mem_flags {
enum { mem_threadgroup = 1 };
}

struct bfloat {  // MSL's bfloat: 8 exponent bits, 7 mantissa bits, round to nearest even
  uint16_t bits;
  bfloat() : bits(0) {}
  explicit bfloat(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) {
      bits = static_cast<uint16_t>((u >> 16) | 0x40);  // quiet NaN
    } else {
      u += 0x7fffu + ((u >> 16) & 1u);
      bits = static_cast<uint16_t>(u >> 16);
    }
  }
  explicit operator float() const {
    const uint32_t u = static_cast<uint32_t>(bits) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
  }
};
inline bfloat operator-(bfloat a, bfloat b) {
  return bfloat(static_cast<float>(a) - static_cast<float>(b));
}

inline float max(float a, float b) { return fmaxf(a, b); }

namespace metal {
namespace fast {
inline float exp(float x) { return expf(x); }
inline float log(float x) { return logf(x); }
}  // namespace fast
}  // namespace metal

// ---------------------------------------------------------------- fibers
struct Group {
  ucontext_t scheduler;
  ucontext_t fiber[kThreads];
  std::vector<char> stacks;
  bool done[kThreads];
  int current = 0;
  // threadgroup barrier
  int bar_count = 0;
  unsigned bar_generation = 0;
  // simdgroup reductions
  float simd_vals[kSimdGroups][kSimdWidth];
  float simd_result[kSimdGroups];
  int simd_count[kSimdGroups];
  unsigned simd_generation[kSimdGroups];
};

Group* g_group = nullptr;

void yield_to_scheduler() {
  Group& g = *g_group;
  swapcontext(&g.fiber[g.current], &g.scheduler);
}

void threadgroup_barrier(int) {
  Group& g = *g_group;
  const unsigned gen = g.bar_generation;
  if (++g.bar_count == kThreads) {
    g.bar_count = 0;
    ++g.bar_generation;
    return;
  }
  while (g.bar_generation == gen) yield_to_scheduler();
}

template <typename Op>
float simd_reduce(float value, Op op) {
  Group& g = *g_group;
  const int group = g.current / kSimdWidth, lane = g.current % kSimdWidth;
  const unsigned gen = g.simd_generation[group];
  g.simd_vals[group][lane] = value;
  if (++g.simd_count[group] == kSimdWidth) {
    float v[kSimdWidth];
    memcpy(v, g.simd_vals[group], sizeof(v));
    for (int offset = kSimdWidth / 2; offset > 0; offset >>= 1) {  // butterfly
      float next[kSimdWidth];
      for (int i = 0; i < kSimdWidth; ++i) next[i] = op(v[i], v[i ^ offset]);
      memcpy(v, next, sizeof(v));
    }
    g.simd_result[group] = v[0];
    g.simd_count[group] = 0;
    ++g.simd_generation[group];
  } else {
    while (g.simd_generation[group] == gen) yield_to_scheduler();
  }
  return g.simd_result[group];
}

float simd_max(float v) {
  return simd_reduce(v, [](float a, float b) { return fmaxf(a, b); });
}
float simd_sum(float v) {
  return simd_reduce(v, [](float a, float b) { return a + b; });
}

// ---------------------------------------------------------------- the reference's kernel
// mx.fast.metal_kernel wraps the body in a function whose parameters are the inputs, the
// outputs and the thread-position attributes the body mentions; T and V are template
// arguments there (model.py:85).  Here V is a run-time value, so the body's `constexpr`
// becomes `const`, and `threadgroup` storage is one static array (one threadgroup runs at a
// time).
template <typename T>
void kernel_body(const T* logits, const float* temp, T* out, const int V,
                 const uint3 threadgroup_position_in_grid, const uint thread_index_in_threadgroup,
                 const uint thread_index_in_simdgroup, const uint simdgroup_index_in_threadgroup) {
#define constexpr const
#define threadgroup static
#include "fused_log_softmax_body.inc"
#undef threadgroup
#undef constexpr
}

template <typename T>
struct Launch {
  const T* logits;
  const float* temp;
  T* out;
  int V;
  uint row;
};

void* g_launch = nullptr;

template <typename T>
void fiber_entry() {
  Group& g = *g_group;
  const Launch<T>& l = *static_cast<const Launch<T>*>(g_launch);
  const uint tid = static_cast<uint>(g.current);
  kernel_body<T>(l.logits, l.temp, l.out, l.V, uint3{0, l.row, 0}, tid, tid % kSimdWidth,
                 tid / kSimdWidth);
  g.done[g.current] = true;
  yield_to_scheduler();  // never resumed
}

template <typename T>
int run(const T* logits, float temperature, T* out, int rows, int V) {
  Group* g = new Group();
  g->stacks.resize(static_cast<size_t>(kThreads) * kStackBytes);
  g_group = g;
  Launch<T> launch{logits, &temperature, out, V, 0};
  g_launch = &launch;
  for (int row = 0; row < rows; ++row) {  // grid=(1024, rows, 1): one threadgroup per row
    launch.row = static_cast<uint>(row);
    g->bar_count = 0;
    memset(g->simd_count, 0, sizeof(g->simd_count));
    for (int t = 0; t < kThreads; ++t) {
      g->done[t] = false;
      getcontext(&g->fiber[t]);
      g->fiber[t].uc_stack.ss_sp = g->stacks.data() + static_cast<size_t>(t) * kStackBytes;
      g->fiber[t].uc_stack.ss_size = kStackBytes;
      g->fiber[t].uc_link = nullptr;
      makecontext(&g->fiber[t], reinterpret_cast<void (*)()>(fiber_entry<T>), 0);
    }
    int remaining = kThreads;
    long rounds = 0;
    while (remaining > 0) {
      remaining = 0;
      for (int t = 0; t < kThreads; ++t) {
        if (g->done[t]) continue;
        g->current = t;
        swapcontext(&g->scheduler, &g->fiber[t]);
        if (!g->done[t]) ++remaining;
      }
      if (++rounds > 1000000) {  // a body that never converges: give up instead of spinning
        g_group = nullptr;
        delete g;
        return -1;
      }
    }
  }
  g_group = nullptr;
  g_launch = nullptr;
  delete g;
  return 0;
}

// ---------------------------------------------------------------- paged KV gather
// mlx-impl/paged_kv.py:57-116: a Metal body assembled as a Python f-string; build_ref.py
// replaces its `{B}`-style fields by the `_arg` parameters below and its `{{ }}` by braces.
// One thread per output element, no barriers, so the grid is walked with plain loops.
template <typename T>
void gather_body(const int32_t* block_tables, const int32_t* offsets, const T* k_pool,
                 const T* v_pool, T* k_out, T* v_out, const uint max_seq_len,
                 const uint3 thread_position_in_grid, const uint B_arg, const uint H_arg,
                 const uint D_arg, const uint block_size_arg, const uint max_blocks_arg) {
#include "gather_paged_kv_body.inc"
}

template <typename T>
void gather_run(const int32_t* block_tables, const int32_t* offsets, const T* k_pool,
                const T* v_pool, T* k_out, T* v_out, uint B, uint H, uint D, uint block_size,
                uint max_blocks, uint max_seq_len) {
  for (uint x = 0; x < B; ++x)  // grid=(B, H, max_seq_len * D), paged_kv.py:110
    for (uint y = 0; y < H; ++y)
      for (uint z = 0; z < max_seq_len * D; ++z)
        gather_body<T>(block_tables, offsets, k_pool, v_pool, k_out, v_out, max_seq_len,
                       uint3{x, y, z}, B, H, D, block_size, max_blocks);
}

}  // namespace

// Pools [num_blocks, H, block_size, D], outputs [B, H, max_seq_len, D]; elem_bytes 2 or 4 (the
// kernel only copies, so elements travel as integers of their width).
extern "C" int metal_gather_paged_kv(const int32_t* block_tables, const int32_t* offsets,
                                     const void* k_pool, const void* v_pool, void* k_out,
                                     void* v_out, int elem_bytes, int B, int H, int D,
                                     int block_size, int max_blocks, int max_seq_len) {
  if (elem_bytes == 2) {
    gather_run<uint16_t>(block_tables, offsets, static_cast<const uint16_t*>(k_pool),
                         static_cast<const uint16_t*>(v_pool), static_cast<uint16_t*>(k_out),
                         static_cast<uint16_t*>(v_out), B, H, D, block_size, max_blocks, max_seq_len);
    return 0;
  }
  if (elem_bytes == 4) {
    gather_run<uint32_t>(block_tables, offsets, static_cast<const uint32_t*>(k_pool),
                         static_cast<const uint32_t*>(v_pool), static_cast<uint32_t*>(k_out),
                         static_cast<uint32_t*>(v_out), B, H, D, block_size, max_blocks, max_seq_len);
    return 0;
  }
  return -1;
}

// logits / out: [rows, V] row-contiguous (ensure_row_contiguous=True, model.py:73).
extern "C" int metal_fused_log_softmax_f32(const float* logits, float temperature, float* out,
                                           int rows, int V) {
  return run<float>(logits, temperature, out, rows, V);
}

extern "C" int metal_fused_log_softmax_bf16(const uint16_t* logits, float temperature,
                                            uint16_t* out, int rows, int V) {
  static_assert(sizeof(bfloat) == 2, "bfloat is its 16 bits");
  return run<bfloat>(reinterpret_cast<const bfloat*>(logits), temperature,
                     reinterpret_cast<bfloat*>(out), rows, V);
}
