// Online softmax arithmetic shared by the streaming kernels: per-thread (max, sum-exp) states,
// their merges, and the packed f32x2 fast path for 16-byte vectors of bf16 / fp32 logits.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "ptx.cuh"

namespace tome {

// ------------------------------------------------------------------ online (max, sum-exp)
struct Online {
  float m;  // running maximum of the raw logits
  float s;  // sum of 2^((x - m) * c)
};

__device__ __forceinline__ void online_init(Online& st) {
  st.m = -FLT_MAX;
  st.s = 0.0f;
}

__device__ __forceinline__ void online_raise(Online& st, float vmax, float c) {
  if (vmax > st.m) {
    st.s *= ex2f((st.m - vmax) * c);
    st.m = vmax;
  }
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ __nv_bfloat162 as_bf162(uint32_t w) {
  return *reinterpret_cast<__nv_bfloat162*>(&w);
}

// ------------------------------------------------------------------ streaming inner loop
// Inside the streaming loop a thread keeps
//   m   running maximum of its raw logits, never below K1_M_FLOOR
//   mc  fl(m * c)
//   a,b packed partial sums of 2^(x*c - mc), two fp32 lanes each
// so that one packed FFMA (fma.rn.f32x2) forms two exponents.  The exponent x*c - fl(m*c)
// differs from (x - m)*c by delta = m*c - fl(m*c), the same for every term of the thread;
// fast_finish() folds 2^-delta back in exactly.  The floor keeps |mc| small enough for that
// to work when a thread has so far seen nothing but mask values (-1e30, -FLT_MAX, -inf).
// Rows whose result is not a positive finite sum (every logit below the floor, or logits
// beyond ~1e7 in magnitude) are redone by exact_row() with the (x - m) form.
constexpr float K1_M_FLOOR = -1048576.0f;

struct Fast {
  float m, mc;
  float2 a, b;
};

__device__ __forceinline__ void fast_init(Fast& f, float c) {
  f.m = K1_M_FLOOR;
  f.mc = K1_M_FLOOR * c;
  f.a = make_float2(0.0f, 0.0f);
  f.b = make_float2(0.0f, 0.0f);
}

// A NaN maximum (the bf16 overload of fast_update() propagates NaN into it) takes the branch
// too and turns the whole state into NaN, which no later update can undo: a row that holds a
// NaN gives NaN, as mx.logsumexp (mlx-impl/node.py:401) does, whichever exponential path
// the NaN itself would have taken.
__device__ __forceinline__ void fast_raise(Fast& f, float vmax, float c) {
  if (!(vmax <= f.m)) {
    const float mc_new = vmax * c;
    const float r = ex2f(f.mc - mc_new);
    const float2 r2 = make_float2(r, r);
    f.a = __fmul2_rn(f.a, r2);
    f.b = __fmul2_rn(f.b, r2);
    f.m = vmax;
    f.mc = mc_new;
  }
}

__device__ __forceinline__ Online fast_finish(const Fast& f, float c) {
  Online st;
  st.m = f.m;
  const float delta = fmaf(f.m, c, -f.mc);  // exact residual of the product
  st.s = ((f.a.x + f.a.y) + (f.b.x + f.b.y)) * ex2f(-delta);
  return st;
}

// 2^x for x <= 0 on the FMA pipe (Cody-Waite split + cubic, relative error 7.5e-5), used
// for a few logits per vector to take load off the exp unit.
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -126.0f);
  const float t = x + 12582912.0f;           // 1.5 * 2^23: low mantissa bits = round(x)
  const float fr = x - (t - 12582912.0f);    // in [-0.5, 0.5]
  float p = fmaf(fr, 0.0551716648f, 0.2426111251f);
  p = fmaf(p, fr, 0.6932609677f);
  p = fmaf(p, fr, 0.9999280572f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}

// The same for two values at once with packed f32x2 arithmetic (12 instructions per pair).
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
  x.x = fmaxf(x.x, -126.0f);
  x.y = fmaxf(x.y, -126.0f);
  const float2 magic = make_float2(12582912.0f, 12582912.0f);
  const float2 t = __fadd2_rn(x, magic);
  const float2 j = __fadd2_rn(t, make_float2(-12582912.0f, -12582912.0f));
  const float2 fr = __ffma2_rn(j, make_float2(-1.0f, -1.0f), x);
  float2 p = __ffma2_rn(fr, make_float2(0.0551716648f, 0.0551716648f),
                        make_float2(0.2426111251f, 0.2426111251f));
  p = __ffma2_rn(p, fr, make_float2(0.6932609677f, 0.6932609677f));
  p = __ffma2_rn(p, fr, make_float2(0.9999280572f, 0.9999280572f));
  float2 r;
  r.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
  return r;
}

// Pair number `slot` (0..3) of an 8-logit vector; the first POLY logits of the vector take
// the polynomial.
template <int POLY>
__device__ __forceinline__ float2 ex2_pair(float2 t, int slot) {
  if (2 * slot + 1 < POLY) return ex2_poly2(t);
  float2 e;
  e.x = (2 * slot < POLY) ? ex2_poly(t.x) : ex2f(t.x);
  e.y = ex2f(t.y);
  return e;
}

// 8 bf16 logits
// (both overloads return the largest logit of the vector; for bf16 it is NaN when the vector
// holds one, because the polynomial exponentials would otherwise lose it; fp32 vectors take
// ex2.approx for every logit, which keeps a NaN in the sum by itself)
template <int POLY>
__device__ __forceinline__ float fast_update(Fast& f, uint4 v, float c, __nv_bfloat16) {
  const __nv_bfloat162 mx = __hmax2_nan(__hmax2_nan(as_bf162(v.x), as_bf162(v.y)),
                                        __hmax2_nan(as_bf162(v.z), as_bf162(v.w)));
  const uint32_t mw = *reinterpret_cast<const uint32_t*>(&mx);
  const float vmax = fmax_nan(bf16_lo(mw), bf16_hi(mw));  // NaN if any of the 8 logits is
  fast_raise(f, vmax, c);
  const float2 c2 = make_float2(c, c);
  const float2 n2 = make_float2(-f.mc, -f.mc);
  const float2 t0 = __ffma2_rn(make_float2(bf16_lo(v.x), bf16_hi(v.x)), c2, n2);
  const float2 t1 = __ffma2_rn(make_float2(bf16_lo(v.y), bf16_hi(v.y)), c2, n2);
  const float2 t2 = __ffma2_rn(make_float2(bf16_lo(v.z), bf16_hi(v.z)), c2, n2);
  const float2 t3 = __ffma2_rn(make_float2(bf16_lo(v.w), bf16_hi(v.w)), c2, n2);
  const float2 e0 = ex2_pair<POLY>(t0, 0);
  const float2 e1 = ex2_pair<POLY>(t1, 1);
  const float2 e2 = ex2_pair<POLY>(t2, 2);
  const float2 e3 = ex2_pair<POLY>(t3, 3);
  f.a = __fadd2_rn(f.a, __fadd2_rn(e0, e1));
  f.b = __fadd2_rn(f.b, __fadd2_rn(e2, e3));
  return vmax;
}

// 4 fp32 logits
template <int POLY>
__device__ __forceinline__ float fast_update(Fast& f, uint4 v, float c, float) {
  const float x0 = __uint_as_float(v.x), x1 = __uint_as_float(v.y);
  const float x2 = __uint_as_float(v.z), x3 = __uint_as_float(v.w);
  const float vmax = fmaxf(fmaxf(x0, x1), fmaxf(x2, x3));
  fast_raise(f, vmax, c);
  const float2 c2 = make_float2(c, c);
  const float2 n2 = make_float2(-f.mc, -f.mc);
  const float2 t0 = __ffma2_rn(make_float2(x0, x1), c2, n2);
  const float2 t1 = __ffma2_rn(make_float2(x2, x3), c2, n2);
  f.a = __fadd2_rn(f.a, make_float2(ex2f(t0.x), ex2f(t0.y)));
  f.b = __fadd2_rn(f.b, make_float2(ex2f(t1.x), ex2f(t1.y)));
  return vmax;
}

// Largest logit of a 16-byte vector, without touching any state.
__device__ __forceinline__ float vec_max(uint4 v, __nv_bfloat16) {
  const __nv_bfloat162 mx = __hmax2(__hmax2(as_bf162(v.x), as_bf162(v.y)),
                                    __hmax2(as_bf162(v.z), as_bf162(v.w)));
  const uint32_t mw = *reinterpret_cast<const uint32_t*>(&mx);
  return fmaxf(bf16_lo(mw), bf16_hi(mw));
}
__device__ __forceinline__ float vec_max(uint4 v, float) {
  return fmaxf(fmaxf(__uint_as_float(v.x), __uint_as_float(v.y)),
               fmaxf(__uint_as_float(v.z), __uint_as_float(v.w)));
}

__device__ __forceinline__ void online_update_scalar(Online& st, float x, float c) {
  online_raise(st, x, c);
  st.s += ex2f((x - st.m) * c);
}

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float from_float_neg_inf(float) { return __int_as_float(0xff800000); }
__device__ __forceinline__ __nv_bfloat16 from_float_neg_inf(__nv_bfloat16) {
  return __ushort_as_bfloat16(static_cast<unsigned short>(0xff80));
}

// Merge the 32 per-thread states of a warp; every lane gets the result.
__device__ __forceinline__ void online_warp_reduce(Online& st, float c) {
  float m = st.m;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float s = st.s * ex2f((st.m - m) * c);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  st.m = m;
  st.s = s;
}

}  // namespace tome
