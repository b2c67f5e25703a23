// Arithmetic of the tcgen05 kernels' softmax: P = 2^(s * scale - m) for a chunk of 32 scores of one
// row, as packed two-wide FP32 instructions (fma/add .f32x2, new on sm_100) and with part of the
// exponentials evaluated by a polynomial on the FMA pipe instead of the MUFU pipe.
//
// Why: a 128 x 128 tile needs 16 384 exponentials, and the MUFU pipe retires 16 per clock per SM:
// 1024 cycles, as long as the tile's two tensor-core products take.  Splitting the exponentials
// between MUFU and FMA pipes shortens that, and the two-wide instructions halve the issue slots of
// the scaling and of the row sum.
#pragma once

#include <cuda_fp8.h>
#include <stdint.h>

#include "ptx.cuh"

namespace atrex_sm100 {

typedef unsigned long long f32x2;   // two floats in one 64-bit register

__device__ __forceinline__ f32x2 pack2(float a, float b) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// 2^x for a pair without the MUFU pipe.  x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f by the
// degree-3 minimax polynomial (relative error 7.5e-5, 26 times below BF16's rounding step), 2^n by
// adding n to the exponent field.  x is clamped at -126, so the result is never below 2^-126:
// callers use it only where every score is finite (tiles without masked columns), where such a term
// is negligible against the row's own maximum; exact zeros for masked scores need ex2.approx.
__device__ __forceinline__ void exp2_poly2(f32x2 x2, float& p0, float& p1) {
  float a, b;
  unpack2(x2, a, b);
  x2 = pack2(fmaxf(a, -126.f), fmaxf(b, -126.f));
  const f32x2 magic = pack2(12582912.f, 12582912.f);   // 1.5 * 2^23: the sum's low mantissa bits hold round(x)
  const f32x2 t2 = add2(x2, magic);
  const f32x2 f2 = sub2(x2, sub2(t2, magic));
  f32x2 p2 = fma2(f2, pack2(0.05517167f, 0.05517167f), pack2(0.24261113f, 0.24261113f));
  p2 = fma2(p2, f2, pack2(0.69326097f, 0.69326097f));
  p2 = fma2(p2, f2, pack2(0.99992806f, 0.99992806f));
  float t0, t1, q0, q1;
  unpack2(t2, t0, t1);
  unpack2(p2, q0, q1);
  p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(t0) << 23));
  p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(t1) << 23));
}

// One pair of probabilities; kPoly selects the pipe.
template <bool kPoly>
__device__ __forceinline__ void exp2_pair(uint32_t s0, uint32_t s1, f32x2 scale2, f32x2 negm2, float& p0, float& p1) {
  const f32x2 x2 = fma2(pack2(__uint_as_float(s0), __uint_as_float(s1)), scale2, negm2);
  if (kPoly) {
    exp2_poly2(x2, p0, p1);
  } else {
    float a, b;
    unpack2(x2, a, b);
    p0 = fast_exp2(a);
    p1 = fast_exp2(b);
  }
}

// 32 scores -> 16 BF16 pairs; the row sum accumulates in two packed registers.
// kPolyOf8: how many of every 8 pairs take the polynomial (0 where scores may be -inf).
template <int kPolyOf8>
__device__ __forceinline__ void exp32_bf16(const uint32_t* s, f32x2 scale2, f32x2 negm2, f32x2 (&sum2)[2],
                                           uint32_t (&packed)[16]) {
#pragma unroll
  for (int q = 0; q < 16; ++q) {
    float p0, p1;
    if ((q & 7) < kPolyOf8) exp2_pair<true>(s[2 * q], s[2 * q + 1], scale2, negm2, p0, p1);
    else exp2_pair<false>(s[2 * q], s[2 * q + 1], scale2, negm2, p0, p1);
    sum2[q & 1] = add2(sum2[q & 1], pack2(p0, p1));
    packed[q] = pack_bf16(p0, p1);
  }
}

// 32 scores -> 8 registers of four E4M3 each.
template <int kPolyOf8>
__device__ __forceinline__ void exp32_e4m3(const uint32_t* s, f32x2 scale2, f32x2 negm2, f32x2 (&sum2)[2],
                                           uint32_t (&packed)[8]) {
#pragma unroll
  for (int q = 0; q < 16; q += 2) {
    float p0, p1, p2, p3;
    if ((q & 7) < kPolyOf8) exp2_pair<true>(s[2 * q], s[2 * q + 1], scale2, negm2, p0, p1);
    else exp2_pair<false>(s[2 * q], s[2 * q + 1], scale2, negm2, p0, p1);
    if (((q + 1) & 7) < kPolyOf8) exp2_pair<true>(s[2 * q + 2], s[2 * q + 3], scale2, negm2, p2, p3);
    else exp2_pair<false>(s[2 * q + 2], s[2 * q + 3], scale2, negm2, p2, p3);
    sum2[0] = add2(sum2[0], pack2(p0, p1));
    sum2[1] = add2(sum2[1], pack2(p2, p3));
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(p0, p1), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(p2, p3), __NV_SATFINITE, __NV_E4M3);
    packed[q >> 1] = lo | (hi << 16);
  }
}

__device__ __forceinline__ float sum_of(const f32x2 (&sum2)[2]) {
  float a, b, c, d;
  unpack2(sum2[0], a, b);
  unpack2(sum2[1], c, d);
  return (a + b) + (c + d);
}

}  // namespace atrex_sm100
