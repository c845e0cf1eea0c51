// Arithmetic of the deterministic alias construction, shared by the table builders and by the
// online walk that evaluates single slots without building a table.
//
//   B = min(40, 62 - ceil(log2 n)), C = 2^B, q_i = trunc(w_i * 2^(B-1-e)) with e = floor(log2 max w),
//   Q_i = q_0 + .. + q_(i-1), W = Q_n, K = n*C / W (one IEEE double division),
//   g(Q) = n*C if Q == W else min(n*C, trunc((double)Q * K)),  M_i = g(Q_i + q_i) - g(Q_i).
#pragma once
#include <math_constants.h>

#include "skw_device.cuh"

namespace skw {

__device__ __forceinline__ float sane_weight(float w) {
  return (w > 0.0f && w < CUDART_INF_F) ? w : 0.0f;
}
__device__ __forceinline__ int bucket_bits(u32 n) {
  const int L = n <= 1 ? 0 : 32 - __clz((int)(n - 1));
  return min(40, 62 - L);
}
__device__ __forceinline__ double pow2d(int e) {
  return __longlong_as_double((long long)(e + 1023) << 52);
}
// 2^(B-1-e), e = exponent of the largest weight.
__device__ __forceinline__ double weight_scale(float wmax, int B) {
  const int e = (int)((__double_as_longlong((double)wmax) >> 52) & 0x7FF) - 1023;
  return pow2d(B - 1 - e);
}
__device__ __forceinline__ u64 quantise(float w, double scale) {
  return __double2ull_rz(__dmul_rn((double)w, scale));
}
// The same value as quantise(w, 2^s) from the bits of w (w > 0 finite or 0), without the fp64
// conversions: w = M * 2^(max(ew, 1) - 150) with M the 24-bit significand (no hidden bit when the
// exponent field ew is 0), so trunc(w * 2^s) = (M * 2^40) >> (190 - s - max(ew, 1)).  The shift
// count is at least 24 for every weight up to the one s was derived from, and the PTX shift gives 0
// for counts of 64 and more (weights too small to register), which C++ leaves undefined.
__device__ __forceinline__ u64 quantise_bits(float w, int s) {
  const u32 b = __float_as_uint(w);
  const u32 ew = b >> 23;
  const u32 M = (b & 0x7FFFFFu) | (ew ? 0x800000u : 0u);
  const u32 r = (u32)(190 - s) - max(ew, 1u);
  u64 q;
  asm("shr.b64 %0, %1, %2;" : "=l"(q) : "l"((u64)(M << 8) << 32), "r"(r));
  return q;
}
// s of quantise_bits for the largest weight wmax (> 0): B - 1 - floor(log2 wmax)
__device__ __forceinline__ int weight_shift(float wmax, int B) {
  const u32 b = __float_as_uint(wmax);
  const u32 ew = b >> 23;
  const int e = ew ? (int)ew - 127 : (31 - __clz((int)(b & 0x7FFFFFu))) - 149;
  return B - 1 - e;
}
__device__ __forceinline__ float mass_to_prob_fast(u64 m, int B) {
  // one rounding (u64 -> fp32, nearest even) then an exact power-of-two scale: the same bits as
  // rounding the exact quotient m / 2^B once
  return __ull2float_rn(m) * __uint_as_float((u32)(127 - B) << 23);
}

__device__ __forceinline__ double mass_factor(u32 n, int B, u64 W) {
  return __ddiv_rn(__ull2double_rn((u64)n << B), __ull2double_rn(W));
}
// g(Q): cumulative mass up to cumulative quantised weight Q.
__device__ __forceinline__ u64 cum_mass(u64 Q, u64 W, u64 nC, double K) {
  if (Q == W) return nC;
  const u64 g = __double2ull_rz(__dmul_rn(__ull2double_rn(Q), K));
  return g < nC ? g : nC;
}
__device__ __forceinline__ float mass_to_prob(u64 m, int B) {
  return __double2float_rn(__dmul_rn(__ull2double_rn(m), pow2d(-B)));
}

}  // namespace skw
