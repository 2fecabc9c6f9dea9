// Rounding helpers shared by the key and the value quantizer (sm_100a).
#pragma once

#include "pq_common.cuh"

namespace pq {
namespace {

// ---------------------------------------------------------------------------------------------
// Fast paths with an exact fallback.
//
// The reference's results are roundings to a 16-bit type of fp32 library results (atan2f, sqrtf, an
// IEEE division).  A cheaper fp32 approximation gives the same 16-bit result whenever it lies farther
// from the nearest rounding tie than its own error; only the remaining fraction of a percent takes the
// library call.  `rounds_safely` implements that test; the margins are validated exhaustively over
// every pair of 16-bit inputs by pq_selftest_quantizer (see tests/test_quantizer_gpu.py).
// fp32 keys always take the exact path.  The exact routines are kept out of line so the unrolled hot
// code stays small enough for the instruction cache.
// ---------------------------------------------------------------------------------------------
constexpr unsigned kTieMargin = 24;     // fp32 units in the last place kept clear on both sides of a tie

template <typename T> __device__ __forceinline__ bool rounds_safely(float v);
template <> __device__ __forceinline__ bool rounds_safely<__nv_bfloat16>(float v) {
  // bf16 keeps the top 16 bits: ties sit at 0x8000 in the low half
  const unsigned low = __float_as_uint(v) & 0xffffu;
  return (low - (0x8000u - kTieMargin)) > 2u * kTieMargin;
}
template <> __device__ __forceinline__ bool rounds_safely<__half>(float v) {
  // fp16 keeps 10 mantissa bits: ties sit at 0x1000 in the low 13 bits, for values in its normal range
  const unsigned bits = __float_as_uint(v);
  const unsigned low = bits & 0x1fffu;
  const unsigned mag = bits & 0x7fffffffu;
  const bool normal = mag >= 0x38800000u && mag < 0x47000000u;     // 2^-14 <= |v| < 32768
  return normal && (low - (0x1000u - kTieMargin)) > 2u * kTieMargin;
}
template <> __device__ __forceinline__ bool rounds_safely<float>(float) { return false; }

// One test for an (angle, radius) pair from the approximations: both lie in the ordinary range (2^-100 .. 2^100
// for bf16, the normal range of fp16) and both keep clear of a rounding tie of T by 32 fp32 units in the last place
// (the zone [tie - 32, tie + 31] of the low bits, found by one addition and one mask).  The angle magnitude never
// exceeds pi and is NaN only when the radius is NaN too, so its upper bound needs no test.
template <typename T> __device__ __forceinline__ bool polar_safe(float a, float r);
template <> __device__ __forceinline__ bool polar_safe<__nv_bfloat16>(float a, float r) {
  const unsigned ua = __float_as_uint(a), ur = __float_as_uint(r);
  const bool range = (ua & 0x7fffffffu) > 0x0d800000u && (ur - 0x0d800001u) < (0x71800000u - 0x0d800001u);
  return range && ((ua + 0x8020u) & 0xffc0u) != 0u && ((ur + 0x8020u) & 0xffc0u) != 0u;
}
template <> __device__ __forceinline__ bool polar_safe<__half>(float a, float r) {
  const unsigned ua = __float_as_uint(a), ur = __float_as_uint(r);
  const bool range = (ua & 0x7fffffffu) >= 0x38800000u && (ur - 0x38800000u) < (0x47000000u - 0x38800000u);
  return range && ((ua + 0x1020u) & 0x1fc0u) != 0u && ((ur + 0x1020u) & 0x1fc0u) != 0u;
}
template <> __device__ __forceinline__ bool polar_safe<float>(float, float) { return false; }

// 2^-100 < |v| < 2^100 and not NaN: the range in which the approximations neither flush nor overflow.
// It is tested on RESULTS: zero, NaN, inf or denormal inputs and underflowing ratios all surface there.
__device__ __forceinline__ bool mid_range(float v) {
  return ((__float_as_uint(v) & 0x7fffffffu) - 0x0d800001u) < (0x71800000u - 0x0d800001u);
}

// round two fp32 values to T and back with one packed conversion (full-rate pipe, unlike the scalar cvt)
template <typename T> __device__ __forceinline__ void round2(float a, float b, float& ra, float& rb) {
  if constexpr (Elem<T>::kDtype == PQ_F32) { ra = a; rb = b; }
  else { const float2 f = unpack2<Elem<T>::kDtype>(pack2<Elem<T>::kDtype>(a, b)); ra = f.x; rb = f.y; }
}

// Reciprocal for the multiply-instead-of-divide fast path: correctly rounded for an ordinary divisor, NaN otherwise
// (zero, denormal, huge, NaN), so that every product with it fails the "quotient < 256" test and takes the exact
// division - the divisor's validity costs nothing per element.
__device__ __forceinline__ float guarded_rcp(float step) {
  return mid_range(step) ? __frcp_rn(step) : __int_as_float(0x7fc00000);
}

// exact IEEE quotient, out of line: taken by a fraction of a percent of the items
__device__ __noinline__ float div_exact(float a, float b) { return __fdiv_rn(a, b); }

// Quotient a / b from the correctly rounded reciprocal r = RN(1 / b): one product and one remainder correction,
//   q0 = RN(a r);  e = a - b q0 (exact, one FMA);  q = RN(q0 + e r).
// For ordinary operands this is the correctly rounded quotient - in particular it is exact whenever a / b is
// exactly representable, which covers the only inputs for which a 16-bit rounding of the quotient could differ
// from the rounding of an approximation: quotients of two 16-bit values that sit exactly on a rounding tie.  No
// tie test and no branch are needed; operands outside the ordinary range arrive with r = NaN (guarded_rcp) and are
// sent to the IEEE division by the caller's range test on q.  Checked against __fdiv_rn for every pair of 16-bit
// operands by pq_selftest_quantizer (which = 1).
__device__ __forceinline__ float div_refined(float a, float b, float r) {
  const float q0 = a * r;
  const float e = __fmaf_rn(-b, q0, a);
  return __fmaf_rn(e, r, q0);
}

// a - b of two packed 16-bit pairs, rounded once to the same type.  torch computes RN_T(RN_fp32(a - b)); the fp32
// difference of two 16-bit values is exact whenever the result is anywhere near a rounding tie of T (the operands'
// exponents are then close), so the single rounding of the packed instruction gives the same value - checked for
// every pair of 16-bit operands by pq_selftest_quantizer (which = 2).
template <int DT> __device__ __forceinline__ uint32_t sub2_packed(uint32_t a, uint32_t b) {
  uint32_t d;
  if constexpr (DT == PQ_BF16) asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  else asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// a + b and a * b of packed 16-bit pairs, rounded once.  torch evaluates both in fp32 and rounds the result to T; a
// product of two 16-bit values is exact in fp32, and the sum obeys the argument given at sub2_packed.
template <int DT> __device__ __forceinline__ uint32_t add2_packed(uint32_t a, uint32_t b) {
  uint32_t d;
  if constexpr (DT == PQ_BF16) asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  else asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
template <int DT> __device__ __forceinline__ uint32_t mul2_packed(uint32_t a, uint32_t b) {
  uint32_t d;
  if constexpr (DT == PQ_BF16) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  else asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// floor of a value in [0, 2^22) by a round-toward-zero addition of 2^23: the integer sits in the low mantissa bits
__device__ __forceinline__ uint32_t floor_bits(float v) { return __float_as_uint(__fadd_rz(v, 8388608.0f)); }

}  // namespace
}  // namespace pq
