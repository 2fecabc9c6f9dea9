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

}  // namespace
}  // namespace pq
