// Polar key quantizer for sm_100a.
//
// One CTA quantises one (batch, kv head, token group) tile: G tokens x 128
// channels.  The arithmetic is the reference's op sequence
// (models/modeling_llama_polar.py:143-155 of ericshwu/PolarQuant) with every
// intermediate rounded to the key dtype exactly where torch rounds it, so codes
// and scales are bit-identical to the eager ops on CUDA:
//
//   phi   = RN(atan2f(y, x));  if phi < 0: phi = RN(phi + float(2*pi))       (:143-144)
//   tstep = RN(RN(max phi - min phi) / 2^tbits)                              (:146-147)
//   theta = min(u8(floor(RN(RN(phi - min phi) / tstep))), 2^tbits - 1)       (:148)
//   r     = RN(sqrtf(RN(x*x) + RN(y*y))), same min/max/step/floor/clamp     (:150-153)
//   code  = (rho << tbits) + theta                                           (:155)
//
// Pair d is channels (d, d + 64) (the (2, 64) view at :141).  Traffic is the
// ideal one pass: every key element is read once (8/16-byte loads, any token /
// head / batch stride) and 64 code bytes per token plus four 64-wide scale rows
// per group are written.
#include <type_traits>

#include "pq_common.cuh"
#include "pq_rounding.cuh"

namespace pq {
namespace {

constexpr int kQuantThreads = 256;

__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float min_nan(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// NaN-propagating max / min of two packed 16-bit pairs of type DT (exact: the operands are already values of DT)
template <int DT> __device__ __forceinline__ uint32_t max2_nan(uint32_t a, uint32_t b) {
  uint32_t r;
  if constexpr (DT == PQ_BF16) asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  else asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
template <int DT> __device__ __forceinline__ uint32_t min2_nan(uint32_t a, uint32_t b) {
  uint32_t r;
  if constexpr (DT == PQ_BF16) asm("min.NaN.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  else asm("min.NaN.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// four consecutive elements starting at p
template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  uint4 u = ldg_stream(p);
  v[0] = __uint_as_float(u.x); v[1] = __uint_as_float(u.y);
  v[2] = __uint_as_float(u.z); v[3] = __uint_as_float(u.w);
}
template <> __device__ __forceinline__ void load4<__half>(const __half* p, float (&v)[4]) {
  uint2 u;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(u.x), "=r"(u.y) : "l"(p));
  float2 a = unpack2<PQ_F16>(u.x), b = unpack2<PQ_F16>(u.y);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  uint2 u;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(u.x), "=r"(u.y) : "l"(p));
  float2 a = unpack2<PQ_BF16>(u.x), b = unpack2<PQ_BF16>(u.y);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

// float -> int64 -> uint8, the cast ATen performs: NaN gives 0, +inf and anything past 2^63 give 0xff
__device__ __forceinline__ unsigned cast_like_aten(float q) {
  return static_cast<unsigned>(static_cast<long long>(q)) & 0xffu;
}

// atan2 by the odd polynomial atan(z) = z * P(z^2) on z = min/max in [0, 1] (relative error 2.4e-7 when
// evaluated in fp32) and the usual octant fix-ups.
__device__ __forceinline__ float atan2_approx(float y, float x) {
  const unsigned ix = __float_as_uint(x) & 0x7fffffffu, iy = __float_as_uint(y) & 0x7fffffffu;
  const unsigned imx = max(ix, iy), imn = min(ix, iy);            // integer order == order of magnitudes
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(__uint_as_float(imx)));
  const float z = __uint_as_float(imn) * r, u = z * z;
  float p = -0.004780454095453024f;
  p = fmaf(p, u, 0.024557121098041534f);
  p = fmaf(p, u, -0.059904709458351135f);
  p = fmaf(p, u, 0.09942758828401566f);
  p = fmaf(p, u, -0.14029419422149658f);
  p = fmaf(p, u, 0.19971375167369843f);
  p = fmaf(p, u, -0.3333209455013275f);
  p = fmaf(p, u, 0.9999999403953552f);
  float a = p * z;
  if (iy > ix) a = 1.5707963267948966f - a;
  if (x < 0.0f) a = 3.141592653589793f - a;
  return __float_as_int(y) < 0 ? -a : a;      // sign bit, so that y = -0 gives -pi (x < 0) like atan2f
}

// exact (library) angle and radius before rounding, out of line: taken by a fraction of a percent of the items
__device__ __forceinline__ float2 polar_exact_inline(float x, float y, bool norm_separate) {
  const float s = norm_separate ? __fadd_rn(__fmul_rn(x, x), __fmul_rn(y, y)) : __fmaf_rn(y, y, __fmul_rn(x, x));
  return make_float2(atan2f(y, x), __fsqrt_rn(s));
}
__device__ __noinline__ float2 polar_exact(float x, float y, bool norm_separate) {
  return polar_exact_inline(x, y, norm_separate);
}

// Which key dtypes use the approximations.  bf16 ties are 2^16 fp32 steps apart, so about one value in a thousand
// needs the exact routine and a warp rarely diverges.  fp16 ties are 2^13 apart: with four tests per pair of items
// half of all warps would take the slow branch (measured: 2.7 ms against 1.9 ms for the exact-only code at the 32k
// prefill shape), so fp16 - like fp32, where nothing is rounded - stays on the exact routines.
template <typename T> struct FastPathPays { static constexpr bool value = false; };
template <> struct FastPathPays<__nv_bfloat16> { static constexpr bool value = true; };

// Angle and radius of the four pairs a thread holds of one token, each rounded to T where torch rounds:
//   phi = RN(atan2f(y, x)); if (phi < 0) phi = RN(phi + wrap);   rad = RN(sqrtf(x^2 + y^2)).
// Fast form (16-bit T): polynomial arctangent and rsqrt-based root, accepted when polar_safe says the approximation
// rounds like the exact value; one branch per token covers the rare items that need the library routines.
template <typename T, bool FAST = true, bool FORCE = false>
__device__ __forceinline__ void polar_of4(const float (&x)[4], const float (&y)[4], float wrap, bool norm_separate,
                                          float (&phi)[4], float (&rad)[4]) {
  constexpr bool kFast = FAST && (FORCE || FastPathPays<T>::value) && Elem<T>::kDtype != PQ_F32;
  float a[4], r[4];
  if constexpr (kFast) {
    bool all_ok = true;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      a[k] = atan2_approx(y[k], x[k]);
      // for 16-bit keys the two products are exact in fp32, so both forms of the sum agree
      const float s = __fmaf_rn(y[k], y[k], __fmul_rn(x[k], x[k]));
      float rs;
      asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(rs) : "f"(s));
      r[k] = s * rs;
      all_ok = all_ok & polar_safe<T>(a[k], r[k]);       // bitwise: no short-circuit branches in the hot path
    }
    if (!all_ok) {                             // rarely taken: redo the unsafe items with the library routines
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (!polar_safe<T>(a[k], r[k])) { const float2 e = polar_exact(x[k], y[k], norm_separate); a[k] = e.x; r[k] = e.y; }
    }
  } else {                                     // exact-only dtypes: the library calls inline, no call overhead
#pragma unroll
    for (int k = 0; k < 4; ++k) { const float2 e = polar_exact_inline(x[k], y[k], norm_separate); a[k] = e.x; r[k] = e.y; }
  }
#pragma unroll
  for (int k = 0; k < 4; k += 2) {
    round2<T>(a[k], a[k + 1], a[k], a[k + 1]);
    float w[2];
    round2<T>(__fadd_rn(a[k], wrap), __fadd_rn(a[k + 1], wrap), w[0], w[1]);
    phi[k] = a[k] < 0.0f ? w[0] : a[k];
    phi[k + 1] = a[k + 1] < 0.0f ? w[1] : a[k + 1];
    round2<T>(r[k], r[k + 1], rad[k], rad[k + 1]);
  }
}

// The same for 16-bit T with the results as packed pairs (pairs 0-1 and 2-3), which is how the kernel keeps them
// between its two passes: one conversion rounds the angle, the wrap is added in fp32 to the rounded value and the
// selected value is packed (packing an already rounded value is exact), the radius is packed once.
template <typename T, bool FAST = true, bool FORCE = false>
__device__ __forceinline__ void polar_of4_packed(const float (&x)[4], const float (&y)[4], float wrap, bool norm_separate,
                                                 uint32_t (&phi_w)[2], uint32_t (&rad_w)[2]) {
  constexpr bool kFast = FAST && (FORCE || FastPathPays<T>::value);
  constexpr int DT16 = Elem<T>::kDtype == PQ_BF16 ? PQ_BF16 : PQ_F16;
  float a[4], r[4];
  if constexpr (kFast) {
    bool all_ok = true;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      a[k] = atan2_approx(y[k], x[k]);
      const float s = __fmaf_rn(y[k], y[k], __fmul_rn(x[k], x[k]));
      float rs;
      asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(rs) : "f"(s));
      r[k] = s * rs;
      all_ok = all_ok & polar_safe<T>(a[k], r[k]);
    }
    if (!all_ok) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (!polar_safe<T>(a[k], r[k])) { const float2 e = polar_exact(x[k], y[k], norm_separate); a[k] = e.x; r[k] = e.y; }
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) { const float2 e = polar_exact_inline(x[k], y[k], norm_separate); a[k] = e.x; r[k] = e.y; }
  }
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const float2 ar = unpack2<DT16>(pack2<DT16>(a[2 * k], a[2 * k + 1]));
    const float p0 = ar.x < 0.0f ? __fadd_rn(ar.x, wrap) : ar.x, p1 = ar.y < 0.0f ? __fadd_rn(ar.y, wrap) : ar.y;
    phi_w[k] = pack2<DT16>(p0, p1);
    rad_w[k] = pack2<DT16>(r[2 * k], r[2 * k + 1]);
  }
}

// Quantisation level of d = RN(v - lo) (already rounded to T): min(u8(floor(RN(d / step))), top), the reference's
// chain floor -> uint8 cast -> clamp.  `exact` is the reference arithmetic verbatim.
template <typename T> __device__ __forceinline__ unsigned level_exact(float d, float step, unsigned top) {
  const float q = Elem<T>::round(__fdiv_rn(d, step));
  // in [0, 256) truncation to int is the floor and equals the reference's cast chain
  const bool small = q >= 0.0f && q < 256.0f;
  unsigned u = static_cast<unsigned>(__float2int_rz(small ? q : 0.0f));
  if (!small) u = cast_like_aten(floorf(q));
  return u < top ? u : top;
}
__device__ __noinline__ unsigned level_exact_bf16(float d, float step, unsigned top) { return level_exact<__nv_bfloat16>(d, step, top); }
__device__ __noinline__ unsigned level_exact_f16(float d, float step, unsigned top) { return level_exact<__half>(d, step, top); }
template <typename T> __device__ __forceinline__ unsigned level_exact_call(float d, float step, unsigned top) {
  if constexpr (Elem<T>::kDtype == PQ_BF16) return level_exact_bf16(d, step, top);
  else if constexpr (Elem<T>::kDtype == PQ_F16) return level_exact_f16(d, step, top);
  else return level_exact<T>(d, step, top);
}

// Code bytes (rho << tbits) + theta of four pairs from the rounded differences dt = RN(phi - tmn), dr = RN(rad - rmn).
// Fast form: the quotient by div_refined (correctly rounded, no tie test), accepted while 0 <= q < 255 - which also
// screens NaN, negative and degenerate steps (their reciprocal is NaN) - then RN to T, clamp and floor in floating
// point (a quotient below 255 cannot round up to 256, where the reference's uint8 cast wraps to 0).
template <typename T, bool FAST = true>
__device__ __forceinline__ uint32_t codes_of4(const float (&dt)[4], const float (&dr)[4], const float (&tstep)[4],
                                              const float (&trcp)[4], const float (&rstep)[4], const float (&rrcp)[4],
                                              unsigned ttop, unsigned rtop, int tbits) {
  constexpr bool kFast = FAST && Elem<T>::kDtype != PQ_F32;
  uint32_t word = 0;
  if constexpr (kFast) {
    float qt[4], qr[4];
    bool all_ok = true;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      qt[k] = div_refined(dt[k], tstep[k], trcp[k]);
      qr[k] = div_refined(dr[k], rstep[k], rrcp[k]);
      all_ok = all_ok & (__float_as_uint(qt[k]) < 0x437f0000u) & (__float_as_uint(qr[k]) < 0x437f0000u);   // [0, 255)
    }
    if (all_ok) {
      // round to T and clamp to the top level on packed pairs (the clamp is exact: both operands are values of T),
      // floor in fp32 by a round-toward-zero addition, gather the low bytes of the four codes with byte permutes
      constexpr int DT16 = Elem<T>::kDtype == PQ_BF16 ? PQ_BF16 : PQ_F16;
      const uint32_t tf2 = pack2<DT16>(static_cast<float>(ttop), static_cast<float>(ttop));
      const uint32_t rf2 = pack2<DT16>(static_cast<float>(rtop), static_cast<float>(rtop));
      uint32_t c[4];
#pragma unroll
      for (int k = 0; k < 4; k += 2) {
        const float2 t = unpack2<DT16>(min2_nan<DT16>(pack2<DT16>(qt[k], qt[k + 1]), tf2));
        const float2 r = unpack2<DT16>(min2_nan<DT16>(pack2<DT16>(qr[k], qr[k + 1]), rf2));
        c[k] = (floor_bits(r.x) << tbits) + floor_bits(t.x);
        c[k + 1] = (floor_bits(r.y) << tbits) + floor_bits(t.y);
      }
      return __byte_perm(__byte_perm(c[0], c[1], 0x0040), __byte_perm(c[2], c[3], 0x0040), 0x5410);
    }
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const unsigned th = kFast ? level_exact_call<T>(dt[k], tstep[k], ttop) : level_exact<T>(dt[k], tstep[k], ttop);
    const unsigned rh = kFast ? level_exact_call<T>(dr[k], rstep[k], rtop) : level_exact<T>(dr[k], rstep[k], rtop);
    word |= (((rh << tbits) + th) & 0xffu) << (8 * k);
  }
  return word;
}

// ---- 6-bit packed container (PQ_KEYS_PACKED6; layout stated in include/polarquant_b200.h at pq_keys_repack) ----
constexpr int kPackedStepBytes = 768;      // 16 tokens x 48 bytes
// upper two code bits of the four code bytes of word W, at their places in the H word
__device__ __forceinline__ uint32_t h_part(uint32_t word, int W) {
  const uint32_t hb = (word >> 4) & 0x03030303u;
  return ((hb & 0x3u) | ((hb >> 6) & 0xcu) | (hb & 0x30000u) | ((hb >> 6) & 0xc0000u)) << (4 * W);
}
// the four code bytes of word W back from A_{W / 2} and H
__device__ __forceinline__ uint32_t unpack_word(uint32_t a, uint32_t h, int W) {
  const uint32_t h4 = h >> (4 * W);
  const uint32_t hs = (h4 & 0x3u) | ((h4 & 0xcu) << 6) | (h4 & 0x30000u) | ((h4 & 0xc0000u) << 6);
  return ((a >> (4 * (W & 1))) & 0x0f0f0f0fu) | (hs << 4);
}

// One warp per 16-token step: lane l = 4 g + t owns pairs 16 t .. 16 t + 15 of tokens g and g + 8 in both containers.
__global__ void keys_repack_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int64_t steps,
                                   int to_packed) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  for (int64_t s = blockIdx.x * static_cast<int64_t>(blockDim.x >> 5) + (threadIdx.x >> 5); s < steps;
       s += static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5)) {
    const uint8_t* bytes = (to_packed ? in : out) + s * 16 * kPairs + g * kPairs + 16 * t;
    const uint8_t* tile = (to_packed ? out : in) + s * kPackedStepBytes;
    if (to_packed) {
      const uint4 lo = *reinterpret_cast<const uint4*>(bytes), hi = *reinterpret_cast<const uint4*>(bytes + 8 * kPairs);
      uint4 a; uint2 h;
      a.x = (lo.x & 0x0f0f0f0fu) | ((lo.y & 0x0f0f0f0fu) << 4); a.y = (lo.z & 0x0f0f0f0fu) | ((lo.w & 0x0f0f0f0fu) << 4);
      a.z = (hi.x & 0x0f0f0f0fu) | ((hi.y & 0x0f0f0f0fu) << 4); a.w = (hi.z & 0x0f0f0f0fu) | ((hi.w & 0x0f0f0f0fu) << 4);
      h.x = h_part(lo.x, 0) | h_part(lo.y, 1) | h_part(lo.z, 2) | h_part(lo.w, 3);
      h.y = h_part(hi.x, 0) | h_part(hi.y, 1) | h_part(hi.z, 2) | h_part(hi.w, 3);
      *reinterpret_cast<uint4*>(const_cast<uint8_t*>(tile) + 16 * lane) = a;
      *reinterpret_cast<uint2*>(const_cast<uint8_t*>(tile) + 512 + 8 * lane) = h;
    } else {
      const uint4 a = *reinterpret_cast<const uint4*>(tile + 16 * lane);
      const uint2 h = *reinterpret_cast<const uint2*>(tile + 512 + 8 * lane);
      uint4 lo, hi;
      lo.x = unpack_word(a.x, h.x, 0); lo.y = unpack_word(a.x, h.x, 1); lo.z = unpack_word(a.y, h.x, 2); lo.w = unpack_word(a.y, h.x, 3);
      hi.x = unpack_word(a.z, h.y, 0); hi.y = unpack_word(a.z, h.y, 1); hi.z = unpack_word(a.w, h.y, 2); hi.w = unpack_word(a.w, h.y, 3);
      *reinterpret_cast<uint4*>(const_cast<uint8_t*>(bytes)) = lo;
      *reinterpret_cast<uint4*>(const_cast<uint8_t*>(bytes) + 8 * kPairs) = hi;
    }
  }
}

// lengths = {token groups, residual tokens} on the device; the kernel runs only when lengths[1] + r_add == full
struct WindowGate { const int* lengths; int r_add, full, max_groups; };

// Rotary embedding fused in front of the quantizer (prefill): keys arrive un-rotated, are rotated with the eager
// arithmetic of apply_rotary_pos_emb (rotate-half: channel d pairs with d + 64, the quantizer's own pairing), written
// out for the prefill attention and the residual window, and quantised from registers.
template <typename T> struct RopeFusion {
  const T* cos; const T* sin; int64_t cs_sb, cs_sl;       // (B or 1, L, 128): batch stride (0 = shared), token stride
  T* out; int64_t o_sb, o_sh, o_sl;                        // rotated keys (may be the input buffer), or nullptr
};
__device__ __forceinline__ uint2 ldg8_nc(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
// out = RN(RN(x * cos) + RN(rotate_half(x) * sin)) for four pairs: xr = x c_lo - y s_lo, yr = y c_hi + x s_hi
template <int DT>
__device__ __forceinline__ void rope4_packed(uint2 xw, uint2 yw, uint2 clo, uint2 chi, uint2 slo, uint2 shi, uint2& xr,
                                             uint2& yr) {
  xr.x = sub2_packed<DT>(mul2_packed<DT>(xw.x, clo.x), mul2_packed<DT>(yw.x, slo.x));
  xr.y = sub2_packed<DT>(mul2_packed<DT>(xw.y, clo.y), mul2_packed<DT>(yw.y, slo.y));
  yr.x = add2_packed<DT>(mul2_packed<DT>(yw.x, chi.x), mul2_packed<DT>(xw.x, shi.x));
  yr.y = add2_packed<DT>(mul2_packed<DT>(yw.y, chi.y), mul2_packed<DT>(xw.y, shi.y));
}
// rotation only, for the tokens behind the quantised ones (the residual window): one thread per (token, 4 pairs)
template <typename T>
__global__ void rope_rows_kernel(const T* __restrict__ keys, int64_t sb, int64_t sh, int64_t sl, int Nk, int tok_first,
                                 int tokens, const RopeFusion<T> rope) {
  constexpr int DT16 = Elem<T>::kDtype == PQ_BF16 ? PQ_BF16 : PQ_F16;
  const int bh = blockIdx.y, h = bh % Nk, b = bh / Nk;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int tok = idx >> 4, p0 = (idx & 15) * 4;
  if (tok >= tokens) return;
  const int64_t pos = tok_first + tok;
  const T* row = keys + b * sb + h * sh + pos * sl + p0;
  const T* c = rope.cos + b * rope.cs_sb + pos * rope.cs_sl + p0;
  const T* sn = rope.sin + b * rope.cs_sb + pos * rope.cs_sl + p0;
  uint2 xr, yr;
  rope4_packed<DT16>(ldg8_nc(row), ldg8_nc(row + kPairs), ldg8_nc(c), ldg8_nc(c + kPairs), ldg8_nc(sn), ldg8_nc(sn + kPairs),
                     xr, yr);
  T* o = rope.out + b * rope.o_sb + h * rope.o_sh + pos * rope.o_sl + p0;
  *reinterpret_cast<uint2*>(o) = xr;
  *reinterpret_cast<uint2*>(o + kPairs) = yr;
}

// 16-bit keys, G a multiple of 16 up to kMaxSmemGroup: angle and radius of the group wait in shared memory between
// the two passes (16 bytes per thread and token, conflict-free), so the token loops stay rolled - a small code
// footprint that the instruction cache holds - and a thread needs 64 registers (four CTAs per SM).
// A CTA of eight warps covers 128 tokens: one group of 128, or 128 / G groups side by side for G = 16, 32, 64
// (`wpg` warps per group), so that the fixed cost per CTA - two barriers, the min/max reduction, the reciprocals of
// the steps - is spread over the same number of pairs whatever the group size.  Other multiples of 16 take one
// group per CTA.
constexpr int kMaxSmemGroup = 128;
#ifndef PQ_QUANT16_MIN_CTAS
#define PQ_QUANT16_MIN_CTAS 4
#endif
template <typename T, int WPG, bool ROPE = false>
__global__ void __launch_bounds__(kQuantThreads, PQ_QUANT16_MIN_CTAS)
quantize_kernel16(const T* __restrict__ keys, int64_t sb, int64_t sh, int64_t sl, int Nk, int nb, int G,
                  int rbits, int tbits, unsigned flags, uint8_t* __restrict__ codes, T* __restrict__ rscale,
                  T* __restrict__ rmn_out, T* __restrict__ tscale, T* __restrict__ tmn_out,
                  int64_t c_sb, int64_t c_sh, int64_t s_sb, int64_t s_sh, const WindowGate gate, int total_groups,
                  const RopeFusion<T> rope) {
  constexpr int wpg = WPG;                                 // warps per group
  using E = Elem<T>;
  constexpr int DT16 = E::kDtype == PQ_BF16 ? PQ_BF16 : PQ_F16;
  int group_off = 0;
  if (gate.lengths) {
    group_off = gate.lengths[0];
    if (gate.lengths[1] + gate.r_add != gate.full || group_off < 0 || group_off + nb > gate.max_groups) return;
  }
  extern __shared__ uint4 s_polar[];                       // [G / 16][kQuantThreads]: phi pairs 0-1, 2-3, rad pairs 0-1, 2-3
  __shared__ float red[4][kQuantThreads / 32][kPairs];
  constexpr int gpc = (kQuantThreads / 32) / wpg;          // groups per CTA
  __shared__ float fin[gpc][4][kPairs];                    // per group of the CTA

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gsub = warp / wpg, wsub = warp % wpg;          // this warp's group within the CTA, its place in it
  const int tile = blockIdx.x * gpc + gsub;                // (b * Nk + h) * nb + j; the host keeps it below 2^31
  const bool live = tile < total_groups;                   // the last CTA may hold fewer groups
  const int tl = live ? tile : 0;
  const int j = tl % nb;
  const int bh = tl / nb;
  const int h = bh % Nk, b = bh / Nk;
  const int tsub = lane >> 4;
  const int p0 = (lane & 15) * 4;             // first of this thread's four pairs
  const int tok_step = 2 * wpg;               // tokens the group's warps cover per iteration
  const int ni = live ? G / tok_step : 0;
  const int tok0 = 2 * wsub + tsub;
  const T* row = keys + b * sb + h * sh + (static_cast<int64_t>(j) * G + tok0) * sl + p0;
  const int64_t row_step = tok_step * sl;

  const float wrap = (flags & PQ_QUANT_WRAP_DTYPE) ? E::round(6.283185307179586f) : 6.283185307179586f;
  const bool norm_sep = (flags & PQ_QUANT_NORM_FMA) == 0;

  // identities of the NaN-propagating max / min: -inf and +inf as packed pairs
  constexpr uint32_t kNegInf2 = DT16 == PQ_BF16 ? 0xff80ff80u : 0xfc00fc00u, kPosInf2 = DT16 == PQ_BF16 ? 0x7f807f80u : 0x7c007c00u;
  uint32_t tmx_w[2] = {kNegInf2, kNegInf2}, tmn_w[2] = {kPosInf2, kPosInf2};
  uint32_t rmx_w[2] = {kNegInf2, kNegInf2}, rmn_w[2] = {kPosInf2, kPosInf2};
#pragma unroll 2
  for (int i = 0; i < ni; ++i) {
    float x[4], y[4];
    if constexpr (ROPE) {
      const int64_t pos = static_cast<int64_t>(j) * G + tok0 + i * tok_step;       // token of the sequence
      const T* c = rope.cos + b * rope.cs_sb + pos * rope.cs_sl + p0;
      const T* sn = rope.sin + b * rope.cs_sb + pos * rope.cs_sl + p0;
      uint2 xr, yr;
      rope4_packed<DT16>(ldg8_nc(row), ldg8_nc(row + kPairs), ldg8_nc(c), ldg8_nc(c + kPairs), ldg8_nc(sn),
                         ldg8_nc(sn + kPairs), xr, yr);
      if (rope.out) {
        T* o = rope.out + b * rope.o_sb + h * rope.o_sh + pos * rope.o_sl + p0;
        *reinterpret_cast<uint2*>(o) = xr;
        *reinterpret_cast<uint2*>(o + kPairs) = yr;
      }
      const float2 x01 = unpack2<DT16>(xr.x), x23 = unpack2<DT16>(xr.y), y01 = unpack2<DT16>(yr.x), y23 = unpack2<DT16>(yr.y);
      x[0] = x01.x; x[1] = x01.y; x[2] = x23.x; x[3] = x23.y; y[0] = y01.x; y[1] = y01.y; y[2] = y23.x; y[3] = y23.y;
    } else {
      load4<T>(row, x);
      load4<T>(row + kPairs, y);
    }
    row += row_step;
    uint32_t pw[2], rw[2];
    polar_of4_packed<T>(x, y, wrap, norm_sep, pw, rw);
    s_polar[i * kQuantThreads + threadIdx.x] = make_uint4(pw[0], pw[1], rw[0], rw[1]);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      tmx_w[k] = max2_nan<DT16>(tmx_w[k], pw[k]); tmn_w[k] = min2_nan<DT16>(tmn_w[k], pw[k]);
      rmx_w[k] = max2_nan<DT16>(rmx_w[k], rw[k]); rmn_w[k] = min2_nan<DT16>(rmn_w[k], rw[k]);
    }
  }
  float tmx[4], tmn[4], rmx[4], rmn[4];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    float2 f;
    f = unpack2<DT16>(tmx_w[k]); tmx[2 * k] = f.x; tmx[2 * k + 1] = f.y;
    f = unpack2<DT16>(tmn_w[k]); tmn[2 * k] = f.x; tmn[2 * k + 1] = f.y;
    f = unpack2<DT16>(rmx_w[k]); rmx[2 * k] = f.x; rmx[2 * k + 1] = f.y;
    f = unpack2<DT16>(rmn_w[k]); rmn[2 * k] = f.x; rmn[2 * k + 1] = f.y;
  }
  // combine the two token halves of the warp, then the eight warps
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    tmx[p] = max_nan(tmx[p], __shfl_xor_sync(0xffffffffu, tmx[p], 16));
    tmn[p] = min_nan(tmn[p], __shfl_xor_sync(0xffffffffu, tmn[p], 16));
    rmx[p] = max_nan(rmx[p], __shfl_xor_sync(0xffffffffu, rmx[p], 16));
    rmn[p] = min_nan(rmn[p], __shfl_xor_sync(0xffffffffu, rmn[p], 16));
  }
  if (tsub == 0) {
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      red[0][warp][p0 + p] = tmx[p]; red[1][warp][p0 + p] = tmn[p];
      red[2][warp][p0 + p] = rmx[p]; red[3][warp][p0 + p] = rmn[p];
    }
  }
  __syncthreads();
  {
    const int stat = threadIdx.x >> 6, pair = threadIdx.x & 63;
#pragma unroll
    for (int gq = 0; gq < gpc; ++gq) {
      float v = red[stat][gq * wpg][pair];
#pragma unroll
      for (int w = 1; w < wpg; ++w)
        v = (stat & 1) ? min_nan(v, red[stat][gq * wpg + w][pair]) : max_nan(v, red[stat][gq * wpg + w][pair]);
      fin[gq][stat][pair] = v;
    }
  }
  __syncthreads();
  if (!live) return;

  float tstep[4], rstep[4], trcp[4], rrcp[4];
  const float inv_t = 1.0f / static_cast<float>(1 << tbits), inv_r = 1.0f / static_cast<float>(1 << rbits);
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    tmx[p] = fin[gsub][0][p0 + p]; tmn[p] = fin[gsub][1][p0 + p];
    rmx[p] = fin[gsub][2][p0 + p]; rmn[p] = fin[gsub][3][p0 + p];
    // dividing by a power of two equals multiplying by its exact reciprocal
    tstep[p] = E::round(__fmul_rn(E::round(__fsub_rn(tmx[p], tmn[p])), inv_t));
    rstep[p] = E::round(__fmul_rn(E::round(__fsub_rn(rmx[p], rmn[p])), inv_r));
    trcp[p] = guarded_rcp(tstep[p]);
    rrcp[p] = guarded_rcp(rstep[p]);
  }
  if (wsub == 0 && tsub == 0) {
    const int64_t so = b * s_sb + h * s_sh + static_cast<int64_t>(j + group_off) * kPairs + p0;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      rscale[so + p] = E::from_float(rstep[p]); rmn_out[so + p] = E::from_float(rmn[p]);
      tscale[so + p] = E::from_float(tstep[p]); tmn_out[so + p] = E::from_float(tmn[p]);
    }
  }
  const uint32_t tlo_w[2] = {pack2<DT16>(tmn[0], tmn[1]), pack2<DT16>(tmn[2], tmn[3])};
  const uint32_t rlo_w[2] = {pack2<DT16>(rmn[0], rmn[1]), pack2<DT16>(rmn[2], rmn[3])};

  const unsigned ttop = (1u << tbits) - 1u, rtop = (1u << rbits) - 1u;
  const bool pack6 = (flags & PQ_QUANT_PACK6) != 0;
  uint8_t* crow = codes + b * c_sb + h * c_sh + static_cast<int64_t>(j + group_off) * G * kPairs + p0;
  uint8_t* ctile = codes + b * c_sb + h * c_sh + static_cast<int64_t>(j + group_off) * G * 48;   // packed container
  // one copy of the loop per container, so that the choice costs no branch per token
  auto second_pass = [&](auto packed_container) {
    constexpr bool kPack6 = decltype(packed_container)::value;
#pragma unroll 2
    for (int i = 0; i < ni; ++i) {
      const uint4 v = s_polar[i * kQuantThreads + threadIdx.x];
      const float2 t01 = unpack2<DT16>(sub2_packed<DT16>(v.x, tlo_w[0])), t23 = unpack2<DT16>(sub2_packed<DT16>(v.y, tlo_w[1]));
      const float2 r01 = unpack2<DT16>(sub2_packed<DT16>(v.z, rlo_w[0])), r23 = unpack2<DT16>(sub2_packed<DT16>(v.w, rlo_w[1]));
      const float dt[4] = {t01.x, t01.y, t23.x, t23.y}, dr[4] = {r01.x, r01.y, r23.x, r23.y};
      const uint32_t word = codes_of4<T>(dt, dr, tstep, trcp, rstep, rrcp, ttop, rtop, tbits);
      const int tok = tok0 + tok_step * i;
      if constexpr (!kPack6) {
        *reinterpret_cast<uint32_t*>(crow + static_cast<int64_t>(tok) * kPairs) = word;
      } else {
        // the 16 lanes that share a token assemble the words of the packed container with shuffles (layout and
        // roles of the lanes as in quantize_kernel's emit)
        const int W = lane & 3, t = (lane >> 2) & 3;
        uint32_t a = (word & 0x0f0f0f0fu) << (4 * (W & 1));
        a |= __shfl_xor_sync(0xffffffffu, a, 1);
        uint32_t hw = h_part(word, W);
        hw |= __shfl_xor_sync(0xffffffffu, hw, 1);
        hw |= __shfl_xor_sync(0xffffffffu, hw, 2);
        const int r = tok & 15, l = 4 * (r & 7) + t, hi = r >> 3;
        uint8_t* tl = ctile + static_cast<int64_t>(tok >> 4) * kPackedStepBytes;
        if (W == 0) *reinterpret_cast<uint32_t*>(tl + 16 * l + 8 * hi) = a;
        else if (W == 2) *reinterpret_cast<uint32_t*>(tl + 16 * l + 8 * hi + 4) = a;
        else if (W == 1) *reinterpret_cast<uint32_t*>(tl + 512 + 8 * l + 4 * hi) = hw;
      }
    }
  };
  if (pack6) second_pass(std::true_type{});
  else second_pass(std::false_type{});
}

// NI > 0: the thread keeps phi and r of its NI tokens x 4 pairs in registers
// (G == 16 * NI).  NI == 0: any G; phi and r are recomputed in the second pass.
template <typename T, int NI>
#ifndef PQ_QUANT_MIN_CTAS
#define PQ_QUANT_MIN_CTAS 3
#endif
__global__ void __launch_bounds__(kQuantThreads, sizeof(T) == 2 ? PQ_QUANT_MIN_CTAS : 2)
quantize_kernel(const T* __restrict__ keys, int64_t sb, int64_t sh, int64_t sl, int Nk, int nb, int G,
                int rbits, int tbits, unsigned flags, uint8_t* __restrict__ codes, T* __restrict__ rscale,
                T* __restrict__ rmn_out, T* __restrict__ tscale, T* __restrict__ tmn_out,
                int64_t c_sb, int64_t c_sh, int64_t s_sb, int64_t s_sh, const WindowGate gate) {
  using E = Elem<T>;
  // Device-side gate (re-quantisation of a cache window inside a replayed CUDA graph): run only on the step that
  // fills the window, and write behind the groups the cache already holds.
  int group_off = 0;
  if (gate.lengths) {
    group_off = gate.lengths[0];
    if (gate.lengths[1] + gate.r_add != gate.full || group_off < 0 || group_off + nb > gate.max_groups) return;
  }
  __shared__ float red[4][kQuantThreads / 32][kPairs];
  __shared__ float fin[4][kPairs];

  const int tile = blockIdx.x;                // (b * Nk + h) * nb + j
  const int j = tile % nb;
  const int bh = tile / nb;
  const int h = bh % Nk, b = bh / Nk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tsub = lane >> 4;
  const int p0 = (lane & 15) * 4;             // first of this thread's four pairs
  const T* base = keys + b * sb + h * sh + static_cast<int64_t>(j) * G * sl;

  const float wrap = (flags & PQ_QUANT_WRAP_DTYPE) ? E::round(6.283185307179586f) : 6.283185307179586f;
  const bool norm_sep = (flags & PQ_QUANT_NORM_FMA) == 0;

  constexpr int NR = NI > 0 ? NI : 1;
  // 16-bit keys: angle and radius are values of T already, so the NI tokens a thread keeps between the two passes
  // are held (and min/max-reduced) as packed pairs - half the registers, half the min/max instructions
  constexpr bool kPacked = NI > 0 && E::kDtype != PQ_F32;
  constexpr int DT16 = E::kDtype == PQ_BF16 ? PQ_BF16 : PQ_F16;
  float phi[kPacked ? 1 : NR][4], rad[kPacked ? 1 : NR][4];
  uint32_t phi_w[kPacked ? NR : 1][2], rad_w[kPacked ? NR : 1][2];
  float tmx[4], tmn[4], rmx[4], rmn[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) { tmx[p] = -INFINITY; tmn[p] = INFINITY; rmx[p] = -INFINITY; rmn[p] = INFINITY; }

  const int tok0 = 2 * warp + tsub;
  if constexpr (kPacked) {
    uint32_t tmx_w[2], tmn_w[2], rmx_w[2], rmn_w[2];
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const T* row = base + static_cast<int64_t>(tok0 + 16 * i) * sl;
      float x[4], y[4], ph[4], rd[4];
      load4<T>(row + p0, x);
      load4<T>(row + p0 + kPairs, y);
      polar_of4<T>(x, y, wrap, norm_sep, ph, rd);
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const uint32_t pw = pack2<DT16>(ph[2 * k], ph[2 * k + 1]), rw = pack2<DT16>(rd[2 * k], rd[2 * k + 1]);   // exact: already rounded
        phi_w[i][k] = pw; rad_w[i][k] = rw;
        if (i == 0) { tmx_w[k] = tmn_w[k] = pw; rmx_w[k] = rmn_w[k] = rw; }
        else {
          tmx_w[k] = max2_nan<DT16>(tmx_w[k], pw); tmn_w[k] = min2_nan<DT16>(tmn_w[k], pw);
          rmx_w[k] = max2_nan<DT16>(rmx_w[k], rw); rmn_w[k] = min2_nan<DT16>(rmn_w[k], rw);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      float2 f;
      f = unpack2<DT16>(tmx_w[k]); tmx[2 * k] = f.x; tmx[2 * k + 1] = f.y;
      f = unpack2<DT16>(tmn_w[k]); tmn[2 * k] = f.x; tmn[2 * k + 1] = f.y;
      f = unpack2<DT16>(rmx_w[k]); rmx[2 * k] = f.x; rmx[2 * k + 1] = f.y;
      f = unpack2<DT16>(rmn_w[k]); rmn[2 * k] = f.x; rmn[2 * k + 1] = f.y;
    }
  } else if constexpr (NI > 0) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const T* row = base + static_cast<int64_t>(tok0 + 16 * i) * sl;
      float x[4], y[4];
      load4<T>(row + p0, x);
      load4<T>(row + p0 + kPairs, y);
      polar_of4<T>(x, y, wrap, norm_sep, phi[i], rad[i]);
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        tmx[p] = max_nan(tmx[p], phi[i][p]); tmn[p] = min_nan(tmn[p], phi[i][p]);
        rmx[p] = max_nan(rmx[p], rad[i][p]); rmn[p] = min_nan(rmn[p], rad[i][p]);
      }
    }
  } else {
    for (int tok = tok0; tok < G; tok += 16) {
      const T* row = base + static_cast<int64_t>(tok) * sl;
      float x[4], y[4], ph[4], rd[4];
      load4<T>(row + p0, x);
      load4<T>(row + p0 + kPairs, y);
      polar_of4<T>(x, y, wrap, norm_sep, ph, rd);
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        tmx[p] = max_nan(tmx[p], ph[p]); tmn[p] = min_nan(tmn[p], ph[p]);
        rmx[p] = max_nan(rmx[p], rd[p]); rmn[p] = min_nan(rmn[p], rd[p]);
      }
    }
  }

  // combine the two token halves of the warp, then the eight warps
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    tmx[p] = max_nan(tmx[p], __shfl_xor_sync(0xffffffffu, tmx[p], 16));
    tmn[p] = min_nan(tmn[p], __shfl_xor_sync(0xffffffffu, tmn[p], 16));
    rmx[p] = max_nan(rmx[p], __shfl_xor_sync(0xffffffffu, rmx[p], 16));
    rmn[p] = min_nan(rmn[p], __shfl_xor_sync(0xffffffffu, rmn[p], 16));
  }
  if (tsub == 0) {
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      red[0][warp][p0 + p] = tmx[p]; red[1][warp][p0 + p] = tmn[p];
      red[2][warp][p0 + p] = rmx[p]; red[3][warp][p0 + p] = rmn[p];
    }
  }
  __syncthreads();
  {
    const int stat = threadIdx.x >> 6, pair = threadIdx.x & 63;
    float v = red[stat][0][pair];
#pragma unroll
    for (int w = 1; w < kQuantThreads / 32; ++w)
      v = (stat & 1) ? min_nan(v, red[stat][w][pair]) : max_nan(v, red[stat][w][pair]);
    fin[stat][pair] = v;
  }
  __syncthreads();

  float tstep[4], rstep[4], trcp[4], rrcp[4];
  const float inv_t = 1.0f / static_cast<float>(1 << tbits), inv_r = 1.0f / static_cast<float>(1 << rbits);
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    tmx[p] = fin[0][p0 + p]; tmn[p] = fin[1][p0 + p];
    rmx[p] = fin[2][p0 + p]; rmn[p] = fin[3][p0 + p];
    // dividing by a power of two equals multiplying by its exact reciprocal
    tstep[p] = E::round(__fmul_rn(E::round(__fsub_rn(tmx[p], tmn[p])), inv_t));
    rstep[p] = E::round(__fmul_rn(E::round(__fsub_rn(rmx[p], rmn[p])), inv_r));
    trcp[p] = guarded_rcp(tstep[p]);
    rrcp[p] = guarded_rcp(rstep[p]);
  }
  if (warp == 0 && tsub == 0) {
    const int64_t so = b * s_sb + h * s_sh + static_cast<int64_t>(j + group_off) * kPairs + p0;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      rscale[so + p] = E::from_float(rstep[p]); rmn_out[so + p] = E::from_float(rmn[p]);
      tscale[so + p] = E::from_float(tstep[p]); tmn_out[so + p] = E::from_float(tmn[p]);
    }
  }

  const unsigned ttop = (1u << tbits) - 1u, rtop = (1u << rbits) - 1u;
  const bool pack6 = (flags & PQ_QUANT_PACK6) != 0;
  uint8_t* crow = codes + b * c_sb + h * c_sh + static_cast<int64_t>(j + group_off) * G * kPairs + p0;
  uint8_t* ctile = codes + b * c_sb + h * c_sh + static_cast<int64_t>(j + group_off) * G * 48;   // packed container
  // Store the four codes (one per byte of `word`) of this thread's pairs for token `tok` of the group.  In the packed
  // container the 16 lanes that share a token assemble their words with shuffles: the lane of code word W = lane % 4
  // of pair block t = (lane / 4) % 4 contributes the nibbles of its codes to A_{W / 2} and their upper bits to H.
  auto emit = [&](int tok, uint32_t word) {
    if (!pack6) { *reinterpret_cast<uint32_t*>(crow + static_cast<int64_t>(tok) * kPairs) = word; return; }
    const int W = lane & 3, t = (lane >> 2) & 3;
    uint32_t a = (word & 0x0f0f0f0fu) << (4 * (W & 1));
    a |= __shfl_xor_sync(0xffffffffu, a, 1);
    uint32_t hw = h_part(word, W);
    hw |= __shfl_xor_sync(0xffffffffu, hw, 1);
    hw |= __shfl_xor_sync(0xffffffffu, hw, 2);
    const int r = tok & 15, l = 4 * (r & 7) + t, hi = r >> 3;
    uint8_t* tile = ctile + static_cast<int64_t>(tok >> 4) * kPackedStepBytes;
    if (W == 0) *reinterpret_cast<uint32_t*>(tile + 16 * l + 8 * hi) = a;
    else if (W == 2) *reinterpret_cast<uint32_t*>(tile + 16 * l + 8 * hi + 4) = a;
    else if (W == 1) *reinterpret_cast<uint32_t*>(tile + 512 + 8 * l + 4 * hi) = hw;
  };
  if constexpr (NI > 0) {
    // the group's minima as packed pairs, for the packed subtraction
    uint32_t tmn_w[2] = {0, 0}, rmn_w[2] = {0, 0};
    if constexpr (kPacked) {
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        tmn_w[k] = pack2<DT16>(tmn[2 * k], tmn[2 * k + 1]); rmn_w[k] = pack2<DT16>(rmn[2 * k], rmn[2 * k + 1]);
      }
    }
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      float dt[4], dr[4];
      if constexpr (kPacked) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const float2 a = unpack2<DT16>(sub2_packed<DT16>(phi_w[i][k], tmn_w[k]));
          const float2 c = unpack2<DT16>(sub2_packed<DT16>(rad_w[i][k], rmn_w[k]));
          dt[2 * k] = a.x; dt[2 * k + 1] = a.y; dr[2 * k] = c.x; dr[2 * k + 1] = c.y;
        }
      } else {
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          dt[p] = E::round(__fsub_rn(phi[i][p], tmn[p])); dr[p] = E::round(__fsub_rn(rad[i][p], rmn[p]));
        }
      }
      emit(tok0 + 16 * i, codes_of4<T>(dt, dr, tstep, trcp, rstep, rrcp, ttop, rtop, tbits));
    }
  } else {
    for (int tok = tok0; tok < G; tok += 16) {
      const T* row = base + static_cast<int64_t>(tok) * sl;
      float x[4], y[4], pv[4], rv[4], dt[4], dr[4];
      load4<T>(row + p0, x);
      load4<T>(row + p0 + kPairs, y);
      polar_of4<T>(x, y, wrap, norm_sep, pv, rv);
#pragma unroll
      for (int p = 0; p < 4; p += 2) {
        round2<T>(__fsub_rn(pv[p], tmn[p]), __fsub_rn(pv[p + 1], tmn[p + 1]), dt[p], dt[p + 1]);
        round2<T>(__fsub_rn(rv[p], rmn[p]), __fsub_rn(rv[p + 1], rmn[p + 1]), dr[p], dr[p + 1]);
      }
      emit(tok, codes_of4<T>(dt, dr, tstep, trcp, rstep, rrcp, ttop, rtop, tbits));
    }
  }
}

// Exhaustive self-test: for every pair of 16-bit patterns, the fast-path functions must return exactly what the
// exact-only functions return.  which = 0: angle and radius of the key pair (x, y); which = 1: quantisation
// level of value x with step y.  Counts the disagreeing pairs.
template <typename T>
__global__ void selftest_kernel(int which, unsigned long long* mismatches) {
  using E = Elem<T>;
  constexpr int DT16 = E::kDtype == PQ_BF16 ? PQ_BF16 : PQ_F16;
  unsigned long long bad = 0;
  const unsigned long long total = 1ull << 32;
  for (unsigned long long i = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
    const unsigned short xb = static_cast<unsigned short>(i & 0xffffu), yb = static_cast<unsigned short>(i >> 16);
    const float x = E::to_float(*reinterpret_cast<const T*>(&xb)), y = E::to_float(*reinterpret_cast<const T*>(&yb));
    if (which == 0) {
      // the pair, its mirror image and the two with the first channel negated
      const float xx[4] = {x, y, -x, -y}, yy[4] = {y, x, y, x};
      float p0[4], r0[4], p1[4], r1[4];
      uint32_t pw[2], rw[2];
      polar_of4_packed<T, true, true>(xx, yy, 6.283185307179586f, true, pw, rw);     // the kernel's form
      const float2 pa = unpack2<DT16>(pw[0]), pb = unpack2<DT16>(pw[1]), ra = unpack2<DT16>(rw[0]), rb = unpack2<DT16>(rw[1]);
      p0[0] = pa.x; p0[1] = pa.y; p0[2] = pb.x; p0[3] = pb.y; r0[0] = ra.x; r0[1] = ra.y; r0[2] = rb.x; r0[3] = rb.y;
      polar_of4<T, false>(xx, yy, 6.283185307179586f, true, p1, r1);
      // values compare equal or both NaN; +0 and -0 count as equal, as they do for torch.equal
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const bool same_p = (p0[k] == p1[k]) || (p0[k] != p0[k] && p1[k] != p1[k]);
        const bool same_r = (r0[k] == r1[k]) || (r0[k] != r0[k] && r1[k] != r1[k]);
        bad += !(same_p && same_r);
      }
    } else if (which == 1) {
      // value x as the rounded difference, y as the step: angle and radius slots, two bit widths
      const float rc = guarded_rcp(y);
      const float d[4] = {x, x, x, x}, st[4] = {y, y, y, y}, rcp[4] = {rc, rc, rc, rc};
      const uint32_t fast = codes_of4<T, true>(d, d, st, rcp, st, rcp, 15u, 15u, 4);
      const uint32_t exact = codes_of4<T, false>(d, d, st, rcp, st, rcp, 15u, 15u, 4);
      const uint32_t fast8 = codes_of4<T, true>(d, d, st, rcp, st, rcp, 255u, 0u, 8);
      const uint32_t exact8 = codes_of4<T, false>(d, d, st, rcp, st, rcp, 255u, 0u, 8);
      bad += fast != exact || fast8 != exact8;
      // and the rounded quotient itself, wherever the refined division is accepted (below 256: the value quantiser's
      // range test)
      const float qf = div_refined(x, y, rc);
      if (qf < 256.0f) {
        const float a = E::round(qf), b = E::round(__fdiv_rn(x, y));
        bad += !(a == b);
      }
    } else {
      // packed subtraction against the fp32 subtraction rounded to T
      const uint32_t w = sub2_packed<DT16>(pack2<DT16>(x, x), pack2<DT16>(y, y));
      const float got = unpack2<DT16>(w).x, want = E::round(__fsub_rn(x, y));
      bad += !((got == want) || (got != got && want != want));
    }
  }
  if (bad) atomicAdd(mismatches, bad);
}

template <typename T>
int launch_quantize(const void* keys, const int64_t* st, int B, int Nk, int L, int G, int rbits, int tbits,
                    unsigned flags, uint8_t* codes, void* rs, void* rm, void* ts, void* tm, const int64_t* os,
                    const WindowGate& gate, cudaStream_t s, const void* rope_ptr = nullptr) {
  const int nb = L / G;
  const int64_t tiles = static_cast<int64_t>(B) * Nk * nb;
  if (tiles == 0) return PQ_OK;
  if (tiles > 0x7fffffffLL) return PQ_ERR_UNSUPPORTED;
  dim3 grid(static_cast<unsigned>(tiles)), block(kQuantThreads);
  const T* k = static_cast<const T*>(keys);
  if constexpr (sizeof(T) == 2) {
    if (G % 16 == 0 && G <= kMaxSmemGroup) {
      const int gpc = (G == 16 || G == 32 || G == 64) ? 128 / G : 1;       // groups per CTA
      const int wpg = (kQuantThreads / 32) / gpc;                          // warps per group
      const size_t smem = static_cast<size_t>(G / (2 * wpg)) * kQuantThreads * sizeof(uint4);
      const dim3 grid16(static_cast<unsigned>((tiles + gpc - 1) / gpc));
      const RopeFusion<T> none{};
      const RopeFusion<T>* rope = static_cast<const RopeFusion<T>*>(rope_ptr);
#define PQ_LAUNCH_Q16(W)                                                                                         \
  if (rope)                                                                                                      \
    quantize_kernel16<T, W, true><<<grid16, block, smem, s>>>(                                                   \
        k, st[0], st[1], st[2], Nk, nb, G, rbits, tbits, flags, codes, static_cast<T*>(rs), static_cast<T*>(rm), \
        static_cast<T*>(ts), static_cast<T*>(tm), os[0], os[1], os[2], os[3], gate, static_cast<int>(tiles), *rope); \
  else                                                                                                           \
    quantize_kernel16<T, W, false><<<grid16, block, smem, s>>>(                                                  \
        k, st[0], st[1], st[2], Nk, nb, G, rbits, tbits, flags, codes, static_cast<T*>(rs), static_cast<T*>(rm), \
        static_cast<T*>(ts), static_cast<T*>(tm), os[0], os[1], os[2], os[3], gate, static_cast<int>(tiles), none)
      switch (wpg) {
        case 1: PQ_LAUNCH_Q16(1); break;
        case 2: PQ_LAUNCH_Q16(2); break;
        case 4: PQ_LAUNCH_Q16(4); break;
        default: PQ_LAUNCH_Q16(8); break;
      }
#undef PQ_LAUNCH_Q16
      PQ_CUDA_TRY(cudaGetLastError());
      return PQ_OK;
    }
  }
  if (rope_ptr) return PQ_ERR_UNSUPPORTED;   // the fused rotation exists for 16-bit keys and groups of 16 k <= 128 tokens
#define PQ_LAUNCH_Q(NI)                                                                                   \
  quantize_kernel<T, NI><<<grid, block, 0, s>>>(k, st[0], st[1], st[2], Nk, nb, G, rbits, tbits, flags, \
                                                codes, static_cast<T*>(rs), static_cast<T*>(rm),        \
                                                static_cast<T*>(ts), static_cast<T*>(tm), os[0], os[1], os[2], os[3], gate)
  switch (G) {
    case 16: PQ_LAUNCH_Q(1); break;
    case 32: PQ_LAUNCH_Q(2); break;
    case 64: PQ_LAUNCH_Q(4); break;
    case 128: PQ_LAUNCH_Q(8); break;
    default: PQ_LAUNCH_Q(0); break;
  }
#undef PQ_LAUNCH_Q
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

// Append one token per (batch, kv head): copy the new key row into slot `res_pos` of the residual window and the new
// value row into slot `ctx_pos` of the value buffer.  One warp per row pair, 16-byte copies where alignment allows.
template <typename T>
__global__ void cache_append_kernel(const T* __restrict__ k_new, const T* __restrict__ v_new, int64_t n_sb, int64_t n_sh,
                                    int64_t vn_sb, int64_t vn_sh, T* __restrict__ k_res, int64_t kr_sb, int64_t kr_sh,
                                    int64_t kr_st, T* __restrict__ values, int64_t v_sb, int64_t v_sh, int64_t v_st,
                                    int Nk, int res_pos, int ctx_pos, const int* __restrict__ lengths, int G,
                                    int values_window, int res_cap, int value_cap) {
  if (lengths) {                                           // positions kept on the device
    res_pos = lengths[1];
    ctx_pos = values_window ? res_pos : lengths[0] * G + res_pos;
    if (res_pos < 0 || res_pos >= res_cap || ctx_pos < 0 || ctx_pos >= value_cap) return;
  }
  const int b = blockIdx.x / Nk, h = blockIdx.x % Nk;
  const int c = threadIdx.x;                               // channel
  k_res[b * kr_sb + h * kr_sh + res_pos * kr_st + c] = k_new[b * n_sb + h * n_sh + c];
  values[b * v_sb + h * v_sh + ctx_pos * v_st + c] = v_new[b * vn_sb + h * vn_sh + c];
}

}  // namespace

int cache_append_device(const void* k_new, const void* v_new, const int64_t* in_strides, void* k_res,
                        const int64_t* kres_strides, void* values, const int64_t* v_strides, int B, int Nk, int hd,
                        int res_pos, int ctx_pos, int dtype, const int* lengths, int G, int values_window,
                        int res_cap, int value_cap, cudaStream_t stream) {
  if (!k_new || !v_new || !k_res || !values || !in_strides || !kres_strides || !v_strides) return PQ_ERR_INVALID;
  if (B <= 0 || Nk <= 0 || res_pos < 0 || ctx_pos < 0 || !dtype_ok(dtype)) return PQ_ERR_INVALID;
  if (lengths && (G <= 0 || res_cap <= 0 || value_cap <= 0)) return PQ_ERR_INVALID;
  if (hd != kHeadDim) return PQ_ERR_UNSUPPORTED;
  const unsigned grid = static_cast<unsigned>(B) * Nk;
#define PQ_APPEND(T)                                                                                              \
  cache_append_kernel<T><<<grid, kHeadDim, 0, stream>>>(                                                         \
      static_cast<const T*>(k_new), static_cast<const T*>(v_new), in_strides[0], in_strides[1], in_strides[2],   \
      in_strides[3], static_cast<T*>(k_res), kres_strides[0], kres_strides[1], kres_strides[2],                  \
      static_cast<T*>(values), v_strides[0], v_strides[1], v_strides[2], Nk, res_pos, ctx_pos, lengths, G,       \
      values_window, res_cap, value_cap)
  if (dtype == PQ_F32) PQ_APPEND(float);
  else if (dtype == PQ_F16) PQ_APPEND(__half);
  else PQ_APPEND(__nv_bfloat16);
#undef PQ_APPEND
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

// ---------------------------------------------------------------------------------------------
// Rotary embedding of one decode token fused with the cache append: the query heads of the fused projection output
// are rotated into q_out, the key heads are rotated straight into their slot of the residual window, the value
// heads are copied into theirs.  Arithmetic is the eager `x * cos + rotate_half(x) * sin` of the attention
// patches (apply_rotary_pos_emb at models/modeling_llama_polar.py:57): both products and the sum are rounded to
// the tensor dtype, so the rotated key that gets quantised later is the one the reference would have produced.
// ---------------------------------------------------------------------------------------------
namespace {
template <typename T>
__global__ void __launch_bounds__(kHeadDim / 2)
rope_append_kernel(const T* __restrict__ qkv, int64_t qkv_sb, const T* __restrict__ cosv, const T* __restrict__ sinv,
                   int64_t cs_sb, T* __restrict__ q_out, T* __restrict__ k_res, int64_t kr_sb, int64_t kr_sh,
                   int64_t kr_st, T* __restrict__ values, int64_t v_sb, int64_t v_sh, int64_t v_st, int N, int Nk,
                   int res_pos, int ctx_pos, const int* __restrict__ lengths, int G, int values_window, int res_cap,
                   int value_cap) {
  constexpr int H = kHeadDim / 2;
  if (lengths) {
    res_pos = lengths[1];
    ctx_pos = values_window ? res_pos : lengths[0] * G + res_pos;
  }
  const bool slot_ok = res_pos >= 0 && res_pos < res_cap && ctx_pos >= 0 && ctx_pos < value_cap;
  const int b = blockIdx.x, j = blockIdx.y, d = threadIdx.x;
  const T* x = qkv + b * qkv_sb + static_cast<int64_t>(j) * kHeadDim;
  if (j >= N + Nk) {                                        // value head: copy
    if (!slot_ok) return;
    T* dst = values + b * v_sb + (j - N - Nk) * v_sh + ctx_pos * v_st;
    dst[d] = x[d]; dst[d + H] = x[d + H];
    return;
  }
  const T* c = cosv + b * cs_sb;
  const T* s = sinv + b * cs_sb;
  const float lo = Elem<T>::to_float(x[d]), hi = Elem<T>::to_float(x[d + H]);
  const float o_lo = Elem<T>::round(__fadd_rn(Elem<T>::round(__fmul_rn(lo, Elem<T>::to_float(c[d]))),
                                              Elem<T>::round(__fmul_rn(-hi, Elem<T>::to_float(s[d])))));
  const float o_hi = Elem<T>::round(__fadd_rn(Elem<T>::round(__fmul_rn(hi, Elem<T>::to_float(c[d + H]))),
                                              Elem<T>::round(__fmul_rn(lo, Elem<T>::to_float(s[d + H])))));
  T* dst;
  if (j < N) dst = q_out + (static_cast<int64_t>(b) * N + j) * kHeadDim;
  else {
    if (!slot_ok) return;
    dst = k_res + b * kr_sb + (j - N) * kr_sh + res_pos * kr_st;
  }
  dst[d] = Elem<T>::from_float(o_lo);
  dst[d + H] = Elem<T>::from_float(o_hi);
}
}  // namespace

int rope_append_device(const void* qkv, int64_t qkv_stride_b, const void* cosv, const void* sinv, int64_t cs_stride_b,
                       void* q_out, void* k_res, const int64_t* kres_strides, void* values, const int64_t* v_strides,
                       int B, int N, int Nk, int hd, int G, const int* lengths, int values_window, int res_cap,
                       int value_cap, int res_pos, int ctx_pos, int dtype, cudaStream_t stream) {
  if (!qkv || !cosv || !sinv || !q_out || !k_res || !values || !kres_strides || !v_strides) return PQ_ERR_INVALID;
  if (B <= 0 || N <= 0 || Nk <= 0 || G <= 0 || res_cap <= 0 || value_cap <= 0 || !dtype_ok(dtype)) return PQ_ERR_INVALID;
  if (!lengths && (res_pos < 0 || ctx_pos < 0 || res_pos >= res_cap || ctx_pos >= value_cap)) return PQ_ERR_INVALID;
  if (hd != kHeadDim) return PQ_ERR_UNSUPPORTED;
  const dim3 grid(static_cast<unsigned>(B), static_cast<unsigned>(N + 2 * Nk));
#define PQ_ROPE(T)                                                                                                \
  rope_append_kernel<T><<<grid, kHeadDim / 2, 0, stream>>>(                                                      \
      static_cast<const T*>(qkv), qkv_stride_b, static_cast<const T*>(cosv), static_cast<const T*>(sinv),        \
      cs_stride_b, static_cast<T*>(q_out), static_cast<T*>(k_res), kres_strides[0], kres_strides[1],             \
      kres_strides[2], static_cast<T*>(values), v_strides[0], v_strides[1], v_strides[2], N, Nk, res_pos,        \
      ctx_pos, lengths, G, values_window, res_cap, value_cap)
  if (dtype == PQ_F32) PQ_ROPE(float);
  else if (dtype == PQ_F16) PQ_ROPE(__half);
  else PQ_ROPE(__nv_bfloat16);
#undef PQ_ROPE
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

// One step of a growing cache, on the device: lengths = {token groups, residual tokens}.  The window that has just
// become full (residual + 1 == full) turns into full / G new groups, otherwise the residual count goes up by one.
namespace {
__global__ void lengths_advance_kernel(int* lengths, int full, int G) {
  const int r = lengths[1] + 1;
  if (r >= full) { lengths[0] += full / G; lengths[1] = 0; }
  else lengths[1] = r;
}
}  // namespace
int lengths_advance_device(int* lengths, int full, int G, cudaStream_t stream) {
  if (!lengths || full <= 0 || G <= 0 || full % G != 0) return PQ_ERR_INVALID;
  lengths_advance_kernel<<<1, 1, 0, stream>>>(lengths, full, G);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

// Largest radius a group can reconstruct, |rmn| + |rscale| * 2^rbits, against the fp16 range of the decode kernels'
// dequantisation.  One pass over the two radius scale tensors; sets *flag when a value is not finite or too large.
namespace {
template <typename T>
__global__ void key_range_check_kernel(const T* __restrict__ rscale, const T* __restrict__ rmn, int64_t count,
                                       float levels, unsigned* __restrict__ flag) {
  bool bad = false;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float top = fabsf(Elem<T>::to_float(rmn[i])) + fabsf(Elem<T>::to_float(rscale[i])) * levels;
    bad |= !(top < 65504.0f);                  // also true for NaN
  }
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) *flag = 1u;
}
}  // namespace

int keys_repack_device(const uint8_t* codes_in, uint8_t* codes_out, int64_t steps, int to_format,
                       cudaStream_t stream) {
  if (steps < 0 || (to_format != PQ_KEYS_BYTE && to_format != PQ_KEYS_PACKED6)) return PQ_ERR_INVALID;
  if (steps == 0) return PQ_OK;
  if (!codes_in || !codes_out) return PQ_ERR_INVALID;
  if (reinterpret_cast<uintptr_t>(codes_in) % 16 || reinterpret_cast<uintptr_t>(codes_out) % 16) return PQ_ERR_ALIGNMENT;
  const int64_t want = (steps + 7) / 8;
  const unsigned grid = static_cast<unsigned>(want < 148 * 16 ? want : 148 * 16);
  keys_repack_kernel<<<grid, 256, 0, stream>>>(codes_in, codes_out, steps, to_format == PQ_KEYS_PACKED6);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

int key_range_check_device(const void* rscale, const void* rmn, int64_t count, int rbits, int dtype,
                           unsigned* flag_dev, cudaStream_t stream) {
  if (count < 0 || rbits < 0 || rbits > 8 || !dtype_ok(dtype)) return PQ_ERR_INVALID;
  if (count == 0) return PQ_OK;
  if (!rscale || !rmn || !flag_dev) return PQ_ERR_INVALID;
  const int64_t want = (count + 255) / 256;
  const unsigned grid = static_cast<unsigned>(want < 148 * 8 ? want : 148 * 8);
  const float levels = static_cast<float>(1 << rbits);
  if (dtype == PQ_F32)
    key_range_check_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(rscale), static_cast<const float*>(rmn), count, levels, flag_dev);
  else if (dtype == PQ_F16)
    key_range_check_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(rscale), static_cast<const __half*>(rmn), count, levels, flag_dev);
  else
    key_range_check_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(rscale), static_cast<const __nv_bfloat16*>(rmn), count, levels, flag_dev);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

int selftest_quantizer_device(int dtype, int which, unsigned long long* mismatches_dev, cudaStream_t stream) {
  if (!mismatches_dev || which < 0 || which > 2) return PQ_ERR_INVALID;
  if (dtype != PQ_F16 && dtype != PQ_BF16) return PQ_ERR_INVALID;
  PQ_CUDA_TRY(cudaMemsetAsync(mismatches_dev, 0, sizeof(unsigned long long), stream));
  if (dtype == PQ_F16) selftest_kernel<__half><<<148 * 8, 256, 0, stream>>>(which, mismatches_dev);
  else selftest_kernel<__nv_bfloat16><<<148 * 8, 256, 0, stream>>>(which, mismatches_dev);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

// out_strides: {codes_stride_b, codes_stride_h} in bytes and {scale_stride_b, scale_stride_h} in elements;
// nullptr means dense outputs.
int quantize_device(const void* keys, const int64_t strides[4], int B, int Nk, int L, int hd, int G,
                    int rbits, int tbits, int dtype, unsigned flags, uint8_t* codes, void* rscale, void* rmn,
                    void* tscale, void* tmn, const int64_t* out_strides, cudaStream_t stream,
                    const int* gate_lengths, int gate_r_add, int gate_full, int gate_max_groups,
                    const void* rope_fusion) {
  if (!strides || B < 0 || Nk < 0 || L < 0 || G <= 0) return PQ_ERR_INVALID;
  const WindowGate gate{gate_lengths, gate_r_add, gate_full, gate_max_groups};
  if (gate_lengths && (!out_strides || gate_full <= 0 || gate_max_groups <= 0)) return PQ_ERR_INVALID;
  if (rbits < 0 || tbits < 0 || rbits + tbits > 8 || (hd & 1) || L % G != 0) return PQ_ERR_INVALID;
  if (!dtype_ok(dtype)) return PQ_ERR_INVALID;
  if (hd != kHeadDim) return PQ_ERR_UNSUPPORTED;
  if (B == 0 || Nk == 0 || L == 0) return PQ_OK;
  if (!keys || !codes || !rscale || !rmn || !tscale || !tmn) return PQ_ERR_INVALID;
  if (strides[3] != 1) return PQ_ERR_INVALID;
  // each thread loads four consecutive elements with one vector load
  const size_t vec = 4 * dtype_bytes(dtype);
  if (reinterpret_cast<uintptr_t>(keys) % vec || strides[0] % 4 || strides[1] % 4 || strides[2] % 4)
    return PQ_ERR_ALIGNMENT;
  if (reinterpret_cast<uintptr_t>(codes) % 4) return PQ_ERR_ALIGNMENT;
  const int64_t nb = L / G;
  const bool pack6 = (flags & PQ_QUANT_PACK6) != 0;
  if (pack6 && (rbits + tbits != 6 || G % 16 != 0)) return PQ_ERR_INVALID;
  const int64_t tok_bytes = pack6 ? 48 : kPairs;                   // code bytes per token
  int64_t os[4] = {nb * G * tok_bytes * Nk, nb * G * tok_bytes, nb * kPairs * Nk, nb * kPairs};
  if (out_strides) {
    for (int i = 0; i < 4; ++i) os[i] = out_strides[i];
    const int64_t span = gate_lengths ? gate_max_groups : nb;      // groups a (b, h) unit must be able to hold
    if (os[0] % 4 || os[1] % 4 || os[1] < span * G * tok_bytes || os[3] < span * kPairs) return PQ_ERR_INVALID;
  }
  switch (dtype) {
    case PQ_F16: return launch_quantize<__half>(keys, strides, B, Nk, L, G, rbits, tbits, flags, codes, rscale, rmn, tscale, tmn, os, gate, stream, rope_fusion);
    case PQ_BF16: return launch_quantize<__nv_bfloat16>(keys, strides, B, Nk, L, G, rbits, tbits, flags, codes, rscale, rmn, tscale, tmn, os, gate, stream, rope_fusion);
    default: return rope_fusion ? PQ_ERR_UNSUPPORTED
                                : launch_quantize<float>(keys, strides, B, Nk, L, G, rbits, tbits, flags, codes, rscale, rmn, tscale, tmn, os, gate, stream);
  }
}

// Prefill-side fusion: rotate the prompt's keys and quantise the first Lq of them in the same pass; the tokens behind
// them (the residual window) are rotated only.
int rope_quantize_device(const void* keys, const int64_t strides[4], const void* cosv, const void* sinv,
                         const int64_t cs_strides[2], void* keys_out, const int64_t out_key_strides[4], int B, int Nk,
                         int L, int Lq, int hd, int G, int rbits, int tbits, int dtype, unsigned flags, uint8_t* codes,
                         void* rscale, void* rmn, void* tscale, void* tmn, const int64_t* out_strides,
                         cudaStream_t stream) {
  if (!strides || !cs_strides || B < 0 || Nk < 0 || L < 0 || Lq < 0 || Lq > L || G <= 0 || Lq % G != 0) return PQ_ERR_INVALID;
  if (dtype != PQ_F16 && dtype != PQ_BF16) return dtype == PQ_F32 ? PQ_ERR_UNSUPPORTED : PQ_ERR_INVALID;
  if (hd != kHeadDim || G % 16 != 0 || G > kMaxSmemGroup) return PQ_ERR_UNSUPPORTED;
  if (B == 0 || Nk == 0 || L == 0) return PQ_OK;
  if (!keys || !cosv || !sinv) return PQ_ERR_INVALID;
  if (keys_out && !out_key_strides) return PQ_ERR_INVALID;
  if (L > Lq && !keys_out) return PQ_ERR_INVALID;            // rotating the tail needs somewhere to put it
  if (strides[3] != 1 || (keys_out && out_key_strides[3] != 1)) return PQ_ERR_INVALID;
  auto mis8 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 8 != 0; };
  if (mis8(keys) || mis8(cosv) || mis8(sinv) || (keys_out && mis8(keys_out)) || strides[0] % 4 || strides[1] % 4 ||
      strides[2] % 4 || cs_strides[0] % 4 || cs_strides[1] % 4 ||
      (keys_out && (out_key_strides[0] % 4 || out_key_strides[1] % 4 || out_key_strides[2] % 4)))
    return PQ_ERR_ALIGNMENT;
  int rc = PQ_OK;
  auto run = [&](auto tag) {
    using T = decltype(tag);
    RopeFusion<T> rope{static_cast<const T*>(cosv), static_cast<const T*>(sinv), cs_strides[0], cs_strides[1],
                       static_cast<T*>(keys_out), keys_out ? out_key_strides[0] : 0, keys_out ? out_key_strides[1] : 0,
                       keys_out ? out_key_strides[2] : 0};
    if (Lq > 0) {
      rc = quantize_device(keys, strides, B, Nk, Lq, hd, G, rbits, tbits, dtype, flags, codes, rscale, rmn, tscale, tmn,
                           out_strides, stream, nullptr, 0, 0, 0, &rope);
      if (rc != PQ_OK) return;
    }
    if (L > Lq) {
      const int tokens = L - Lq;
      const dim3 grid((tokens * 16 + 255) / 256, static_cast<unsigned>(B) * Nk);
      rope_rows_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(keys), strides[0], strides[1], strides[2], Nk, Lq,
                                                   tokens, rope);
      if (cudaGetLastError() != cudaSuccess) rc = PQ_ERR_CUDA;
    }
  };
  if (dtype == PQ_F16) run(__half{}); else run(__nv_bfloat16{});
  return rc;
}

}  // namespace pq
