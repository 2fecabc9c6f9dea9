// Shared device/host helpers for the polar key-cache kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/polarquant_b200.h"

namespace pq {

constexpr int kHeadDim = 128;  // channels per head
constexpr int kPairs = 64;     // 2-D pairs per head: pair d = channels (d, d + 64)

// thread-local record of the last failing CUDA call
int& last_cuda_error();
inline int cuda_fail(cudaError_t e) {
  last_cuda_error() = static_cast<int>(e);
  return PQ_ERR_CUDA;
}
#define PQ_CUDA_TRY(expr)                                   \
  do {                                                      \
    cudaError_t e__ = (expr);                               \
    if (e__ != cudaSuccess) return ::pq::cuda_fail(e__);    \
  } while (0)

inline size_t dtype_bytes(int dt) { return dt == PQ_F32 ? 4 : 2; }
inline bool dtype_ok(int dt) { return dt == PQ_F16 || dt == PQ_BF16 || dt == PQ_F32; }

// ---------------------------------------------------------------------------
// element <-> fp32 conversions, round-to-nearest-even
// ---------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__half> {
  static constexpr int kDtype = PQ_F16;
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int kDtype = PQ_BF16;
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};
template <> struct Elem<float> {
  static constexpr int kDtype = PQ_F32;
  static __device__ __forceinline__ float to_float(float v) { return v; }
  static __device__ __forceinline__ float from_float(float v) { return v; }
  static __device__ __forceinline__ float round(float v) { return v; }
};

// 16-bit pair (lo, hi) packed in a 32-bit word -> two floats, by dtype tag
template <int DT> __device__ __forceinline__ float2 unpack2(uint32_t w);
template <> __device__ __forceinline__ float2 unpack2<PQ_F16>(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <> __device__ __forceinline__ float2 unpack2<PQ_BF16>(uint32_t w) {
  // a bf16 is the high half of an fp32
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <int DT> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<PQ_F16>(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<PQ_BF16>(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// ---------------------------------------------------------------------------
// 128-bit global loads.  The key/value/code streams are read once, so they
// bypass L1 allocation; everything else uses the default path.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// ---------------------------------------------------------------------------
// warp-level tensor-core primitives (mma.sync path; see the decode kernel for
// why the single-query decode shape does not fit tcgen05's M >= 64 tiles)
// ---------------------------------------------------------------------------
// plain (not volatile) asm: an MMA has no effect beyond its outputs, so the compiler may schedule it freely
__device__ __forceinline__ void mma_16816_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_16816_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <int DT>
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  if constexpr (DT == PQ_BF16) mma_16816_bf16(c, a0, a1, a2, a3, b0, b1);
  else mma_16816_f16(c, a0, a1, a2, a3, b0, b1);
}
// transpose an 8x8 matrix of 16-bit elements held one row per 4 lanes
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace pq
