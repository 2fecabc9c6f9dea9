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
#include "pq_common.cuh"

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

template <typename T>
__device__ __forceinline__ void polar_of(float x, float y, float wrap, bool norm_separate,
                                         float& phi, float& rad) {
  using E = Elem<T>;
  float a = E::round(atan2f(y, x));
  if (a < 0.0f) a = E::round(__fadd_rn(a, wrap));
  phi = a;
  float s = norm_separate ? __fadd_rn(__fmul_rn(x, x), __fmul_rn(y, y)) : __fmaf_rn(y, y, __fmul_rn(x, x));
  rad = E::round(__fsqrt_rn(s));
}

template <typename T>
__device__ __forceinline__ unsigned level_of(float v, float lo, float step, unsigned top) {
  using E = Elem<T>;
  float q = floorf(E::round(__fdiv_rn(E::round(__fsub_rn(v, lo)), step)));
  // float -> int64 -> uint8, the cast ATen performs: NaN gives 0, +inf gives 0xff
  unsigned u = static_cast<unsigned>(static_cast<long long>(q)) & 0xffu;
  return u < top ? u : top;
}

// NI > 0: the thread keeps phi and r of its NI tokens x 4 pairs in registers
// (G == 16 * NI).  NI == 0: any G; phi and r are recomputed in the second pass.
template <typename T, int NI>
__global__ void __launch_bounds__(kQuantThreads)
quantize_kernel(const T* __restrict__ keys, int64_t sb, int64_t sh, int64_t sl, int Nk, int nb, int G,
                int rbits, int tbits, unsigned flags, uint8_t* __restrict__ codes, T* __restrict__ rscale,
                T* __restrict__ rmn_out, T* __restrict__ tscale, T* __restrict__ tmn_out) {
  using E = Elem<T>;
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
  float phi[NR][4], rad[NR][4];
  float tmx[4], tmn[4], rmx[4], rmn[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) { tmx[p] = -INFINITY; tmn[p] = INFINITY; rmx[p] = -INFINITY; rmn[p] = INFINITY; }

  const int tok0 = 2 * warp + tsub;
  if constexpr (NI > 0) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const T* row = base + static_cast<int64_t>(tok0 + 16 * i) * sl;
      float x[4], y[4];
      load4<T>(row + p0, x);
      load4<T>(row + p0 + kPairs, y);
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        polar_of<T>(x[p], y[p], wrap, norm_sep, phi[i][p], rad[i][p]);
        tmx[p] = max_nan(tmx[p], phi[i][p]); tmn[p] = min_nan(tmn[p], phi[i][p]);
        rmx[p] = max_nan(rmx[p], rad[i][p]); rmn[p] = min_nan(rmn[p], rad[i][p]);
      }
    }
  } else {
    for (int tok = tok0; tok < G; tok += 16) {
      const T* row = base + static_cast<int64_t>(tok) * sl;
      float x[4], y[4];
      load4<T>(row + p0, x);
      load4<T>(row + p0 + kPairs, y);
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        float a, r;
        polar_of<T>(x[p], y[p], wrap, norm_sep, a, r);
        tmx[p] = max_nan(tmx[p], a); tmn[p] = min_nan(tmn[p], a);
        rmx[p] = max_nan(rmx[p], r); rmn[p] = min_nan(rmn[p], r);
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

  float tstep[4], rstep[4];
  const float inv_t = 1.0f / static_cast<float>(1 << tbits), inv_r = 1.0f / static_cast<float>(1 << rbits);
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    tmx[p] = fin[0][p0 + p]; tmn[p] = fin[1][p0 + p];
    rmx[p] = fin[2][p0 + p]; rmn[p] = fin[3][p0 + p];
    // dividing by a power of two equals multiplying by its exact reciprocal
    tstep[p] = E::round(__fmul_rn(E::round(__fsub_rn(tmx[p], tmn[p])), inv_t));
    rstep[p] = E::round(__fmul_rn(E::round(__fsub_rn(rmx[p], rmn[p])), inv_r));
  }
  if (warp == 0 && tsub == 0) {
    const int64_t so = static_cast<int64_t>(tile) * kPairs + p0;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      rscale[so + p] = E::from_float(rstep[p]); rmn_out[so + p] = E::from_float(rmn[p]);
      tscale[so + p] = E::from_float(tstep[p]); tmn_out[so + p] = E::from_float(tmn[p]);
    }
  }

  const unsigned ttop = (1u << tbits) - 1u, rtop = (1u << rbits) - 1u;
  uint8_t* crow = codes + static_cast<int64_t>(tile) * G * kPairs + p0;
  if constexpr (NI > 0) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      uint32_t word = 0;
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        unsigned th = level_of<T>(phi[i][p], tmn[p], tstep[p], ttop);
        unsigned rh = level_of<T>(rad[i][p], rmn[p], rstep[p], rtop);
        word |= (((rh << tbits) + th) & 0xffu) << (8 * p);
      }
      *reinterpret_cast<uint32_t*>(crow + static_cast<int64_t>(tok0 + 16 * i) * kPairs) = word;
    }
  } else {
    for (int tok = tok0; tok < G; tok += 16) {
      const T* row = base + static_cast<int64_t>(tok) * sl;
      float x[4], y[4];
      load4<T>(row + p0, x);
      load4<T>(row + p0 + kPairs, y);
      uint32_t word = 0;
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        float a, r;
        polar_of<T>(x[p], y[p], wrap, norm_sep, a, r);
        unsigned th = level_of<T>(a, tmn[p], tstep[p], ttop);
        unsigned rh = level_of<T>(r, rmn[p], rstep[p], rtop);
        word |= (((rh << tbits) + th) & 0xffu) << (8 * p);
      }
      *reinterpret_cast<uint32_t*>(crow + static_cast<int64_t>(tok) * kPairs) = word;
    }
  }
}

template <typename T>
int launch_quantize(const void* keys, const int64_t* st, int B, int Nk, int L, int G, int rbits, int tbits,
                    unsigned flags, uint8_t* codes, void* rs, void* rm, void* ts, void* tm, cudaStream_t s) {
  const int nb = L / G;
  const int64_t tiles = static_cast<int64_t>(B) * Nk * nb;
  if (tiles == 0) return PQ_OK;
  if (tiles > 0x7fffffffLL) return PQ_ERR_UNSUPPORTED;
  dim3 grid(static_cast<unsigned>(tiles)), block(kQuantThreads);
  const T* k = static_cast<const T*>(keys);
#define PQ_LAUNCH_Q(NI)                                                                                   \
  quantize_kernel<T, NI><<<grid, block, 0, s>>>(k, st[0], st[1], st[2], Nk, nb, G, rbits, tbits, flags, \
                                                codes, static_cast<T*>(rs), static_cast<T*>(rm),        \
                                                static_cast<T*>(ts), static_cast<T*>(tm))
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

}  // namespace

int quantize_device(const void* keys, const int64_t strides[4], int B, int Nk, int L, int hd, int G,
                    int rbits, int tbits, int dtype, unsigned flags, uint8_t* codes, void* rscale, void* rmn,
                    void* tscale, void* tmn, cudaStream_t stream) {
  if (!strides || B < 0 || Nk < 0 || L < 0 || G <= 0) return PQ_ERR_INVALID;
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
  switch (dtype) {
    case PQ_F16: return launch_quantize<__half>(keys, strides, B, Nk, L, G, rbits, tbits, flags, codes, rscale, rmn, tscale, tmn, stream);
    case PQ_BF16: return launch_quantize<__nv_bfloat16>(keys, strides, B, Nk, L, G, rbits, tbits, flags, codes, rscale, rmn, tscale, tmn, stream);
    default: return launch_quantize<float>(keys, strides, B, Nk, L, G, rbits, tbits, flags, codes, rscale, rmn, tscale, tmn, stream);
  }
}

}  // namespace pq
