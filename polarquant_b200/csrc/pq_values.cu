// Packed value cache for sm_100a: per-token 4-bit min/max quantiser, layout conversion, and the
// dequantise-and-multiply used when attention probabilities already exist.
//
// The reference's mixed key/value class (LlamaPolarMixedGroupAttention, models/modeling_llama_polar.py:160-292 of
// ericshwu/PolarQuant) packs values with `triton_quantize_and_pack_along_last_dim(values, 128, 4)` (:242, :285) and
// multiplies with `cuda_bmm_fA_qB_outer(128, probs, codes, scale, mn, 4)` (:230-237).  Both come from the KIVI
// project, which the reference imports but does not ship; the arithmetic below restates KIVI's published
// algorithm with torch's CUDA rounding at every step:
//
//   mn, mx = min / max over the 128 channels of a token (NaN propagates)
//   scale  = RN(RN(mx - mn) * (1.0f / 15.0f))     torch divides a CUDA tensor by a Python scalar by multiplying
//                                                 with the fp32 reciprocal
//   level  = rint(clamp(RN(RN(v - mn) / scale), 0, 15))      IEEE division; NaN (0 / 0 of a constant token) -> 0
//   word c // 8 of the token gets level << 4 * (c % 8)       ("kivi" layout)
//
// The fused attention kernel reads a second, "tiled" layout of the same 64 bytes per token: eight 64-bit slots,
// slot g holding channels g + 8 j at 4-bit field j = 0..15 - the rows (g, g + 8) of all eight 16-channel output
// tiles that lane group g of a warp owns in the P.V tensor-core product.
#include "pq_common.cuh"
#include "pq_rounding.cuh"

namespace pq {
namespace {

constexpr int kValThreads = 256;
constexpr int kTokPerIter = kValThreads / 16;   // 16 lanes x 8 channels per token
constexpr int kValIters = 4;                    // tokens per CTA = 64

struct ValArgs {
  const void* v; int64_t sb, sh, st;            // element strides of (B, Nk, T, 128), inner stride 1
  uint32_t* codes; int64_t c_sb, c_sh;          // byte strides; 64 bytes per token, tokens contiguous
  void* scale; void* mn; int64_t s_sb, s_sh;    // element strides; one element per token, tokens contiguous
  int Nk, T;
  int unit0;                                    // first (b * Nk + h) unit of this launch (grid.y counts from it)
  float inv_levels;
  // device-side gate, as in the key quantizer: run only when lengths[1] + r_add == full, write behind the
  // lengths[0] * G tokens the cache already holds
  const int* gate_lengths; int gate_r_add, gate_full, gate_G, gate_max_tokens;
};

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

template <typename T> __device__ __forceinline__ void load8(const T* p, bool ok, float (&v)[8]) {
  if constexpr (Elem<T>::kDtype == PQ_F32) {
    uint4 a = make_uint4(0, 0, 0, 0), b = a;
    if (ok) { a = ldg_stream(p); b = ldg_stream(p + 4); }
    v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y); v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
    v[4] = __uint_as_float(b.x); v[5] = __uint_as_float(b.y); v[6] = __uint_as_float(b.z); v[7] = __uint_as_float(b.w);
  } else {
    uint4 a = make_uint4(0, 0, 0, 0);
    if (ok) a = ldg_stream(p);
    const float2 f0 = unpack2<Elem<T>::kDtype>(a.x), f1 = unpack2<Elem<T>::kDtype>(a.y);
    const float2 f2 = unpack2<Elem<T>::kDtype>(a.z), f3 = unpack2<Elem<T>::kDtype>(a.w);
    v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y; v[4] = f2.x; v[5] = f2.y; v[6] = f3.x; v[7] = f3.y;
  }
}

// 8 x 8 transpose of 4-bit fields among the eight lanes of a group: lane r holds the kivi word of channels
// 8 (8 h + r) .. + 7 (h = which half of the 16-lane token group); afterwards it holds tiled word 2 r + h, whose field
// j' is channel r + 8 (8 h + j'), i.e. field r of the word lane j' held.
__device__ __forceinline__ uint32_t to_tiled_word(uint32_t kivi_word, int lane) {
  const int r = lane & 7, base = lane & ~7;
  uint32_t out = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t w = __shfl_sync(0xffffffffu, kivi_word, base + j);
    out |= ((w >> (4 * r)) & 0xfu) << (4 * j);
  }
  return out;
}
// position of a lane's word in the 16-word token row
__device__ __forceinline__ int word_index(int sub, bool tiled) {
  return tiled ? 2 * (sub & 7) + (sub >> 3) : sub;
}

template <typename T, bool TILED>
__global__ void __launch_bounds__(kValThreads) quantize_values_kernel(const ValArgs a) {
  const int sub = threadIdx.x & 15;
  const int lane = threadIdx.x & 31;
  int tok_off = 0;
  if (a.gate_lengths) {
    tok_off = a.gate_lengths[0] * a.gate_G;
    if (a.gate_lengths[1] + a.gate_r_add != a.gate_full || tok_off < 0 || tok_off + a.T > a.gate_max_tokens) return;
  }
  // grid (token blocks, units): no per-thread division
  const int unit = a.unit0 + blockIdx.y;
  const int h = unit % a.Nk;
  const int64_t b = unit / a.Nk;
  const T* unit_in = static_cast<const T*>(a.v) + b * a.sb + h * a.sh + 8 * sub;
#pragma unroll
  for (int it = 0; it < kValIters; ++it) {
    const int tok = (blockIdx.x * kValIters + it) * kTokPerIter + (threadIdx.x >> 4);
    const bool ok = tok < a.T;
    const int t = ok ? tok : 0;
    float v[8];
    load8<T>(unit_in + static_cast<int64_t>(t) * a.st, ok, v);
    float mn = v[0], mx = v[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) { mn = min_nan(mn, v[i]); mx = max_nan(mx, v[i]); }
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
      mn = min_nan(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = max_nan(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    const float scale = Elem<T>::round(__fmul_rn(Elem<T>::round(__fsub_rn(mx, mn)), a.inv_levels));
    // RN(d / scale) from the correctly rounded reciprocal and one remainder correction (div_refined: the IEEE
    // quotient for ordinary operands, checked for every (d, scale) pair of 16-bit values by pq_selftest_quantizer,
    // which = 1), the IEEE division itself for degenerate scales and for fp32.  Roundings are packed conversions, the final round-half-even and the
    // conversion to an integer are one addition of 1.5 * 2^23: nothing per element runs on the quarter-rate pipe.
    constexpr bool kFast = Elem<T>::kDtype != PQ_F32;
    const float rcp = guarded_rcp(scale);
    // levels are assembled with FMAs (level * 16^k summed exactly in fp32, four levels per accumulator): the
    // multiply-add pipe has room, the integer/logic pipe is the one this kernel saturates
    float acc_lo = 0.0f, acc_hi = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      float d0, d1, q0, q1;
      round2<T>(__fsub_rn(v[i], mn), __fsub_rn(v[i + 1], mn), d0, d1);
      if constexpr (kFast) {
        q0 = div_refined(d0, scale, rcp); q1 = div_refined(d1, scale, rcp);
        const bool ok0 = q0 < 256.0f, ok1 = q1 < 256.0f;           // false for the NaN of a degenerate scale
        if (!(ok0 & ok1)) {
          if (!ok0) q0 = div_exact(d0, scale);
          if (!ok1) q1 = div_exact(d1, scale);
        }
      } else {
        q0 = __fdiv_rn(d0, scale); q1 = __fdiv_rn(d1, scale);
      }
      round2<T>(q0, q1, q0, q1);
      // fmaxf / fminf return the other operand for NaN: a NaN quotient becomes level 0, as the cast does in torch;
      // adding and subtracting 1.5 * 2^23 rounds half to even
      const float r0 = __fsub_rn(__fadd_rn(fminf(fmaxf(q0, 0.0f), 15.0f), 12582912.0f), 12582912.0f);
      const float r1 = __fsub_rn(__fadd_rn(fminf(fmaxf(q1, 0.0f), 15.0f), 12582912.0f), 12582912.0f);
      const float w0 = static_cast<float>(1u << (4 * (i & 3))), w1 = static_cast<float>(1u << (4 * (i & 3) + 4));
      if (i < 4) { acc_lo = __fmaf_rn(r0, w0, acc_lo); acc_lo = __fmaf_rn(r1, w1, acc_lo); }
      else { acc_hi = __fmaf_rn(r0, w0, acc_hi); acc_hi = __fmaf_rn(r1, w1, acc_hi); }
    }
    // both sums are integers below 2^16: after adding 2^23 they sit in the low mantissa bits
    uint32_t word = __byte_perm(__float_as_uint(__fadd_rn(acc_lo, 8388608.0f)),
                                __float_as_uint(__fadd_rn(acc_hi, 8388608.0f)), 0x5410);
    if constexpr (TILED) word = to_tiled_word(word, lane);
    if (ok) {
      char* row = reinterpret_cast<char*>(a.codes) + b * a.c_sb + h * a.c_sh + static_cast<int64_t>(t + tok_off) * 64;
      reinterpret_cast<uint32_t*>(row)[word_index(sub, TILED)] = word;
      if (sub == 0) {
        const int64_t at = b * a.s_sb + h * a.s_sh + t + tok_off;
        static_cast<T*>(a.scale)[at] = Elem<T>::from_float(scale);
        static_cast<T*>(a.mn)[at] = Elem<T>::from_float(mn);
      }
    }
  }
}

// kivi <-> tiled conversion of packed rows: the field transpose is an involution up to the word order
__global__ void __launch_bounds__(kValThreads) relayout_values_kernel(const uint32_t* in, uint32_t* out,
                                                                       long long tokens, int to_tiled) {
  const long long tok = (static_cast<long long>(blockIdx.x) * kValThreads + threadIdx.x) >> 4;
  const int sub = threadIdx.x & 15, lane = threadIdx.x & 31;
  const bool ok = tok < tokens;
  const long long tk = ok ? tok : 0;
  // lane r of half h must hold the word whose fields are spread over the eight output words of its group:
  // kivi word 8 h + r on the way in, tiled word 2 r + h on the way back
  const uint32_t w = in[tk * 16 + word_index(sub, !to_tiled)];
  const uint32_t o = to_tiled_word(w, lane);
  if (ok) out[tk * 16 + word_index(sub, to_tiled != 0)] = o;
}

// out[b, h, m, :] = sum_t probs[b, h, m, t] * (level[b, h, t, :] * scale[b, h, t] + mn[b, h, t]), kivi layout.
// One CTA per (b, h, m): 64 tokens in flight (16 lanes x 8 channels each), fp32 accumulation, one shared-memory
// reduction over the 64 token lanes.
constexpr int kMatThreads = 1024;
template <typename T>
__global__ void __launch_bounds__(kMatThreads) values_matmul_kernel(const T* probs, const uint32_t* codes,
                                                                     const T* scale, const T* mn, T* out, int M,
                                                                     int Tn) {
  __shared__ float red[kMatThreads / 16][128 + 4];
  const int sub = threadIdx.x & 15, tl = threadIdx.x >> 4;
  const long long bhm = blockIdx.x, bh = bhm / M;
  const T* p = probs + bhm * Tn;
  const uint32_t* c = codes + bh * Tn * 16;
  const T* s = scale + bh * Tn;
  const T* z = mn + bh * Tn;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int t = tl; t < Tn; t += kMatThreads / 16) {
    const float pt = Elem<T>::to_float(p[t]);
    const float ps = pt * Elem<T>::to_float(s[t]), pz = pt * Elem<T>::to_float(z[t]);
    const uint32_t w = c[static_cast<long long>(t) * 16 + sub];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += fmaf(static_cast<float>((w >> (4 * i)) & 0xfu), ps, pz);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[tl][8 * sub + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < 128) {
    float sum = 0.f;
    for (int r = 0; r < kMatThreads / 16; ++r) sum += red[r][threadIdx.x];
    out[bhm * 128 + threadIdx.x] = Elem<T>::from_float(sum);
  }
}

template <typename T>
int launch_quantize_values(ValArgs a, long long units, bool tiled, cudaStream_t s) {
  const int per_cta = kTokPerIter * kValIters;
  const unsigned gx = static_cast<unsigned>((a.T + per_cta - 1) / per_cta);
  for (long long u0 = 0; u0 < units; u0 += 65535) {          // grid.y is limited to 65535 units per launch
    const unsigned gy = static_cast<unsigned>(units - u0 < 65535 ? units - u0 : 65535);
    a.unit0 = static_cast<int>(u0);
    if (tiled) quantize_values_kernel<T, true><<<dim3(gx, gy), kValThreads, 0, s>>>(a);
    else quantize_values_kernel<T, false><<<dim3(gx, gy), kValThreads, 0, s>>>(a);
    PQ_CUDA_TRY(cudaGetLastError());
  }
  return PQ_OK;
}

}  // namespace

int quantize_values_device(const void* values, const int64_t strides[4], int B, int Nk, int T, int hd, int vbits,
                           int dtype, int layout, void* codes, void* scale, void* mn, const int64_t* out_strides,
                           cudaStream_t stream, const int* gate_lengths, int gate_r_add, int gate_full, int gate_G,
                           int gate_max_tokens) {
  if (gate_lengths && (!out_strides || gate_full <= 0 || gate_G <= 0 || gate_max_tokens < T)) return PQ_ERR_INVALID;
  if (B < 0 || Nk <= 0 || T < 0 || !dtype_ok(dtype) || !strides) return PQ_ERR_INVALID;
  if (layout != PQ_VALUES_KIVI && layout != PQ_VALUES_TILED) return PQ_ERR_INVALID;
  if (hd != kHeadDim || vbits != 4) return PQ_ERR_UNSUPPORTED;
  if (strides[3] != 1) return PQ_ERR_UNSUPPORTED;
  if (B == 0 || T == 0) return PQ_OK;
  if (!values || !codes || !scale || !mn) return PQ_ERR_INVALID;
  const size_t es = dtype_bytes(dtype);
  if (reinterpret_cast<uintptr_t>(values) % 16 || (strides[0] * es) % 16 || (strides[1] * es) % 16 ||
      (strides[2] * es) % 16 || reinterpret_cast<uintptr_t>(codes) % 16)
    return PQ_ERR_ALIGNMENT;
  ValArgs a{};
  a.v = values; a.sb = strides[0]; a.sh = strides[1]; a.st = strides[2];
  a.codes = static_cast<uint32_t*>(codes); a.scale = scale; a.mn = mn;
  a.c_sh = static_cast<int64_t>(T) * 64; a.c_sb = a.c_sh * Nk;
  a.s_sh = T; a.s_sb = a.s_sh * Nk;
  if (out_strides) {
    a.c_sb = out_strides[0]; a.c_sh = out_strides[1]; a.s_sb = out_strides[2]; a.s_sh = out_strides[3];
    if (a.c_sb % 16 || a.c_sh % 16) return PQ_ERR_ALIGNMENT;
  }
  a.Nk = Nk; a.T = T;
  a.gate_lengths = gate_lengths; a.gate_r_add = gate_r_add; a.gate_full = gate_full; a.gate_G = gate_G;
  a.gate_max_tokens = gate_max_tokens;
  a.inv_levels = 1.0f / 15.0f;
  const long long units = static_cast<long long>(B) * Nk;
  if (units > 0x7fffffffLL) return PQ_ERR_UNSUPPORTED;
  const bool tiled = layout == PQ_VALUES_TILED;
  switch (dtype) {
    case PQ_F16: return launch_quantize_values<__half>(a, units, tiled, stream);
    case PQ_BF16: return launch_quantize_values<__nv_bfloat16>(a, units, tiled, stream);
    default: return launch_quantize_values<float>(a, units, tiled, stream);
  }
}

int values_relayout_device(const void* codes_in, void* codes_out, int64_t tokens, int to_layout, cudaStream_t stream) {
  if (tokens < 0 || (to_layout != PQ_VALUES_KIVI && to_layout != PQ_VALUES_TILED)) return PQ_ERR_INVALID;
  if (tokens == 0) return PQ_OK;
  if (!codes_in || !codes_out || codes_in == codes_out) return PQ_ERR_INVALID;
  if (reinterpret_cast<uintptr_t>(codes_in) % 4 || reinterpret_cast<uintptr_t>(codes_out) % 4) return PQ_ERR_ALIGNMENT;
  const long long ctas = (tokens * 16 + kValThreads - 1) / kValThreads;
  if (ctas > 0x7fffffffLL) return PQ_ERR_UNSUPPORTED;
  relayout_values_kernel<<<static_cast<unsigned>(ctas), kValThreads, 0, stream>>>(
      static_cast<const uint32_t*>(codes_in), static_cast<uint32_t*>(codes_out), tokens, to_layout == PQ_VALUES_TILED);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

int values_matmul_device(const void* probs, const void* codes, const void* scale, const void* mn, void* out,
                         int64_t BH, int M, int T, int hd, int vbits, int dtype, cudaStream_t stream) {
  if (BH < 0 || M <= 0 || T < 0 || !dtype_ok(dtype)) return PQ_ERR_INVALID;
  if (hd != kHeadDim || vbits != 4) return PQ_ERR_UNSUPPORTED;
  if (BH == 0) return PQ_OK;
  if (!out || (T > 0 && (!probs || !codes || !scale || !mn))) return PQ_ERR_INVALID;
  if (BH * M > 0x7fffffffLL) return PQ_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(codes) % 4) return PQ_ERR_ALIGNMENT;
  const unsigned grid = static_cast<unsigned>(BH * M);
  switch (dtype) {
    case PQ_F16:
      values_matmul_kernel<__half><<<grid, kMatThreads, 0, stream>>>(
          static_cast<const __half*>(probs), static_cast<const uint32_t*>(codes), static_cast<const __half*>(scale),
          static_cast<const __half*>(mn), static_cast<__half*>(out), M, T);
      break;
    case PQ_BF16:
      values_matmul_kernel<__nv_bfloat16><<<grid, kMatThreads, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(probs), static_cast<const uint32_t*>(codes),
          static_cast<const __nv_bfloat16*>(scale), static_cast<const __nv_bfloat16*>(mn),
          static_cast<__nv_bfloat16*>(out), M, T);
      break;
    default:
      values_matmul_kernel<float><<<grid, kMatThreads, 0, stream>>>(
          static_cast<const float*>(probs), static_cast<const uint32_t*>(codes), static_cast<const float*>(scale),
          static_cast<const float*>(mn), static_cast<float*>(out), M, T);
      break;
  }
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

}  // namespace pq
