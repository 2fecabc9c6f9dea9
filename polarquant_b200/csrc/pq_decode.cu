// Decode-time kernels over the packed polar key cache (sm_100a):
//   * qk_decode_kernel        - un-scaled fp32 logits q.K^T over the codes
//                               (the reference's Triton kernel, models/kernel4group.py:14-80)
//   * decode_attention_kernel - fused: logits over codes + logits over the
//                               full-precision residual keys + scale + mask +
//                               online softmax + P.V, one partial per warp segment
//                               (models/modeling_llama_polar.py:66-99)
//   * merge_partials_kernel / merge_lse_kernel - log-sum-exp merges.
//
// Work decomposition.  A "step" is 16 consecutive tokens of one (batch, kv head)
// unit.  All steps of all units form one flat sequence that is cut into equal
// contiguous ranges, one per warp; warps never synchronise with each other.
// A warp whose range crosses a unit boundary emits one partial (m, l, O) per
// unit it touched; the merge kernel finds a unit's partials by the same
// arithmetic, so no counters, atomics or zero-initialised scratch are needed.
//
// Per step (one warp, 16 tokens, all query heads of the kv head):
//   1. 128-bit loads of the 16 x 64 code bytes: lane (g, t) [g = lane / 4,
//      t = lane % 4] gets the codes of pairs 16t..16t+15 of tokens g and g+8.
//   2. Dequantise in registers: the angle code indexes a per-group table of
//      (cos, sin) half2 entries in shared memory (64 pairs x 2^tbits levels,
//      rebuilt per token group because the angle step and offset are per
//      (group, pair), models/kernel4group.py:67); the radius code becomes a
//      half directly through an exponent trick and one HFMA2.  The products
//      land in the A-fragment layout of mma.m16n8k16 (tokens x pair-channels).
//   3. S^T[token, head] = K^[token, :] . q[head, :] on the tensor cores, the
//      query heads of the kv head (<= 8) as the N dimension.  The lookup-table
//      form of the reference (one table per query head) needs one shared-memory
//      gather per (token, pair, head); the dequantise-then-MMA form needs one
//      per (token, pair) whatever the GQA group size.
//   4. Online softmax in the log2 domain on the accumulator fragment, warp
//      shuffles across the eight token rows.
//   5. P^T is transposed in registers (movmatrix) into the B operand and
//      O^T[channel, head] += V^T[channel, token] . P^T[token, head]; value tiles are
//      copied global -> shared with cp.async two steps ahead (three stages per
//      warp, rows padded to 272 bytes) and read as A fragments with
//      ldmatrix.trans, which needs no registers while the tile is in flight.
//
// tcgen05/TMEM is not used: one decode query per head gives M = 16 tokens x
// N <= 8 heads tiles, far below the 64-row minimum of tcgen05.mma, and the path
// is bound by HBM and the shared-memory gathers, not by tensor throughput.
#include <stdlib.h>

#include <mutex>

#include "pq_exchange.cuh"

namespace pq {
namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;
constexpr int kStep = 16;          // tokens per step
constexpr int kHeadTile = 8;       // query heads per unit (N of the MMA)
constexpr int kPartialFloats = kHeadDim * kHeadTile;   // O^T partial, [channel][head]
#ifndef PQ_PREFETCH_STEPS
#define PQ_PREFETCH_STEPS 4
#endif
constexpr int kPrefetch = PQ_PREFETCH_STEPS;   // steps between the L2 prefetch and the use of a tile (0 = off)

struct DecodeArgs {
  const void* q; int64_t q_sb, q_sh;
  const uint8_t* codes; int64_t c_sb, c_sh;
  int key_format;       // PQ_KEYS_BYTE: one byte per pair; PQ_KEYS_PACKED6: 48 bytes per token, tiled per 16-token step
  const void *rscale, *rmn, *tscale, *tmn; int64_t s_sb, s_sh;
  const void* kres; int64_t kr_sb, kr_sh, kr_st;
  const void* v; int64_t v_sb, v_sh, v_st;
  int v_tok0;           // token of `v` that holds the first residual value: Nb*G, or 0 with packed values
  const void* vq_codes; int64_t vq_sb, vq_sh;            // packed values, byte strides
  const void *vq_scale, *vq_mn; int64_t vs_sb, vs_sh;    // their per-token scale / minimum, element strides
  const uint8_t* mask; int64_t m_sb;
  float* part_o;        // [slot][128][8]
  float2* part_ml;      // [slot][8]  (running max in log2 units, running sum)
  float* logits;        // qk-only output (B, N, Nb*G)
  int B, N, Nk, Nb, G, R;
  int nrep, head_tiles;
  int spg;              // steps per token group = G / 16
  int nq, nr, slots_per_unit;   // quantised steps, residual steps, nq + 2*nr
  long long total_slots; int total_warps; int max_seg;
  float scale_log2;     // sm_scale * log2(e)
  // Lengths read on the device (CUDA-graph replay of a growing cache): dyn[0] = token groups, dyn[1] + dyn_r_add =
  // residual tokens.  The kernels then redo the partition themselves from these and from the launch's CTA count.
  const int* dyn; int dyn_r_add;
  long long plan_ctas; int plan_forced;
};

constexpr int kMinSlotsPerWarp = 16;   // below this a partial costs more than the work it covers

// The partition of the flat step space over warps, from the problem's dimensions and the CTAs available.  Host
// and device evaluate the same integer arithmetic, so a kernel that reads its lengths on the device arrives at
// the plan the host would have made.
__host__ __device__ inline void plan_core(DecodeArgs& a, long long ctas, bool forced) {
  a.nrep = a.N / a.Nk;
  a.head_tiles = (a.nrep + kHeadTile - 1) / kHeadTile;
  a.spg = a.G / kStep;
  a.nq = a.Nb * a.spg;
  a.nr = (a.R + kStep - 1) / kStep;
  a.slots_per_unit = a.nq + 2 * a.nr;
  const long long units = static_cast<long long>(a.B) * a.Nk * a.head_tiles;
  a.total_slots = units * a.slots_per_unit;
  const long long useful = (a.total_slots + static_cast<long long>(kMinSlotsPerWarp) * kWarps - 1) /
                           (static_cast<long long>(kMinSlotsPerWarp) * kWarps);
  if (!forced && ctas > useful) ctas = useful;
  if (ctas < 1) ctas = 1;
  long long warps = ctas * kWarps;
  if (warps > a.total_slots) warps = a.total_slots > 0 ? a.total_slots : 1;   // every warp range is non-empty
  a.total_warps = static_cast<int>(warps);
  const long long per_warp = (a.total_slots + a.total_warps - 1) / a.total_warps;
  // an empty problem (device-side lengths of an empty cache) has no slots and no partials
  a.max_seg = a.slots_per_unit > 0 ? static_cast<int>((per_warp + a.slots_per_unit - 1) / a.slots_per_unit) + 1 : 0;
}
__device__ __forceinline__ void plan_on_device(DecodeArgs& a) {
  // the host's Nb / R are the capacities of the buffers: lengths beyond them are clamped, never followed
  a.Nb = min(max(a.dyn[0], 0), a.Nb);
  a.R = min(max(a.dyn[1] + a.dyn_r_add, 0), a.R);
  if (!a.vq_codes) a.v_tok0 = a.Nb * a.G;
  plan_core(a, a.plan_ctas, a.plan_forced != 0);
}
// partial slots no plan over the given CTAs can exceed: total_warps * max_seg <= units + 3 * warps
__host__ __device__ inline long long slot_bound(long long units, long long ctas) { return units + 3 * ctas * kWarps; }

__device__ __forceinline__ long long range_lo(long long w, long long total, int nwarps) {
  return (w * total) / nwarps;
}

// A CTA whose four warp ranges all lie inside one unit combines its four partials in shared memory and
// emits a single one (in the slot of its first warp): four times fewer partials for the merge kernel when a
// unit is spread over many warps.  Both kernels evaluate this predicate the same way.
__device__ __forceinline__ bool cta_in_one_unit(long long cta, long long total_slots, int total_warps,
                                                int slots_per_unit) {
  const long long w_first = cta * 4, w_end = w_first + 4;
  if (w_end > total_warps) return false;
  const long long lo = range_lo(w_first, total_slots, total_warps), hi = range_lo(w_end, total_slots, total_warps);
  return lo / slots_per_unit == (hi - 1) / slots_per_unit;
}

// ---- per-group constants staged in shared memory ------------------------------------
// The four scale rows of a token group (rscale, rmn, tscale, tmn: 4 x 64 elements) are
// copied global -> shared with cp.async one group ahead of their use, double-buffered,
// so the dependent table build never waits on DRAM.
template <int SDT, bool COMMIT = true>
__device__ __forceinline__ void stage_scales_async(uint32_t dst_addr, const char* rs_row, const char* rm_row,
                                                   const char* ts_row, const char* tm_row, int lane) {
  constexpr int kChunks = (SDT == PQ_F32 ? 16 : 8);          // 16-byte chunks per row
#pragma unroll
  for (int i = lane; i < 4 * kChunks; i += 32) {
    const int tensor = i / kChunks, chunk = i % kChunks;
    const char* src = (tensor == 0 ? rs_row : tensor == 1 ? rm_row : tensor == 2 ? ts_row : tm_row) + 16 * chunk;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_addr + 16u * i), "l"(src) : "memory");
  }
  if constexpr (COMMIT) asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void wait_staged() {
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncwarp();
}

// ---- shared-memory table of (cos, sin) bin centres for one token group ----------
// word index = (row_pos << TBITS) + (level ^ x), row_pos = 4 * (d % 16) + d / 16, so the
// four rows a warp gathers from in one instruction (pairs 16t + m, t = 0..3) are adjacent
// and the lane-dependent part of the byte offset fits in the low byte.  The XOR with
// x = (m / 2 + 8 * (t / 2)) mod 2^TBITS (m = d % 16, t = d / 16) spreads a gather's lanes over
// the banks; the gather side folds the same XOR into the constant it already applies to the
// code bytes.
template <int TBITS> __device__ __forceinline__ uint32_t table_xor(int m, int t) {
  return static_cast<uint32_t>((m >> 1) + 8 * (t >> 1)) & ((1u << TBITS) - 1u);
}

// The build writes whole quads of adjacent positions with 128-bit stores.  Lane l = 8 a + 4 b + c owns the pairs
// (m, t) = (4 a + 2 half + c / 2, b + 2 (c % 2)), half = 0, 1, and walks the quads of a row in the order
// jq ^ (c or c / 2): in every quarter-warp phase of a store the eight lanes then hit eight different 16-byte bank
// groups, for every table size.  Position p of a row holds level p ^ x; the level enters the angle as a float built
// by bit insertion - 16 + level has the mantissa level / 16 - so phi = ts * ((16 + level) - 15.5) + tm is one FMA.
template <int TBITS, int SDT>
__device__ __forceinline__ void build_angle_table(uint32_t tbl_addr, const char* sc, int lane) {
  constexpr int A = 1 << TBITS;
  constexpr int ES = SDT == PQ_F32 ? 4 : 2;
  constexpr int ROW = 64 * ES;                               // bytes per staged scale row
  auto scale_at = [&](int row, int d) {
    if constexpr (SDT == PQ_F32) return *reinterpret_cast<const float*>(sc + row * ROW + 4 * d);
    else if constexpr (SDT == PQ_F16) return __half2float(*reinterpret_cast<const __half*>(sc + row * ROW + 2 * d));
    else return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sc + row * ROW + 2 * d));
  };
  if constexpr (A >= 4) {
    const int a = lane >> 3, b = (lane >> 2) & 1, c = lane & 3;
    const int t = b + 2 * (c & 1);
    const uint32_t walk = TBITS == 4 ? c : TBITS == 3 ? (c >> 1) : 0;      // quad order of this lane
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = 4 * a + 2 * half + (c >> 1), d = 16 * t + m;
      const float ts = scale_at(2, d), tm_c = fmaf(-15.5f, ts, scale_at(3, d));
      const uint32_t base = tbl_addr + (static_cast<uint32_t>(4 * m + t) << (TBITS + 2));
      const uint32_t xs = (table_xor<TBITS>(m, t) ^ (walk << 2)) << 19;      // level = (4 jq + i) ^ (4 walk) ^ x
#pragma unroll
      for (int jq = 0; jq < A / 4; ++jq) {
        uint32_t cs[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          // |phi| stays small (a quantiser emits [0, 2 pi]); the hardware sine/cosine take the
          // fraction of phi / (2 pi), precise to ~1e-6 for |phi| < 100, far below fp16 spacing
          const float lv = __uint_as_float((0x41800000u | (static_cast<uint32_t>(4 * jq + i) << 19)) ^ xs);
          const float phi = fmaf(ts, lv, tm_c);
          cs[i] = pack2<PQ_F16>(__cosf(phi), __sinf(phi));
        }
        const uint32_t at = base + ((static_cast<uint32_t>(jq) ^ walk) << 4);
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(at), "r"(cs[0]), "r"(cs[1]), "r"(cs[2]), "r"(cs[3])
                     : "memory");
      }
    }
  } else {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int d = 2 * lane + half, m = d & 15, t = d >> 4;
      const float ts = scale_at(2, d), tm = scale_at(3, d);
      const uint32_t base = tbl_addr + (static_cast<uint32_t>(4 * m + t) << (TBITS + 2));
      const uint32_t bx = base ^ (table_xor<TBITS>(m, t) << 2);
#pragma unroll
      for (int k = 0; k < A; ++k) {
        const float phi = fmaf(ts, static_cast<float>(k) + 0.5f, tm);
        const uint32_t cs = pack2<PQ_F16>(__cosf(phi), __sinf(phi));
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(bx ^ (static_cast<uint32_t>(k) << 2)), "r"(cs) : "memory");
      }
    }
  }
  __syncwarp();
}

template <int SDT> __device__ __forceinline__ void load16f(const void* p, float (&v)[16]) {
  if constexpr (SDT == PQ_F32) {
    const float4* f = static_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float4 x = f[i];
      v[4 * i] = x.x; v[4 * i + 1] = x.y; v[4 * i + 2] = x.z; v[4 * i + 3] = x.w;
    }
  } else {
    const uint4* u = static_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 x = u[i];
      float2 a = unpack2<SDT>(x.x), b = unpack2<SDT>(x.y), c = unpack2<SDT>(x.z), d = unpack2<SDT>(x.w);
      v[8 * i] = a.x; v[8 * i + 1] = a.y; v[8 * i + 2] = b.x; v[8 * i + 3] = b.y;
      v[8 * i + 4] = c.x; v[8 * i + 5] = c.y; v[8 * i + 6] = d.x; v[8 * i + 7] = d.y;
    }
  }
}

// Radius constants of this lane's 16 pairs for one group.  The radius code rho is
// turned into the half value 2^RBITS + rho by OR-ing it into the mantissa of
// 2^RBITS, so r = rscale * (rho + 0.5) + rmn = rscale * (2^RBITS + rho) + c with
// c = rmn + (0.5 - 2^RBITS) * rscale.  rs2/rc2[w][e] hold the constants of pairs
// (4w + e, 4w + e + 2), the two code bytes one HFMA2 handles.
template <int RBITS, int SDT>
__device__ __forceinline__ void load_radius_consts(const char* sc, int t,
                                                   uint32_t (&rs2)[4][2], uint32_t (&rc2)[4][2]) {
  constexpr int ES = SDT == PQ_F32 ? 4 : 2;
  float rs[16], rm[16];
  load16f<SDT>(sc + 16 * t * ES, rs);
  load16f<SDT>(sc + 64 * ES + 16 * t * ES, rm);
  const float k = 0.5f - static_cast<float>(1 << RBITS);
#pragma unroll
  for (int w = 0; w < 4; ++w)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int a = 4 * w + e, b = a + 2;
      rs2[w][e] = pack2<PQ_F16>(rs[a], rs[b]);
      rc2[w][e] = pack2<PQ_F16>(fmaf(k, rs[a], rm[a]), fmaf(k, rs[b], rm[b]));
    }
}

__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
  __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b),
                      *reinterpret_cast<__half2*>(&c));
  return *reinterpret_cast<uint32_t*>(&r);
}
// cs * (rr.lo, rr.lo) and cs * (rr.hi, rr.hi): the half selection folds into the multiply
__device__ __forceinline__ uint32_t hmul2_lo(uint32_t cs, uint32_t rr) {
  __half2 r = __hmul2(*reinterpret_cast<__half2*>(&cs), __low2half2(*reinterpret_cast<__half2*>(&rr)));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t hmul2_hi(uint32_t cs, uint32_t rr) {
  __half2 r = __hmul2(*reinterpret_cast<__half2*>(&cs), __high2half2(*reinterpret_cast<__half2*>(&rr)));
  return *reinterpret_cast<uint32_t*>(&r);
}

// The gathers are plain (movable) asm so the compiler may schedule them freely inside a step; the step loop ties
// them to the table build that precedes it.
template <int IMM> __device__ __forceinline__ uint32_t lds_u32_imm(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(IMM));
  return v;
}

// One k-step of S^T += K^ . q^T: code bytes E and E + 2 of word W of the two tokens this
// lane holds (pairs 16t + 4W + E and + 2), dequantised and fed to one MMA.
//   * gather address = byte permute splicing ((theta ^ x) << 2) | (t << (TBITS + 2)) from the
//     prepared code word into the low byte of the 256-byte aligned table address; the row
//     block offset (4W + E) << (TBITS + 4) rides in the load's immediate field;
//   * radius = HFMA2 on the two codes at once (hg / hh: the half pair 2^RBITS + rho of pairs
//     4W + E and 4W + E + 2 of the two tokens); the multiply selects the half it needs.
template <int TBITS, int W, int E>
__device__ __forceinline__ void qk_kstep(float (&S)[4], uint32_t hg, uint32_t hh, uint32_t og, uint32_t oh,
                                         uint32_t tbl_addr, uint32_t rs, uint32_t rc, uint32_t qb0, uint32_t qb1) {
  constexpr int ROW_A = (4 * W + E) << (TBITS + 4), ROW_B = (4 * W + E + 2) << (TBITS + 4);
  const uint32_t rg = hfma2_u(hg, rs, rc);
  const uint32_t rh = hfma2_u(hh, rs, rc);
  const uint32_t csAg = lds_u32_imm<ROW_A>(__byte_perm(og, tbl_addr, 0x7650 | E));
  const uint32_t csBg = lds_u32_imm<ROW_B>(__byte_perm(og, tbl_addr, 0x7650 | (E + 2)));
  const uint32_t csAh = lds_u32_imm<ROW_A>(__byte_perm(oh, tbl_addr, 0x7650 | E));
  const uint32_t csBh = lds_u32_imm<ROW_B>(__byte_perm(oh, tbl_addr, 0x7650 | (E + 2)));
  mma_16816_f16(S, hmul2_lo(csAg, rg), hmul2_lo(csAh, rh), hmul2_hi(csBg, rg), hmul2_hi(csBh, rh), qb0, qb1);
}

// shift right by SR bits (left when SR is negative), SR a compile-time constant
template <int SR> __device__ __forceinline__ uint32_t shift_by(uint32_t x) {
  if constexpr (SR >= 0) return x >> SR; else return x << (-SR);
}

// Byte container: radius code of byte E (and E + 2) of a code word -> mantissa of the half 2^RBITS.
template <int RBITS, int TBITS, int E> __device__ __forceinline__ uint32_t radius_half_bytes(uint32_t cw) {
  constexpr int MSH = 10 - RBITS;                                // mantissa shift of rho
  constexpr uint32_t RM = (((1u << RBITS) - 1u) << MSH) * 0x00010001u;
  constexpr uint32_t MAGIC = (static_cast<uint32_t>(15 + RBITS) << 10) * 0x00010001u;
  return (shift_by<8 * E + TBITS + RBITS - 10>(cw) & RM) | MAGIC;
}

// S^T (16 tokens x 8 heads) += K^ (16 tokens x 128 pair-channels) . q^T for one step.
// cg4 / ch4: this lane's 16 code bytes of tokens g and g + 8.  lane_xor[w] carries, per code
// byte of word w, (x << 2) | (t << (TBITS + 2)) for this lane's t (x: the table's bank swizzle).
template <int RBITS, int TBITS>
__device__ __forceinline__ void qk_step_quant(float (&S)[4], const uint4& cg4, const uint4& ch4,
                                              uint32_t tbl_addr, const uint32_t (&lane_xor)[4],
                                              const uint32_t (&rs2)[4][2], const uint32_t (&rc2)[4][2],
                                              const uint32_t (&qb)[8][2]) {
  constexpr uint32_t TM4 = (((1u << TBITS) - 1u) << 2) * 0x01010101u;
  // two accumulator sets halve the chain of dependent MMAs
  float S2[4] = {0.f, 0.f, 0.f, 0.f};
#define PQ_WORD(W, CG, CH)                                                                                     \
  {                                                                                                            \
    const uint32_t og = (((CG) << 2) & TM4) ^ lane_xor[W];                                                     \
    const uint32_t oh = (((CH) << 2) & TM4) ^ lane_xor[W];                                                     \
    qk_kstep<TBITS, W, 0>(S, radius_half_bytes<RBITS, TBITS, 0>(CG), radius_half_bytes<RBITS, TBITS, 0>(CH),  \
                          og, oh, tbl_addr, rs2[W][0], rc2[W][0], qb[2 * W][0], qb[2 * W][1]);                 \
    qk_kstep<TBITS, W, 1>(S2, radius_half_bytes<RBITS, TBITS, 1>(CG), radius_half_bytes<RBITS, TBITS, 1>(CH), \
                          og, oh, tbl_addr, rs2[W][1], rc2[W][1], qb[2 * W + 1][0], qb[2 * W + 1][1]);         \
  }
  PQ_WORD(0, cg4.x, ch4.x)
  PQ_WORD(1, cg4.y, ch4.y)
  PQ_WORD(2, cg4.z, ch4.z)
  PQ_WORD(3, cg4.w, ch4.w)
#undef PQ_WORD
#pragma unroll
  for (int i = 0; i < 4; ++i) S[i] += S2[i];
}

// ---- 6-bit packed keys (PQ_KEYS_PACKED6) -----------------------------------------------------
// 48 bytes per token instead of 64, for the bit splits whose code has 6 bits (3/3 and 2/4).  The format is tiled
// per 16-token step (768 bytes) in the order the warp consumes it, so that a lane's share of a step is one 16-byte
// and one 8-byte load and the unpacking costs what the byte container costs:
//   bytes [0, 512):   lane l = 4 g + t holds words A0, A1 of token g, then A0, A1 of token g + 8;
//   bytes [512, 768): lane l holds word H of token g, then H of token g + 8.
// With c[p] the code of pair 16 t + p (p = 0..15) of a token:
//   A_k (k = 0, 1): nibble 2 i = c[8 k + i] & 15, nibble 2 i + 1 = c[8 k + 4 + i] & 15   (i = 0..3), so the even
//                   nibbles of A_k are the low code bits of code word 2 k and the odd ones of code word 2 k + 1;
//   H: bits 2 j .. 2 j + 1 = c[4 W + E] >> 4 and bits 16 + 2 j .. = c[4 W + E + 2] >> 4 with j = 2 W + E
//                   (W = 0..3, E = 0..1): the two codes one HFMA2 handles sit 16 bits apart.
// The low nibble holds the angle code (and, for 3/3, the lowest radius bit); H holds the upper two radius bits.
constexpr int kPackedStepBytes = 768;
template <int RBITS, int TBITS, int W, int E>
__device__ __forceinline__ uint32_t radius_half_packed(uint32_t aw, uint32_t hw) {
  static_assert((RBITS == 2 && TBITS == 4) || (RBITS == 3 && TBITS == 3), "6-bit codes: 2/4 or 3/3");
  constexpr uint32_t MAGIC = (static_cast<uint32_t>(15 + RBITS) << 10) * 0x00010001u;
  constexpr uint32_t HI = (3u << 8) * 0x00010001u;               // the two upper radius bits at mantissa bits 8..9
  const uint32_t top = (shift_by<2 * (2 * W + E) - 8>(hw) & HI) | MAGIC;
  if constexpr (RBITS == 2) return top;
  else {
    // lowest radius bit: bit 3 of nibble 2 E + (W & 1) of the A word, to mantissa bit 7
    constexpr uint32_t LO = (1u << 7) * 0x00010001u;
    return (shift_by<8 * E + 4 * (W & 1) + 3 - 7>(aw) & LO) | top;
  }
}
template <int RBITS, int TBITS>
__device__ __forceinline__ void qk_step_packed6(float (&S)[4], const uint4& ca, const uint2& chh,
                                                uint32_t tbl_addr, const uint32_t (&lane_xor)[4],
                                                const uint32_t (&rs2)[4][2], const uint32_t (&rc2)[4][2],
                                                const uint32_t (&qb)[8][2]) {
  constexpr uint32_t TM4 = (((1u << TBITS) - 1u) << 2) * 0x01010101u;
  float S2[4] = {0.f, 0.f, 0.f, 0.f};
  // AG / AH: the A word of tokens g / g + 8 that holds code word W (A_{W / 2}); even W reads its even nibbles
#define PQ_WORD6(W, AG, AH)                                                                                          \
  {                                                                                                                  \
    const uint32_t og = (shift_by<((W) & 1) ? 2 : -2>(AG) & TM4) ^ lane_xor[W];                                      \
    const uint32_t oh = (shift_by<((W) & 1) ? 2 : -2>(AH) & TM4) ^ lane_xor[W];                                      \
    qk_kstep<TBITS, W, 0>(S, radius_half_packed<RBITS, TBITS, W, 0>(AG, chh.x),                                      \
                          radius_half_packed<RBITS, TBITS, W, 0>(AH, chh.y), og, oh, tbl_addr, rs2[W][0], rc2[W][0], \
                          qb[2 * W][0], qb[2 * W][1]);                                                               \
    qk_kstep<TBITS, W, 1>(S2, radius_half_packed<RBITS, TBITS, W, 1>(AG, chh.x),                                     \
                          radius_half_packed<RBITS, TBITS, W, 1>(AH, chh.y), og, oh, tbl_addr, rs2[W][1], rc2[W][1], \
                          qb[2 * W + 1][0], qb[2 * W + 1][1]);                                                       \
  }
  PQ_WORD6(0, ca.x, ca.z)
  PQ_WORD6(1, ca.x, ca.z)
  PQ_WORD6(2, ca.y, ca.w)
  PQ_WORD6(3, ca.y, ca.w)
#undef PQ_WORD6
#pragma unroll
  for (int i = 0; i < 4; ++i) S[i] += S2[i];
}

// Ask the L2 to fetch `bytes` (a multiple of 16) starting at the 16-byte aligned address p.
__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// Query B fragments for the quantised path: k-step s = 2w + e pairs lanes' slots with
// pairs pA = 16t + 4w + e and pB = pA + 2; a register holds (q[p], q[p + 64]) as half2.
template <int QDT>
__device__ __forceinline__ void load_q_quant(const void* q_head, bool valid, int t, uint32_t (&qb)[8][2]) {
#pragma unroll
  for (int s = 0; s < 8; ++s)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int p = 16 * t + 4 * (s >> 1) + (s & 1) + 2 * j;
      float x = 0.f, y = 0.f;
      if (valid) {
        if constexpr (QDT == PQ_F32) {
          x = static_cast<const float*>(q_head)[p]; y = static_cast<const float*>(q_head)[p + kPairs];
        } else if constexpr (QDT == PQ_F16) {
          x = __half2float(static_cast<const __half*>(q_head)[p]);
          y = __half2float(static_cast<const __half*>(q_head)[p + kPairs]);
        } else {
          x = __bfloat162float(static_cast<const __nv_bfloat16*>(q_head)[p]);
          y = __bfloat162float(static_cast<const __nv_bfloat16*>(q_head)[p + kPairs]);
        }
      }
      qb[s][j] = pack2<PQ_F16>(x, y);
    }
}

// eight consecutive elements at p as four packed 16-bit pairs; fp32 is rounded to fp16
template <int DT> __device__ __forceinline__ uint4 load8_as16(const void* p, bool valid) {
  uint4 r = make_uint4(0, 0, 0, 0);
  if (valid) {
    if constexpr (DT == PQ_F32) {
      const float4* f = static_cast<const float4*>(p);
      float4 a = f[0], b = f[1];
      r.x = pack2<PQ_F16>(a.x, a.y); r.y = pack2<PQ_F16>(a.z, a.w);
      r.z = pack2<PQ_F16>(b.x, b.y); r.w = pack2<PQ_F16>(b.z, b.w);
    } else {
      r = ldg_stream(p);
    }
  }
  return r;
}

// element size helper for byte arithmetic on typed-by-tag buffers
__device__ __forceinline__ constexpr int esize(int dt) { return dt == PQ_F32 ? 4 : 2; }

// m0/m1: reference exponent of heads (2t, 2t+1) in the scaled log2 domain - at least the running maximum minus
// kMaxSlack, not necessarily the maximum itself; t0/t1: raw-logit thresholds above which it must be raised.
struct SoftmaxState { float m0, m1, l0, l1, t0, t1; };
constexpr float kMaxSlack = 8.0f;     // probabilities may reach 2^8 before the reference exponent is raised

// Online-softmax update for one step.  S holds logits of tokens (g, g+8) x heads
// (2t, 2t+1).  Returns the P^T B-fragment (b0, b1) in the value dtype and rescales O.
// The running maximum lives in the scaled log2 domain; the scale is applied inside the
// exponent's FMA.  GUARDED adds the per-token validity / mask handling (residual window,
// masked batches); the unguarded form is the hot loop's.
template <int VDT, bool GUARDED, int NT>
__device__ __forceinline__ void softmax_step(float (&S)[4], float scale_log2, bool ok_g, bool ok_h,
                                             bool masked_g, bool masked_h, SoftmaxState& st,
                                             float (&O)[NT][4], uint32_t& b0, uint32_t& b1) {
  if constexpr (GUARDED) {
    // a finite stand-in for "+ finfo.min" keeps an all-masked row uniform, as in the reference
    const float kMasked = -1.0e30f / scale_log2;
    if (masked_g) { S[0] = kMasked; S[1] = kMasked; }
    if (masked_h) { S[2] = kMasked; S[3] = kMasked; }
    if (!ok_g) { S[0] = -INFINITY; S[1] = -INFINITY; }
    if (!ok_h) { S[2] = -INFINITY; S[3] = -INFINITY; }
  }
  float mx0 = fmaxf(S[0], S[2]), mx1 = fmaxf(S[1], S[3]);
  // Raising the reference exponent costs a warp-wide reduction and a rescale of O; it is only needed when a
  // logit exceeds it by more than kMaxSlack (any exponent gives the same softmax, the slack only bounds the
  // magnitude of the unnormalised probabilities).  The guarded form always takes the exact maximum.
  const bool raise = GUARDED || mx0 > st.t0 || mx1 > st.t1;
  if (__any_sync(0xffffffffu, raise)) {
#pragma unroll
    for (int o = 4; o <= 16; o <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
    }
    const float n0 = fmaxf(st.m0, mx0 * scale_log2), n1 = fmaxf(st.m1, mx1 * scale_log2);   // scale > 0
    if (n0 > st.m0 || n1 > st.m1) {                  // uniform over the lanes that share these heads' rows
      const float a0 = exp2_approx(st.m0 - n0), a1 = exp2_approx(st.m1 - n1);
      st.l0 *= a0; st.l1 *= a1;
#pragma unroll
      for (int j = 0; j < NT; ++j) { O[j][0] *= a0; O[j][1] *= a1; O[j][2] *= a0; O[j][3] *= a1; }
      st.m0 = n0; st.m1 = n1;
      const float inv = 1.0f / scale_log2;
      st.t0 = (n0 + kMaxSlack) * inv; st.t1 = (n1 + kMaxSlack) * inv;
    }
  }
  const float n0 = st.m0, n1 = st.m1;
  const float p0 = exp2_approx(fmaf(S[0], scale_log2, -n0)), p1 = exp2_approx(fmaf(S[1], scale_log2, -n1));
  const float p2 = exp2_approx(fmaf(S[2], scale_log2, -n0)), p3 = exp2_approx(fmaf(S[3], scale_log2, -n1));
  st.l0 += p0 + p2; st.l1 += p1 + p3;
  b0 = movmatrix_trans(pack2<VDT>(p0, p1));
  b1 = movmatrix_trans(pack2<VDT>(p2, p3));
}

// ---- value tiles through shared memory ------------------------------------------------
// A value tile is 16 token rows of 256 bytes.  It is copied global -> shared with cp.async
// (16 bytes per lane, 8 per lane per tile) into rows padded to 272 bytes, so that the eight
// rows of every 8x8 block ldmatrix reads fall in eight different 16-byte bank groups.
constexpr int kVRowSmem = 272;
constexpr int kVTileSmem = kStep * kVRowSmem;      // 4352 bytes
#ifndef PQ_V_STAGES
#define PQ_V_STAGES 3
#endif
constexpr int kVStages = PQ_V_STAGES;              // value tiles in flight per warp: kVStages - 1
__device__ __forceinline__ void load_v_tile_async(uint32_t stage_addr, const char* tile, int64_t v_row,
                                                  int valid_rows, int lane) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = i * 32 + lane, row = c >> 4, col = c & 15;
    const bool ok = row < valid_rows;
    const char* src = tile + (ok ? row : 0) * v_row + col * 16;
    const uint32_t dst = stage_addr + row * kVRowSmem + col * 16;
    const int bytes = ok ? 16 : 0;                 // rows past the end are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
  }
}
// Hot-loop form: dst_lane = stage address + this lane's fixed offset, src_lane = tile address + this lane's
// fixed offset; the eight copies of a lane are two rows apart.  With dense token rows (256 bytes) every
// offset is an immediate.
template <bool DENSE>
__device__ __forceinline__ void load_v_tile_fast(uint32_t dst_lane, const char* src_lane, int64_t two_rows) {
#define PQ_CP(I)                                                                                              \
  if constexpr (DENSE)                                                                                        \
    asm volatile("cp.async.cg.shared.global [%0+%2], [%1+%3], 16;" ::"r"(dst_lane), "l"(src_lane),          \
                 "n"((I) * 2 * kVRowSmem), "n"((I) * 2 * kHeadDim * 2) : "memory");                           \
  else                                                                                                        \
    asm volatile("cp.async.cg.shared.global [%0+%2], [%1], 16;" ::"r"(dst_lane), "l"(src_lane + (I) * two_rows), \
                 "n"((I) * 2 * kVRowSmem) : "memory");
  PQ_CP(0) PQ_CP(1) PQ_CP(2) PQ_CP(3) PQ_CP(4) PQ_CP(5) PQ_CP(6) PQ_CP(7)
#undef PQ_CP
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// O^T[channel, head] += V^T . P^T for all eight 16-channel tiles of one staged value tile.
// ldmatrix.trans hands lane (g, t) the pairs {V[2t][c], V[2t+1][c]}: m-tile j row g is channel
// 16j + g, row g + 8 channel 16j + 8 + g.
// lane supplies the row address of matrix (lane / 8), row (lane % 8); the matrices are
// (tokens 0-7, ch +0), (tokens 0-7, ch +8), (tokens 8-15, ch +0), (tokens 8-15, ch +8)
__device__ __forceinline__ uint32_t ldsm_lane_offset(int lane) {
  const int mi = lane >> 3, r = lane & 7;
  return (r + 8 * (mi >> 1)) * kVRowSmem + (mi & 1) * 16;
}
template <int VDT, int NT>
__device__ __forceinline__ void pv_from_smem(float (&O)[NT][4], uint32_t base, uint32_t b0, uint32_t b1) {
#define PQ_PV(J)                                                                                   \
  {                                                                                                \
    uint32_t a0, a1, a2, a3;                                                                       \
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4+%5];"         \
                 : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3)                                          \
                 : "r"(base), "n"((J) * 32));                                                      \
    mma_16816<VDT>(O[J], a0, a1, a2, a3, b0, b1);                                                  \
  }
  PQ_PV(0) PQ_PV(1) PQ_PV(2) PQ_PV(3) PQ_PV(4) PQ_PV(5) PQ_PV(6) PQ_PV(7)
#undef PQ_PV
}

// ---- packed (4-bit) values ---------------------------------------------------------------
// A lane's share of a 16-token value tile in the tiled layout: the 64-bit slot g of tokens 2t, 2t+1, 2t+8, 2t+9
// (fields j = 0..15 = channels g + 8 j), straight from global memory, plus the scale and minimum pairs of those
// tokens.  No shared memory is involved.
struct VqTile { uint2 a, b, c, d; uint32_t s01, s89, m01, m89; };
__device__ __forceinline__ uint2 ldg8_stream(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg4_nc(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ VqTile load_vq_tile(const char* code_lane, const char* scale_lane, const char* mn_lane) {
  VqTile x;
  x.a = ldg8_stream(code_lane); x.b = ldg8_stream(code_lane + 64);
  x.c = ldg8_stream(code_lane + 8 * 64); x.d = ldg8_stream(code_lane + 9 * 64);
  x.s01 = ldg4_nc(scale_lane); x.s89 = ldg4_nc(scale_lane + 16);
  x.m01 = ldg4_nc(mn_lane); x.m89 = ldg4_nc(mn_lane + 16);
  return x;
}
// a pair of 16-bit values of type DT as an fp16 pair
template <int DT> __device__ __forceinline__ uint32_t as_half2(uint32_t w) {
  if constexpr (DT == PQ_F16) return w;
  else { const float2 f = unpack2<PQ_BF16>(w); return pack2<PQ_F16>(f.x, f.y); }
}
__device__ __forceinline__ uint32_t hmul2_u(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// O^T += V^T . P^T with V = level * scale + mn.  The levels enter the tensor core as they are stored: a 4-bit
// field at bits 0-3 (4-7) of a 16-bit lane IS the fp16 subnormal level * 2^-24 (level * 2^-20), so the A operand
// costs one AND per register pair and the powers of two are folded into the accumulators afterwards (rows g hold
// 2^-24, rows g + 8 hold 2^-20 times the true sum).  The scale multiplies P instead of V, and the minimum's
// contribution sum_t mn_t p_t - the same for all channels of a head - is one more MMA into O[8] whose A rows all
// equal the minimum pair.  b0 / b1: P^T in fp16.
template <int VDT>
__device__ __forceinline__ void pv_quant(float (&O)[9][4], const VqTile& x, uint32_t b0, uint32_t b1) {
  const uint32_t m01 = as_half2<VDT>(x.m01), m89 = as_half2<VDT>(x.m89);
  mma_16816_f16(O[8], m01, m01, m89, m89, b0, b1);
  b0 = hmul2_u(b0, as_half2<VDT>(x.s01));
  b1 = hmul2_u(b1, as_half2<VDT>(x.s89));
#define PQ_PVQ(J, Z, Y)                                                                          \
  mma_16816_f16(O[J], (Z) & 0x000f000fu, (Z) & 0x00f000f0u, (Y) & 0x000f000fu, (Y) & 0x00f000f0u, b0, b1);
  {
    const uint32_t zl = __byte_perm(x.a.x, x.b.x, 0x5410), zh = __byte_perm(x.a.x, x.b.x, 0x7632);
    const uint32_t yl = __byte_perm(x.c.x, x.d.x, 0x5410), yh = __byte_perm(x.c.x, x.d.x, 0x7632);
    PQ_PVQ(0, zl, yl) PQ_PVQ(1, zl >> 8, yl >> 8) PQ_PVQ(2, zh, yh) PQ_PVQ(3, zh >> 8, yh >> 8)
  }
  {
    const uint32_t zl = __byte_perm(x.a.y, x.b.y, 0x5410), zh = __byte_perm(x.a.y, x.b.y, 0x7632);
    const uint32_t yl = __byte_perm(x.c.y, x.d.y, 0x5410), yh = __byte_perm(x.c.y, x.d.y, 0x7632);
    PQ_PVQ(4, zl, yl) PQ_PVQ(5, zl >> 8, yl >> 8) PQ_PVQ(6, zh, yh) PQ_PVQ(7, zh >> 8, yh >> 8)
  }
#undef PQ_PVQ
}

// ---------------------------------------------------------------------------------
// fused decode attention
// ---------------------------------------------------------------------------------
#ifndef PQ_MIN_CTAS
#define PQ_MIN_CTAS 3
#endif
// value stages a warp owns: the cp.async pipeline of full-precision values, one tile for the residual window
// when the packed tokens' values are packed too (VQ), none for the logits-only kernel
constexpr int v_stages(bool qk_only, int vq) { return qk_only ? 0 : (vq ? 1 : kVStages); }

template <int RBITS, int TBITS, int QDT, int VDT, bool QK_ONLY, int VQ, bool DYN, int KF = PQ_KEYS_BYTE>
__global__ void __launch_bounds__(kThreads, QK_ONLY ? 4 : PQ_MIN_CTAS)
decode_kernel(const DecodeArgs a_in) {
  // with device-side lengths the plan is recomputed here; otherwise `a` is the parameter itself
  DecodeArgs a_dyn;
  if constexpr (DYN) { a_dyn = a_in; plan_on_device(a_dyn); }
  const DecodeArgs& a = DYN ? a_dyn : a_in;
  constexpr int A = 1 << TBITS;
  constexpr bool kVPipe = !QK_ONLY && VQ == 0;   // values of the packed tokens stream through shared memory
  constexpr int NT = VQ ? 9 : 8;                 // accumulator tiles: 8 channel tiles (+ the minimum term)
  constexpr int QES = QDT == PQ_F32 ? 4 : 2;     // bytes per q / scale / residual-key element
  constexpr int kStageBytes = 4 * kPairs * QES;   // four scale rows of one group
  extern __shared__ __align__(256) unsigned char smem_dyn[];
  constexpr int kWarpSmem = kPairs * A * 4 + 2 * kStageBytes + v_stages(QK_ONLY, VQ) * kVTileSmem;
  unsigned char* warp_smem = smem_dyn + (threadIdx.x >> 5) * kWarpSmem;
  uint32_t* s_tbl_w = reinterpret_cast<uint32_t*>(warp_smem);
  char* s_sc_w = reinterpret_cast<char*>(warp_smem + kPairs * A * 4);

  // A grid launched behind this one with programmatic stream serialisation (the merge kernel) may be
  // set up now; it waits for this grid's completion itself before it reads the partials.
  asm volatile("griddepcontrol.launch_dependents;");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const long long gw = static_cast<long long>(blockIdx.x) * kWarps + warp;
  if (gw >= a.total_warps) return;
  long long lo = range_lo(gw, a.total_slots, a.total_warps);
  const long long hi = range_lo(gw + 1, a.total_slots, a.total_warps);
  if (lo >= hi) return;

  const uint32_t tbl_addr = static_cast<uint32_t>(__cvta_generic_to_shared(s_tbl_w));
  const uint32_t vst_addr = tbl_addr + kPairs * A * 4 + 2 * kStageBytes;   // two value stages
  uint32_t lane_xor[4];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    lane_xor[w] = (static_cast<uint32_t>(t) << (TBITS + 2)) * 0x01010101u;
#pragma unroll
    for (int i = 0; i < 4; ++i) lane_xor[w] |= (table_xor<TBITS>(4 * w + i, t) << 2) << (8 * i);
  }
  constexpr int KRDT = QDT == PQ_BF16 ? PQ_BF16 : PQ_F16;   // MMA type of the residual-key product

  long long unit = lo / a.slots_per_unit;
  int pos = static_cast<int>(lo - unit * a.slots_per_unit);
  int seg = 0;
  // block-uniform: all four warps of such a CTA have exactly one segment, in the same unit
  const bool combine = !QK_ONLY && cta_in_one_unit(blockIdx.x, a.total_slots, a.total_warps, a.slots_per_unit);

  while (lo < hi) {
    const long long unit_end = (unit + 1) * a.slots_per_unit;
    const long long seg_hi = hi < unit_end ? hi : unit_end;
    const int pos_end = pos + static_cast<int>(seg_hi - lo);

    const int ht = static_cast<int>(unit % a.head_tiles);
    const long long bk = unit / a.head_tiles;
    const int kvh = static_cast<int>(bk % a.Nk);
    const int b = static_cast<int>(bk / a.Nk);
    const int head0 = kvh * a.nrep + ht * kHeadTile;
    const int nheads = min(kHeadTile, a.nrep - ht * kHeadTile);
    const bool head_ok = g < nheads;
    const char* q_head = static_cast<const char*>(a.q) + (b * a.q_sb + (head0 + g) * a.q_sh) * QES;

    SoftmaxState st = {-INFINITY, -INFINITY, 0.f, 0.f, -INFINITY, -INFINITY};
    float O[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { O[j][0] = O[j][1] = O[j][2] = O[j][3] = 0.f; }

    const char* v_unit = static_cast<const char*>(a.v) + (b * a.v_sb + kvh * a.v_sh) * 2;
    const int64_t v_row = a.v_st * 2;                       // bytes between tokens
    const uint8_t* mask_row = a.mask ? a.mask + b * a.m_sb : nullptr;
    const int Lq = a.Nb * a.G;

    // ------------------------------ quantised steps ------------------------------
    const int qs_end = pos_end < a.nq ? pos_end : a.nq;
    if (pos < qs_end) {
      uint32_t qb[8][2];
      load_q_quant<QDT>(q_head, head_ok, t, qb);
      const uint8_t* c_unit = a.codes + b * a.c_sb + kvh * a.c_sh;
      const char* rs_unit = static_cast<const char*>(a.rscale) + (b * a.s_sb + kvh * a.s_sh) * QES;
      const char* rm_unit = static_cast<const char*>(a.rmn) + (b * a.s_sb + kvh * a.s_sh) * QES;
      const char* ts_unit = static_cast<const char*>(a.tscale) + (b * a.s_sb + kvh * a.s_sh) * QES;
      const char* tm_unit = static_cast<const char*>(a.tmn) + (b * a.s_sb + kvh * a.s_sh) * QES;
      uint32_t rs2[4][2], rc2[4][2];

      // lane's code bytes: token row * 64 + 16 t (byte container); with packed keys its 16-byte and 8-byte
      // chunks of the step's 768-byte tile (cg: A words of tokens g and g + 8, ch.x / ch.y: their H words)
      constexpr int kCodeStep = KF == PQ_KEYS_PACKED6 ? kPackedStepBytes : kStep * kPairs;   // code bytes per step
      const uint8_t* c_lane = KF == PQ_KEYS_PACKED6
                                  ? c_unit + static_cast<int64_t>(pos) * kCodeStep + 16 * lane
                                  : c_unit + static_cast<int64_t>(pos) * kCodeStep + g * kPairs + 16 * t;
      auto load_second = [&](const uint8_t* cl) {
        if constexpr (KF == PQ_KEYS_PACKED6) {
          const uint2 h = ldg8_stream(cl + 512 - 8 * lane);      // 512 + 8 * lane from the tile's start
          return make_uint4(h.x, h.y, 0u, 0u);
        } else {
          return ldg_stream(cl + 8 * kPairs);
        }
      };
      uint4 cg = ldg_stream(c_lane), ch = load_second(c_lane);
      // value tiles go global -> shared (cp.async) one step ahead, two stages per warp
      // this lane's fixed part of the copy addresses: row lane / 16 (+ 2 per copy), 16-byte column lane % 16
      const char* v_tile = v_unit + static_cast<int64_t>(pos) * kStep * v_row + (lane >> 4) * v_row + (lane & 15) * 16;
      const uint32_t cp_dst = vst_addr + (lane >> 4) * kVRowSmem + (lane & 15) * 16;
      const uint32_t ldsm_base = vst_addr + ldsm_lane_offset(lane);
      const int64_t v_step = kStep * v_row, two_rows = 2 * v_row;
      const bool v_dense = v_row == kHeadDim * 2;
      int vstage = 0;
      auto fetch_tile = [&](int stage) {
        if (v_dense) load_v_tile_fast<true>(cp_dst + stage * kVTileSmem, v_tile, two_rows);
        else load_v_tile_fast<false>(cp_dst + stage * kVTileSmem, v_tile, two_rows);
      };
      if constexpr (kVPipe) {
        cp_async_wait<0>();               // nothing of an earlier segment may still be landing in the stages
        __syncwarp();
        fetch_tile(0);                    // committed with the first scales below
      }
      // packed values: this lane's slot of tokens 2t, 2t+1 (+8, +9) of the step and their scale / minimum pairs
      const char* vq_lane = nullptr; const char* vs_lane = nullptr; const char* vm_lane = nullptr;
      VqTile vq{};
      if constexpr (VQ != 0) {
        const int64_t tok0 = static_cast<int64_t>(pos) * kStep + 2 * t;
        vq_lane = static_cast<const char*>(a.vq_codes) + b * a.vq_sb + kvh * a.vq_sh + tok0 * 64 + 8 * g;
        vs_lane = static_cast<const char*>(a.vq_scale) + (b * a.vs_sb + kvh * a.vs_sh + tok0) * 2;
        vm_lane = static_cast<const char*>(a.vq_mn) + (b * a.vs_sb + kvh * a.vs_sh + tok0) * 2;
        vq = load_vq_tile(vq_lane, vs_lane, vm_lane);
      }
      const int last_tile = qs_end - 1;   // tiles past the segment are never fetched: the last one is re-read
      int next_tile = pos;

      // The register loads run one step ahead; the L2 is asked for the tiles kPrefetch steps
      // ahead so those loads find their lines on chip.  One lane issues a bulk prefetch per
      // tile (codes: 1 KB contiguous; values: 4 KB when token rows are dense, else row by row).
      auto prefetch_tiles = [&](int step, int count) {
        if (lane == 0) prefetch_l2(c_unit + static_cast<int64_t>(step) * kCodeStep, count * kCodeStep);
        if constexpr (kVPipe) {
          const char* vt = v_unit + static_cast<int64_t>(step) * kStep * v_row;
          if (v_dense) { if (lane == 1) prefetch_l2(vt, count * kStep * kHeadDim * 2); }
          else if (lane < count * kStep) prefetch_l2(vt + lane * v_row, kHeadDim * 2);
        }
        if constexpr (VQ != 0) {
          if (lane == 1)
            prefetch_l2(static_cast<const char*>(a.vq_codes) + b * a.vq_sb + kvh * a.vq_sh +
                            static_cast<int64_t>(step) * kStep * 64, count * kStep * 64);
        }
      };
      if (kPrefetch > 2 && pos + 2 < qs_end) prefetch_tiles(pos + 2, min(kPrefetch - 2, qs_end - pos - 2));

      int in_group = pos % a.spg;
      int grp = pos / a.spg;
      const int last_grp = (qs_end - 1) / a.spg;
      const uint32_t sc_addr = static_cast<uint32_t>(__cvta_generic_to_shared(s_sc_w));
      constexpr bool kCommitScales = !kVPipe;   // with a value pipeline the scale copies join the next value-tile group
      auto stage_group = [&](int gidx, int buf) {
        const int64_t row = static_cast<int64_t>(gidx) * kPairs * QES;
        stage_scales_async<QDT, kCommitScales>(sc_addr + buf * kStageBytes, rs_unit + row, rm_unit + row,
                                               ts_unit + row, tm_unit + row, lane);
      };
      __syncwarp();                       // earlier readers of the staging buffers are done
      int buf = 0;
      stage_group(grp, buf);
      if constexpr (kVPipe) {
        cp_async_commit();                           // first value tile + first scales
#pragma unroll
        for (int d = 1; d < kVStages - 1; ++d) {     // fill the pipeline: tiles pos+1 .. pos+kVStages-2
          if (next_tile < last_tile) { ++next_tile; v_tile += v_step; }
          fetch_tile(d);
          cp_async_commit();
        }
      }
      int s = pos;
      int prev_run = 0;
      while (s < qs_end) {
        // ---- one run of steps inside one token group: constants first, then a lean step loop ----
        const int run_end = min(qs_end, s - in_group + a.spg);
        // this group's scale rows must have landed.  In the fused kernel they rode in the value-tile
        // group committed at the first step of the previous run; when that run had at least kVStages
        // steps the group is older than the kVStages - 1 groups allowed in flight and nothing needs
        // draining.  (The first run of a segment may be shorter than a token group.)
        if (kVPipe && prev_run >= kVStages) { cp_async_wait<kVStages - 1>(); __syncwarp(); }
        else wait_staged();
        prev_run = run_end - s;
        if (grp < last_grp) stage_group(grp + 1, buf ^ 1);
        build_angle_table<TBITS, QDT>(tbl_addr, s_sc_w + buf * kStageBytes, lane);
        uint32_t tbl_run = tbl_addr;
        // the gathers are plain (movable) asm: tie them to this build of the table
        asm volatile("" : "+r"(tbl_run) :: "memory");
        load_radius_consts<RBITS, QDT>(s_sc_w + buf * kStageBytes, t, rs2, rc2);
        buf ^= 1;
#pragma unroll 1
        for (; s < run_end; ++s) {
          if (kPrefetch > 0 && s + kPrefetch < qs_end) prefetch_tiles(s + kPrefetch, 1);
          // next tile; the last step of the segment re-reads its own tile rather than branching
          const bool more = s + 1 < qs_end;
          if (more) c_lane += kCodeStep;
          const uint4 ng = ldg_stream(c_lane), nh = load_second(c_lane);
          if constexpr (kVPipe) {
            if (next_tile < last_tile) { ++next_tile; v_tile += v_step; }
            int fill = vstage + kVStages - 1;
            if (fill >= kVStages) fill -= kVStages;
            fetch_tile(fill);
            cp_async_commit();              // also carries scale rows staged since the last commit
          }
          VqTile nvq{};
          if constexpr (VQ != 0) {
            if (more) { vq_lane += kStep * 64; vs_lane += kStep * 2; vm_lane += kStep * 2; }
            nvq = load_vq_tile(vq_lane, vs_lane, vm_lane);
          }

          float S[4] = {0.f, 0.f, 0.f, 0.f};
          if constexpr (KF == PQ_KEYS_PACKED6)
            qk_step_packed6<RBITS, TBITS>(S, cg, make_uint2(ch.x, ch.y), tbl_run, lane_xor, rs2, rc2, qb);
          else
            qk_step_quant<RBITS, TBITS>(S, cg, ch, tbl_run, lane_xor, rs2, rc2, qb);

          if constexpr (QK_ONLY) {
            // logits (B, N, Nb*G): lane holds tokens (g, g+8) x heads (2t, 2t+1)
            const int tok = s * kStep + g;
            float* orow = a.logits + (static_cast<int64_t>(b) * a.N + head0 + 2 * t) * Lq + tok;
            if (2 * t < nheads) { orow[0] = S[0]; orow[8] = S[2]; }
            if (2 * t + 1 < nheads) { orow[Lq] = S[1]; orow[Lq + 8] = S[3]; }
          } else {
            uint32_t b0, b1;
            constexpr int PDT = VQ ? PQ_F16 : VDT;      // packed values are multiplied in fp16 whatever VDT is
            if (mask_row) {
              const bool mg = mask_row[s * kStep + g] == 0, mh = mask_row[s * kStep + g + 8] == 0;
              softmax_step<PDT, true>(S, a.scale_log2, true, true, mg, mh, st, O, b0, b1);
            } else {
              softmax_step<PDT, false>(S, a.scale_log2, true, true, false, false, st, O, b0, b1);
            }
            if constexpr (VQ != 0) {
              pv_quant<VDT>(O, vq, b0, b1);
              vq = nvq;
            } else {
              cp_async_wait<kVStages - 1>();  // this step's tile has landed; the newer ones may be in flight
              __syncwarp();
              pv_from_smem<VDT>(O, ldsm_base + vstage * kVTileSmem, b0, b1);
              __syncwarp();                   // every lane is done with the stage before it is refilled
              if (++vstage == kVStages) vstage = 0;
            }
          }
          cg = ng; ch = nh;
        }
        in_group = 0;
        ++grp;
      }
      cp_async_wait<0>();                 // the last (redundant) prefetch of the segment
      if constexpr (VQ != 0) {
        // back to true scale: undo the subnormal encoding of the levels and add the minimum term
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          O[j][0] = fmaf(O[j][0], 16777216.0f, O[8][0]); O[j][1] = fmaf(O[j][1], 16777216.0f, O[8][1]);
          O[j][2] = fmaf(O[j][2], 1048576.0f, O[8][2]);  O[j][3] = fmaf(O[j][3], 1048576.0f, O[8][3]);
        }
        O[8][0] = O[8][1] = O[8][2] = O[8][3] = 0.f;
      }
    }

    // ------------------------------ residual steps -------------------------------
    if constexpr (!QK_ONLY) {
      const int rv0 = pos > a.nq ? pos - a.nq : 0;          // virtual residual slots [rv0, rv1)
      const int rv1 = pos_end - a.nq;
      if (rv1 > rv0) {
        // query fragments in natural channel order: chunk c = channels 8t + 32c .. +7
        uint4 qr[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) qr[c] = load8_as16<QDT>(q_head + (8 * t + 32 * c) * QES, head_ok);
        const char* kr_unit = static_cast<const char*>(a.kres) + (b * a.kr_sb + kvh * a.kr_sh) * QES;
        const int64_t kr_row = a.kr_st * QES;
        for (int rv = rv0 + (rv0 & 1); rv < rv1; rv += 2) {   // a step is owned by its even slot
          const int r0 = (rv >> 1) * kStep;
          const bool ok_g = r0 + g < a.R, ok_h = r0 + g + 8 < a.R;
          uint4 kg[4], kh[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            kg[c] = load8_as16<QDT>(kr_unit + (r0 + g) * kr_row + (8 * t + 32 * c) * QES, ok_g);
            kh[c] = load8_as16<QDT>(kr_unit + (r0 + g + 8) * kr_row + (8 * t + 32 * c) * QES, ok_h);
          }
          cp_async_wait<0>();
          __syncwarp();
          load_v_tile_async(vst_addr, v_unit + static_cast<int64_t>(a.v_tok0 + r0) * v_row, v_row, a.R - r0, lane);
          cp_async_commit();
          float S[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            mma_16816<KRDT>(S, kg[c].x, kh[c].x, kg[c].y, kh[c].y, qr[c].x, qr[c].y);
            mma_16816<KRDT>(S, kg[c].z, kh[c].z, kg[c].w, kh[c].w, qr[c].z, qr[c].w);
          }
          if constexpr (QDT != PQ_F32) {
            // the reference computes these logits with a matmul in the query dtype and only then
            // casts to fp32 (models/modeling_llama_polar.py:79): one rounding to that dtype
            const float2 lo2 = unpack2<QDT>(pack2<QDT>(S[0], S[1])), hi2 = unpack2<QDT>(pack2<QDT>(S[2], S[3]));
            S[0] = lo2.x; S[1] = lo2.y; S[2] = hi2.x; S[3] = hi2.y;
          }
          bool mg = false, mh = false;
          if (mask_row) {
            mg = ok_g && mask_row[Lq + r0 + g] == 0;
            mh = ok_h && mask_row[Lq + r0 + g + 8] == 0;
          }
          uint32_t b0, b1;
          softmax_step<VDT, true>(S, a.scale_log2, ok_g, ok_h, mg, mh, st, O, b0, b1);
          cp_async_wait<0>();
          __syncwarp();
          pv_from_smem<VDT>(O, vst_addr + ldsm_lane_offset(lane), b0, b1);
          __syncwarp();
        }
      }

      // ------------------------------ emit the partial -----------------------------
#pragma unroll
      for (int o = 4; o <= 16; o <<= 1) {
        st.l0 += __shfl_xor_sync(0xffffffffu, st.l0, o);
        st.l1 += __shfl_xor_sync(0xffffffffu, st.l1, o);
      }
      if (combine) {
        // stage this warp's partial in its own (now idle) value stages, then one warp-wide pass per channel
        cp_async_wait<0>();
        __syncwarp();
        float* so = reinterpret_cast<float*>(warp_smem + kPairs * A * 4 + 2 * kStageBytes);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int chn = 16 * j + g, chn2 = chn + 8;
          *reinterpret_cast<float2*>(so + chn * kHeadTile + 2 * t) = make_float2(O[j][0], O[j][1]);
          *reinterpret_cast<float2*>(so + chn2 * kHeadTile + 2 * t) = make_float2(O[j][2], O[j][3]);
        }
        if (g == 0) {
          float2* sml = reinterpret_cast<float2*>(so + kPartialFloats);
          sml[2 * t] = make_float2(st.m0, st.l0);
          sml[2 * t + 1] = make_float2(st.m1, st.l1);
        }
        __syncthreads();
        // thread = channel: merge the four staged partials and write one
        const int ch = threadIdx.x;
        const long long slot = static_cast<long long>(blockIdx.x) * kWarps * a.max_seg;     // first warp, segment 0
        float mx[kHeadTile], ls[kHeadTile], acc[kHeadTile];
#pragma unroll
        for (int h = 0; h < kHeadTile; ++h) { mx[h] = -INFINITY; ls[h] = 0.f; acc[h] = 0.f; }
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          const float2* sml = reinterpret_cast<const float2*>(smem_dyn + w * kWarpSmem + kPairs * A * 4 + 2 * kStageBytes) +
                              kPartialFloats / 2;
#pragma unroll
          for (int h = 0; h < kHeadTile; ++h) mx[h] = fmaxf(mx[h], sml[h].x);
        }
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          const float* sw = reinterpret_cast<const float*>(smem_dyn + w * kWarpSmem + kPairs * A * 4 + 2 * kStageBytes);
          const float2* sml = reinterpret_cast<const float2*>(sw + kPartialFloats);
          const float4 o0 = *reinterpret_cast<const float4*>(sw + ch * kHeadTile);
          const float4 o1 = *reinterpret_cast<const float4*>(sw + ch * kHeadTile + 4);
          const float ov[kHeadTile] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
#pragma unroll
          for (int h = 0; h < kHeadTile; ++h) {
            const float2 ml = sml[h];
            const float wgt = ml.x == -INFINITY ? 0.f : exp2_approx(ml.x - mx[h]);
            ls[h] = fmaf(wgt, ml.y, ls[h]);
            acc[h] = fmaf(wgt, ov[h], acc[h]);
          }
        }
        float4* po = reinterpret_cast<float4*>(a.part_o + slot * kPartialFloats + ch * kHeadTile);
        po[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        po[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
        if (ch < kHeadTile) {
          float m = -INFINITY, l = 0.f;
#pragma unroll
          for (int h = 0; h < kHeadTile; ++h) if (h == ch) { m = mx[h]; l = ls[h]; }
          a.part_ml[slot * kHeadTile + ch] = make_float2(m, l);
        }
      } else {
      const long long slot = gw * a.max_seg + seg;
      float* po = a.part_o + slot * kPartialFloats;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // m-tile j: row g is channel 16j + g, row g+8 channel 16j + 8 + g
        const int chn = 16 * j + g, chn2 = chn + 8;
        *reinterpret_cast<float2*>(po + chn * kHeadTile + 2 * t) = make_float2(O[j][0], O[j][1]);
        *reinterpret_cast<float2*>(po + chn2 * kHeadTile + 2 * t) = make_float2(O[j][2], O[j][3]);
      }
      if (g == 0) {
        a.part_ml[slot * kHeadTile + 2 * t] = make_float2(st.m0, st.l0);
        a.part_ml[slot * kHeadTile + 2 * t + 1] = make_float2(st.m1, st.l1);
      }
      }
    }

    lo = seg_hi; ++unit; pos = 0; ++seg;
  }
}

// warp that owns flat slot x: the largest w with range_lo(w) <= x
__device__ __forceinline__ long long warp_of(long long x, long long total, int nwarps) {
  return ((x + 1) * nwarps - 1) / total;
}

// Combine a unit's partials, normalise, write out (and lse).  Grid (units, 2): each CTA owns
// 64 of the 128 channels.  Pass 1 finds the per-head maximum over the unit's partials; pass 2
// stages, chunk by chunk, the weights 2^(m_i - M) and weighted sums once per (partial, head)
// in shared memory, and 8 groups of 64 threads stride over the partial rows, four rows in
// flight per thread, with one FMA per (partial, head, channel).  Every warp range of the
// attention kernel is non-empty (total_warps <= total_slots), so a unit is covered by the
// consecutive warps w0..w1; which of them left a partial follows from the CTA-level combine
// of the attention kernel and is enumerated densely (see below), so every load issued is a
// partial that exists.
constexpr int kMergeGroups = 8;
constexpr int kMergeCh = 64;
constexpr int kMergeChunk = 128;      // partials whose weights are staged at a time
static_assert(kMergeGroups == kHeadTile, "each thread group finishes one head");

template <int ODT>
__global__ void __launch_bounds__(kMergeCh * kMergeGroups)
merge_partials_kernel(const DecodeArgs a_in, void* __restrict__ out, int64_t o_sb, int64_t o_sh,
                      float* __restrict__ lse, const __grid_constant__ PushArgs px) {
  DecodeArgs a = a_in;
  if (a.dyn) plan_on_device(a);
  constexpr int kThreadsM = kMergeCh * kMergeGroups;
  __shared__ float s_w[kMergeChunk][kHeadTile];                // weight of partial i for head h
  __shared__ float s_red[kThreadsM / 32][kHeadTile];
  __shared__ float s_acc[kMergeGroups][kHeadTile][kMergeCh];
  __shared__ float s_max[kHeadTile], s_sum[kHeadTile];

  // a dependent of this kernel (the peer-memory exchange of a sequence split) may become resident now
  asm volatile("griddepcontrol.launch_dependents;");
  // no-op unless launched with programmatic stream serialisation: wait until the attention kernel has
  // completed and its partials are visible
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const long long unit = blockIdx.x;
  const int chl = threadIdx.x & (kMergeCh - 1), grp = threadIdx.x / kMergeCh;
  const int ch = blockIdx.y * kMergeCh + chl;
  const int ht = static_cast<int>(unit % a.head_tiles);
  const long long bk = unit / a.head_tiles;
  const int kvh = static_cast<int>(bk % a.Nk), b = static_cast<int>(bk / a.Nk);
  const int head0 = kvh * a.nrep + ht * kHeadTile;
  const int nheads = min(kHeadTile, a.nrep - ht * kHeadTile);

  if (a.slots_per_unit == 0) {
    // Device-side lengths that describe an empty cache: there are no keys to attend over and the attention
    // kernel wrote no partial.  The result is defined - zeros, log-sum-exp = -inf - rather than a division by zero.
    const int hh = grp;
    if (hh < nheads) {
      const int64_t off = b * o_sb + (head0 + hh) * o_sh + ch;
      if constexpr (ODT == PQ_F32) static_cast<float*>(out)[off] = 0.f;
      else if constexpr (ODT == PQ_F16) static_cast<__half*>(out)[off] = __float2half_rn(0.f);
      else static_cast<__nv_bfloat16*>(out)[off] = __float2bfloat16_rn(0.f);
      if (lse && ch == 0) lse[static_cast<int64_t>(b) * a.N + head0 + hh] = -INFINITY;
      if (px.world > 0) push_row_value(px, static_cast<long long>(b) * a.N + head0 + hh, ch, 0.f, -INFINITY);
    }
    if (px.world > 0) {
      __syncthreads();
      if (threadIdx.x == 0) finish_exchange_cta(px, gridDim.x * gridDim.y);
    }
    return;
  }
  const long long first = unit * a.slots_per_unit, last = first + a.slots_per_unit - 1;
  const long long w0 = warp_of(first, a.total_slots, a.total_warps);
  const long long w1 = warp_of(last, a.total_slots, a.total_warps);
  const int seg0 = static_cast<int>(unit - range_lo(w0, a.total_slots, a.total_warps) / a.slots_per_unit);
  // The unit's partials, in a fixed order.  Warps strictly between w0 and w1 lie wholly inside the unit, so every
  // CTA strictly between the first and the last one combined its four partials into one (in the slot of its
  // first warp); only the two CTAs at the ends can straddle a unit boundary and hold one partial per warp.
  //   [ nf partials of the first CTA | ni = one per interior CTA | nl partials of the last CTA ]
  const long long c0 = w0 >> 2, c1 = w1 >> 2;
  const bool single0 = cta_in_one_unit(c0, a.total_slots, a.total_warps, a.slots_per_unit);
  const bool single1 = c1 != c0 && cta_in_one_unit(c1, a.total_slots, a.total_warps, a.slots_per_unit);
  const long long wf_end = c1 == c0 ? w1 : 4 * c0 + 3;                 // last warp of the unit in the first CTA
  const int nf = single0 ? 1 : static_cast<int>(wf_end - w0 + 1);
  const int ni = c1 > c0 + 1 ? static_cast<int>(c1 - c0 - 1) : 0;
  const int nl = c1 == c0 ? 0 : (single1 ? 1 : static_cast<int>(w1 - 4 * c1 + 1));
  const int n = nf + ni + nl;
  auto slot_of = [&](int k) -> long long {
    if (k < nf) return (w0 + k) * a.max_seg + (k == 0 ? seg0 : 0);       // a single first CTA starts at w0 = 4 c0
    if (k < nf + ni) return 4 * (c0 + 1 + (k - nf)) * a.max_seg;
    return (4 * c1 + (k - nf - ni)) * a.max_seg;
  };
  auto has_partial = [](int) { return true; };       // every index below n is a partial that exists

  // The first batch of partial rows is requested before anything else so that its DRAM round trip
  // overlaps the one of the (m, l) entries.
  float4 o_first[4][2];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i = grp + u * kMergeGroups;
    o_first[u][0] = o_first[u][1] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < n && has_partial(i)) {
      const float4* po = reinterpret_cast<const float4*>(a.part_o + slot_of(i) * kPartialFloats + ch * kHeadTile);
      o_first[u][0] = po[0]; o_first[u][1] = po[1];
    }
  }

  // ---- pass 1: per-head maximum; thread (i, h) pairs stride over the n x 8 (m, l) entries.
  // The entries of the first chunk stay in registers for pass 2. ----
  constexpr int kKeep = kMergeChunk * kHeadTile / kThreadsM;     // entries per thread in one chunk
  float2 kept[kKeep];
  const int h_mine = threadIdx.x & (kHeadTile - 1);
  {
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < kKeep; ++k) {
      const int i = (threadIdx.x >> 3) + k * (kThreadsM >> 3);
      kept[k] = (i < n && has_partial(i)) ? a.part_ml[slot_of(i) * kHeadTile + h_mine] : make_float2(-INFINITY, 0.f);
      m = fmaxf(m, kept[k].x);
    }
    for (int i = (threadIdx.x >> 3) + kKeep * (kThreadsM >> 3); i < n; i += kThreadsM >> 3)
      if (has_partial(i)) m = fmaxf(m, a.part_ml[slot_of(i) * kHeadTile + h_mine].x);
    // lanes with equal (lane & 7) hold the same head
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
    if ((threadIdx.x & 31) < kHeadTile) s_red[threadIdx.x >> 5][h_mine] = m;
    __syncthreads();
    if (threadIdx.x < kHeadTile) {
      float mm = s_red[0][threadIdx.x];
      for (int w = 1; w < kThreadsM / 32; ++w) mm = fmaxf(mm, s_red[w][threadIdx.x]);
      s_max[threadIdx.x] = mm;
      s_sum[threadIdx.x] = 0.f;
    }
    __syncthreads();
  }

  // ---- pass 2 ----
  float acc[kHeadTile];
#pragma unroll
  for (int h = 0; h < kHeadTile; ++h) acc[h] = 0.f;
  float lsum = 0.f;                                             // thread (i, h): sum of w * l
  for (int c0 = 0; c0 < n; c0 += kMergeChunk) {
    const int cn = min(kMergeChunk, n - c0);
    __syncthreads();
    if (c0 == 0) {
#pragma unroll
      for (int k = 0; k < kKeep; ++k) {
        const int i = (threadIdx.x >> 3) + k * (kThreadsM >> 3);
        if (i < cn) {
          const float w = kept[k].x == -INFINITY ? 0.f : exp2_approx(kept[k].x - s_max[h_mine]);
          s_w[i][h_mine] = w;
          lsum = fmaf(w, kept[k].y, lsum);
        }
      }
    } else {
      for (int e = threadIdx.x; e < cn * kHeadTile; e += kThreadsM) {
        const int i = e >> 3;
        const float2 ml = has_partial(c0 + i) ? a.part_ml[slot_of(c0 + i) * kHeadTile + h_mine]
                                              : make_float2(-INFINITY, 0.f);
        const float w = ml.x == -INFINITY ? 0.f : exp2_approx(ml.x - s_max[h_mine]);
        s_w[i][h_mine] = w;
        lsum = fmaf(w, ml.y, lsum);
      }
    }
    __syncthreads();
    for (int i0 = grp; i0 < cn; i0 += 4 * kMergeGroups) {
      float4 o[4][2];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kMergeGroups;
        o[u][0] = o[u][1] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c0 == 0 && i0 == grp) { o[u][0] = o_first[u][0]; o[u][1] = o_first[u][1]; }
        else if (i < cn && has_partial(c0 + i)) {
          const float4* po = reinterpret_cast<const float4*>(a.part_o + slot_of(c0 + i) * kPartialFloats + ch * kHeadTile);
          o[u][0] = po[0]; o[u][1] = po[1];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kMergeGroups;
        if (i < cn) {
          const float4 wa = *reinterpret_cast<const float4*>(&s_w[i][0]);
          const float4 wb = *reinterpret_cast<const float4*>(&s_w[i][4]);
          acc[0] = fmaf(wa.x, o[u][0].x, acc[0]); acc[1] = fmaf(wa.y, o[u][0].y, acc[1]);
          acc[2] = fmaf(wa.z, o[u][0].z, acc[2]); acc[3] = fmaf(wa.w, o[u][0].w, acc[3]);
          acc[4] = fmaf(wb.x, o[u][1].x, acc[4]); acc[5] = fmaf(wb.y, o[u][1].y, acc[5]);
          acc[6] = fmaf(wb.z, o[u][1].z, acc[6]); acc[7] = fmaf(wb.w, o[u][1].w, acc[7]);
        }
      }
    }
  }
  // reduce sum(w * l): thread's head is (threadIdx.x & 7) in every chunk
  lsum += __shfl_xor_sync(0xffffffffu, lsum, 8);
  lsum += __shfl_xor_sync(0xffffffffu, lsum, 16);
  // per-warp sums are combined in a fixed order so that results do not depend on timing
  if ((threadIdx.x & 31) < kHeadTile) s_red[threadIdx.x >> 5][threadIdx.x & (kHeadTile - 1)] = lsum;
#pragma unroll
  for (int h = 0; h < kHeadTile; ++h) s_acc[grp][h][chl] = acc[h];
  __syncthreads();
  if (threadIdx.x < kHeadTile) {
    float l = 0.f;
    for (int w = 0; w < kThreadsM / 32; ++w) l += s_red[w][threadIdx.x];
    s_sum[threadIdx.x] = l;
  }
  __syncthreads();
  const int h = grp;                                            // group g finishes head g
  if (h < nheads) {
    float o = 0.f;
#pragma unroll
    for (int k = 0; k < kMergeGroups; ++k) o += s_acc[k][h][chl];
    const float l = s_sum[h];
    const float val = o / l;
    const int64_t off = b * o_sb + (head0 + h) * o_sh + ch;
    if constexpr (ODT == PQ_F32) static_cast<float*>(out)[off] = val;
    else if constexpr (ODT == PQ_F16) static_cast<__half*>(out)[off] = __float2half_rn(val);
    else static_cast<__nv_bfloat16*>(out)[off] = __float2bfloat16_rn(val);
    const float lse_val = (s_max[h] + log2f(l)) * 0.6931471805599453f;
    if (lse && ch == 0) lse[static_cast<int64_t>(b) * a.N + head0 + h] = lse_val;
    // sequence split over peer memory: the row goes straight into the peers' inboxes, paired with the epoch
    if (px.world > 0) push_row_value(px, static_cast<long long>(b) * a.N + head0 + h, ch, val, lse_val);
  }
  if (px.world > 0) {
    __syncthreads();
    if (threadIdx.x == 0) finish_exchange_cta(px, gridDim.x * gridDim.y);
  }
}

// Merge P normalised partial results: part p holds outs (rows, 128) at outs + p * out_ps and lses (rows) at
// lses + p * lse_ps (element strides between parts; dense tensors have out_ps = rows * 128, lse_ps = rows).
template <int ODT>
__global__ void __launch_bounds__(kHeadDim)
merge_lse_kernel(const float* __restrict__ outs, int64_t out_ps, const float* __restrict__ lses, int64_t lse_ps, int P,
                 void* __restrict__ out, float* __restrict__ lse_out) {
  const int64_t row = blockIdx.x;
  const int ch = threadIdx.x;
  float M = -INFINITY;
  for (int p = 0; p < P; ++p) M = fmaxf(M, lses[p * lse_ps + row]);
  float L = 0.f, acc = 0.f;
  for (int p = 0; p < P; ++p) {
    const float l = lses[p * lse_ps + row];
    const float w = l == -INFINITY ? 0.f : __expf(l - M);
    L += w;
    acc = fmaf(w, outs[p * out_ps + row * kHeadDim + ch], acc);
  }
  const float val = acc / L;
  const int64_t off = row * kHeadDim + ch;
  if constexpr (ODT == PQ_F32) static_cast<float*>(out)[off] = val;
  else if constexpr (ODT == PQ_F16) static_cast<__half*>(out)[off] = __float2half_rn(val);
  else static_cast<__nv_bfloat16*>(out)[off] = __float2bfloat16_rn(val);
  if (lse_out && ch == 0) lse_out[row] = M + __logf(L);
}

// ---------------------------------------------------------------------------------
// host side: partition, dispatch
// ---------------------------------------------------------------------------------
int sm_count() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached = n; cached_dev = dev;
  }
  return cached;
}

void plan(DecodeArgs& a, int ctas_per_sm, int num_ctas) {
  a.plan_ctas = num_ctas > 0 ? num_ctas : static_cast<long long>(sm_count()) * ctas_per_sm;
  a.plan_forced = num_ctas > 0;
  plan_core(a, a.plan_ctas, a.plan_forced != 0);
}

size_t workspace_bytes_for(const DecodeArgs& a) {
  const size_t slots = static_cast<size_t>(a.total_warps) * a.max_seg;
  return slots * (kPartialFloats * sizeof(float) + kHeadTile * sizeof(float2));
}

template <int RBITS, int TBITS, int QDT, int VDT, bool QK_ONLY, int VQ = 0, bool DYN = false, int KF = PQ_KEYS_BYTE>
int launch_decode(const DecodeArgs& a, cudaStream_t s) {
  constexpr int kStageBytes = 4 * kPairs * (QDT == PQ_F32 ? 4 : 2);
  constexpr int kWarpSmem = kPairs * (1 << TBITS) * 4 + 2 * kStageBytes + v_stages(QK_ONLY, VQ) * kVTileSmem;
  constexpr int kSmem = kWarps * kWarpSmem;
  if (kSmem > 48 * 1024)
    PQ_CUDA_TRY(cudaFuncSetAttribute(decode_kernel<RBITS, TBITS, QDT, VDT, QK_ONLY, VQ, DYN, KF>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  // device-side lengths: always the full grid, the kernel retires the warps its own plan does not use
  const unsigned grid = DYN ? static_cast<unsigned>(a.plan_ctas) : (a.total_warps + kWarps - 1) / kWarps;
  decode_kernel<RBITS, TBITS, QDT, VDT, QK_ONLY, VQ, DYN, KF><<<grid, kThreads, kSmem, s>>>(a);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

// 6-bit packed keys: the two 6-bit splits, 16-bit caches (query, keys and values of one dtype), every variant of
// the fused kernel (full-precision or packed values, host- or device-side lengths)
template <int RBITS, int TBITS>
int dispatch_packed6(const DecodeArgs& a, int qdt, int vdt, cudaStream_t s) {
  if constexpr ((RBITS == 2 && TBITS == 4) || (RBITS == 3 && TBITS == 3)) {
#define PQ_P6(DT)                                                                                              \
  if (qdt == DT && vdt == DT) {                                                                                \
    if (a.dyn) return a.vq_codes ? launch_decode<RBITS, TBITS, DT, DT, false, 4, true, PQ_KEYS_PACKED6>(a, s)  \
                                 : launch_decode<RBITS, TBITS, DT, DT, false, 0, true, PQ_KEYS_PACKED6>(a, s); \
    return a.vq_codes ? launch_decode<RBITS, TBITS, DT, DT, false, 4, false, PQ_KEYS_PACKED6>(a, s)            \
                      : launch_decode<RBITS, TBITS, DT, DT, false, 0, false, PQ_KEYS_PACKED6>(a, s);           \
  }
    PQ_P6(PQ_F16)
    PQ_P6(PQ_BF16)
#undef PQ_P6
  }
  return PQ_ERR_UNSUPPORTED;
}

template <int RBITS, int TBITS, bool QK_ONLY>
int dispatch_dtypes(const DecodeArgs& a, int qdt, int vdt, cudaStream_t s) {
  if constexpr (!QK_ONLY) {
    if (a.key_format == PQ_KEYS_PACKED6) return dispatch_packed6<RBITS, TBITS>(a, qdt, vdt, s);
    if (a.dyn) {            // device-side lengths: one instance per 16-bit dtype, with and without packed values
      if (qdt == PQ_F16 && vdt == PQ_F16)
        return a.vq_codes ? launch_decode<RBITS, TBITS, PQ_F16, PQ_F16, false, 4, true>(a, s)
                          : launch_decode<RBITS, TBITS, PQ_F16, PQ_F16, false, 0, true>(a, s);
      if (qdt == PQ_BF16 && vdt == PQ_BF16)
        return a.vq_codes ? launch_decode<RBITS, TBITS, PQ_BF16, PQ_BF16, false, 4, true>(a, s)
                          : launch_decode<RBITS, TBITS, PQ_BF16, PQ_BF16, false, 0, true>(a, s);
      return PQ_ERR_UNSUPPORTED;
    }
    if (a.vq_codes) {       // packed values: one instance per 16-bit dtype
      if (qdt == PQ_F16 && vdt == PQ_F16) return launch_decode<RBITS, TBITS, PQ_F16, PQ_F16, false, 4>(a, s);
      if (qdt == PQ_BF16 && vdt == PQ_BF16) return launch_decode<RBITS, TBITS, PQ_BF16, PQ_BF16, false, 4>(a, s);
      return PQ_ERR_UNSUPPORTED;
    }
  }
#define PQ_CASE(Q, V) if (qdt == Q && vdt == V) return launch_decode<RBITS, TBITS, Q, V, QK_ONLY>(a, s)
  if constexpr (QK_ONLY) {
    PQ_CASE(PQ_F16, PQ_F16); PQ_CASE(PQ_BF16, PQ_F16); PQ_CASE(PQ_F32, PQ_F16);
  } else {
    PQ_CASE(PQ_F16, PQ_F16); PQ_CASE(PQ_BF16, PQ_BF16); PQ_CASE(PQ_F32, PQ_F16);
    PQ_CASE(PQ_F32, PQ_BF16); PQ_CASE(PQ_F16, PQ_BF16); PQ_CASE(PQ_BF16, PQ_F16);
  }
#undef PQ_CASE
  return PQ_ERR_UNSUPPORTED;
}

template <bool QK_ONLY>
int dispatch_bits(const DecodeArgs& a, int rbits, int tbits, int qdt, int vdt, cudaStream_t s) {
#define PQ_BITS(R, T) if (rbits == R && tbits == T) return dispatch_dtypes<R, T, QK_ONLY>(a, qdt, vdt, s)
  PQ_BITS(4, 4); PQ_BITS(3, 3); PQ_BITS(2, 4);
  PQ_BITS(4, 3); PQ_BITS(3, 4); PQ_BITS(2, 2); PQ_BITS(2, 3); PQ_BITS(3, 2); PQ_BITS(4, 2);
#undef PQ_BITS
  return PQ_ERR_UNSUPPORTED;
}

}  // namespace

int qk_decode_device(const void* q, int64_t q_sb, int64_t q_sh, const uint8_t* codes, const void* rscale,
                     const void* rmn, const void* tscale, const void* tmn, float* out, int B, int N, int Nk,
                     int Nb, int G, int D, int rbits, int tbits, int dtype, cudaStream_t stream) {
  if (B < 0 || N <= 0 || Nk <= 0 || Nb < 0 || G <= 0 || N % Nk != 0) return PQ_ERR_INVALID;
  if (rbits < 0 || tbits < 0 || rbits + tbits > 8 || !dtype_ok(dtype)) return PQ_ERR_INVALID;
  if (D != kPairs || G % kStep != 0) return PQ_ERR_UNSUPPORTED;
  if (B == 0 || Nb == 0) return PQ_OK;
  if (!q || !codes || !rscale || !rmn || !tscale || !tmn || !out) return PQ_ERR_INVALID;
  if (reinterpret_cast<uintptr_t>(codes) % 16 || reinterpret_cast<uintptr_t>(rscale) % 16 ||
      reinterpret_cast<uintptr_t>(rmn) % 16 || reinterpret_cast<uintptr_t>(tscale) % 16 ||
      reinterpret_cast<uintptr_t>(tmn) % 16)
    return PQ_ERR_ALIGNMENT;
  DecodeArgs a{};
  a.q = q; a.q_sb = q_sb; a.q_sh = q_sh;
  a.codes = codes; a.c_sh = static_cast<int64_t>(Nb) * G * kPairs; a.c_sb = a.c_sh * Nk;
  a.rscale = rscale; a.rmn = rmn; a.tscale = tscale; a.tmn = tmn;
  a.s_sh = static_cast<int64_t>(Nb) * kPairs; a.s_sb = a.s_sh * Nk;
  a.logits = out;
  a.B = B; a.N = N; a.Nk = Nk; a.Nb = Nb; a.G = G; a.R = 0;
  plan(a, 4, 0);
  return dispatch_bits<true>(a, rbits, tbits, dtype, PQ_F16, stream);
}

size_t decode_workspace_bytes(int B, int N, int Nk, int Nb, int G, int R, int num_ctas) {
  if (B <= 0 || N <= 0 || Nk <= 0 || Nb < 0 || G <= 0 || R < 0 || N % Nk != 0 || G % kStep != 0) return 0;
  DecodeArgs a{};
  a.B = B; a.N = N; a.Nk = Nk; a.Nb = Nb; a.G = G; a.R = R;
  plan(a, PQ_MIN_CTAS, num_ctas);
  return workspace_bytes_for(a);
}

// scratch that suffices for every (Nb, R) a growing cache passes through with device-side lengths
size_t decode_workspace_bytes_dyn(int B, int N, int Nk, int num_ctas) {
  if (B <= 0 || N <= 0 || Nk <= 0 || N % Nk != 0) return 0;
  DecodeArgs a{};
  a.B = B; a.N = N; a.Nk = Nk; a.Nb = 0; a.G = kStep; a.R = 1;
  plan(a, PQ_MIN_CTAS, num_ctas);
  const long long units = static_cast<long long>(B) * Nk * a.head_tiles;
  return static_cast<size_t>(slot_bound(units, a.plan_ctas)) * (kPartialFloats * sizeof(float) + kHeadTile * sizeof(float2));
}

int decode_attention_device(const pq_decode_params* p, cudaStream_t stream) {
  if (!p) return PQ_ERR_INVALID;
  if (p->B < 0 || p->N <= 0 || p->Nk <= 0 || p->Nb < 0 || p->G <= 0 || p->R < 0 || p->N % p->Nk != 0)
    return PQ_ERR_INVALID;
  if (p->rbits < 0 || p->tbits < 0 || p->rbits + p->tbits > 8) return PQ_ERR_INVALID;
  if (!dtype_ok(p->qk_dtype) || !dtype_ok(p->out_dtype)) return PQ_ERR_INVALID;
  if (p->v_dtype != PQ_F16 && p->v_dtype != PQ_BF16) return PQ_ERR_UNSUPPORTED;
  if (p->hd != kHeadDim || p->G % kStep != 0) return PQ_ERR_UNSUPPORTED;
  if (p->key_format != PQ_KEYS_BYTE && p->key_format != PQ_KEYS_PACKED6) return PQ_ERR_INVALID;
  if (p->key_format == PQ_KEYS_PACKED6 && p->rbits + p->tbits != 6) return PQ_ERR_INVALID;
  if (p->B == 0) return PQ_OK;
  if (p->Nb == 0 && p->R == 0) return PQ_ERR_INVALID;          // softmax over nothing
  const bool packed_v = p->vbits != 0 && p->Nb > 0;
  if (p->vbits != 0 && p->vbits != 4) return PQ_ERR_UNSUPPORTED;
  if (!p->q || !p->out || (!p->v && !(packed_v && p->R == 0))) return PQ_ERR_INVALID;
  if (p->Nb > 0 && (!p->codes || !p->rscale || !p->rmn || !p->tscale || !p->tmn)) return PQ_ERR_INVALID;
  if (p->R > 0 && !p->k_res) return PQ_ERR_INVALID;
  // Sequence split over peer memory: the merge pushes the result rows into the peers' exchange buffers.  The result
  // itself must then be this rank's block of its own buffer: fp32 rows (B N, 128) at its start, log-sum-exps behind.
  PushArgs px{};
  if (p->exchange_world > 0) {
    const long long rows = static_cast<long long>(p->B) * p->N;
    const int rc = exchange_push_args(p->exchange_bufs, p->exchange_world,
                                      p->exchange_rank, rows, &px);
    if (rc != PQ_OK) return rc;
    if (p->out_dtype != PQ_F32 || p->out != p->exchange_bufs[p->exchange_rank] || !p->lse ||
        p->lse != static_cast<float*>(p->out) + rows * kHeadDim || p->out_stride_h != kHeadDim ||
        p->out_stride_b != static_cast<int64_t>(p->N) * kHeadDim)
      return PQ_ERR_INVALID;
    if (p->exchange_out) {                     // the merge also collects the peers' rows and writes the final result
      if (!dtype_ok(p->exchange_out_dtype)) return PQ_ERR_INVALID;
      px.collect = 1;
      px.final_out = p->exchange_out; px.final_lse = p->exchange_lse_out; px.final_dtype = p->exchange_out_dtype;
    }
  } else if (p->exchange_world < 0) {
    return PQ_ERR_INVALID;
  }
  const int qes = static_cast<int>(dtype_bytes(p->qk_dtype));
  auto mis = [](const void* ptr, size_t al) { return reinterpret_cast<uintptr_t>(ptr) % al != 0; };
  // 128-bit loads: pointers 16-byte aligned, strides multiples of 16 bytes
  if (p->v && (mis(p->v, 16) || (p->v_stride_b * 2) % 16 || (p->v_stride_h * 2) % 16 || (p->v_stride_t * 2) % 16))
    return PQ_ERR_ALIGNMENT;
  if (packed_v) {
    if (!p->v_codes || !p->v_scale || !p->v_mn) return PQ_ERR_INVALID;
    if (p->qk_dtype != p->v_dtype) return PQ_ERR_UNSUPPORTED;
    // 8-byte code loads at 8-byte offsets within 64-byte rows; 4-byte loads of (scale, scale) token pairs
    if (mis(p->v_codes, 16) || p->vcodes_stride_b % 16 || p->vcodes_stride_h % 16 || mis(p->v_scale, 4) ||
        mis(p->v_mn, 4) || p->vscale_stride_b % 2 || p->vscale_stride_h % 2)
      return PQ_ERR_ALIGNMENT;
  }
  if (mis(p->q, 16) || (p->q_stride_b * qes) % 16 || (p->q_stride_h * qes) % 16) return PQ_ERR_ALIGNMENT;
  if (p->Nb > 0) {
    if (mis(p->codes, 16) || p->codes_stride_b % 16 || p->codes_stride_h % 16) return PQ_ERR_ALIGNMENT;
    if (mis(p->rscale, 16) || mis(p->rmn, 16) || mis(p->tscale, 16) || mis(p->tmn, 16) ||
        (p->scale_stride_b * qes) % 16 || (p->scale_stride_h * qes) % 16)
      return PQ_ERR_ALIGNMENT;
  }
  if (p->R > 0 && (mis(p->k_res, 16) || (p->kres_stride_b * qes) % 16 || (p->kres_stride_h * qes) % 16 ||
                   (p->kres_stride_t * qes) % 16))
    return PQ_ERR_ALIGNMENT;

  DecodeArgs a{};
  a.q = p->q; a.q_sb = p->q_stride_b; a.q_sh = p->q_stride_h;
  a.codes = p->codes; a.c_sb = p->codes_stride_b; a.c_sh = p->codes_stride_h;
  a.key_format = p->key_format;
  a.rscale = p->rscale; a.rmn = p->rmn; a.tscale = p->tscale; a.tmn = p->tmn;
  a.s_sb = p->scale_stride_b; a.s_sh = p->scale_stride_h;
  a.kres = p->k_res; a.kr_sb = p->kres_stride_b; a.kr_sh = p->kres_stride_h; a.kr_st = p->kres_stride_t;
  a.v = p->v; a.v_sb = p->v_stride_b; a.v_sh = p->v_stride_h; a.v_st = p->v_stride_t;
  a.v_tok0 = packed_v ? 0 : p->Nb * p->G;
  if (packed_v) {
    a.vq_codes = p->v_codes; a.vq_sb = p->vcodes_stride_b; a.vq_sh = p->vcodes_stride_h;
    a.vq_scale = p->v_scale; a.vq_mn = p->v_mn; a.vs_sb = p->vscale_stride_b; a.vs_sh = p->vscale_stride_h;
  }
  a.mask = p->mask; a.m_sb = p->mask_stride_b;
  a.B = p->B; a.N = p->N; a.Nk = p->Nk; a.Nb = p->Nb; a.G = p->G; a.R = p->R;
  plan(a, PQ_MIN_CTAS, p->num_ctas);
  size_t need = workspace_bytes_for(a);
  size_t slots = static_cast<size_t>(a.total_warps) * a.max_seg;
  if (p->dyn_lengths) {
    if (mis(p->dyn_lengths, 4)) return PQ_ERR_ALIGNMENT;
    if (p->dyn_r_add < 0) return PQ_ERR_INVALID;
    if (p->qk_dtype != p->v_dtype || p->qk_dtype == PQ_F32) return PQ_ERR_UNSUPPORTED;
    a.dyn = p->dyn_lengths; a.dyn_r_add = p->dyn_r_add;
    slots = static_cast<size_t>(slot_bound(static_cast<long long>(a.B) * a.Nk * a.head_tiles, a.plan_ctas));
    need = slots * (kPartialFloats * sizeof(float) + kHeadTile * sizeof(float2));
  }
  if (!p->workspace || p->workspace_bytes < need) return PQ_ERR_WORKSPACE;
  if (mis(p->workspace, 256)) return PQ_ERR_ALIGNMENT;
  a.part_o = static_cast<float*>(p->workspace);
  a.part_ml = reinterpret_cast<float2*>(a.part_o + slots * kPartialFloats);
  const float sm = p->sm_scale != 0.f ? p->sm_scale : 0.08838834764831845f;   // 1/sqrt(128)
  a.scale_log2 = sm * 1.4426950408889634f;

  // a kernel instance exists per (rbits, tbits); without packed keys any instance serves
  const int rb = (p->Nb > 0 || p->dyn_lengths) ? p->rbits : 4, tb = (p->Nb > 0 || p->dyn_lengths) ? p->tbits : 4;
  int rc = dispatch_bits<false>(a, rb, tb, p->qk_dtype, p->v_dtype, stream);
  if (rc != PQ_OK) return rc;
  if (p->mid_event) PQ_CUDA_TRY(cudaEventRecord(static_cast<cudaEvent_t>(p->mid_event), stream));
  const unsigned units = static_cast<unsigned>(static_cast<long long>(a.B) * a.Nk * a.head_tiles);
  // The merge is launched with programmatic stream serialisation when it directly follows the attention
  // kernel in the stream, so its launch overlaps that kernel's tail; with an event in between it is a plain launch.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(units, kHeadDim / kMergeCh);
  cfg.blockDim = dim3(kMergeCh * kMergeGroups);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool no_pdl = getenv("POLARQUANT_B200_NO_PDL") != nullptr;   // field switch: plain launches only
  cfg.numAttrs = (p->mid_event || no_pdl) ? 0 : 1;
  void* out_ptr = p->out;
  int64_t osb = p->out_stride_b, osh = p->out_stride_h;
  float* lse_ptr = p->lse;
  switch (p->out_dtype) {
    case PQ_F16: PQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, merge_partials_kernel<PQ_F16>, a, out_ptr, osb, osh, lse_ptr, px)); break;
    case PQ_BF16: PQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, merge_partials_kernel<PQ_BF16>, a, out_ptr, osb, osh, lse_ptr, px)); break;
    default: PQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, merge_partials_kernel<PQ_F32>, a, out_ptr, osb, osh, lse_ptr, px)); break;
  }
  return PQ_OK;
}

int merge_lse_strided_device(const float* outs, int64_t out_part_stride, const float* lses, int64_t lse_part_stride,
                             int P, int64_t rows, int hd, void* out, int out_dtype, float* lse_out,
                             cudaStream_t stream) {
  if (P <= 0 || rows < 0 || !dtype_ok(out_dtype)) return PQ_ERR_INVALID;
  if (hd != kHeadDim) return PQ_ERR_UNSUPPORTED;
  if (rows == 0) return PQ_OK;
  if (!outs || !lses || !out) return PQ_ERR_INVALID;
  if (rows > 0x7fffffffLL) return PQ_ERR_UNSUPPORTED;
  const unsigned grid = static_cast<unsigned>(rows);
  switch (out_dtype) {
    case PQ_F16: merge_lse_kernel<PQ_F16><<<grid, kHeadDim, 0, stream>>>(outs, out_part_stride, lses, lse_part_stride, P, out, lse_out); break;
    case PQ_BF16: merge_lse_kernel<PQ_BF16><<<grid, kHeadDim, 0, stream>>>(outs, out_part_stride, lses, lse_part_stride, P, out, lse_out); break;
    default: merge_lse_kernel<PQ_F32><<<grid, kHeadDim, 0, stream>>>(outs, out_part_stride, lses, lse_part_stride, P, out, lse_out); break;
  }
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

int merge_lse_device(const float* outs, const float* lses, int P, int64_t rows, int hd, void* out,
                     int out_dtype, float* lse_out, cudaStream_t stream) {
  return merge_lse_strided_device(outs, rows * kHeadDim, lses, rows, P, rows, hd, out, out_dtype, lse_out, stream);
}

// ---------------------------------------------------------------------------------
// Fused decode attention for callers that must not allocate.
//
// Some hosts of this library cannot hand over scratch memory: a serving runtime whose
// device heap is fully carved up at start-up, a plugin loaded into a process that forbids
// allocation calls after initialisation, code running inside a region where any allocator
// call (the CUDA runtime's or a framework's caching allocator) is off limits.  For them the
// partial results of the split-sequence kernel live in a fixed array inside the library
// image instead of a caller-provided buffer.  The array costs kStaticScratchBytes of device
// memory on every GPU whose context loads the library, until the process exits.
//
// In host code the array's name is only a handle, not a device address, so the address is
// looked up once per device with cudaGetSymbolAddress (with that device current) and cached.
// ---------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = size_t(16) << 20;     // 16 MiB; the 32k-context benchmark shape needs 14.8 MB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_addr[kMaxDevices] = {};
}  // namespace

size_t decode_static_scratch_bytes() { return kStaticScratchBytes; }

int decode_attention_static_device(const pq_decode_params* p, cudaStream_t stream) {
  if (!p) return PQ_ERR_INVALID;
  // the size check needs only the dimensions and comes first, so an oversized problem is
  // refused before anything touches the device
  pq_decode_params q = *p;
  if (p->dyn_lengths) {
    // Device-side lengths: the scratch must hold the bound over every length, units + 12 partial slots per CTA.
    // With num_ctas == 0 the grid is shrunk, if need be, to the largest one whose bound fits the array
    // (fewer, longer warp ranges: the same result up to the order of the merge); an explicit num_ctas is
    // taken as given and refused when its bound does not fit.
    if (p->B <= 0 || p->N <= 0 || p->Nk <= 0 || p->N % p->Nk != 0) return p->B == 0 ? PQ_OK : PQ_ERR_INVALID;
    constexpr long long kSlotBytes = kPartialFloats * sizeof(float) + kHeadTile * sizeof(float2);
    const long long cap_slots = static_cast<long long>(kStaticScratchBytes) / kSlotBytes;
    const int nrep = p->N / p->Nk;
    const long long units = static_cast<long long>(p->B) * p->Nk * ((nrep + kHeadTile - 1) / kHeadTile);
    const long long fit = (cap_slots - units) / (3 * kWarps);            // largest CTA count with slot_bound <= cap
    if (fit < 1) return PQ_ERR_SCRATCH_LIMIT;
    if (p->num_ctas > 0) {
      if (p->num_ctas > fit) return PQ_ERR_SCRATCH_LIMIT;
    } else {
      const long long dflt = static_cast<long long>(sm_count()) * PQ_MIN_CTAS;
      if (dflt > fit) q.num_ctas = static_cast<int>(fit);
    }
  } else {
    const size_t need = decode_workspace_bytes(p->B, p->N, p->Nk, p->Nb, p->G, p->R, p->num_ctas);
    if (need > kStaticScratchBytes) return PQ_ERR_SCRATCH_LIMIT;
  }
  int dev = -1;
  PQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return PQ_ERR_UNSUPPORTED;
  void* addr = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    addr = g_scratch_addr[dev];
    if (!addr) {
      // first call on this device: resolve the device address of the array (no allocation;
      // it may load the library's device code, so make this call before any stream capture).
      // The address is cached per device ordinal for the life of the process: a host that
      // destroys the device's context (cudaDeviceReset) must not call this entry point afterwards.
      PQ_CUDA_TRY(cudaGetSymbolAddress(&addr, g_static_scratch));
      if (!addr) return PQ_ERR_CUDA;
      g_scratch_addr[dev] = addr;
    }
  }
  q.workspace = addr;
  q.workspace_bytes = kStaticScratchBytes;
  return decode_attention_device(&q, stream);
}

}  // namespace pq
