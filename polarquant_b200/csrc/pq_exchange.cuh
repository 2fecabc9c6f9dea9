// Layout of the sequence-split exchange buffer and the argument block with which the attention kernel's merge
// pushes a rank's partial straight into the peers' inboxes (pq_exchange.cu holds the protocol's description).
#pragma once

#include "pq_common.cuh"

namespace pq {

constexpr int kExchangeRowsPerCta = 4;
constexpr int kInboxRowWords = 2 * kHeadDim + 4;             // 64 + 1 stores of 4 words per row

__host__ __device__ inline long long exchange_block_floats(long long rows) { return (rows * (kHeadDim + 1) + 3) / 4 * 4; }
__host__ __device__ inline int exchange_slices(long long rows) {
  return static_cast<int>((rows + kExchangeRowsPerCta - 1) / kExchangeRowsPerCta);
}
__host__ __device__ inline long long exchange_inbox_words(long long rows) { return rows * kInboxRowWords; }
__host__ __device__ inline long long exchange_buffer_words(int world, long long rows) {
  return exchange_block_floats(rows) + 2ll * world * exchange_inbox_words(rows) + 4;
}

// What a producer kernel needs to push this rank's rows: for every peer the base of the inbox slot (parity 0) this
// rank writes to, the distance to the parity-1 slot, and this rank's control words (the epoch is ctrl[0] + 1).  With
// `collect` set the producer also gathers the peers' rows from this rank's own inbox and writes the merged result,
// i.e. it does the whole exchange and no exchange kernel follows.
struct PushArgs {
  float* inbox[PQ_EXCHANGE_MAX_RANKS];
  unsigned* ctrl;
  long long parity_stride, rows;
  int world, rank;                         // world == 0: nothing to push
  const float* local_inbox;                // this rank's inbox (parity 0, sender 0)
  long long inbox_words;                   // one (parity, sender) slot
  void* final_out; float* final_lse;       // merged result (rows, 128) of final_dtype, log-sum-exp (rows) or null
  int final_dtype, collect;
};

constexpr unsigned long long kExchangeWaitLimitNs = 1000000000ull;   // a wait on a peer gives up after one second ...
constexpr int kExchangeSpinLimit = 1 << 24;                          // ... or after this many polls

// one (value, epoch) pair: an aligned 8-byte store arrives whole
__device__ __forceinline__ void push_pair(float* p, float v, unsigned e) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(e) : "memory");
}
// two pairs in one 16-byte store
__device__ __forceinline__ void push_pairs(float* p, float a, float b, unsigned e) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};" ::"l"(p), "r"(__float_as_uint(a)), "r"(e),
               "r"(__float_as_uint(b)) : "memory");
}
__device__ __forceinline__ uint2 look_pair(const float* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 look_pairs(const float* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long exchange_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Called by the thread that has just computed channel `ch` of output row `row` (and holds the row's log-sum-exp):
// pushes the value - and, from the thread with ch == 0, the log-sum-exp - to every peer; with px.collect it then waits
// (bounded) for the same channel of the same row from every peer in this rank's inbox, merges in rank order with the
// arithmetic of the gathered merge and writes the final result.
__device__ __forceinline__ void push_row_value(const PushArgs& px, long long row, int ch, float val, float lse) {
  const unsigned e = *reinterpret_cast<const volatile unsigned*>(px.ctrl) + 1u;
  const long long par = (e & 1u) ? px.parity_stride : 0;
#pragma unroll
  for (int p = 0; p < PQ_EXCHANGE_MAX_RANKS; ++p) {          // constant indices: the pointers stay in parameter space
    if (p >= px.world || p == px.rank) continue;
    float* dst = px.inbox[p] + par;
    push_pair(dst + row * 2 * kHeadDim + 2 * ch, val, e);
    if (ch == 0) push_pairs(dst + px.rows * 2 * kHeadDim + row * 4, lse, 0.f, e);
  }
  if (!px.collect) return;
  const float* base = px.local_inbox + par;
  uint2 lv[PQ_EXCHANGE_MAX_RANKS];
  uint4 ll[PQ_EXCHANGE_MAX_RANKS];
  bool ok = false;
  unsigned long long t0 = 0;
  for (int it = 0; it < kExchangeSpinLimit; ++it) {          // one poll: all awaited words, their loads in flight together
    ok = true;
#pragma unroll
    for (int p = 0; p < PQ_EXCHANGE_MAX_RANKS; ++p) {
      if (p >= px.world || p == px.rank) continue;
      const float* src = base + p * px.inbox_words;
      ll[p] = look_pairs(src + px.rows * 2 * kHeadDim + row * 4);
      lv[p] = look_pair(src + row * 2 * kHeadDim + 2 * ch);
    }
#pragma unroll
    for (int p = 0; p < PQ_EXCHANGE_MAX_RANKS; ++p) {
      if (p >= px.world || p == px.rank) continue;
      ok &= ll[p].y == e && ll[p].w == e && lv[p].y == e;
    }
    if (ok) break;
    if (it == 0) t0 = exchange_ns();
    else if (exchange_ns() - t0 > kExchangeWaitLimitNs) break;
  }
  if (!ok) atomicOr(px.ctrl + 2, 2u);
  float M = -INFINITY;
#pragma unroll
  for (int p = 0; p < PQ_EXCHANGE_MAX_RANKS; ++p)
    if (p < px.world) M = fmaxf(M, p == px.rank ? lse : __uint_as_float(ll[p].x));
  float L = 0.f, acc = 0.f;
#pragma unroll
  for (int p = 0; p < PQ_EXCHANGE_MAX_RANKS; ++p) {
    if (p >= px.world) continue;
    const float l = p == px.rank ? lse : __uint_as_float(ll[p].x);
    const float v = p == px.rank ? val : __uint_as_float(lv[p].x);
    const float w = l == -INFINITY ? 0.f : __expf(l - M);
    L += w;
    acc = fmaf(w, v, acc);
  }
  const float merged = acc / L;
  const long long off = row * kHeadDim + ch;
  if (px.final_dtype == PQ_F32) static_cast<float*>(px.final_out)[off] = merged;
  else if (px.final_dtype == PQ_F16) static_cast<__half*>(px.final_out)[off] = __float2half_rn(merged);
  else static_cast<__nv_bfloat16*>(px.final_out)[off] = __float2bfloat16_rn(merged);
  if (px.final_lse && ch == 0) px.final_lse[row] = M + __logf(L);
}

// With px.collect the producer kernel is the whole exchange: its last CTA to finish advances the epoch.  Called once
// per CTA by one thread after the CTA's rows are done (all CTAs have read the epoch by then).
__device__ __forceinline__ void finish_exchange_cta(const PushArgs& px, unsigned ctas) {
  if (!px.collect) return;
  const unsigned e = *reinterpret_cast<const volatile unsigned*>(px.ctrl) + 1u;
  if (atomicAdd(px.ctrl + 1, 1u) == ctas - 1) {
    px.ctrl[1] = 0u;
    *reinterpret_cast<volatile unsigned*>(px.ctrl) = e;
  }
}

// fills `px` for rank `rank` of `world` from the ranks' buffer pointers as this process sees them
int exchange_push_args(void* const* bufs, int world, int rank, long long rows, PushArgs* px);

}  // namespace pq
