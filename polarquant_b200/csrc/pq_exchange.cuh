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
  return exchange_block_floats(rows) + 2ll * world * exchange_inbox_words(rows) +
         static_cast<long long>(world) * exchange_slices(rows) + 4;
}

// What a producer kernel needs to push this rank's rows: for every peer the base of the inbox slot (parity 0) this
// rank writes to, the distance to the parity-1 slot, and this rank's control words (the epoch is ctrl[0] + 1).
struct PushArgs {
  float* inbox[PQ_EXCHANGE_MAX_RANKS];
  const unsigned* ctrl;
  long long parity_stride, rows;
  int world, rank;                         // world == 0: nothing to push
};

// one (value, epoch) pair: an aligned 8-byte store arrives whole
__device__ __forceinline__ void push_pair(float* p, float v, unsigned e) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(e) : "memory");
}
// two pairs in one 16-byte store
__device__ __forceinline__ void push_pairs(float* p, float a, float b, unsigned e) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};" ::"l"(p), "r"(__float_as_uint(a)), "r"(e),
               "r"(__float_as_uint(b)) : "memory");
}
// Push channel `ch` of output row `row` (and, from the thread with ch == 0, the row's log-sum-exp) to every peer.
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
}

// fills `px` for rank `rank` of `world` from the ranks' buffer pointers as this process sees them
int exchange_push_args(const void* const* bufs, int world, int rank, long long rows, PushArgs* px);

}  // namespace pq
