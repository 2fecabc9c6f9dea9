// Sequence-split exchange over NVLink peer memory (sm_100a): one kernel pushes this GPU's partial attention result
// into every peer's buffer, picks up the peers' pushes and merges all partials by log-sum-exp.  It replaces the
// all-gather + merge pair of the sequence split (two launches, one of them a library collective) by one launch whose
// only remote operations are plain stores into peer memory.
//
// The pushed data validates itself: every 16-byte store carries two (value, epoch) pairs, and the receiver polls
// the words in its own memory until both epochs match (8-byte halves of an aligned 16-byte store arrive whole).  No
// fence, no separate "data ready" flag and no second round trip sit on the critical path: the latency of the
// exchange is one store's flight over NVLink plus whatever the ranks' attention kernels are apart.
//
// Every rank owns one exchange buffer of the same layout (32-bit words):
//
//   own     block                 [out (rows, 128) | lse (rows)] fp32, padded to a multiple of 4: this rank's partial,
//                                 written in place by its attention kernel
//   inbox   2 x world x rows*260  per epoch parity and sending rank: rows x 64 stores {v0, e, v1, e} of the output
//                                 and rows stores {lse, e, 0, e}
//   ctrl    4 words               epoch of the last finished call, finished-CTA counter, status bits, unused
//
// CTA s owns the row slice s (kRowsPerCta rows) on every rank, so CTAs of one launch never wait on each other - only
// on the CTA of the same index on the peers - and no grid-wide barrier exists.  Per call (epoch e, parity e & 1):
//   1. store the slice, paired with e, into this rank's inbox slot on every peer;
//   2. poll the local inbox slots of the peers until the slice has arrived, merge in rank order with the arithmetic
//      of the gathered merge (bit-identical results), write the output.
// No "slot consumed" handshake is needed before a slot is overwritten: the slot of epoch e was last read by the peer's
// call of epoch e - 2, and that call had ended before the peer produced the rows of epoch e - 1, which this rank's
// call of epoch e - 1 waited for before it ended.  (It does rely on the calls of one rank being ordered on a stream.)
// Step 1 is normally done by the producer instead: the merge kernel that ends the attention call stores each result
// value as a {v, e} pair into the peers' inboxes as it writes it locally (push_row_value, pq_exchange.cuh), and this
// kernel is told so (PQ_EXCHANGE_PUSHED).
// The epoch lives in the buffer and is advanced by the last CTA to finish, so a captured CUDA graph replays the call.
// Every wait is bounded (one second); on expiry the kernel records a status bit and carries on, so that a peer that
// never arrives leaves a wrong result and a readable status rather than a hung GPU.
#include <stdlib.h>
#include <string.h>

#include "pq_exchange.cuh"

namespace pq {
namespace {

constexpr int kRowsPerCta = kExchangeRowsPerCta;
static_assert(kRowsPerCta * 32 == kHeadDim, "one float4 per thread covers the output rows of a slice");
constexpr unsigned long long kWaitLimitNs = kExchangeWaitLimitNs;
constexpr int kSpinLimit = kExchangeSpinLimit;

struct ExchangeArgs {
  float* buf[PQ_EXCHANGE_MAX_RANKS];
  void* out[PQ_EXCHANGE_MAX_RANKS];        // a real launch uses entry `rank` only
  float* lse_out[PQ_EXCHANGE_MAX_RANKS];
  int world, rank;                         // rank < 0: all ranks emulated by one launch, rank = blockIdx.y
  long long rows, block_f, inbox_words;    // inbox_words: one (parity, sender) slot
  int slices;
  int pushed;                              // the producer of this rank's block already pushed it to the peers
};

inline long long block_floats(long long rows) { return exchange_block_floats(rows); }
inline int slices_of(long long rows) { return exchange_slices(rows); }
inline long long inbox_slot_words(long long rows) { return exchange_inbox_words(rows); }
inline long long buffer_words(int world, long long rows) { return exchange_buffer_words(world, rows); }

template <int ODT>
__global__ void __launch_bounds__(kHeadDim) exchange_merge_kernel(const ExchangeArgs a) {
  const int rank = a.rank < 0 ? static_cast<int>(blockIdx.y) : a.rank;
  const int s = blockIdx.x, tid = threadIdx.x;
  float* mine = a.buf[rank];
  const long long inbox0 = a.block_f;
  unsigned* ctrl = reinterpret_cast<unsigned*>(mine) + inbox0 + 2ll * a.world * a.inbox_words;
  __shared__ unsigned s_epoch;
  if (tid == 0) s_epoch = *reinterpret_cast<volatile unsigned*>(ctrl) + 1u;
  __syncthreads();
  const unsigned epoch = s_epoch;
  const long long slot = static_cast<long long>(epoch & 1u) * a.world;     // inbox slots of this epoch's parity
  const long long r0 = static_cast<long long>(s) * kRowsPerCta;
  const int row = tid >> 5, col = tid & 31;
  const bool active = r0 + row < a.rows;
  const long long grow = r0 + row;

  // launched as a programmatic dependent of the kernel that writes this rank's partial: everything above overlaps
  // that kernel's tail (a no-op for an ordinary launch)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (active) {
    // 1. push: this thread's four output values (and, once per row, the log-sum-exp), each pair with the epoch
    const float4 v = *reinterpret_cast<const float4*>(mine + grow * kHeadDim + 4 * col);
    const float l = mine[a.rows * kHeadDim + grow];
    for (int p = 0; p < a.world; ++p) {
      if (p == rank || a.pushed) continue;
      float* dst = a.buf[p] + inbox0 + (slot + rank) * a.inbox_words;
      push_pairs(dst + grow * 2 * kHeadDim + 8 * col, v.x, v.y, epoch);
      push_pairs(dst + grow * 2 * kHeadDim + 8 * col + 4, v.z, v.w, epoch);
      if (col == 0) push_pairs(dst + a.rows * 2 * kHeadDim + grow * 4, l, 0.f, epoch);
    }

    // 2. collect the peers' values of this row and these four channels from the local inbox.  One poll looks at
    // every word (all loads in flight together: one L2 round trip per poll whatever the number of peers) and the
    // loop ends once each carries this epoch in both halves, or when the time limit is reached.
    uint4 look[PQ_EXCHANGE_MAX_RANKS][3];
    bool ok = false;
    unsigned long long t0 = 0;
    for (int it = 0; it < kSpinLimit; ++it) {
      ok = true;
#pragma unroll
      for (int p = 0; p < PQ_EXCHANGE_MAX_RANKS; ++p) {
        if (p >= a.world || p == rank) continue;
        const float* src = mine + inbox0 + (slot + p) * a.inbox_words;
        look[p][0] = look_pairs(src + a.rows * 2 * kHeadDim + grow * 4);
        look[p][1] = look_pairs(src + grow * 2 * kHeadDim + 8 * col);
        look[p][2] = look_pairs(src + grow * 2 * kHeadDim + 8 * col + 4);
      }
#pragma unroll
      for (int p = 0; p < PQ_EXCHANGE_MAX_RANKS; ++p) {
        if (p >= a.world || p == rank) continue;
#pragma unroll
        for (int k = 0; k < 3; ++k) ok &= look[p][k].y == epoch && look[p][k].w == epoch;
      }
      if (ok) break;
      if (it == 0) t0 = exchange_ns();
      else if (exchange_ns() - t0 > kWaitLimitNs) break;
    }
    float4 vp[PQ_EXCHANGE_MAX_RANKS];
    float lp[PQ_EXCHANGE_MAX_RANKS];
#pragma unroll
    for (int p = 0; p < PQ_EXCHANGE_MAX_RANKS; ++p) {
      if (p >= a.world) continue;
      if (p == rank) { vp[p] = v; lp[p] = l; continue; }
      lp[p] = __uint_as_float(look[p][0].x);
      vp[p] = make_float4(__uint_as_float(look[p][1].x), __uint_as_float(look[p][1].z),
                          __uint_as_float(look[p][2].x), __uint_as_float(look[p][2].z));
    }
    if (!ok) atomicOr(ctrl + 2, 2u);

    // merge in rank order: the arithmetic of the merge over a gathered buffer, four channels per thread
    float M = -INFINITY;
#pragma unroll
    for (int p = 0; p < PQ_EXCHANGE_MAX_RANKS; ++p)
      if (p < a.world) M = fmaxf(M, lp[p]);
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int p = 0; p < PQ_EXCHANGE_MAX_RANKS; ++p) {
      if (p >= a.world) continue;
      const float w = lp[p] == -INFINITY ? 0.f : __expf(lp[p] - M);
      L += w;
      acc.x = fmaf(w, vp[p].x, acc.x); acc.y = fmaf(w, vp[p].y, acc.y);
      acc.z = fmaf(w, vp[p].z, acc.z); acc.w = fmaf(w, vp[p].w, acc.w);
    }
    const float4 val = make_float4(acc.x / L, acc.y / L, acc.z / L, acc.w / L);
    const long long off = grow * kHeadDim + 4 * col;
    if constexpr (ODT == PQ_F32) {
      *reinterpret_cast<float4*>(static_cast<float*>(a.out[rank]) + off) = val;
    } else {
      constexpr int DT16 = ODT == PQ_F16 ? PQ_F16 : PQ_BF16;
      *reinterpret_cast<uint2*>(static_cast<char*>(a.out[rank]) + off * 2) =
          make_uint2(pack2<DT16>(val.x, val.y), pack2<DT16>(val.z, val.w));
    }
    if (a.lse_out[rank] && col == 0) a.lse_out[rank][grow] = M + __logf(L);
  }
  __syncthreads();

  // the last CTA of this rank advances the epoch
  // (no fence: the counter only elects the last CTA, and what it writes is read by the next launch)
  if (tid == 0) {
    if (atomicAdd(ctrl + 1, 1u) == gridDim.x - 1) {
      ctrl[1] = 0u;
      *reinterpret_cast<volatile unsigned*>(ctrl) = epoch;
    }
  }
}

}  // namespace

int exchange_push_args(void* const* bufs, int world, int rank, long long rows, PushArgs* px) {
  if (!bufs || !px || world < 1 || world > PQ_EXCHANGE_MAX_RANKS || rank < 0 || rank >= world || rows <= 0)
    return PQ_ERR_INVALID;
  *px = PushArgs{};
  for (int p = 0; p < world; ++p) {
    if (!bufs[p]) return PQ_ERR_INVALID;
    if (reinterpret_cast<uintptr_t>(bufs[p]) & 15) return PQ_ERR_ALIGNMENT;
    px->inbox[p] = static_cast<float*>(bufs[p]) + block_floats(rows) + rank * inbox_slot_words(rows);
  }
  px->ctrl = static_cast<unsigned*>(bufs[rank]) + buffer_words(world, rows) - 4;
  px->parity_stride = world * inbox_slot_words(rows);
  px->rows = rows; px->world = world; px->rank = rank;
  px->local_inbox = static_cast<const float*>(bufs[rank]) + block_floats(rows);
  px->inbox_words = inbox_slot_words(rows);
  return PQ_OK;
}

namespace {

int check_common(void* const* bufs, int world, long long rows, int hd, int out_dtype) {
  if (!bufs || world < 1 || world > PQ_EXCHANGE_MAX_RANKS || rows <= 0 || hd != kHeadDim) return PQ_ERR_INVALID;
  if (out_dtype != PQ_F16 && out_dtype != PQ_BF16 && out_dtype != PQ_F32) return PQ_ERR_INVALID;
  for (int p = 0; p < world; ++p) {
    if (!bufs[p]) return PQ_ERR_INVALID;
    if (reinterpret_cast<uintptr_t>(bufs[p]) & 15) return PQ_ERR_ALIGNMENT;
  }
  return PQ_OK;
}

int launch(const ExchangeArgs& a, int out_dtype, dim3 grid, bool cooperative, bool dependent, cudaStream_t stream) {
  void* params[] = {const_cast<ExchangeArgs*>(&a)};
  const void* fn = out_dtype == PQ_F16    ? reinterpret_cast<const void*>(exchange_merge_kernel<PQ_F16>)
                   : out_dtype == PQ_BF16 ? reinterpret_cast<const void*>(exchange_merge_kernel<PQ_BF16>)
                                          : reinterpret_cast<const void*>(exchange_merge_kernel<PQ_F32>);
  if (cooperative) {
    PQ_CUDA_TRY(cudaLaunchCooperativeKernel(fn, grid, dim3(kHeadDim), params, 0, stream));
  } else {
    // programmatic dependent launch, when the caller says the preceding kernel of the stream is the merge of the
    // attention partials: the grid may become resident while that kernel drains and waits for its results on the
    // device.  (Behind another exchange kernel it must not be used: the epoch is read before that wait.)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(kHeadDim); cfg.dynamicSmemBytes = 0; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    static const bool no_pdl = getenv("POLARQUANT_B200_NO_PDL") != nullptr;   // field switch: plain launches only
    cfg.attrs = attr; cfg.numAttrs = (dependent && !no_pdl) ? 1 : 0;
    PQ_CUDA_TRY(cudaLaunchKernelExC(&cfg, fn, params));
  }
  return PQ_OK;
}

}  // namespace
}  // namespace pq

using namespace pq;

extern "C" {

int64_t pq_exchange_bytes(int world, int64_t rows, int hd) {
  if (world < 1 || world > PQ_EXCHANGE_MAX_RANKS || rows <= 0 || hd != kHeadDim) return 0;
  return buffer_words(world, rows) * 4;
}

int64_t pq_exchange_slot_offset(int world, int64_t rows, int hd, int rank) {
  if (world < 1 || world > PQ_EXCHANGE_MAX_RANKS || rows <= 0 || hd != kHeadDim || rank < 0 || rank >= world) return -1;
  return 0;      // the rank's own partial opens its buffer; the peers' partials arrive in the inbox behind it
}

int pq_peer_alloc(int64_t bytes, void** ptr, unsigned char* handle) {
  if (bytes <= 0 || !ptr || !handle) return PQ_ERR_INVALID;
  static_assert(sizeof(cudaIpcMemHandle_t) == PQ_IPC_HANDLE_BYTES, "handle size");
  void* p = nullptr;
  PQ_CUDA_TRY(cudaMalloc(&p, static_cast<size_t>(bytes)));
  cudaError_t e = cudaMemset(p, 0, static_cast<size_t>(bytes));
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { cudaFree(p); return cuda_fail(e); }
  memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return PQ_OK;
}

int pq_peer_open(const unsigned char* handle, void** ptr) {
  if (!handle || !ptr) return PQ_ERR_INVALID;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  PQ_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return PQ_OK;
}

int pq_peer_close(void* ptr) {
  if (!ptr) return PQ_ERR_INVALID;
  PQ_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return PQ_OK;
}

int pq_peer_free(void* ptr) {
  if (!ptr) return PQ_ERR_INVALID;
  PQ_CUDA_TRY(cudaFree(ptr));
  return PQ_OK;
}

int pq_exchange_merge(void* const* bufs, int world, int rank, int64_t rows, int hd, void* out, int out_dtype,
                      float* lse_out, unsigned flags, void* stream) {
  const int rc = check_common(bufs, world, rows, hd, out_dtype);
  if (rc != PQ_OK) return rc;
  if (rank < 0 || rank >= world || !out || (flags & ~(PQ_EXCHANGE_AFTER_ATTENTION | PQ_EXCHANGE_PUSHED)))
    return PQ_ERR_INVALID;
  if (reinterpret_cast<uintptr_t>(out) & 15) return PQ_ERR_ALIGNMENT;      // four channels per vector store
  ExchangeArgs a{};
  for (int p = 0; p < world; ++p) a.buf[p] = static_cast<float*>(bufs[p]);
  a.out[rank] = out; a.lse_out[rank] = lse_out;
  a.world = world; a.rank = rank; a.rows = rows; a.block_f = block_floats(rows); a.slices = slices_of(rows);
  a.inbox_words = inbox_slot_words(rows);
  a.pushed = (flags & PQ_EXCHANGE_PUSHED) != 0;
  return launch(a, out_dtype, dim3(a.slices), false, (flags & PQ_EXCHANGE_AFTER_ATTENTION) != 0,
                static_cast<cudaStream_t>(stream));
}

int pq_exchange_merge_emulated(void* const* bufs, int world, int64_t rows, int hd, void* const* outs, int out_dtype,
                               float* const* lse_outs, unsigned flags, void* stream) {
  const int rc = check_common(bufs, world, rows, hd, out_dtype);
  if (rc != PQ_OK) return rc;
  if (!outs || (flags & ~PQ_EXCHANGE_PUSHED)) return PQ_ERR_INVALID;
  ExchangeArgs a{};
  for (int p = 0; p < world; ++p) {
    if (!outs[p]) return PQ_ERR_INVALID;
    if (reinterpret_cast<uintptr_t>(outs[p]) & 15) return PQ_ERR_ALIGNMENT;
    a.buf[p] = static_cast<float*>(bufs[p]);
    a.out[p] = outs[p];
    a.lse_out[p] = lse_outs ? lse_outs[p] : nullptr;
  }
  a.world = world; a.rank = -1; a.rows = rows; a.block_f = block_floats(rows); a.slices = slices_of(rows);
  a.inbox_words = inbox_slot_words(rows);
  a.pushed = (flags & PQ_EXCHANGE_PUSHED) != 0;
  // the emulated ranks wait on one another inside one launch: a cooperative launch guarantees that all of its CTAs
  // are resident together (and is refused, not deadlocked, when they cannot be)
  return launch(a, out_dtype, dim3(a.slices, world), true, false, static_cast<cudaStream_t>(stream));
}

int pq_exchange_status(const void* local_buf, int world, int64_t rows, int hd, unsigned* status, void* stream) {
  if (!local_buf || !status || pq_exchange_bytes(world, rows, hd) == 0) return PQ_ERR_INVALID;
  const unsigned* ctrl = static_cast<const unsigned*>(local_buf) + buffer_words(world, rows) - 4;
  PQ_CUDA_TRY(cudaMemcpyAsync(status, ctrl + 2, sizeof(unsigned), cudaMemcpyDeviceToHost,
                              static_cast<cudaStream_t>(stream)));
  PQ_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return PQ_OK;
}

}  // extern "C"
