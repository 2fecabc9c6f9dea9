// Sequence-split exchange over NVLink peer memory (sm_100a): one kernel pushes this GPU's partial attention result
// into every peer's buffer, waits for the peers' pushes and merges all partials by log-sum-exp.  It replaces the
// all-gather + merge pair of the sequence split (two launches, one of them a library collective) by one launch whose
// only remote operations are plain stores into peer memory and two flag words per (peer, row slice).
//
// Every rank owns one exchange buffer of the same layout (float / 32-bit units):
//
//   slots   world x block      block = [out (rows, 128) | lse (rows)], padded to a multiple of 4 floats; slot r holds
//                              rank r's partial.  A rank's attention kernel writes its own slot of its own buffer.
//   ready   world x slices     ready[r][s] = epoch once rank r's rows of slice s have landed in THIS buffer
//   free    world x slices     free[r][s]  = epoch once rank r has finished reading what THIS rank pushed to it
//   ctrl    4 words            epoch of the last finished call, finished-CTA counter, status bits, unused
//
// CTA s of the kernel owns the row slice s (kRowsPerCta rows) on every rank, so CTAs of one launch never wait on each
// other - only on the CTA of the same index on the peers - and the protocol needs no grid-wide barrier:
//   1. wait until every peer released the slice pushed in the previous call (free[p][s] >= epoch - 1, flags in the
//      local buffer), 2. store the slice into slot `rank` of every peer, 3. system-scope fence, then ready[rank][s] =
//   epoch on every peer, 4. wait for ready[p][s] == epoch from every peer (local flags), 5. merge the slice from the
//   local slots, 6. free[rank][s] = epoch on every peer.  The epoch lives in the buffer and is advanced by the last
//   CTA to finish, so a captured CUDA graph replays the call unchanged.
// Every wait is bounded (about a second); on expiry the kernel records a status bit and carries on, so that a peer
// that never arrives leaves a wrong result and a readable status rather than a hung GPU.
#include <string.h>

#include "pq_common.cuh"

namespace pq {
namespace {

constexpr int kRowsPerCta = 4;
static_assert(kRowsPerCta * 32 == kHeadDim, "one float4 per thread covers the output rows of a slice");
constexpr unsigned long long kWaitLimitNs = 1000000000ull;   // a wait on a peer gives up after one second ...
constexpr int kSpinLimit = 1 << 24;                          // ... or after this many polls, whichever comes first

struct ExchangeArgs {
  float* buf[PQ_EXCHANGE_MAX_RANKS];
  void* out[PQ_EXCHANGE_MAX_RANKS];        // a real launch uses entry `rank` only
  float* lse_out[PQ_EXCHANGE_MAX_RANKS];
  int world, rank;                         // rank < 0: all ranks emulated by one launch, rank = blockIdx.y
  long long rows, block_f;
  int slices;
};

inline long long block_floats(long long rows) { return (rows * (kHeadDim + 1) + 3) / 4 * 4; }
inline int slices_of(long long rows) { return static_cast<int>((rows + kRowsPerCta - 1) / kRowsPerCta); }
inline long long buffer_words(int world, long long rows) {
  return world * block_floats(rows) + 2ll * world * slices_of(rows) + 4;
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// true once *flag has reached `want` (epochs only grow; the signed difference tolerates wrap-around)
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool wait_reached(const unsigned* flag, unsigned want) {
  if (static_cast<int>(ld_acquire_sys(flag) - want) >= 0) return true;
  const unsigned long long t0 = global_ns();
  for (int it = 0; it < kSpinLimit; ++it) {
    __nanosleep(100);
    if (static_cast<int>(ld_acquire_sys(flag) - want) >= 0) return true;
    if (global_ns() - t0 > kWaitLimitNs) break;
  }
  return false;
}

template <int ODT>
__global__ void __launch_bounds__(kHeadDim) exchange_merge_kernel(const ExchangeArgs a) {
  const int rank = a.rank < 0 ? static_cast<int>(blockIdx.y) : a.rank;
  const int s = blockIdx.x, tid = threadIdx.x;
  float* mine = a.buf[rank];
  const long long flags0 = a.world * a.block_f;
  unsigned* ready = reinterpret_cast<unsigned*>(mine) + flags0;
  unsigned* freed = ready + static_cast<long long>(a.world) * a.slices;
  unsigned* ctrl = freed + static_cast<long long>(a.world) * a.slices;
  __shared__ unsigned s_epoch;
  if (tid == 0) s_epoch = *reinterpret_cast<volatile unsigned*>(ctrl) + 1u;
  __syncthreads();
  const unsigned epoch = s_epoch;
  const long long r0 = static_cast<long long>(s) * kRowsPerCta;
  const int nr = static_cast<int>(min(static_cast<long long>(kRowsPerCta), a.rows - r0));

  // 1. the peers have consumed what the previous call pushed into their slot `rank`
  if (tid < a.world && tid != rank && !wait_reached(freed + tid * a.slices + s, epoch - 1u)) atomicOr(ctrl + 2, 1u);
  __syncthreads();

  // 2. push the slice: 32 float4 per output row, one float per lse row
  {
    const float* src = mine + rank * a.block_f;
    const int row = tid >> 5, col = tid & 31;
    if (row < nr) {
      const long long off = (r0 + row) * kHeadDim + 4 * col;
      const float4 v = *reinterpret_cast<const float4*>(src + off);
      for (int p = 0; p < a.world; ++p)
        if (p != rank) *reinterpret_cast<float4*>(a.buf[p] + rank * a.block_f + off) = v;
    }
    if (tid < nr) {
      const long long off = a.rows * kHeadDim + r0 + tid;
      const float v = src[off];
      for (int p = 0; p < a.world; ++p)
        if (p != rank) a.buf[p][rank * a.block_f + off] = v;
    }
  }
  __syncthreads();
  // 3. publish: the fence orders every thread's stores (observed through the barrier) before the flags
  if (tid == 0) {
    __threadfence_system();
    for (int p = 0; p < a.world; ++p)
      if (p != rank)
        st_release_sys(reinterpret_cast<unsigned*>(a.buf[p]) + flags0 + rank * a.slices + s, epoch);
  }
  // 4. the peers' slices have landed here
  if (tid < a.world && tid != rank && !wait_reached(ready + tid * a.slices + s, epoch)) atomicOr(ctrl + 2, 2u);
  __syncthreads();

  // 5. merge, in rank order (the same arithmetic as the merge of a gathered buffer).  Remote ranks wrote these lines
  // into local memory: read them past L1.
  for (int r = 0; r < nr; ++r) {
    const long long row = r0 + r;
    float M = -INFINITY;
    for (int p = 0; p < a.world; ++p) M = fmaxf(M, __ldcg(mine + p * a.block_f + a.rows * kHeadDim + row));
    float L = 0.f, acc = 0.f;
    for (int p = 0; p < a.world; ++p) {
      const float l = __ldcg(mine + p * a.block_f + a.rows * kHeadDim + row);
      const float w = l == -INFINITY ? 0.f : __expf(l - M);
      L += w;
      acc = fmaf(w, __ldcg(mine + p * a.block_f + row * kHeadDim + tid), acc);
    }
    const float val = acc / L;
    const long long off = row * kHeadDim + tid;
    if constexpr (ODT == PQ_F32) static_cast<float*>(a.out[rank])[off] = val;
    else if constexpr (ODT == PQ_F16) static_cast<__half*>(a.out[rank])[off] = __float2half_rn(val);
    else static_cast<__nv_bfloat16*>(a.out[rank])[off] = __float2bfloat16_rn(val);
    if (a.lse_out[rank] && tid == 0) a.lse_out[rank][row] = M + __logf(L);
  }
  __syncthreads();

  // 6. release the peers' slices; the last CTA of this rank advances the epoch
  if (tid == 0) {
    for (int p = 0; p < a.world; ++p)
      if (p != rank)
        st_release_sys(reinterpret_cast<unsigned*>(a.buf[p]) + flags0 + static_cast<long long>(a.world) * a.slices +
                           rank * a.slices + s, epoch);
    __threadfence();
    if (atomicAdd(ctrl + 1, 1u) == gridDim.x - 1) {
      ctrl[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned*>(ctrl) = epoch;
    }
  }
}

int check_common(void* const* bufs, int world, long long rows, int hd, int out_dtype) {
  if (!bufs || world < 1 || world > PQ_EXCHANGE_MAX_RANKS || rows <= 0 || hd != kHeadDim) return PQ_ERR_INVALID;
  if (out_dtype != PQ_F16 && out_dtype != PQ_BF16 && out_dtype != PQ_F32) return PQ_ERR_INVALID;
  for (int p = 0; p < world; ++p) {
    if (!bufs[p]) return PQ_ERR_INVALID;
    if (reinterpret_cast<uintptr_t>(bufs[p]) & 15) return PQ_ERR_ALIGNMENT;
  }
  return PQ_OK;
}

int launch(const ExchangeArgs& a, int out_dtype, dim3 grid, bool cooperative, cudaStream_t stream) {
  void* params[] = {const_cast<ExchangeArgs*>(&a)};
  const void* fn = out_dtype == PQ_F16    ? reinterpret_cast<const void*>(exchange_merge_kernel<PQ_F16>)
                   : out_dtype == PQ_BF16 ? reinterpret_cast<const void*>(exchange_merge_kernel<PQ_BF16>)
                                          : reinterpret_cast<const void*>(exchange_merge_kernel<PQ_F32>);
  if (cooperative) PQ_CUDA_TRY(cudaLaunchCooperativeKernel(fn, grid, dim3(kHeadDim), params, 0, stream));
  else PQ_CUDA_TRY(cudaLaunchKernel(fn, grid, dim3(kHeadDim), params, 0, stream));
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
  return rank * block_floats(rows) * 4;
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
                      float* lse_out, void* stream) {
  const int rc = check_common(bufs, world, rows, hd, out_dtype);
  if (rc != PQ_OK) return rc;
  if (rank < 0 || rank >= world || !out) return PQ_ERR_INVALID;
  ExchangeArgs a{};
  for (int p = 0; p < world; ++p) a.buf[p] = static_cast<float*>(bufs[p]);
  a.out[rank] = out; a.lse_out[rank] = lse_out;
  a.world = world; a.rank = rank; a.rows = rows; a.block_f = block_floats(rows); a.slices = slices_of(rows);
  return launch(a, out_dtype, dim3(a.slices), false, static_cast<cudaStream_t>(stream));
}

int pq_exchange_merge_emulated(void* const* bufs, int world, int64_t rows, int hd, void* const* outs, int out_dtype,
                               float* const* lse_outs, void* stream) {
  const int rc = check_common(bufs, world, rows, hd, out_dtype);
  if (rc != PQ_OK) return rc;
  if (!outs) return PQ_ERR_INVALID;
  ExchangeArgs a{};
  for (int p = 0; p < world; ++p) {
    if (!outs[p]) return PQ_ERR_INVALID;
    a.buf[p] = static_cast<float*>(bufs[p]);
    a.out[p] = outs[p];
    a.lse_out[p] = lse_outs ? lse_outs[p] : nullptr;
  }
  a.world = world; a.rank = -1; a.rows = rows; a.block_f = block_floats(rows); a.slices = slices_of(rows);
  // the emulated ranks wait on one another inside one launch: a cooperative launch guarantees that all of its CTAs
  // are resident together (and is refused, not deadlocked, when they cannot be)
  return launch(a, out_dtype, dim3(a.slices, world), true, static_cast<cudaStream_t>(stream));
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
