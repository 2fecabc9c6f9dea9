// C ABI of the library (declarations and contracts: include/polarquant_b200.h).
#include <string.h>

#include "pq_common.cuh"

namespace pq {
int& last_cuda_error() {
  static thread_local int e = 0;
  return e;
}
int quantize_device(const void* keys, const int64_t strides[4], int B, int Nk, int L, int hd, int G, int rbits,
                    int tbits, int dtype, unsigned flags, uint8_t* codes, void* rscale, void* rmn, void* tscale,
                    void* tmn, const int64_t* out_strides, cudaStream_t stream, const int* gate_lengths = nullptr,
                    int gate_r_add = 0, int gate_full = 0, int gate_max_groups = 0, const void* rope_fusion = nullptr);
int rope_quantize_device(const void* keys, const int64_t strides[4], const void* cosv, const void* sinv,
                         const int64_t cs_strides[2], void* keys_out, const int64_t out_key_strides[4], int B, int Nk,
                         int L, int Lq, int hd, int G, int rbits, int tbits, int dtype, unsigned flags, uint8_t* codes,
                         void* rscale, void* rmn, void* tscale, void* tmn, const int64_t* out_strides,
                         cudaStream_t stream);
int lengths_advance_device(int* lengths, int full, int G, cudaStream_t stream);
int cache_append_device(const void* k_new, const void* v_new, const int64_t* in_strides, void* k_res,
                        const int64_t* kres_strides, void* values, const int64_t* v_strides, int B, int Nk, int hd,
                        int res_pos, int ctx_pos, int dtype, const int* lengths, int G, int values_window,
                        int res_cap, int value_cap, cudaStream_t stream);
size_t decode_workspace_bytes_dyn(int B, int N, int Nk, int num_ctas);
int rope_append_device(const void* qkv, int64_t qkv_stride_b, const void* cosv, const void* sinv, int64_t cs_stride_b,
                       void* q_out, void* k_res, const int64_t* kres_strides, void* values, const int64_t* v_strides,
                       int B, int N, int Nk, int hd, int G, const int* lengths, int values_window, int res_cap,
                       int value_cap, int res_pos, int ctx_pos, int dtype, cudaStream_t stream);
int selftest_quantizer_device(int dtype, int which, unsigned long long* mismatches_dev, cudaStream_t stream);
int keys_repack_device(const uint8_t* codes_in, uint8_t* codes_out, int64_t steps, int to_format,
                       cudaStream_t stream);
int key_range_check_device(const void* rscale, const void* rmn, int64_t count, int rbits, int dtype,
                           unsigned* flag_dev, cudaStream_t stream);
int qk_decode_device(const void* q, int64_t q_sb, int64_t q_sh, const uint8_t* codes, const void* rscale,
                     const void* rmn, const void* tscale, const void* tmn, float* out, int B, int N, int Nk,
                     int Nb, int G, int D, int rbits, int tbits, int dtype, cudaStream_t stream);
size_t decode_workspace_bytes(int B, int N, int Nk, int Nb, int G, int R, int num_ctas);
int decode_attention_device(const pq_decode_params* p, cudaStream_t stream);
int decode_attention_static_device(const pq_decode_params* p, cudaStream_t stream);
size_t decode_static_scratch_bytes();
int quantize_values_device(const void* values, const int64_t strides[4], int B, int Nk, int T, int hd, int vbits,
                           int dtype, int layout, void* codes, void* scale, void* mn, const int64_t* out_strides,
                           cudaStream_t stream, const int* gate_lengths = nullptr, int gate_r_add = 0,
                           int gate_full = 0, int gate_G = 0, int gate_max_tokens = 0);
int values_relayout_device(const void* codes_in, void* codes_out, int64_t tokens, int to_layout, cudaStream_t stream);
int values_matmul_device(const void* probs, const void* codes, const void* scale, const void* mn, void* out,
                         int64_t BH, int M, int T, int hd, int vbits, int dtype, cudaStream_t stream);
int merge_lse_device(const float* outs, const float* lses, int P, int64_t rows, int hd, void* out, int out_dtype,
                     float* lse_out, cudaStream_t stream);
int merge_lse_strided_device(const float* outs, int64_t out_part_stride, const float* lses, int64_t lse_part_stride,
                             int P, int64_t rows, int hd, void* out, int out_dtype, float* lse_out,
                             cudaStream_t stream);

namespace {
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
// carve a 256-byte aligned block out of a staging area
struct Carver {
  char* base; size_t off = 0;
  explicit Carver(void* b) : base(static_cast<char*>(b)) {}
  void* take(size_t bytes) { void* p = base ? base + off : nullptr; off += align_up(bytes, 256); return p; }
};
}  // namespace
}  // namespace pq

using namespace pq;

extern "C" {

int pq_abi_version(void) { return 8; }
size_t pq_decode_params_size(void) { return sizeof(pq_decode_params); }
int pq_last_cuda_error(void) { return last_cuda_error(); }

const char* pq_strerror(int status) {
  switch (status) {
    case PQ_OK: return "ok";
    case PQ_ERR_INVALID: return "invalid argument (shape, null pointer, or rbits + tbits > 8)";
    case PQ_ERR_UNSUPPORTED: return "configuration not built into this library (head_dim must be 128, group a multiple of 16, 1 <= tbits <= 4)";
    case PQ_ERR_WORKSPACE: return "workspace missing or smaller than pq_decode_workspace_bytes()";
    case PQ_ERR_CUDA: return "a CUDA runtime call failed (pq_last_cuda_error() has the code)";
    case PQ_ERR_ALIGNMENT: return "pointer or stride is not aligned for vector loads";
    case PQ_ERR_SCRATCH_LIMIT: return "problem needs more scratch than the built-in 16 MiB array of pq_decode_attention_static; use pq_decode_attention with a caller-provided workspace";
    default: return "unknown status";
  }
}

int pq_quantize(const void* keys, const int64_t strides[4], int B, int Nk, int L, int hd, int G, int rbits,
                int tbits, int dtype, unsigned flags, uint8_t* codes, void* rscale, void* rmn, void* tscale,
                void* tmn, void* stream) {
  return quantize_device(keys, strides, B, Nk, L, hd, G, rbits, tbits, dtype, flags, codes, rscale, rmn, tscale,
                         tmn, nullptr, static_cast<cudaStream_t>(stream));
}

int pq_quantize_into(const void* keys, const int64_t strides[4], int B, int Nk, int L, int hd, int G, int rbits,
                     int tbits, int dtype, unsigned flags, uint8_t* codes, void* rscale, void* rmn, void* tscale,
                     void* tmn, const int64_t out_strides[4], void* stream) {
  if (!out_strides) return PQ_ERR_INVALID;
  return quantize_device(keys, strides, B, Nk, L, hd, G, rbits, tbits, dtype, flags, codes, rscale, rmn, tscale,
                         tmn, out_strides, static_cast<cudaStream_t>(stream));
}

int pq_quantize_into_dyn(const void* keys, const int64_t strides[4], int B, int Nk, int L, int hd, int G, int rbits,
                         int tbits, int dtype, unsigned flags, uint8_t* codes, void* rscale, void* rmn, void* tscale,
                         void* tmn, const int64_t out_strides[4], int max_groups, const int* lengths, int r_add,
                         void* stream) {
  if (!out_strides || !lengths) return PQ_ERR_INVALID;
  return quantize_device(keys, strides, B, Nk, L, hd, G, rbits, tbits, dtype, flags, codes, rscale, rmn, tscale,
                         tmn, out_strides, static_cast<cudaStream_t>(stream), lengths, r_add, L, max_groups);
}

int pq_quantize_values_dyn(const void* values, const int64_t strides[4], int B, int Nk, int T, int hd, int vbits,
                           int dtype, int layout, void* codes, void* scale, void* mn, const int64_t out_strides[4],
                           int G, int max_tokens, const int* lengths, int r_add, void* stream) {
  if (!out_strides || !lengths) return PQ_ERR_INVALID;
  return quantize_values_device(values, strides, B, Nk, T, hd, vbits, dtype, layout, codes, scale, mn, out_strides,
                                static_cast<cudaStream_t>(stream), lengths, r_add, T, G, max_tokens);
}

int pq_lengths_advance(int* lengths, int full, int G, void* stream) {
  return lengths_advance_device(lengths, full, G, static_cast<cudaStream_t>(stream));
}

int pq_cache_append(const void* k_new, const void* v_new, const int64_t in_strides[4], void* k_res,
                    const int64_t kres_strides[3], void* values, const int64_t v_strides[3], int B, int Nk, int hd,
                    int res_pos, int ctx_pos, int dtype, void* stream) {
  return cache_append_device(k_new, v_new, in_strides, k_res, kres_strides, values, v_strides, B, Nk, hd, res_pos,
                             ctx_pos, dtype, nullptr, 0, 0, 0, 0, static_cast<cudaStream_t>(stream));
}

int pq_cache_append_dyn(const void* k_new, const void* v_new, const int64_t in_strides[4], void* k_res,
                        const int64_t kres_strides[3], void* values, const int64_t v_strides[3], int B, int Nk,
                        int hd, int G, const int* lengths, int values_window, int res_cap, int value_cap, int dtype,
                        void* stream) {
  if (!lengths) return PQ_ERR_INVALID;
  return cache_append_device(k_new, v_new, in_strides, k_res, kres_strides, values, v_strides, B, Nk, hd, 0, 0,
                             dtype, lengths, G, values_window, res_cap, value_cap, static_cast<cudaStream_t>(stream));
}

int pq_rope_append(const void* qkv, int64_t qkv_stride_b, const void* cos, const void* sin, int64_t cs_stride_b,
                   void* q_out, void* k_res, const int64_t kres_strides[3], void* values, const int64_t v_strides[3],
                   int B, int N, int Nk, int hd, int G, const int* lengths, int values_window, int res_cap,
                   int value_cap, int res_pos, int ctx_pos, int dtype, void* stream) {
  return rope_append_device(qkv, qkv_stride_b, cos, sin, cs_stride_b, q_out, k_res, kres_strides, values, v_strides,
                            B, N, Nk, hd, G, lengths, values_window, res_cap, value_cap, res_pos, ctx_pos, dtype,
                            static_cast<cudaStream_t>(stream));
}

int pq_merge_lse_strided(const float* outs, int64_t out_part_stride, const float* lses, int64_t lse_part_stride, int P,
                         int64_t rows, int hd, void* out, int out_dtype, float* lse_out, void* stream) {
  return merge_lse_strided_device(outs, out_part_stride, lses, lse_part_stride, P, rows, hd, out, out_dtype, lse_out,
                                  static_cast<cudaStream_t>(stream));
}

int pq_rope_quantize(const void* keys, const int64_t strides[4], const void* cos, const void* sin,
                     const int64_t cs_strides[2], void* keys_out, const int64_t out_key_strides[4], int B, int Nk, int L,
                     int Lq, int hd, int G, int rbits, int tbits, int dtype, unsigned flags, uint8_t* codes, void* rscale,
                     void* rmn, void* tscale, void* tmn, const int64_t* out_strides, void* stream) {
  return rope_quantize_device(keys, strides, cos, sin, cs_strides, keys_out, out_key_strides, B, Nk, L, Lq, hd, G, rbits,
                              tbits, dtype, flags, codes, rscale, rmn, tscale, tmn, out_strides,
                              static_cast<cudaStream_t>(stream));
}

int pq_keys_repack(const uint8_t* codes_in, uint8_t* codes_out, int64_t steps, int to_format, void* stream) {
  return keys_repack_device(codes_in, codes_out, steps, to_format, static_cast<cudaStream_t>(stream));
}

int pq_key_range_check(const void* rscale, const void* rmn, int64_t count, int rbits, int dtype, unsigned* flag_dev,
                       void* stream) {
  return key_range_check_device(rscale, rmn, count, rbits, dtype, flag_dev, static_cast<cudaStream_t>(stream));
}

int pq_selftest_quantizer(int dtype, int which, unsigned long long* mismatches_dev, void* stream) {
  return selftest_quantizer_device(dtype, which, mismatches_dev, static_cast<cudaStream_t>(stream));
}

int pq_qk_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h, const uint8_t* codes, const void* rscale,
                 const void* rmn, const void* tscale, const void* tmn, float* out, int B, int N, int Nk, int Nb,
                 int G, int D, int rbits, int tbits, int dtype, void* stream) {
  return qk_decode_device(q, q_stride_b, q_stride_h, codes, rscale, rmn, tscale, tmn, out, B, N, Nk, Nb, G, D,
                          rbits, tbits, dtype, static_cast<cudaStream_t>(stream));
}

size_t pq_decode_workspace_bytes(int B, int N, int Nk, int Nb, int G, int R, int num_ctas) {
  return decode_workspace_bytes(B, N, Nk, Nb, G, R, num_ctas);
}
size_t pq_decode_workspace_bytes_dyn(int B, int N, int Nk, int num_ctas) {
  return decode_workspace_bytes_dyn(B, N, Nk, num_ctas);
}

int pq_decode_attention(const pq_decode_params* p, void* stream) {
  return decode_attention_device(p, static_cast<cudaStream_t>(stream));
}

int pq_decode_attention_static(const pq_decode_params* p, void* stream) {
  return decode_attention_static_device(p, static_cast<cudaStream_t>(stream));
}
size_t pq_decode_static_scratch_bytes(void) { return decode_static_scratch_bytes(); }

int pq_quantize_values(const void* values, const int64_t strides[4], int B, int Nk, int T, int hd, int vbits,
                       int dtype, int layout, void* codes, void* scale, void* mn, const int64_t* out_strides,
                       void* stream) {
  return quantize_values_device(values, strides, B, Nk, T, hd, vbits, dtype, layout, codes, scale, mn, out_strides,
                                static_cast<cudaStream_t>(stream));
}
int pq_values_relayout(const void* codes_in, void* codes_out, int64_t tokens, int to_layout, void* stream) {
  return values_relayout_device(codes_in, codes_out, tokens, to_layout, static_cast<cudaStream_t>(stream));
}
int pq_values_matmul(const void* probs, const void* codes, const void* scale, const void* mn, void* out, int64_t BH,
                     int M, int T, int hd, int vbits, int dtype, void* stream) {
  return values_matmul_device(probs, codes, scale, mn, out, BH, M, T, hd, vbits, dtype,
                              static_cast<cudaStream_t>(stream));
}

int pq_merge_lse(const float* outs, const float* lses, int P, int64_t rows, int hd, void* out, int out_dtype,
                 float* lse_out, void* stream) {
  return merge_lse_device(outs, lses, P, rows, hd, out, out_dtype, lse_out, static_cast<cudaStream_t>(stream));
}

int pq_event_create(void** event) {
  if (!event) return PQ_ERR_INVALID;
  cudaEvent_t e;
  PQ_CUDA_TRY(cudaEventCreate(&e));
  *event = e;
  return PQ_OK;
}
int pq_event_destroy(void* event) {
  if (!event) return PQ_OK;
  PQ_CUDA_TRY(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
  return PQ_OK;
}
int pq_event_record(void* event, void* stream) {
  if (!event) return PQ_ERR_INVALID;
  PQ_CUDA_TRY(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
  return PQ_OK;
}
int pq_event_elapsed_ms(void* start, void* end, float* ms) {
  if (!start || !end || !ms) return PQ_ERR_INVALID;
  PQ_CUDA_TRY(cudaEventSynchronize(static_cast<cudaEvent_t>(end)));
  PQ_CUDA_TRY(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(end)));
  return PQ_OK;
}

// ----------------------------- host-buffer forms -----------------------------

size_t pq_quantize_host_staging_bytes(int B, int Nk, int L, int hd, int G, int dtype) {
  if (B <= 0 || Nk <= 0 || L <= 0 || hd <= 0 || G <= 0 || !dtype_ok(dtype)) return 0;
  const size_t es = dtype_bytes(dtype);
  const size_t tokens = static_cast<size_t>(B) * Nk * L;
  const size_t scale = static_cast<size_t>(B) * Nk * (L / G) * (hd / 2) * es;
  return align_up(tokens * hd * es, 256) + align_up(tokens * (hd / 2), 256) + 4 * align_up(scale, 256);
}

int pq_quantize_host(const void* keys_host, int B, int Nk, int L, int hd, int G, int rbits, int tbits, int dtype,
                     unsigned flags, uint8_t* codes_host, void* rscale_host, void* rmn_host, void* tscale_host,
                     void* tmn_host, void* staging, size_t staging_bytes, void* stream) {
  if (B <= 0 || Nk <= 0 || L <= 0 || G <= 0 || L % G != 0 || !dtype_ok(dtype)) return PQ_ERR_INVALID;
  if (!keys_host || !codes_host || !rscale_host || !rmn_host || !tscale_host || !tmn_host) return PQ_ERR_INVALID;
  if (!staging || staging_bytes < pq_quantize_host_staging_bytes(B, Nk, L, hd, G, dtype)) return PQ_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t es = dtype_bytes(dtype);
  const size_t tokens = static_cast<size_t>(B) * Nk * L;
  const size_t kbytes = tokens * hd * es, cbytes = tokens * (hd / 2);
  const size_t sbytes = static_cast<size_t>(B) * Nk * (L / G) * (hd / 2) * es;
  Carver c(staging);
  void* d_keys = c.take(kbytes);
  uint8_t* d_codes = static_cast<uint8_t*>(c.take(cbytes));
  void* d_rs = c.take(sbytes); void* d_rm = c.take(sbytes); void* d_ts = c.take(sbytes); void* d_tm = c.take(sbytes);
  PQ_CUDA_TRY(cudaMemcpyAsync(d_keys, keys_host, kbytes, cudaMemcpyHostToDevice, s));
  const int64_t st[4] = {static_cast<int64_t>(Nk) * L * hd, static_cast<int64_t>(L) * hd, hd, 1};
  int rc = quantize_device(d_keys, st, B, Nk, L, hd, G, rbits, tbits, dtype, flags, d_codes, d_rs, d_rm, d_ts, d_tm, nullptr, s);
  if (rc != PQ_OK) return rc;
  PQ_CUDA_TRY(cudaMemcpyAsync(codes_host, d_codes, cbytes, cudaMemcpyDeviceToHost, s));
  PQ_CUDA_TRY(cudaMemcpyAsync(rscale_host, d_rs, sbytes, cudaMemcpyDeviceToHost, s));
  PQ_CUDA_TRY(cudaMemcpyAsync(rmn_host, d_rm, sbytes, cudaMemcpyDeviceToHost, s));
  PQ_CUDA_TRY(cudaMemcpyAsync(tscale_host, d_ts, sbytes, cudaMemcpyDeviceToHost, s));
  PQ_CUDA_TRY(cudaMemcpyAsync(tmn_host, d_tm, sbytes, cudaMemcpyDeviceToHost, s));
  return PQ_OK;
}

size_t pq_decode_host_staging_bytes(int B, int N, int Nk, int Nb, int G, int R, int hd, int qk_dtype, int v_dtype,
                                    int out_dtype, int has_mask) {
  if (B <= 0 || N <= 0 || Nk <= 0 || Nb < 0 || G <= 0 || R < 0 || hd <= 0) return 0;
  if (!dtype_ok(qk_dtype) || !dtype_ok(v_dtype) || !dtype_ok(out_dtype)) return 0;
  const size_t qe = dtype_bytes(qk_dtype), ve = dtype_bytes(v_dtype), oe = dtype_bytes(out_dtype);
  const size_t units = static_cast<size_t>(B) * Nk, ctx = static_cast<size_t>(Nb) * G + R;
  size_t total = 0;
  total += align_up(static_cast<size_t>(B) * N * hd * qe, 256);          // q
  total += align_up(units * Nb * G * (hd / 2), 256);                     // codes
  total += 4 * align_up(units * Nb * (hd / 2) * qe, 256);                // scales
  total += align_up(units * R * hd * qe, 256);                           // residual keys
  total += align_up(units * ctx * hd * ve, 256);                         // values
  if (has_mask) total += align_up(static_cast<size_t>(B) * ctx, 256);
  total += align_up(static_cast<size_t>(B) * N * hd * oe, 256);          // out
  total += align_up(static_cast<size_t>(B) * N * sizeof(float), 256);    // lse
  total += align_up(decode_workspace_bytes(B, N, Nk, Nb, G, R, 0), 256);
  return total;
}

int pq_decode_attention_host(const pq_decode_params* hp, void* staging, size_t staging_bytes, void* stream) {
  if (!hp) return PQ_ERR_INVALID;
  const int B = hp->B, N = hp->N, Nk = hp->Nk, Nb = hp->Nb, G = hp->G, R = hp->R, hd = hp->hd;
  if (B <= 0 || N <= 0 || Nk <= 0 || Nb < 0 || G <= 0 || R < 0 || hd <= 0) return PQ_ERR_INVALID;
  if (!dtype_ok(hp->qk_dtype) || !dtype_ok(hp->v_dtype) || !dtype_ok(hp->out_dtype)) return PQ_ERR_INVALID;
  const size_t need = pq_decode_host_staging_bytes(B, N, Nk, Nb, G, R, hd, hp->qk_dtype, hp->v_dtype,
                                                   hp->out_dtype, hp->mask != nullptr);
  if (!staging || staging_bytes < need) return PQ_ERR_WORKSPACE;
  if (!hp->q || !hp->v || !hp->out) return PQ_ERR_INVALID;
  if (hp->vbits != 0 || hp->dyn_lengths) return PQ_ERR_UNSUPPORTED;   // packed values, device-side lengths: resident caches only
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t qe = dtype_bytes(hp->qk_dtype), ve = dtype_bytes(hp->v_dtype), oe = dtype_bytes(hp->out_dtype);
  const size_t units = static_cast<size_t>(B) * Nk, ctx = static_cast<size_t>(Nb) * G + R;
  const size_t q_b = static_cast<size_t>(B) * N * hd * qe, c_b = units * Nb * G * (hd / 2);
  const size_t s_b = units * Nb * (hd / 2) * qe, kr_b = units * R * hd * qe, v_b = units * ctx * hd * ve;
  const size_t m_b = static_cast<size_t>(B) * ctx, o_b = static_cast<size_t>(B) * N * hd * oe;
  const size_t l_b = static_cast<size_t>(B) * N * sizeof(float);

  Carver c(staging);
  pq_decode_params d = *hp;
  void* dq = c.take(q_b); void* dc = c.take(c_b);
  void* drs = c.take(s_b); void* drm = c.take(s_b); void* dts = c.take(s_b); void* dtm = c.take(s_b);
  void* dkr = c.take(kr_b); void* dv = c.take(v_b);
  void* dm = hp->mask ? c.take(m_b) : nullptr;
  void* dout = c.take(o_b); void* dl = c.take(l_b);
  d.workspace_bytes = decode_workspace_bytes(B, N, Nk, Nb, G, R, 0);
  d.workspace = c.take(d.workspace_bytes);
  d.num_ctas = 0;
  d.mid_event = nullptr;
  d.exchange_bufs = nullptr; d.exchange_world = 0; d.exchange_rank = 0;      // device-buffer feature only
  d.exchange_out = nullptr; d.exchange_lse_out = nullptr;

  PQ_CUDA_TRY(cudaMemcpyAsync(dq, hp->q, q_b, cudaMemcpyHostToDevice, s));
  if (Nb > 0) {
    if (!hp->codes || !hp->rscale || !hp->rmn || !hp->tscale || !hp->tmn) return PQ_ERR_INVALID;
    PQ_CUDA_TRY(cudaMemcpyAsync(dc, hp->codes, c_b, cudaMemcpyHostToDevice, s));
    PQ_CUDA_TRY(cudaMemcpyAsync(drs, hp->rscale, s_b, cudaMemcpyHostToDevice, s));
    PQ_CUDA_TRY(cudaMemcpyAsync(drm, hp->rmn, s_b, cudaMemcpyHostToDevice, s));
    PQ_CUDA_TRY(cudaMemcpyAsync(dts, hp->tscale, s_b, cudaMemcpyHostToDevice, s));
    PQ_CUDA_TRY(cudaMemcpyAsync(dtm, hp->tmn, s_b, cudaMemcpyHostToDevice, s));
  }
  if (R > 0) {
    if (!hp->k_res) return PQ_ERR_INVALID;
    PQ_CUDA_TRY(cudaMemcpyAsync(dkr, hp->k_res, kr_b, cudaMemcpyHostToDevice, s));
  }
  PQ_CUDA_TRY(cudaMemcpyAsync(dv, hp->v, v_b, cudaMemcpyHostToDevice, s));
  if (hp->mask) PQ_CUDA_TRY(cudaMemcpyAsync(dm, hp->mask, m_b, cudaMemcpyHostToDevice, s));

  d.q = dq; d.q_stride_b = static_cast<int64_t>(N) * hd; d.q_stride_h = hd;
  d.codes = static_cast<const uint8_t*>(dc);
  d.codes_stride_h = static_cast<int64_t>(Nb) * G * (hd / 2); d.codes_stride_b = d.codes_stride_h * Nk;
  d.rscale = drs; d.rmn = drm; d.tscale = dts; d.tmn = dtm;
  d.scale_stride_h = static_cast<int64_t>(Nb) * (hd / 2); d.scale_stride_b = d.scale_stride_h * Nk;
  d.k_res = dkr; d.kres_stride_t = hd; d.kres_stride_h = static_cast<int64_t>(R) * hd; d.kres_stride_b = d.kres_stride_h * Nk;
  d.v = dv; d.v_stride_t = hd; d.v_stride_h = static_cast<int64_t>(ctx) * hd; d.v_stride_b = d.v_stride_h * Nk;
  d.mask = static_cast<const uint8_t*>(dm); d.mask_stride_b = static_cast<int64_t>(ctx);
  d.out = dout; d.out_stride_b = static_cast<int64_t>(N) * hd; d.out_stride_h = hd;
  d.lse = hp->lse ? static_cast<float*>(dl) : nullptr;
  int rc = decode_attention_device(&d, s);
  if (rc != PQ_OK) return rc;
  PQ_CUDA_TRY(cudaMemcpyAsync(hp->out, dout, o_b, cudaMemcpyDeviceToHost, s));
  if (hp->lse) PQ_CUDA_TRY(cudaMemcpyAsync(hp->lse, dl, l_b, cudaMemcpyDeviceToHost, s));
  return PQ_OK;
}

}  // extern "C"
