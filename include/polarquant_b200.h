/*
 * polarquant_b200 - C ABI of the B200 (sm_100a) polar key-cache hot path.
 *
 * Every entry point takes raw device pointers (unless its name ends in _host),
 * explicit sizes and strides, and a CUDA stream handle (cudaStream_t passed as
 * void*).  Work is enqueued on that stream and the call returns without
 * synchronising.  The library owns no memory: outputs and scratch are the
 * caller's (one exception: the peer-mappable exchange buffer of pq_peer_alloc,
 * freed by pq_peer_free).  Return value: PQ_OK (0) or a negative pq_status; nothing throws or
 * aborts.  Strides are in ELEMENTS of the tensor's dtype.
 *
 * The reference project (ericshwu/PolarQuant) is Python; the interface each
 * function stands behind is cited as file:line of that project.
 */
#ifndef POLARQUANT_B200_H
#define POLARQUANT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { PQ_F16 = 0, PQ_BF16 = 1, PQ_F32 = 2 } pq_dtype;

typedef enum {
  PQ_OK = 0,
  PQ_ERR_INVALID = -1,     /* bad shape, null pointer, rbits + tbits > 8, ...   */
  PQ_ERR_UNSUPPORTED = -2, /* valid for the reference, not built into this lib  */
  PQ_ERR_WORKSPACE = -3,   /* scratch buffer missing or too small               */
  PQ_ERR_CUDA = -4,        /* a CUDA runtime call failed (see pq_last_cuda_error) */
  PQ_ERR_ALIGNMENT = -5,   /* a pointer or stride breaks a 16-byte requirement  */
  PQ_ERR_SCRATCH_LIMIT = -6 /* problem needs more scratch than the built-in array of pq_decode_attention_static holds */
} pq_status;

/* pq_quantize flag bits */
#define PQ_QUANT_WRAP_DTYPE 1u /* add RN_dtype(2*pi) to negative angles (what torch does on CPU) \
                                  instead of float32(2*pi) (what torch does on CUDA, the default) */
#define PQ_QUANT_NORM_FMA 2u /* fp32 keys only: radius^2 = fma(y, y, RN(x*x)) instead of RN(x*x) + RN(y*y), the \
                                 form torch evaluates on both CPU and CUDA (for 16-bit keys the two coincide) */
#define PQ_QUANT_PACK6 4u /* write the codes in the 48-byte-per-token PQ_KEYS_PACKED6 container (see pq_keys_repack) \
                             instead of one byte per pair; needs rbits + tbits == 6 and G % 16 == 0 */

/*
 * Polar key quantizer.  Replaces the method quantize_and_pack_nbit
 * (models/modeling_llama_polar.py:135-157, models/modeling_qwen_polar.py:134-156).
 *
 * keys: (B, Nk, L, hd) of `dtype`, strides[4] in elements with strides[3] == 1;
 * pair d is channels (d, d + hd/2).  L % G == 0, rbits + tbits <= 8, hd == 128.
 * Outputs are contiguous: codes (B, Nk, L/G, G, hd/2) uint8 with
 * code = (rho << tbits) + theta; rscale, rmn, tscale, tmn (B, Nk, L/G, 1, hd/2)
 * of `dtype`.  Bit-exact with the reference ops executed by torch on CUDA.
 */
int pq_quantize(const void* keys, const int64_t strides[4], int B, int Nk, int L, int hd, int G,
                int rbits, int tbits, int dtype, unsigned flags,
                uint8_t* codes, void* rscale, void* rmn, void* tscale, void* tmn, void* stream);

/*
 * pq_quantize writing into a preallocated cache: the outputs of (batch b, kv head h) start at
 * b * out_strides[0] + h * out_strides[1] bytes (codes) and b * out_strides[2] + h * out_strides[3] elements
 * (each scale tensor); within a (b, h) unit the L/G groups are contiguous as in pq_quantize.  Pass pointers to
 * the first group to be written.  This is how an in-place cache appends a freshly quantised group without the
 * torch.cat of the reference's decode branch (models/modeling_llama_polar.py:84-90).
 */
int pq_quantize_into(const void* keys, const int64_t strides[4], int B, int Nk, int L, int hd, int G,
                     int rbits, int tbits, int dtype, unsigned flags,
                     uint8_t* codes, void* rscale, void* rmn, void* tscale, void* tmn,
                     const int64_t out_strides[4], void* stream);

/*
 * Append the current token to an in-place cache: for every (batch, kv head) copy the key row k_new[b, h, :] into
 * slot res_pos of the residual window k_res (B, Nk, RL, hd) and the value row v_new[b, h, :] into slot ctx_pos of
 * the value buffer (B, Nk, max_tokens, hd).  in_strides = {k_new stride_b, stride_h, v_new stride_b, stride_h},
 * kres_strides / v_strides = {stride_b, stride_h, stride_token}, all in elements.  Replaces the two torch.cat
 * calls of the reference's decode branch (models/modeling_llama_polar.py:77,98).
 */
int pq_cache_append(const void* k_new, const void* v_new, const int64_t in_strides[4], void* k_res,
                    const int64_t kres_strides[3], void* values, const int64_t v_strides[3], int B, int Nk, int hd,
                    int res_pos, int ctx_pos, int dtype, void* stream);
/*
 * The same with the positions read on the device from lengths = {token groups, residual tokens} (see
 * pq_decode_params.dyn_lengths): key slot lengths[1]; value slot lengths[1] when `values` is only the residual
 * window (values_window != 0, packed-value caches), else lengths[0] * G + lengths[1].  Slots at or beyond res_cap /
 * value_cap tokens are not written.  The lengths are not modified: advance lengths[1] once per step, after the
 * attention calls of all layers that share the array.
 */
int pq_cache_append_dyn(const void* k_new, const void* v_new, const int64_t in_strides[4], void* k_res,
                        const int64_t kres_strides[3], void* values, const int64_t v_strides[3], int B, int Nk,
                        int hd, int G, const int* lengths, int values_window, int res_cap, int value_cap, int dtype,
                        void* stream);

/*
 * Re-quantisation of a full residual window with everything decided on the device, so that it can sit inside a
 * replayed CUDA graph: same arguments as pq_quantize_into / pq_quantize_values (L = T = the window length, pass the
 * BASE pointers of the cache buffers, out_strides required), plus lengths = {token groups, residual tokens}.  The
 * kernels do nothing unless lengths[1] + r_add equals the window length, and then write groups lengths[0]..
 * (tokens lengths[0] * G ..) of every (b, h) unit; max_groups / max_tokens bound what a unit can hold (beyond that
 * nothing is written).  pq_lengths_advance is the matching bookkeeping step: residual + 1, or - when that fills the
 * window - groups += full / G and residual = 0.  Replaces the `% self.residual_length == 0` branches of the
 * reference's decode step (models/modeling_llama_polar.py:83-92, 240-248) for a device-driven loop.
 */
int pq_quantize_into_dyn(const void* keys, const int64_t strides[4], int B, int Nk, int L, int hd, int G, int rbits,
                         int tbits, int dtype, unsigned flags, uint8_t* codes, void* rscale, void* rmn, void* tscale,
                         void* tmn, const int64_t out_strides[4], int max_groups, const int* lengths, int r_add,
                         void* stream);
int pq_quantize_values_dyn(const void* values, const int64_t strides[4], int B, int Nk, int T, int hd, int vbits,
                           int dtype, int layout, void* codes, void* scale, void* mn, const int64_t out_strides[4],
                           int G, int max_tokens, const int* lengths, int r_add, void* stream);
int pq_lengths_advance(int* lengths, int full, int G, void* stream);

/*
 * Rotary embedding of one decode token fused with the cache append.  qkv (B, (N + 2 Nk) * hd) is the fused
 * projection output of the step, [query heads | key heads | value heads], row stride qkv_stride_b elements; cos /
 * sin hold hd elements of `dtype` per sequence (cs_stride_b elements apart, 0 = shared).  Query heads are rotated
 * into q_out (B, N, hd) contiguous, key heads are rotated into slot res_pos of k_res, value heads are copied into
 * slot ctx_pos of `values`; with `lengths` the slots come from the device as in pq_cache_append_dyn (res_pos and
 * ctx_pos are then ignored).  Arithmetic: out = RN(RN(x * cos) + RN(rotate_half(x) * sin)), the eager ops of
 * apply_rotary_pos_emb as called at models/modeling_llama_polar.py:57, rounded where they round.  Replaces that
 * call plus the torch.cat appends at :77,98 for the decode step.
 */
int pq_rope_append(const void* qkv, int64_t qkv_stride_b, const void* cos, const void* sin, int64_t cs_stride_b,
                   void* q_out, void* k_res, const int64_t kres_strides[3], void* values, const int64_t v_strides[3],
                   int B, int N, int Nk, int hd, int G, const int* lengths, int values_window, int res_cap,
                   int value_cap, int res_pos, int ctx_pos, int dtype, void* stream);

/*
 * Prefill-side fusion: rotary embedding of the prompt's keys and their polar quantisation in one pass over the keys.
 * In the reference the prefill rotates the keys (apply_rotary_pos_emb, models/modeling_llama_polar.py:57), runs the
 * attention on them and then quantises all but the last L % 128 of them (:116-126): the rotated keys are written
 * once and read again by the quantizer.  Here keys (B, Nk, L, hd) arrive UN-rotated (element strides[4], inner 1 -
 * typically the (B, L, Nk, hd) projection output), cos / sin hold hd elements of `dtype` per position, element
 * strides cs_strides = {batch (0 = shared by all sequences), position}; the rotated keys
 * RN(RN(x * cos) + RN(rotate_half(x) * sin)) - every product and the sum rounded to `dtype` as the eager ops round
 * them - are written to keys_out (element strides out_key_strides[4]; may be the input buffer itself; NULL only when
 * Lq == L) and the first Lq tokens (a multiple of G) are quantised from registers exactly as pq_quantize[_into]
 * quantises the rotated keys: codes and scales are bit-identical to quantising keys_out.  Tokens [Lq, L) are rotated
 * only.  out_strides as in pq_quantize_into, or NULL for dense outputs of the Lq tokens.  16-bit dtypes, hd == 128,
 * G a multiple of 16 up to 128; PQ_QUANT_PACK6 is honoured.
 */
int pq_rope_quantize(const void* keys, const int64_t strides[4], const void* cos, const void* sin,
                     const int64_t cs_strides[2], void* keys_out, const int64_t out_key_strides[4], int B, int Nk, int L,
                     int Lq, int hd, int G, int rbits, int tbits, int dtype, unsigned flags, uint8_t* codes, void* rscale,
                     void* rmn, void* tscale, void* tmn, const int64_t* out_strides, void* stream);

/*
 * Self-test of the quantizer's fast paths (no reference counterpart).  The kernel replaces atan2f, sqrtf and the
 * IEEE division by cheaper approximations wherever the approximation provably rounds to the same 16-bit value,
 * and calls the exact routine otherwise.  This entry point checks that claim exhaustively on the device: for all
 * 2^32 pairs of 16-bit patterns of `dtype` (PQ_F16 or PQ_BF16) it compares the fast-path result with the
 * exact-only result - which = 0: angle and radius of the key pair (x, y), its mirror image and both with the first
 * channel negated; which = 1: quantisation level of the rounded difference x with step y; which = 2: the packed
 * 16-bit subtraction x - y against the fp32 subtraction rounded to `dtype` - and writes the number of disagreeing
 * cases to *mismatches_dev (device memory, 8 bytes).
 */
int pq_selftest_quantizer(int dtype, int which, unsigned long long* mismatches_dev, void* stream);

/*
 * Un-scaled fp32 query-key logits over the packed keys.  Replaces
 * attention_decode_forward_triton_impl and its Triton kernel
 * (models/kernel4group.py:14-109).
 *
 * q: (B, N, 2*D) of `dtype` with element strides q_stride_b / q_stride_h and unit
 * inner stride; codes (B, Nk, Nb, G, D) and the four scale tensors (B, Nk, Nb, D)
 * contiguous; out (B, N, Nb*G) fp32 contiguous.  Query head kvh*(N/Nk)+h reads
 * kv head kvh.  D == 64, G % 16 == 0, 1 <= tbits <= 4.
 *
 * Limits narrower than the reference's (which only asserts rbits + tbits <= 8,
 * models/modeling_llama_polar.py:138): bit splits with tbits > 4 (or rbits > 4) are accepted
 * by pq_quantize but refused here with PQ_ERR_UNSUPPORTED - the angle table of 64 x 2^tbits
 * entries per warp is built for at most 16 levels.  The dequantised keys are formed in fp16,
 * so every reconstructed |key channel| (at most the group's largest radius, rmn + rscale * 2^rbits)
 * must stay below 65504; bf16 keys beyond that would give inf / NaN logits, not an error.
 * pq_key_range_check tests a cache's radius scales against this bound on the device.
 */
int pq_qk_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                 const uint8_t* codes, const void* rscale, const void* rmn,
                 const void* tscale, const void* tmn, float* out,
                 int B, int N, int Nk, int Nb, int G, int D, int rbits, int tbits, int dtype,
                 void* stream);

/*
 * Sub-byte key codes (an opt-in second format; the reference keeps one byte per pair,
 * models/modeling_llama_polar.py:155, and names real packing as future work, models/kernel4group.py:1-3).
 * For the bit splits whose code has 6 bits (3/3 and 2/4) PQ_KEYS_PACKED6 stores 48 bytes per token instead of 64.
 * The format is tiled per step of 16 consecutive tokens (768 bytes), in the order a warp of the decode kernel
 * consumes it: bytes [0, 512) hold, for lane l = 4 g + t (g = 0..7, t = 0..3), the words A0, A1 of token g and A0,
 * A1 of token g + 8; bytes [512, 768) hold, per lane, the word H of token g and of token g + 8.  With c[p] the code
 * of pair 16 t + p of the token: nibble 2 i of A_k is c[8 k + i] & 15 and nibble 2 i + 1 is c[8 k + 4 + i] & 15
 * (i = 0..3, k = 0..1); bits 2 j, 2 j + 1 of H are c[4 W + E] >> 4 and bits 16 + 2 j, 17 + 2 j are
 * c[4 W + E + 2] >> 4 for j = 2 W + E (W = 0..3, E = 0..1).  Token counts are multiples of 16.
 *
 * pq_quantize / pq_quantize_into[_dyn] write it directly when PQ_QUANT_PACK6 is set in `flags` (the codes buffer
 * then takes 48 bytes per token, out_strides[0..1] in bytes of that format); pq_keys_repack converts `steps`
 * 16-token blocks between the two containers (to_format = PQ_KEYS_PACKED6 or PQ_KEYS_BYTE, out of place; code
 * bits above the sixth are dropped when packing).  Packing is lossless for 6-bit codes: unpack(pack(c)) == c, and
 * pq_decode_attention gives bit-identical results on either container.
 */
#define PQ_KEYS_BYTE 0
#define PQ_KEYS_PACKED6 1
int pq_keys_repack(const uint8_t* codes_in, uint8_t* codes_out, int64_t steps, int to_format, void* stream);

/*
 * Range check for the fp16 dequantisation of the decode kernels (no reference counterpart: the reference
 * dequantises in fp32 inside its Triton kernel, models/kernel4group.py:67-75).  rscale / rmn: `count` elements of
 * `dtype` each (any of the (B, Nk, Nb, 1, 64) tensors, contiguous).  Sets *flag_dev (device memory, 4 bytes,
 * zeroed by the caller) to 1 when some largest reconstructible radius |rmn| + |rscale| * 2^rbits is not finite or
 * reaches 65504; leaves it untouched otherwise.  Costs one pass over the scales (1/32 of the code bytes at G = 128).
 */
int pq_key_range_check(const void* rscale, const void* rmn, int64_t count, int rbits, int dtype,
                       unsigned* flag_dev, void* stream);

/*
 * Fused decode attention over the polar cache: lookup-table QK over the packed
 * keys + QK over the full-precision residual keys + scale + optional mask +
 * online softmax + P.V, split over the sequence with a log-sum-exp merge.
 * Replaces the decode branch of the patched attention forward
 * (models/modeling_llama_polar.py:61-101, models/modeling_qwen_polar.py:60-100),
 * i.e. the composition of the call at :66-75 with the eager ops at :77-99.
 * The limits stated at pq_qk_decode (tbits and rbits at most 4, reconstructed keys below
 * 65504 in magnitude) hold here too.
 */
typedef struct pq_decode_params {
  /* query (B, N, hd), dtype qk_dtype */
  const void* q;
  int64_t q_stride_b, q_stride_h;
  /* packed keys: codes (B, Nk, Nb, G, hd/2) uint8; unit (b, kvh) starts at
     b * codes_stride_b + kvh * codes_stride_h bytes and holds Nb*G*(hd/2)
     contiguous bytes.  NULL allowed when Nb == 0. */
  const uint8_t* codes;
  int64_t codes_stride_b, codes_stride_h;
  /* scales (B, Nk, Nb, hd/2), dtype qk_dtype; unit (b, kvh) starts at
     b * scale_stride_b + kvh * scale_stride_h elements, rows contiguous */
  const void* rscale;
  const void* rmn;
  const void* tscale;
  const void* tmn;
  int64_t scale_stride_b, scale_stride_h;
  /* full-precision residual keys (B, Nk, R, hd), dtype qk_dtype, including the
     current token.  NULL allowed when R == 0. */
  const void* k_res;
  int64_t kres_stride_b, kres_stride_h, kres_stride_t;
  /* values (B, Nk, Nb*G + R, hd), dtype v_dtype (PQ_F16 or PQ_BF16); with vbits == 4 only the last R tokens */
  const void* v;
  int64_t v_stride_b, v_stride_h, v_stride_t;
  /* optional key mask (B, Nb*G + R) uint8, 1 = attend, 0 = masked; NULL = none */
  const uint8_t* mask;
  int64_t mask_stride_b;
  /* output (B, N, hd) of out_dtype; optional natural-log log-sum-exp (B, N) fp32 */
  void* out;
  int64_t out_stride_b, out_stride_h;
  float* lse;
  /* caller-owned scratch of at least pq_decode_workspace_bytes(...) bytes, 256-byte aligned */
  void* workspace;
  size_t workspace_bytes;
  int B, N, Nk, Nb, G, R, hd;
  int rbits, tbits;
  int qk_dtype, v_dtype, out_dtype;
  float sm_scale;  /* logits multiplier; 0 means 1/sqrt(hd) as at modeling_llama_polar.py:80 */
  int num_ctas;    /* 0 = choose from the device's SM count */
  void* mid_event; /* optional cudaEvent_t recorded between the attention kernel and the merge kernel */
  /* Optional packed values (vbits == 4; 0 = none): the values of the Nb*G packed-key tokens as 4-bit codes in
     the PQ_VALUES_TILED layout of pq_quantize_values, 64 bytes per token, tokens contiguous per (b, kvh) unit,
     unit at b * vcodes_stride_b + kvh * vcodes_stride_h BYTES; v_scale / v_mn one element of v_dtype per token,
     unit at b * vscale_stride_b + kvh * vscale_stride_h ELEMENTS (even).  `v` then holds only the R
     full-precision values of the residual window, (B, Nk, R, hd).  Requires qk_dtype == v_dtype (fp16 or bf16).
     This is the decode branch of LlamaPolarMixedGroupAttention (models/modeling_llama_polar.py:189-246). */
  const void* v_codes;
  int64_t vcodes_stride_b, vcodes_stride_h;
  const void* v_scale;
  const void* v_mn;
  int64_t vscale_stride_b, vscale_stride_h;
  int vbits;
  /* Optional device-side lengths, for replaying one captured CUDA graph over a growing cache: a device pointer
     to two ints {token groups, residual tokens}.  When set, the kernels use dyn_lengths[0] and
     dyn_lengths[1] + dyn_r_add instead of Nb and R and partition the work themselves; Nb and R then state the
     CAPACITY of the buffers (lengths beyond them are clamped), the workspace must hold
     pq_decode_workspace_bytes_dyn() bytes, and qk_dtype == v_dtype (fp16 or bf16). */
  const int* dyn_lengths;
  int dyn_r_add;
  /* Layout of `codes`: PQ_KEYS_BYTE (0, the reference's container: one byte per pair, 64 bytes per token) or
     PQ_KEYS_PACKED6 (48 bytes per token, see pq_keys_repack; rbits + tbits must be 6: 3/3 or 2/4; 16-bit caches
     with qk_dtype == v_dtype).  A unit then holds Nb * G * 48 contiguous bytes. */
  int key_format;
  /* Sequence split over peer memory (pq_exchange_merge below): with exchange_world > 0 the merge that ends this call
     also stores every result row, paired with the exchange's epoch, into the inboxes of the peers - the push of
     pq_exchange_merge done by the producer, so that the transfer is in flight before the exchange kernel starts; call
     pq_exchange_merge with PQ_EXCHANGE_PUSHED afterwards.  exchange_bufs: the `world` exchange buffers in rank order
     as this process sees them (host array, read during the call); out must be exchange_bufs[exchange_rank] (fp32,
     dense (B N, 128)), lse must be out + B * N * 128.  Zero / NULL: off. */
  void* const* exchange_bufs;
  int exchange_world;
  int exchange_rank;
  /* With exchange_out set the merge that ends this call does the whole exchange: after pushing its rows it waits
     (bounded) for the peers' rows in this rank's own buffer, merges them in rank order and writes the final result
     (B N, 128) of exchange_out_dtype to exchange_out (and its log-sum-exp to exchange_lse_out unless NULL); no
     pq_exchange_merge follows on this rank.  A rank that has no keys in a step calls pq_exchange_merge instead (after
     writing zeros / -inf to its block); the two forms interoperate. */
  void* exchange_out;
  int exchange_out_dtype;
  float* exchange_lse_out;
} pq_decode_params;

int pq_decode_attention(const pq_decode_params* p, void* stream);
/* sizeof(pq_decode_params) as this library was compiled, for bindings to verify their mirror of the struct */
size_t pq_decode_params_size(void);

/* Scratch bytes pq_decode_attention needs for this problem on the current device. */
size_t pq_decode_workspace_bytes(int B, int N, int Nk, int Nb, int G, int R, int num_ctas);
/* Scratch bytes that suffice for every length when dyn_lengths is used. */
size_t pq_decode_workspace_bytes_dyn(int B, int N, int Nk, int num_ctas);

/*
 * pq_decode_attention for callers that cannot provide scratch memory or call an allocator
 * at all (a runtime that hands out its whole device heap at start-up, a plugin host that
 * forbids allocation after initialisation).  It has no counterpart in the reference, whose
 * Python code allocates freely.  Same arguments and results as pq_decode_attention; the
 * workspace fields of `p` are ignored.  The partial results go to an array built into the
 * library image: pq_decode_static_scratch_bytes() bytes (16 MiB) of device memory, held on
 * every GPU that loads the library until the process exits.  A problem whose
 * pq_decode_workspace_bytes() exceeds that is refused with PQ_ERR_SCRATCH_LIMIT before any
 * work is enqueued.  The call itself performs no cudaMalloc / cudaFree and calls no
 * allocating library routine.
 *
 * With dyn_lengths set the array must hold the bound over every length,
 * B * Nk * ceil(N / Nk / 8) + 12 * num_ctas partial slots of 4160 bytes (4032 slots fit).  The default grid of a
 * 148-SM GPU (444 CTAs, 5328 slots) does not fit, so with num_ctas == 0 this entry point runs the largest grid
 * that does - (4032 - units) / 12 CTAs, e.g. 325 for batch 16 x 8 kv heads - and an explicit num_ctas beyond
 * that, or a problem with more than 4020 units, is refused with PQ_ERR_SCRATCH_LIMIT.
 *
 * The first call on each device looks up the array's device address (with that device
 * current) and caches it for the life of the process; make that first call outside any
 * CUDA stream capture.  The cache is keyed by device ordinal: after the host destroys the
 * device's context (cudaDeviceReset) the address is stale and this entry point must not be
 * called again in that process.
 * All calls on a device share the one array, and it keeps whatever the previous call left
 * in it.  Nothing in it has to start at zero: every slot a call reads was written earlier
 * by the same call.  Two calls whose kernels overlap in time on the same GPU (different
 * streams, or different host threads) would overwrite each other's partials: serialise them.
 */
int pq_decode_attention_static(const pq_decode_params* p, void* stream);
size_t pq_decode_static_scratch_bytes(void);

/*
 * Packed value cache (the reference's LlamaPolarMixedGroupAttention, models/modeling_llama_polar.py:160-292).
 * pq_quantize_values replaces `triton_quantize_and_pack_along_last_dim(values, 128, 4)` (:242, :285; a KIVI routine
 * the reference imports without shipping it): per token, min/max over the 128 channels, scale = (mx - mn) / 15,
 * level = round(clamp((v - mn) / scale, 0, 15)), every step rounded to `dtype` as torch on CUDA rounds it.
 * values (B, Nk, T, hd) with element strides[4], strides[3] == 1; codes 64 bytes per token; scale, mn one element
 * of `dtype` per token.  out_strides NULL: outputs contiguous, codes (B, Nk, T, 16) int32, scale / mn
 * (B, Nk, T, 1).  Otherwise unit (b, h) starts at b * out_strides[0] + h * out_strides[1] bytes (codes) and
 * b * out_strides[2] + h * out_strides[3] elements (scale, mn), tokens contiguous within a unit: pass pointers to
 * the first token to be written (in-place cache).  hd == 128, vbits == 4.
 *
 * layout PQ_VALUES_KIVI: channel c at bits 4 * (c % 8) of word c / 8 (what `cuda_bmm_fA_qB_outer` and
 * pq_values_matmul read).  PQ_VALUES_TILED: channel c at 4-bit field c / 8 of the 64-bit slot c % 8 - the order in
 * which pq_decode_attention consumes them.  pq_values_relayout converts `tokens` rows of 64 bytes between the two
 * (out of place).
 */
#define PQ_VALUES_KIVI 0
#define PQ_VALUES_TILED 1
int pq_quantize_values(const void* values, const int64_t strides[4], int B, int Nk, int T, int hd, int vbits,
                       int dtype, int layout, void* codes, void* scale, void* mn, const int64_t* out_strides,
                       void* stream);
int pq_values_relayout(const void* codes_in, void* codes_out, int64_t tokens, int to_layout, void* stream);
/*
 * out (BH, M, hd) = probs (BH, M, T) x dequantised values (BH, T, hd), all contiguous, `dtype` throughout, fp32
 * accumulation; codes in the PQ_VALUES_KIVI layout.  Replaces `cuda_bmm_fA_qB_outer(128, probs, codes, scale, mn, 4)`
 * as called at models/modeling_llama_polar.py:230-237 (the reference passes per-query-head copies: BH = B * N).
 */
int pq_values_matmul(const void* probs, const void* codes, const void* scale, const void* mn, void* out,
                     int64_t BH, int M, int T, int hd, int vbits, int dtype, void* stream);

/*
 * Merge P partial attention results over disjoint key ranges (sequence split
 * across chunks or GPUs).  outs (P, rows, hd) fp32 softmax-normalised, lses
 * (P, rows) fp32 natural log; out (rows, hd) of out_dtype, lse_out (rows) fp32 or
 * NULL.  No counterpart in the reference, which never splits the sequence.
 */
int pq_merge_lse(const float* outs, const float* lses, int P, int64_t rows, int hd,
                 void* out, int out_dtype, float* lse_out, void* stream);
/*
 * The same with explicit strides (in elements) between the parts, so that the buffer an all-gather fills - every
 * rank's [outs (rows, hd) | lses (rows)] block back to back - is merged in place: outs = buffer,
 * out_part_stride = rows * (hd + 1), lses = buffer + rows * hd, lse_part_stride = rows * (hd + 1).
 */
int pq_merge_lse_strided(const float* outs, int64_t out_part_stride, const float* lses, int64_t lse_part_stride, int P,
                         int64_t rows, int hd, void* out, int out_dtype, float* lse_out, void* stream);

/*
 * Sequence split across the GPUs of one node without a library collective: ONE kernel per step pushes this rank's
 * partial ([out (rows, hd) fp32 | lse (rows) fp32], the block pq_decode_attention writes when out / lse point into it)
 * into every peer's exchange buffer with plain peer stores over NVLink, picks up the peers' pushes from local memory
 * and merges all partials by log-sum-exp - the same arithmetic, in rank order, as pq_merge_lse_strided over an
 * all-gathered buffer (bit-identical results).  Pushed values travel paired with the step's epoch in 16-byte stores,
 * so the receiver validates every word by itself and no fence or "ready" flag sits on the critical path.  No
 * counterpart in the reference, which never splits the sequence (test4long.py:38-43 runs one replica per GPU).
 *
 * Every rank owns one exchange buffer of pq_exchange_bytes(world, rows, hd) bytes, created with pq_peer_alloc (the
 * one allocation this library makes: peer mapping needs an allocation of its own; it is zero-filled, which is the
 * protocol's initial state), exports its handle (PQ_IPC_HANDLE_BYTES bytes, to be carried to the peers by the host
 * program, e.g. an all-gather of bytes) and opens the peers' handles with pq_peer_open.  `bufs` lists the `world`
 * buffers in rank order as seen from this process: bufs[rank] the local one, the others the opened mappings.  The
 * attention output of the step goes to bufs[rank] + pq_exchange_slot_offset(world, rows, hd, rank).
 *
 * pq_exchange_merge enqueues the kernel (grid rows / 4, 128 threads; hd must be 128; world <= PQ_EXCHANGE_MAX_RANKS;
 * out 16-byte aligned).  All ranks must call it once per step with the same world / rows; calls on one buffer must
 * not overlap.  The epoch lives in the buffer, so the call can be captured in a CUDA graph and replayed.  Every wait
 * on a peer is bounded (one second): if a peer never arrives the kernel finishes with a wrong result and sets a
 * status bit (2: a peer's data did not arrive), which
 * pq_exchange_status reads back (it synchronises the stream).  Ranks may only leave between steps: free the buffer
 * (pq_peer_close on the mappings, pq_peer_free on the own one) after all ranks finished their last call.
 *
 * pq_exchange_merge_emulated runs all `world` ranks' CTAs in ONE cooperative launch on one GPU over `world` local
 * buffers (plain allocations of the same layout, zero-filled) - the protocol's test on a single GPU, where separate
 * launches that wait on one another must not be used.
 */
#define PQ_EXCHANGE_MAX_RANKS 8
/* flag of pq_exchange_merge: the kernel directly before it on the stream is pq_decode_attention's own merge (the call
   that wrote this rank's block): the exchange is then launched as its programmatic dependent and its prologue overlaps
   that kernel's tail.  Leave it clear after anything else. */
#define PQ_EXCHANGE_AFTER_ATTENTION 1u
/* flag of pq_exchange_merge: this rank's block was already pushed to the peers by the pq_decode_attention call that
   wrote it (pq_decode_params.exchange_bufs); the kernel then only collects and merges. */
#define PQ_EXCHANGE_PUSHED 2u
#define PQ_IPC_HANDLE_BYTES 64
int64_t pq_exchange_bytes(int world, int64_t rows, int hd);
int64_t pq_exchange_slot_offset(int world, int64_t rows, int hd, int rank);
int pq_peer_alloc(int64_t bytes, void** ptr, unsigned char* handle);
int pq_peer_open(const unsigned char* handle, void** ptr);
int pq_peer_close(void* ptr);
int pq_peer_free(void* ptr);
int pq_exchange_merge(void* const* bufs, int world, int rank, int64_t rows, int hd, void* out, int out_dtype,
                      float* lse_out, unsigned flags, void* stream);
int pq_exchange_merge_emulated(void* const* bufs, int world, int64_t rows, int hd, void* const* outs, int out_dtype,
                               float* const* lse_outs, unsigned flags, void* stream);
int pq_exchange_status(const void* local_buf, int world, int64_t rows, int hd, unsigned* status, void* stream);

/*
 * Host-buffer forms: the same operations for callers whose tensors live in host
 * memory.  Inputs are copied to the device staging area the caller provides,
 * the kernels run, results are copied back; everything is enqueued on `stream`
 * (the caller synchronises).  Host buffers should be pinned for the copies to
 * overlap.  staging must hold pq_*_host_staging_bytes bytes.
 */
int pq_quantize_host(const void* keys_host, int B, int Nk, int L, int hd, int G, int rbits, int tbits,
                     int dtype, unsigned flags, uint8_t* codes_host, void* rscale_host, void* rmn_host,
                     void* tscale_host, void* tmn_host, void* staging, size_t staging_bytes, void* stream);
size_t pq_quantize_host_staging_bytes(int B, int Nk, int L, int hd, int G, int dtype);

/* p holds HOST pointers for q, codes, scales, k_res, v, mask, out, lse (contiguous
   tensors; the stride fields are ignored and recomputed); workspace fields are
   ignored, scratch is carved from staging. */
int pq_decode_attention_host(const pq_decode_params* p, void* staging, size_t staging_bytes, void* stream);
size_t pq_decode_host_staging_bytes(int B, int N, int Nk, int Nb, int G, int R, int hd,
                                    int qk_dtype, int v_dtype, int out_dtype, int has_mask);

/*
 * CUDA-event helpers so a host program without its own CUDA binding can time the
 * kernels on the stream they are launched on.  pq_event_elapsed_ms synchronises
 * on `end` first.
 */
int pq_event_create(void** event);
int pq_event_destroy(void* event);
int pq_event_record(void* event, void* stream);
int pq_event_elapsed_ms(void* start, void* end, float* ms);

const char* pq_strerror(int status);
/* cudaError_t of the most recent failing CUDA call made by this library on the calling thread */
int pq_last_cuda_error(void);
/* library ABI version, bumped when a signature or struct layout changes */
int pq_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* POLARQUANT_B200_H */
