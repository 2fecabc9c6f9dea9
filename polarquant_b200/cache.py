"""Preallocated, in-place polar KV cache for one attention layer, and the decode step over it.

The reference grows its cache with ``torch.cat`` on every step and re-materialises GQA copies of keys and values
(``repeat_kv``) before each matmul (models/modeling_llama_polar.py:77,86-90,98-99): per generated token the whole
value cache is copied twice.  Here all buffers are allocated once for ``max_tokens``; a step writes the new key and
value into their slots, runs the fused attention kernel over views of the buffers, and - every ``residual_length``
steps - quantises the full-precision window straight into the next free group of the code buffer
(``pq_quantize_into``).  Semantics follow the reference's decode branch exactly: attention sees the residual window
in full precision, including the current token, and only afterwards the window is quantised (:79 precedes :83).

Cache layout (what the reference's 8-tuple holds, with capacity):
    codes   (B, Nk, max_groups, G, 64) uint8        rscale/rmn/tscale/tmn (B, Nk, max_groups, 1, 64)
    k_res   (B, Nk, residual_length, 128)           values (B, Nk, max_tokens, 128)

With ``vbits=4`` the values are packed too, as in the reference's LlamaPolarMixedGroupAttention
(models/modeling_llama_polar.py:160-292): the values of the quantised tokens live as 4-bit codes with a scale and a
minimum per token, the values of the residual window in full precision, and both windows are quantised together
when the window fills (:240-248):
    v_codes (B, Nk, max_tokens, 16) int32, tiled layout     v_scale / v_mn (B, Nk, max_tokens, 1)
    v_res   (B, Nk, residual_length, 128)
136 bytes per token and kv head instead of 324.

With ``key_format="packed6"`` (bit splits 3/3 and 2/4) the codes live in the 48-byte-per-token container instead of one
byte per pair; everything else is unchanged and the attention results are bit-identical.

CUDA-graph replay.  With ``lengths`` (an int32 device tensor ``[token groups, residual tokens]``, shared by the
caches of all layers) ``decode_step_graph`` enqueues the append and the attention with the lengths read on the
device, and changes nothing on the host: one captured graph of the whole model step is replayed for every token.
The owner of the tensor advances ``lengths[1]`` once per step inside the graph (after the last layer) and calls
``after_replay()`` on every cache afterwards, which mirrors the step on the host and, every ``residual_length``
steps, quantises the full window outside the graph.  Fully device-driven variant: ``requantize_graph()`` after each
layer's attention and one ``advance_graph()`` at the end of the captured step make the window's re-quantisation part
of the graph too (a no-op launch except on the step that fills the window); the host then only counts
(``after_replay(device_requantized=True)``).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, ops


class PolarKVCache:
    def __init__(self, batch: int, kv_heads: int, max_tokens: int, dtype=torch.bfloat16, device="cuda",
                 rbits: int = 4, tbits: int = 4, group_size: int = 128, residual_length: int = 128,
                 head_dim: int = 128, vbits: int = 0, lengths: torch.Tensor | None = None,
                 num_q_heads: int | None = None, key_format: str = "byte"):
        if residual_length % group_size:
            raise ValueError("residual_length must be a multiple of group_size")
        if head_dim != 128:
            raise NotImplementedError("head_dim must be 128")
        if vbits not in (0, 4):
            raise NotImplementedError("values are kept in full precision (vbits=0) or packed to 4 bits")
        self.vbits = vbits
        self.B, self.Nk, self.G, self.RL = batch, kv_heads, group_size, residual_length
        self.rbits, self.tbits, self.dtype = rbits, tbits, dtype
        self.max_groups = max_tokens // group_size
        self.max_tokens = max_tokens
        dev = torch.device(device)
        if key_format == "packed6":
            # 48 instead of 64 key bytes per token: the 6-bit container of the 3/3 and 2/4 bit splits
            if rbits + tbits != 6 or group_size % 16:
                raise ValueError("key_format='packed6' holds 6-bit codes (rbits + tbits == 6) of groups of 16 k tokens")
            self.codes = torch.empty((batch, kv_heads, self.max_groups, group_size // 16, 768), dtype=torch.uint8,
                                     device=dev)
        elif key_format == "byte":
            self.codes = torch.empty((batch, kv_heads, self.max_groups, group_size, 64), dtype=torch.uint8, device=dev)
        else:
            raise ValueError("key_format must be 'byte' or 'packed6'")
        self.key_format = key_format
        self._tok_bytes = 48 if key_format == "packed6" else 64          # code bytes per token
        self._qflags = _lib.PQ_QUANT_PACK6 if key_format == "packed6" else 0
        self.scales = [torch.empty((batch, kv_heads, self.max_groups, 1, 64), dtype=dtype, device=dev)
                       for _ in range(4)]                     # rscale, rmn, tscale, tmn
        self.k_res = torch.empty((batch, kv_heads, residual_length, head_dim), dtype=dtype, device=dev)
        if vbits:
            cap = max(self.max_groups * group_size, group_size)      # packed tokens come in whole groups
            self.v_codes = torch.empty((batch, kv_heads, cap, 16), dtype=torch.int32, device=dev)
            self.v_scale = torch.empty((batch, kv_heads, cap, 1), dtype=dtype, device=dev)
            self.v_mn = torch.empty((batch, kv_heads, cap, 1), dtype=dtype, device=dev)
            self.values = torch.empty((batch, kv_heads, residual_length, head_dim), dtype=dtype, device=dev)
        else:
            self.values = torch.empty((batch, kv_heads, max_tokens, head_dim), dtype=dtype, device=dev)
        self.num_groups = 0        # quantised token groups
        self.res_len = 0           # full-precision keys in the window
        self.lengths = lengths
        if lengths is not None:
            if lengths.dtype != torch.int32 or lengths.numel() != 2 or not lengths.is_cuda or \
                    (dev.index is not None and lengths.device.index != dev.index):
                raise ValueError("lengths must be an int32 tensor of two elements on the cache's device")
        # The scratch of the attention call grows with the number of 8-head tiles per kv head.  It is sized for
        # ``num_q_heads`` (default: a GQA ratio of 8) and regrown by ``_ensure_workspace`` when a call brings more.
        self._dev = dev
        self._ws_heads = 0
        self.workspace = None
        self._ensure_workspace(num_q_heads if num_q_heads else kv_heads * 8)
        # everything that does not change from step to step is marshalled once
        self._dt = ops._DT[dtype]
        p = _lib.DecodeParams()
        p.codes, p.codes_stride_b, p.codes_stride_h = self.codes.data_ptr(), self.codes.stride(0), self.codes.stride(1)
        p.rscale, p.rmn, p.tscale, p.tmn = (t.data_ptr() for t in self.scales)
        p.scale_stride_b, p.scale_stride_h = self.scales[0].stride(0), self.scales[0].stride(1)
        p.k_res = self.k_res.data_ptr()
        p.kres_stride_b, p.kres_stride_h, p.kres_stride_t = self.k_res.stride(0), self.k_res.stride(1), self.k_res.stride(2)
        p.v = self.values.data_ptr()
        p.v_stride_b, p.v_stride_h, p.v_stride_t = self.values.stride(0), self.values.stride(1), self.values.stride(2)
        p.workspace, p.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        p.B, p.Nk, p.G, p.hd = batch, kv_heads, group_size, head_dim
        p.rbits, p.tbits = rbits, tbits
        p.key_format = ops._KEY_FORMATS[key_format]
        p.qk_dtype = p.v_dtype = self._dt
        if vbits:
            p.v_codes = self.v_codes.data_ptr()
            p.vcodes_stride_b, p.vcodes_stride_h = self.v_codes.stride(0) * 4, self.v_codes.stride(1) * 4
            p.v_scale, p.v_mn = self.v_scale.data_ptr(), self.v_mn.data_ptr()
            p.vscale_stride_b, p.vscale_stride_h = self.v_scale.stride(0), self.v_scale.stride(1)
            p.vbits = vbits
        self._params = p
        self._kres_strides = (ctypes.c_int64 * 3)(self.k_res.stride(0), self.k_res.stride(1), self.k_res.stride(2))
        self._v_strides = (ctypes.c_int64 * 3)(self.values.stride(0), self.values.stride(1), self.values.stride(2))

    def _ensure_workspace(self, num_q_heads: int) -> None:
        """Make the scratch buffer large enough for attention calls with ``num_q_heads`` query heads.  Growing
        allocates, so it must happen outside CUDA-graph capture: construct the cache with ``num_q_heads`` (or run
        one eager step first) when the GQA ratio exceeds 8."""
        if num_q_heads <= self._ws_heads:
            return
        if num_q_heads % self.Nk:
            raise ValueError("query heads must be a multiple of the cache's kv heads")
        lib = _lib.load()
        need = lib.pq_decode_workspace_bytes(self.B, num_q_heads, self.Nk, self.max_groups, self.G, self.RL, 0)
        if self.lengths is not None:
            need = max(need, lib.pq_decode_workspace_bytes_dyn(self.B, num_q_heads, self.Nk, 0))
        if self.workspace is not None and torch.cuda.is_current_stream_capturing():
            raise RuntimeError(f"PolarKVCache scratch was sized for {self._ws_heads} query heads; pass "
                               f"num_q_heads={num_q_heads} to the constructor before capturing a CUDA graph")
        self.workspace = torch.empty(max(need, 1 << 20) + 256, dtype=torch.uint8, device=self._dev)
        self._ws_heads = num_q_heads
        if getattr(self, "_params", None) is not None:
            self._params.workspace, self._params.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()

    @property
    def seq_len(self) -> int:
        return self.num_groups * self.G + self.res_len

    # ------------------------------------------------------------------ writes
    def _quantize_into(self, keys: torch.Tensor, first_group: int, batch_start: int = 0) -> None:
        """Quantise ``keys`` (b, Nk, n*G, 128; any strides with unit inner stride) into groups
        [first_group, first_group + n) of the code and scale buffers of sequences [batch_start, batch_start + b)."""
        n = keys.shape[2] // self.G
        if n == 0:
            return
        if first_group + n > self.max_groups:
            raise RuntimeError("PolarKVCache is full")
        if not ops._vec_ok(keys, 4):
            keys = keys.contiguous()
        lib = _lib.load()
        dev = keys.device
        in_strides = (ctypes.c_int64 * 4)(*keys.stride())
        out_strides = (ctypes.c_int64 * 4)(self.codes.stride(0), self.codes.stride(1),
                                           self.scales[0].stride(0), self.scales[0].stride(1))
        es = self.scales[0].element_size()
        code_ptr = self.codes.data_ptr() + first_group * self.G * self._tok_bytes + batch_start * self.codes.stride(0)
        scale_ptrs = [s.data_ptr() + (first_group * 64 + batch_start * s.stride(0)) * es for s in self.scales]
        with ops._on_device(dev):
            rc = lib.pq_quantize_into(keys.data_ptr(), in_strides, keys.shape[0], self.Nk, n * self.G, 128, self.G,
                                      self.rbits, self.tbits, ops._DT[keys.dtype], self._qflags, code_ptr, *scale_ptrs,
                                      out_strides, ops._stream(dev))
        _lib.check(rc, "pq_quantize_into")

    def _quantize_values_into(self, values: torch.Tensor, first_token: int, batch_start: int = 0) -> None:
        """Pack ``values`` (b, Nk, n, 128; unit inner stride) into tokens [first_token, first_token + n) of the
        packed value buffers of sequences [batch_start, batch_start + b) (models/modeling_llama_polar.py:242,285)."""
        n = values.shape[2]
        if n == 0:
            return
        if not ops._vec_ok(values, 8):
            values = values.contiguous()
        lib = _lib.load()
        in_strides = (ctypes.c_int64 * 4)(*values.stride())
        out_strides = (ctypes.c_int64 * 4)(self.v_codes.stride(0) * 4, self.v_codes.stride(1) * 4,
                                           self.v_scale.stride(0), self.v_scale.stride(1))
        es = self.v_scale.element_size()
        with ops._on_device(values.device):
            cb, sb = batch_start * self.v_codes.stride(0) * 4, batch_start * self.v_scale.stride(0) * es
            rc = lib.pq_quantize_values(values.data_ptr(), in_strides, values.shape[0], self.Nk, n, 128, self.vbits,
                                        ops._DT[values.dtype], _lib.PQ_VALUES_TILED,
                                        self.v_codes.data_ptr() + first_token * 64 + cb,
                                        self.v_scale.data_ptr() + first_token * es + sb,
                                        self.v_mn.data_ptr() + first_token * es + sb, out_strides,
                                        ops._stream(values.device))
        _lib.check(rc, "pq_quantize_values")

    def prefill(self, key_states: torch.Tensor, value_states: torch.Tensor, batch_start: int = 0) -> None:
        """Store a prompt: keys/values (b, Nk, L, 128), strided views allowed (the (B, L, Nk, hd) layout the
        projections produce).  The first L - L % residual_length keys are quantised, the rest stay in full
        precision, as at models/modeling_llama_polar.py:116-126.  ``batch_start`` places a chunk of b <= B
        sequences (chunked prefill); every chunk must have the same length L, which becomes the cache's."""
        bsz, _, length, _ = key_states.shape
        if length > self.max_tokens:
            raise RuntimeError("prompt longer than the cache")
        if batch_start < 0 or batch_start + bsz > self.B:
            raise ValueError("batch chunk does not fit the cache")
        sl = slice(batch_start, batch_start + bsz)
        rest = length % self.RL
        nq = length - rest
        self.num_groups = 0
        self._quantize_into(key_states[:, :, :nq], 0, batch_start)
        self.num_groups = nq // self.G
        self.res_len = rest
        if self.lengths is not None:
            self.sync_lengths()
        if rest:
            self.k_res[sl, :, :rest].copy_(key_states[:, :, nq:])
        if self.vbits:
            self._quantize_values_into(value_states[:, :, :nq].to(self.dtype), 0, batch_start)
            if rest:
                self.values[sl, :, :rest].copy_(value_states[:, :, nq:])
        else:
            self.values[sl, :, :length].copy_(value_states)

    def prefill_rope(self, key_states: torch.Tensor, value_states: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                     batch_start: int = 0, rotated_out: torch.Tensor | None = None) -> torch.Tensor:
        """``prefill`` for UN-rotated keys: the rotary embedding is applied while the keys are quantised into the
        cache (one pass over the keys instead of a rotation pass plus a quantisation pass).  ``cos`` / ``sin``
        (L, 128) or (b, L, 128).  Returns the rotated keys (for the prompt's own attention), written to
        ``rotated_out`` if given - ``key_states`` itself is allowed - else to a new tensor."""
        bsz, _, length, _ = key_states.shape
        if length > self.max_tokens:
            raise RuntimeError("prompt longer than the cache")
        if batch_start < 0 or batch_start + bsz > self.B:
            raise ValueError("batch chunk does not fit the cache")
        if key_states.dtype != self.dtype:
            raise ValueError("prefill_rope takes keys in the cache dtype")
        dev = key_states.device
        rest = length % self.RL
        nq = length - rest
        if not ops._vec_ok(key_states, 4):
            key_states = key_states.contiguous()
        cos, sin = cos.to(self.dtype), sin.to(self.dtype)
        if cos.dim() == 2:
            cos, sin = cos[None], sin[None]
        if not ops._vec_ok(cos, 4) or not ops._vec_ok(sin, 4) or cos.stride() != sin.stride():
            cos, sin = cos.contiguous(), sin.contiguous()
        out = rotated_out if rotated_out is not None else torch.empty_like(key_states)
        i64 = ctypes.c_int64
        es = self.scales[0].element_size()
        code_ptr = self.codes.data_ptr() + batch_start * self.codes.stride(0)
        scale_ptrs = [s.data_ptr() + batch_start * s.stride(0) * es for s in self.scales]
        out_strides = (i64 * 4)(self.codes.stride(0), self.codes.stride(1), self.scales[0].stride(0),
                                self.scales[0].stride(1))
        lib = _lib.load()
        with ops._on_device(dev):
            rc = lib.pq_rope_quantize(key_states.data_ptr(), (i64 * 4)(*key_states.stride()), cos.data_ptr(),
                                      sin.data_ptr(), (i64 * 2)(0 if cos.shape[0] == 1 else cos.stride(0), cos.stride(1)),
                                      out.data_ptr(), (i64 * 4)(*out.stride()), bsz, self.Nk, length, nq, 128, self.G,
                                      self.rbits, self.tbits, self._dt, self._qflags, code_ptr, *scale_ptrs, out_strides,
                                      ops._stream(dev))
        _lib.check(rc, "pq_rope_quantize")
        sl = slice(batch_start, batch_start + bsz)
        self.num_groups = nq // self.G
        self.res_len = rest
        if self.lengths is not None:
            self.sync_lengths()
        if rest:
            self.k_res[sl, :, :rest].copy_(out[:, :, nq:])
        if self.vbits:
            self._quantize_values_into(value_states[:, :, :nq].to(self.dtype), 0, batch_start)
            if rest:
                self.values[sl, :, :rest].copy_(value_states[:, :, nq:])
        else:
            self.values[sl, :, :length].copy_(value_states)
        return out

    def decode_step(self, query_states: torch.Tensor, key_new: torch.Tensor, value_new: torch.Tensor,
                    attention_mask=None, sm_scale=None, out_dtype=None) -> torch.Tensor:
        """Append one token per sequence and attend.  query_states (B, N, 1, 128); key_new / value_new
        (B, Nk, 1, 128), any batch/head strides.  Returns (B, N, 1, 128).  Three library calls (append, attention,
        and - every residual_length steps - quantise); no allocation proportional to the context, no copy of the
        cache."""
        pos = self.seq_len
        if pos + 1 > self.max_tokens:
            raise RuntimeError("PolarKVCache is full")
        if attention_mask is not None or query_states.dtype != self.dtype or key_new.dtype != self.dtype \
                or value_new.dtype != self.dtype or key_new.stride(-1) != 1 or value_new.stride(-1) != 1:
            return self._decode_step_general(query_states, key_new, value_new, attention_mask, sm_scale, out_dtype)
        lib = _lib.load()
        dev = self._dev
        stream = ops._stream(dev)
        in_strides = (ctypes.c_int64 * 4)(key_new.stride(0), key_new.stride(1), value_new.stride(0),
                                          value_new.stride(1))
        with ops._on_device(dev):
            rc = lib.pq_cache_append(key_new.data_ptr(), value_new.data_ptr(), in_strides, self.k_res.data_ptr(),
                                     self._kres_strides, self.values.data_ptr(), self._v_strides, self.B, self.Nk,
                                     128, self.res_len, self.res_len if self.vbits else pos, self._dt, stream)
            _lib.check(rc, "pq_cache_append")
            self.res_len += 1
            bsz, nq, _, hd = query_states.shape
            self._ensure_workspace(nq)
            q = query_states.reshape(bsz, nq, hd)
            if not ops._vec_ok(q, 8):
                q = q.contiguous()
            out_dtype = out_dtype or self.dtype
            out = torch.empty((bsz, nq, 1, hd), dtype=out_dtype, device=dev)
            p = self._params
            p.q, p.q_stride_b, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
            p.out, p.out_stride_b, p.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
            p.N, p.Nb, p.R = nq, self.num_groups, self.res_len
            p.out_dtype = ops._DT[out_dtype]
            p.sm_scale = 0.0 if sm_scale is None else float(sm_scale)
            rc = lib.pq_decode_attention(ctypes.byref(p), stream)
        _lib.check(rc, "pq_decode_attention")
        if self.res_len == self.RL:                      # window full: quantise it in place (:83-92)
            self._requantize_window()
            if self.lengths is not None:
                self.sync_lengths()
        elif self.lengths is not None:                   # host-driven step on a cache that also has device lengths
            self.lengths[1:2].add_(1)
        return out

    # ------------------------------------------------------------------ CUDA-graph replay
    def decode_step_graph(self, query_states: torch.Tensor, key_new: torch.Tensor, value_new: torch.Tensor,
                          out: torch.Tensor | None = None) -> torch.Tensor:
        """``decode_step`` with every length read on the device from ``self.lengths``: safe to capture in a CUDA
        graph and to replay as the cache grows.  Tensors must already have the cache dtype and unit inner
        strides; their addresses are what a captured graph will reuse.  Host state is not touched - call
        ``after_replay()`` once per executed step."""
        if self.lengths is None:
            raise RuntimeError("this cache was built without a device-side lengths tensor")
        lib = _lib.load()
        dev = self._dev
        if key_new.dtype != self.dtype or value_new.dtype != self.dtype or key_new.stride(-1) != 1 \
                or value_new.stride(-1) != 1:
            raise ValueError("decode_step_graph needs cache-dtype tensors with unit inner stride")
        in_strides = (ctypes.c_int64 * 4)(key_new.stride(0), key_new.stride(1), value_new.stride(0),
                                          value_new.stride(1))
        with ops._on_device(dev):
            rc = lib.pq_cache_append_dyn(key_new.data_ptr(), value_new.data_ptr(), in_strides, self.k_res.data_ptr(),
                                         self._kres_strides, self.values.data_ptr(), self._v_strides, self.B,
                                         self.Nk, 128, self.G, self.lengths.data_ptr(), 1 if self.vbits else 0,
                                         self.RL, self.values.shape[2], self._dt, ops._stream(dev))
        _lib.check(rc, "pq_cache_append_dyn")
        return self.attend_graph(query_states, out)

    def rope_append_graph(self, qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """Rotary embedding + append of one decode token in a single kernel, lengths read on the device.
        ``qkv`` (B, (N + 2 Nk) * 128): the fused projection output [query heads | key heads | value heads];
        ``cos`` / ``sin`` (128,) or (B, 128) in the cache dtype.  Returns the rotated queries (B, N, 1, 128) for
        ``attend_graph``.  Same arithmetic as ``x * cos + rotate_half(x) * sin`` in eager torch."""
        if self.lengths is None:
            raise RuntimeError("this cache was built without a device-side lengths tensor")
        bsz = qkv.shape[0]
        qkv = qkv.reshape(bsz, -1)
        nq = qkv.shape[1] // 128 - 2 * self.Nk
        if qkv.dtype != self.dtype or qkv.stride(1) != 1 or cos.dtype != self.dtype or sin.dtype != self.dtype \
                or nq <= 0 or bsz != self.B:
            raise ValueError("rope_append_graph: qkv must be (B, (N + 2 Nk) * 128) in the cache dtype")
        cos, sin = cos.reshape(-1, 128), sin.reshape(-1, 128)
        cs_stride = cos.stride(0) if cos.shape[0] > 1 else 0
        if sin.shape != cos.shape or (sin.shape[0] > 1 and sin.stride(0) != cs_stride) or cos.stride(1) != 1 \
                or sin.stride(1) != 1:
            raise ValueError("rope_append_graph: cos and sin must have the same (1 or B, 128) layout")
        q_out = torch.empty((bsz, nq, 1, 128), dtype=self.dtype, device=self._dev)
        lib = _lib.load()
        with ops._on_device(self._dev):
            rc = lib.pq_rope_append(qkv.data_ptr(), qkv.stride(0), cos.data_ptr(), sin.data_ptr(), cs_stride,
                                    q_out.data_ptr(), self.k_res.data_ptr(), self._kres_strides,
                                    self.values.data_ptr(), self._v_strides, self.B, nq, self.Nk, 128, self.G,
                                    self.lengths.data_ptr(), 1 if self.vbits else 0, self.RL, self.values.shape[2],
                                    0, 0, self._dt, ops._stream(self._dev))
        _lib.check(rc, "pq_rope_append")
        return q_out

    def attend_graph(self, query_states: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Fused attention of the step whose token was appended by ``rope_append_graph`` / ``decode_step_graph``
        (the appended token is not yet counted in ``lengths``: the kernels add it)."""
        lib = _lib.load()
        dev = self._dev
        bsz, nq, _, hd = query_states.shape
        q = query_states.reshape(bsz, nq, hd)
        if not ops._vec_ok(q, 8) or query_states.dtype != self.dtype:
            raise ValueError("attend_graph needs cache-dtype queries with unit inner stride and aligned rows")
        if out is None:
            out = torch.empty((bsz, nq, 1, hd), dtype=self.dtype, device=dev)
        self._ensure_workspace(nq)
        p = _lib.DecodeParams()
        ctypes.memmove(ctypes.byref(p), ctypes.byref(self._params), ctypes.sizeof(p))
        p.q, p.q_stride_b, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
        p.out, p.out_stride_b, p.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
        p.N, p.Nb, p.R = nq, self.max_groups, self.RL             # capacities; the lengths come from the device
        p.out_dtype = self._dt
        p.dyn_lengths, p.dyn_r_add = self.lengths.data_ptr(), 1   # the appended token is not counted yet
        with ops._on_device(dev):
            rc = lib.pq_decode_attention(ctypes.byref(p), ops._stream(dev))
        _lib.check(rc, "pq_decode_attention")
        return out

    def requantize_graph(self) -> None:
        """Inside the captured step, after ``attend_graph``: quantise the residual window into the next groups IF this
        step has filled it - decided on the device (``lengths[1] + 1 == residual_length``), a no-op launch otherwise.
        With it and ``advance_graph`` a replayed graph needs nothing from the host between tokens."""
        if self.lengths is None:
            raise RuntimeError("this cache was built without a device-side lengths tensor")
        lib = _lib.load()
        dev = self._dev
        stream = ops._stream(dev)
        lp = self.lengths.data_ptr()
        with ops._on_device(dev):
            if self.vbits:
                vin = (ctypes.c_int64 * 4)(*self.values.stride())
                vout = (ctypes.c_int64 * 4)(self.v_codes.stride(0) * 4, self.v_codes.stride(1) * 4,
                                            self.v_scale.stride(0), self.v_scale.stride(1))
                rc = lib.pq_quantize_values_dyn(self.values.data_ptr(), vin, self.B, self.Nk, self.RL, 128,
                                                self.vbits, self._dt, _lib.PQ_VALUES_TILED, self.v_codes.data_ptr(),
                                                self.v_scale.data_ptr(), self.v_mn.data_ptr(), vout, self.G,
                                                self.v_codes.shape[2], lp, 1, stream)
                _lib.check(rc, "pq_quantize_values_dyn")
            kin = (ctypes.c_int64 * 4)(*self.k_res.stride())
            kout = (ctypes.c_int64 * 4)(self.codes.stride(0), self.codes.stride(1),
                                        self.scales[0].stride(0), self.scales[0].stride(1))
            rc = lib.pq_quantize_into_dyn(self.k_res.data_ptr(), kin, self.B, self.Nk, self.RL, 128, self.G,
                                          self.rbits, self.tbits, self._dt, self._qflags, self.codes.data_ptr(),
                                          *(t.data_ptr() for t in self.scales), kout, self.max_groups, lp, 1, stream)
            _lib.check(rc, "pq_quantize_into_dyn")

    def advance_graph(self) -> None:
        """Once per captured step, after the last layer: residual + 1, or - when that fills the window - the new
        groups are counted and the residual starts over.  One call for all caches that share ``lengths``."""
        with ops._on_device(self._dev):
            rc = _lib.load().pq_lengths_advance(self.lengths.data_ptr(), self.RL, self.G, ops._stream(self._dev))
        _lib.check(rc, "pq_lengths_advance")

    def after_replay(self, device_requantized: bool = False) -> bool:
        """Mirror one executed graph step on the host.  Returns True when the step filled the window.  Without
        ``device_requantized`` the window is quantised here, outside the graph, and the caller must then store the
        new lengths into the shared tensor (``sync_lengths``); with it the graph already did both
        (``requantize_graph`` + ``advance_graph``) and only the host's counters move."""
        self.res_len += 1
        if self.res_len == self.RL:
            if device_requantized:
                self.num_groups += self.RL // self.G
                self.res_len = 0
            else:
                self._requantize_window()
            return True
        return False

    def sync_lengths(self) -> None:
        """Write this cache's host-side lengths into the device tensor (after prefill, after a re-quantisation)."""
        self.lengths.copy_(torch.tensor([self.num_groups, self.res_len], dtype=torch.int32), non_blocking=False)

    def _requantize_window(self) -> None:
        if self.vbits:                                   # values of the window first: they sit at the same tokens
            self._quantize_values_into(self.values, self.num_groups * self.G)
        self._quantize_into(self.k_res, self.num_groups)
        self.num_groups += self.RL // self.G
        self.res_len = 0

    def _decode_step_general(self, query_states, key_new, value_new, attention_mask, sm_scale, out_dtype):
        """Same step through the general tensor-level entry points (masks, dtype conversions, odd strides)."""
        pos = self.seq_len
        self.k_res[:, :, self.res_len:self.res_len + 1].copy_(key_new)
        vpos = self.res_len if self.vbits else pos
        self.values[:, :, vpos:vpos + 1].copy_(value_new)
        self.res_len += 1
        ng = self.num_groups
        packed = (self.codes[:, :, :ng], *(s[:, :, :ng] for s in self.scales)) if ng else (None,) * 5
        kw = {}
        if self.vbits and ng:
            nq = ng * self.G
            kw = dict(value_codes=self.v_codes[:, :, :nq], value_scale=self.v_scale[:, :, :nq],
                      value_mn=self.v_mn[:, :, :nq], vbits=self.vbits)
        self._ensure_workspace(query_states.shape[1])
        out = ops.decode_attention(query_states, self.k_res[:, :, :self.res_len], *packed,
                                   self.values[:, :, :vpos + 1], attention_mask=attention_mask, rbits=self.rbits,
                                   tbits=self.tbits, sm_scale=sm_scale, out_dtype=out_dtype,
                                   workspace=self.workspace, key_format=self.key_format, **kw)
        if self.res_len == self.RL:
            self._requantize_window()
            if self.lengths is not None:
                self.sync_lengths()
        elif self.lengths is not None:
            self.lengths[1:2].add_(1)
        return out

    def as_reference_tuple(self):
        """The reference's 8-tuple view of the cache (models/modeling_llama_polar.py:62,101): views, no copies -
        except the codes of a packed-key cache, which are unpacked into the reference's byte container."""
        ng = self.num_groups
        codes = self.codes[:, :, :ng]
        if ng and self.key_format == "packed6":
            codes = ops.keys_repack(codes, "byte")
        packed = (codes, *(s[:, :, :ng] for s in self.scales)) if ng else (None,) * 5
        k_full = self.k_res[:, :, :self.res_len] if self.res_len else None
        if self.vbits:
            # the mixed class's 11-tuple (models/modeling_llama_polar.py:190,246); its value codes are in the
            # kivi layout, so this one member is a converted copy
            nq = ng * self.G
            v_full = self.values[:, :, :self.res_len] if self.res_len else None
            if not nq:
                return (k_full, *packed, v_full, None, None, None, self.seq_len)
            v_quant = ops.values_relayout(self.v_codes[:, :, :nq], "kivi")
            return (k_full, *packed, v_full, v_quant, self.v_scale[:, :, :nq], self.v_mn[:, :, :nq], self.seq_len)
        return (k_full, *packed, self.values[:, :, :self.seq_len], self.seq_len)
