"""Tensor-level entry points over the C ABI: quantizer, QK logits, fused decode attention, LSE merge.

Every function takes CUDA tensors, enqueues on the current torch stream of the
tensors' device and returns without synchronising.  torch only supplies device
memory and the stream handle.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib

_DT = {torch.float16: _lib.PQ_F16, torch.bfloat16: _lib.PQ_BF16, torch.float32: _lib.PQ_F32}


def _dtype_code(t: torch.Tensor, what: str) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise ValueError(f"{what}: dtype {t.dtype} is not supported (float16, bfloat16, float32)") from None


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("polarquant_b200 runs on CUDA tensors only; there is no CPU path")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError("all tensors must live on the same CUDA device")
    return dev


def _stream(dev: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


class _on_device:
    """Device guard that costs nothing when the tensors' device is already current (the usual case)."""
    __slots__ = ("dev", "guard")

    def __init__(self, dev: torch.device):
        self.dev, self.guard = dev, None

    def __enter__(self):
        if torch.cuda.current_device() != self.dev.index:
            self.guard = torch.cuda.device(self.dev)
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)
        return False


def _vec_ok(t: torch.Tensor, elems: int) -> bool:
    """True when 4/8-element vector loads are legal on every row of ``t``."""
    if t.stride(-1) != 1:
        return False
    es = t.element_size()
    if t.data_ptr() % (elems * es):
        return False
    return all(s % elems == 0 for s in t.stride()[:-1])


def quantize_and_pack_nbit(key_states: torch.Tensor, rbits: int = 4, tbits: int = 4, group_size: int = 128,
                           flags: int = 0, key_format: str = "byte"):
    """Polar-quantise keys (B, Nk, L, 128); same contract as the reference method.

    Reference: ``quantize_and_pack_nbit`` at models/modeling_llama_polar.py:135-157.
    Returns ``(indices, rscale, rmn, tscale, tmn)`` with shapes (B, Nk, L/G, G, 64)
    uint8 and four (B, Nk, L/G, 1, 64) tensors in the key dtype.  Strided inputs
    (the (B, L, Nk, hd) layout the prefill hands over) are read in place.

    ``key_format="packed6"`` (bit splits 3/3 and 2/4 only) writes the codes in the 48-byte-per-token container
    instead: ``indices`` is then (B, Nk, L/G, G/16, 768) uint8, one 768-byte tile per 16 tokens (layout:
    ``pq_keys_repack`` in the C header); scales are unchanged.  ``decode_attention(key_format="packed6")`` reads it.
    """
    if key_states.dim() != 4:
        raise ValueError("key_states must be (batch, kv_heads, length, head_dim)")
    bsz, heads, length, hd = key_states.shape
    # the reference's assertion (models/modeling_llama_polar.py:138)
    assert hd % 2 == 0 and length % group_size == 0 and rbits + tbits <= 8
    dev = _require_cuda(key_states)
    dt = _dtype_code(key_states, "quantize_and_pack_nbit")
    if not _vec_ok(key_states, 4):
        key_states = key_states.contiguous()
    nb = length // group_size
    if key_format == "packed6":
        if rbits + tbits != 6 or group_size % 16:
            raise ValueError("the packed container holds 6-bit codes (rbits + tbits == 6) of groups of 16 k tokens")
        flags |= _lib.PQ_QUANT_PACK6
        codes = torch.empty((bsz, heads, nb, group_size // 16, 768), dtype=torch.uint8, device=dev)
    elif key_format == "byte":
        codes = torch.empty((bsz, heads, nb, group_size, hd // 2), dtype=torch.uint8, device=dev)
    else:
        raise ValueError("key_format must be 'byte' or 'packed6'")
    scales = [torch.empty((bsz, heads, nb, 1, hd // 2), dtype=key_states.dtype, device=dev) for _ in range(4)]
    strides = (ctypes.c_int64 * 4)(*key_states.stride())
    lib = _lib.load()
    with _on_device(dev):
        rc = lib.pq_quantize(key_states.data_ptr(), strides, bsz, heads, length, hd, group_size, rbits, tbits, dt,
                             flags, codes.data_ptr(), scales[0].data_ptr(), scales[1].data_ptr(),
                             scales[2].data_ptr(), scales[3].data_ptr(), _stream(dev))
    _lib.check(rc, "pq_quantize")
    return (codes, *scales)


def qk_decode(query_states: torch.Tensor, indices: torch.Tensor, rscale, rmn, tscale, tmn,
              rbits: int = 4, tbits: int = 4) -> torch.Tensor:
    """Un-scaled fp32 logits (B, N, 1, Nb*G) over the packed keys.

    Reference: ``attention_decode_forward_triton_impl`` at models/kernel4group.py:83-109.
    ``Nk = indices.shape[1]`` and query head ``kvh * (N // Nk) + h`` reads kv head kvh.
    """
    bsz, kvh, nb, grp, half = indices.shape
    nq = query_states.shape[1]
    dev = _require_cuda(query_states, indices, rscale, rmn, tscale, tmn)
    dt = _dtype_code(query_states, "attention_decode_forward")
    if nq % kvh:
        raise ValueError("query heads must be a multiple of the kv heads of the code tensor")
    if indices.dtype != torch.uint8:
        raise ValueError("indices must be uint8")
    q = query_states.reshape(bsz, nq, 2 * half)
    if q.stride(-1) != 1:
        q = q.contiguous()
    indices = indices.contiguous()
    scales = []
    for s in (rscale, rmn, tscale, tmn):
        if s.dtype != query_states.dtype:
            s = s.to(query_states.dtype)
        scales.append(s.contiguous())
    out = torch.empty((bsz, nq, 1, nb * grp), dtype=torch.float32, device=dev)
    lib = _lib.load()
    with _on_device(dev):
        rc = lib.pq_qk_decode(q.data_ptr(), q.stride(0), q.stride(1), indices.data_ptr(), scales[0].data_ptr(),
                              scales[1].data_ptr(), scales[2].data_ptr(), scales[3].data_ptr(), out.data_ptr(),
                              bsz, nq, kvh, nb, grp, half, rbits, tbits, dt, _stream(dev))
    _lib.check(rc, "pq_qk_decode")
    return out


_KEY_FORMATS = {"byte": _lib.PQ_KEYS_BYTE, "packed6": _lib.PQ_KEYS_PACKED6}


def rope_quantize(key_states: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rbits: int = 4, tbits: int = 4,
                  group_size: int = 128, quantize_tokens: int | None = None, out: torch.Tensor | None = None,
                  key_format: str = "byte"):
    """Prefill-side fusion: rotate the prompt's keys and polar-quantise them in one pass.

    ``key_states`` (B, Nk, L, 128) are the UN-rotated keys (fp16 / bf16, strided views allowed - the (B, L, Nk, hd)
    layout of the projection); ``cos`` / ``sin`` (L, 128) or (B, L, 128) as ``apply_rotary_pos_emb`` takes them
    (models/modeling_llama_polar.py:55-57).  Returns ``(rotated keys, (indices, rscale, rmn, tscale, tmn))``: the
    rotated keys (written to ``out`` if given - it may be ``key_states`` itself - else to a new tensor in the
    input's layout) equal the eager ``k * cos + rotate_half(k) * sin`` bit for bit, and the first
    ``quantize_tokens`` of them (default: all but the last L % 128, as at :116-126) are quantised exactly as
    ``quantize_and_pack_nbit`` quantises the rotated keys.
    """
    if key_states.dim() != 4:
        raise ValueError("key_states must be (batch, kv_heads, length, head_dim)")
    bsz, heads, length, hd = key_states.shape
    dev = _require_cuda(key_states, cos, sin, out)
    dt = _dtype_code(key_states, "rope_quantize")
    if cos.dtype != key_states.dtype or sin.dtype != key_states.dtype:
        cos, sin = cos.to(key_states.dtype), sin.to(key_states.dtype)
    if cos.dim() == 2:
        cos, sin = cos[None], sin[None]
    if cos.shape[-2:] != (length, hd) or sin.shape != cos.shape or cos.shape[0] not in (1, bsz):
        raise ValueError("cos / sin must be (L, head_dim) or (B, L, head_dim)")
    lq = length - length % 128 if quantize_tokens is None else quantize_tokens
    assert hd % 2 == 0 and lq % group_size == 0 and rbits + tbits <= 8
    if not _vec_ok(key_states, 4):
        key_states = key_states.contiguous()
    if not _vec_ok(cos, 4) or not _vec_ok(sin, 4) or cos.stride() != sin.stride():
        cos, sin = cos.contiguous(), sin.contiguous()
    if out is None:
        out = torch.empty_like(key_states)               # keeps the (dense) layout of a transposed projection output
    elif out.shape != key_states.shape or out.dtype != key_states.dtype or not _vec_ok(out, 4):
        raise ValueError("out must match key_states in shape and dtype, with aligned rows")
    nb = lq // group_size
    flags = 0
    if key_format == "packed6":
        if rbits + tbits != 6 or group_size % 16:
            raise ValueError("the packed container holds 6-bit codes (rbits + tbits == 6) of groups of 16 k tokens")
        flags |= _lib.PQ_QUANT_PACK6
        codes = torch.empty((bsz, heads, nb, group_size // 16, 768), dtype=torch.uint8, device=dev)
    else:
        codes = torch.empty((bsz, heads, nb, group_size, hd // 2), dtype=torch.uint8, device=dev)
    scales = [torch.empty((bsz, heads, nb, 1, hd // 2), dtype=key_states.dtype, device=dev) for _ in range(4)]
    i64 = ctypes.c_int64
    lib = _lib.load()
    with _on_device(dev):
        rc = lib.pq_rope_quantize(key_states.data_ptr(), (i64 * 4)(*key_states.stride()), cos.data_ptr(), sin.data_ptr(),
                                  (i64 * 2)(0 if cos.shape[0] == 1 else cos.stride(0), cos.stride(1)), out.data_ptr(),
                                  (i64 * 4)(*out.stride()), bsz, heads, length, lq, hd, group_size, rbits, tbits, dt,
                                  flags, codes.data_ptr(), scales[0].data_ptr(), scales[1].data_ptr(),
                                  scales[2].data_ptr(), scales[3].data_ptr(), None, _stream(dev))
    _lib.check(rc, "pq_rope_quantize")
    return out, (codes, *scales)


def keys_repack(indices: torch.Tensor, to_format: str) -> torch.Tensor:
    """Convert key codes between the byte container (..., G, 64) and the 6-bit packed container
    (..., G/16, 768); returns a new tensor.  Lossless for 6-bit codes (bit splits 3/3 and 2/4)."""
    dev = _require_cuda(indices)
    if indices.dtype != torch.uint8:
        raise ValueError("indices must be uint8")
    indices = indices.contiguous()
    if to_format == "packed6":
        if indices.shape[-1] != 64 or indices.shape[-2] % 16:
            raise ValueError("byte container: (..., G, 64) with G a multiple of 16")
        steps = indices.numel() // (16 * 64)
        out = torch.empty((*indices.shape[:-2], indices.shape[-2] // 16, 768), dtype=torch.uint8, device=dev)
    elif to_format == "byte":
        if indices.shape[-1] != 768:
            raise ValueError("packed container: (..., G/16, 768)")
        steps = indices.numel() // 768
        out = torch.empty((*indices.shape[:-2], indices.shape[-2] * 16, 64), dtype=torch.uint8, device=dev)
    else:
        raise ValueError("to_format must be 'byte' or 'packed6'")
    lib = _lib.load()
    with _on_device(dev):
        rc = lib.pq_keys_repack(indices.data_ptr(), out.data_ptr(), steps, _KEY_FORMATS[to_format], _stream(dev))
    _lib.check(rc, "pq_keys_repack")
    return out


def key_range_check(rscale: torch.Tensor, rmn: torch.Tensor, rbits: int = 4) -> torch.Tensor:
    """Device-side check that the packed keys stay inside the fp16 range of the decode kernels' dequantisation.

    The kernels form the dequantised key in fp16 (the reference's Triton kernel works in fp32,
    models/kernel4group.py:67-75), so the largest radius a group can reconstruct, |rmn| + |rscale| * 2^rbits, must
    stay below 65504.  Returns a one-element int32 CUDA tensor: 1 when some group breaks that bound or holds a
    non-finite scale, else 0.  Nothing synchronises; read the tensor when convenient.
    """
    dev = _require_cuda(rscale, rmn)
    if rscale.dtype != rmn.dtype or rscale.numel() != rmn.numel():
        raise ValueError("rscale and rmn must have the same dtype and size")
    rscale, rmn = rscale.contiguous(), rmn.contiguous()
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    lib = _lib.load()
    with _on_device(dev):
        rc = lib.pq_key_range_check(rscale.data_ptr(), rmn.data_ptr(), rscale.numel(), rbits,
                                    _dtype_code(rscale, "key_range_check"), flag.data_ptr(), _stream(dev))
    _lib.check(rc, "pq_key_range_check")
    return flag


_workspaces: dict = {}


def _workspace(dev: torch.device, nbytes: int) -> torch.Tensor:
    """Per-(device, stream) scratch, grown on demand and reused across calls."""
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)
        _workspaces[key] = ws
    return ws


def _unit_strides(t: torch.Tensor, inner: int):
    """(stride_b, stride_h) of a (B, Nk, ...) tensor whose trailing dims are dense, else None."""
    expect = 1
    for size, stride in zip(reversed(t.shape[2:]), reversed(t.stride()[2:])):
        if size != 1 and stride != expect:
            return None
        expect *= size
    return t.stride(0), t.stride(1)


def decode_attention(query_states: torch.Tensor, key_residual, indices, rscale, rmn, tscale, tmn,
                     value_states: torch.Tensor, attention_mask=None, rbits: int = 4, tbits: int = 4,
                     sm_scale: float | None = None, out_dtype: torch.dtype | None = None,
                     return_lse: bool = False, workspace: torch.Tensor | None = None, num_ctas: int = 0,
                     mid_event=None, value_codes=None, value_scale=None, value_mn=None, vbits: int = 4,
                     key_format: str = "byte", out: torch.Tensor | None = None, lse_out: torch.Tensor | None = None,
                     push_to=None, collect_out: torch.Tensor | None = None):
    """One fused decode-attention step over the polar cache.

    Computes what the reference's decode branch computes with separate ops
    (models/modeling_llama_polar.py:66-99): logits over the packed keys, logits
    over the full-precision residual keys (which already include the current
    token), ``/ sqrt(head_dim)``, optional key mask, softmax, and the product with
    the values (which already include the current token).

    query_states (B, N, 1, 128); key_residual (B, Nk, R, 128) or None; indices
    (B, Nk, Nb, G, 64) uint8 or None with scales (B, Nk, Nb, 1, 64);
    value_states (B, Nk, Nb*G + R, 128) fp16/bf16, any batch/head/token strides;
    attention_mask (B, Nb*G + R), nonzero = attend.  Returns (B, N, 1, 128) in
    ``out_dtype`` (default: the query dtype) and, with ``return_lse``, the
    natural-log log-sum-exp (B, N) fp32.

    Packed values (the decode branch of LlamaPolarMixedGroupAttention,
    models/modeling_llama_polar.py:189-246): pass ``value_codes`` (B, Nk, Nb*G, 16) int32 in the TILED layout of
    ``quantize_values`` with ``value_scale`` / ``value_mn`` (B, Nk, Nb*G, 1); ``value_states`` then holds only
    the R full-precision values of the residual window (or is None when R == 0).

    ``key_format="packed6"``: ``indices`` is the 48-byte-per-token container (B, Nk, Nb, G/16, 768) written by
    ``quantize_and_pack_nbit(key_format="packed6")`` or ``keys_repack`` (bit splits 3/3 and 2/4, fp16/bf16 caches);
    the result is bit-identical to the byte container's.

    ``out`` (B, N, 1, 128) / ``lse_out`` (B, N) fp32: write the results into these tensors instead of new ones
    (``out`` may have any batch / head strides with a dense last dimension; ``lse_out`` must be contiguous).

    ``push_to``: a ``distributed.PeerExchange``; the results are written to its ``out_view`` / ``lse_view`` and the
    merge that ends the call also stores every row into the peers' exchange buffers (sequence split over peer
    memory: follow with ``push_to.merge(after_attention=True, pushed=True)``).  With ``collect_out`` (B, N, 1, 128)
    as well, that merge also waits for the peers' rows, merges them and writes the final result there: the call is
    the whole sequence-split step and nothing follows it.
    """
    dev = _require_cuda(query_states, key_residual, indices, value_states, attention_mask, value_codes)
    bsz, nq, qlen, hd = query_states.shape
    if qlen != 1:
        raise ValueError("decode attention takes exactly one query position")
    packed_v = value_codes is not None and value_codes.shape[2] > 0
    if packed_v and value_states is None:
        value_states = torch.empty((bsz, value_codes.shape[1], 0, hd), dtype=value_scale.dtype, device=dev)
    kvh = value_states.shape[1]
    qdt = _dtype_code(query_states, "decode_attention")
    vdt = _dtype_code(value_states, "decode_attention")
    out_dtype = out_dtype or query_states.dtype
    nb = grp = 0
    if indices is not None and indices.shape[2] > 0:
        _, _, nb, grp, _ = indices.shape
        if key_format == "packed6":
            if indices.shape[-1] != 768:
                raise ValueError("packed keys must be (B, Nk, Nb, G/16, 768) uint8")
            grp *= 16
    else:
        indices = None
        grp = 128
    res = 0 if key_residual is None else key_residual.shape[2]
    ctx = nb * grp + res
    if packed_v:
        if value_codes.shape[2] != nb * grp or value_states.shape[2] != res:
            raise ValueError("packed values must cover exactly the packed keys, value_states the residual window")
    elif value_states.shape[2] != ctx:
        raise ValueError(f"value_states holds {value_states.shape[2]} tokens, keys hold {ctx}")

    p = _lib.DecodeParams()
    q = query_states.reshape(bsz, nq, hd)
    if not _vec_ok(q, 8):
        q = q.contiguous()
    p.q, p.q_stride_b, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    keep = [q]
    if indices is not None:
        if indices.dtype != torch.uint8:
            raise ValueError("indices must be uint8")
        if _unit_strides(indices, 1) is None or indices.data_ptr() % 16 or indices.stride(0) % 16 or indices.stride(1) % 16:
            indices = indices.contiguous()
        p.codes, (p.codes_stride_b, p.codes_stride_h) = indices.data_ptr(), _unit_strides(indices, 1)
        sc = []
        for s in (rscale, rmn, tscale, tmn):
            if s.dtype != query_states.dtype:
                s = s.to(query_states.dtype)
            if _unit_strides(s, 1) is None or not _vec_ok(s, 8):
                s = s.contiguous()
            sc.append(s)
        if len({(s.stride(0), s.stride(1)) for s in sc}) != 1:
            sc = [s.contiguous() for s in sc]
        p.rscale, p.rmn, p.tscale, p.tmn = (s.data_ptr() for s in sc)
        p.scale_stride_b, p.scale_stride_h = sc[0].stride(0), sc[0].stride(1)
        keep += [indices, *sc]
    if res:
        kr = key_residual
        if kr.dtype != query_states.dtype:
            kr = kr.to(query_states.dtype)
        if not _vec_ok(kr, 8):
            kr = kr.contiguous()
        p.k_res = kr.data_ptr()
        p.kres_stride_b, p.kres_stride_h, p.kres_stride_t = kr.stride(0), kr.stride(1), kr.stride(2)
        keep.append(kr)
    v = value_states
    if vdt == _lib.PQ_F32:
        v = v.to(torch.float16 if query_states.dtype != torch.bfloat16 else torch.bfloat16)
        vdt = _DT[v.dtype]
    if not _vec_ok(v, 8):
        v = v.contiguous()
    p.v, p.v_stride_b, p.v_stride_h, p.v_stride_t = v.data_ptr(), v.stride(0), v.stride(1), v.stride(2)
    keep.append(v)
    if packed_v:
        if value_codes.dtype != torch.int32 or value_codes.shape[-1] != 16:
            raise ValueError("value_codes must be (B, Nk, T, 16) int32")
        vc = value_codes
        if _unit_strides(vc, 1) is None or vc.data_ptr() % 16 or (vc.stride(0) * 4) % 16 or (vc.stride(1) * 4) % 16:
            vc = vc.contiguous()
        vs, vm = (x if x.dtype == v.dtype else x.to(v.dtype) for x in (value_scale, value_mn))
        if _unit_strides(vs, 1) is None or _unit_strides(vm, 1) is None or vs.stride()[:2] != vm.stride()[:2] \
                or vs.stride(0) % 2 or vs.stride(1) % 2 or vs.data_ptr() % 4 or vm.data_ptr() % 4:
            vs, vm = vs.contiguous(), vm.contiguous()
        p.v_codes, p.vcodes_stride_b, p.vcodes_stride_h = vc.data_ptr(), vc.stride(0) * 4, vc.stride(1) * 4
        p.v_scale, p.v_mn = vs.data_ptr(), vm.data_ptr()
        p.vscale_stride_b, p.vscale_stride_h = vs.stride(0), vs.stride(1)
        p.vbits = vbits
        keep += [vc, vs, vm]
    if attention_mask is not None:
        m = (attention_mask != 0).to(torch.uint8)
        if m.shape != (bsz, ctx):
            raise ValueError(f"attention_mask must be (batch, {ctx})")
        m = m.contiguous()
        p.mask, p.mask_stride_b = m.data_ptr(), m.stride(0)
        keep.append(m)
    if out is None:
        out = torch.empty((bsz, nq, 1, hd), dtype=out_dtype, device=dev)
    elif out.shape != (bsz, nq, 1, hd) or out.dtype != out_dtype or out.stride(-1) != 1 or out.device != dev:
        raise ValueError("out must be (B, N, 1, 128) of the output dtype on the inputs' device")
    p.out, p.out_stride_b, p.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    if lse_out is not None:
        if lse_out.shape != (bsz, nq) or lse_out.dtype != torch.float32 or not lse_out.is_contiguous():
            raise ValueError("lse_out must be a contiguous (B, N) float32 tensor")
        return_lse = True
    lse = lse_out if lse_out is not None else (torch.empty((bsz, nq), dtype=torch.float32, device=dev)
                                               if return_lse else None)
    p.lse = lse.data_ptr() if return_lse else None
    p.B, p.N, p.Nk, p.Nb, p.G, p.R, p.hd = bsz, nq, kvh, nb, grp, res, hd
    p.rbits, p.tbits = rbits, tbits
    p.key_format = _KEY_FORMATS[key_format]
    if push_to is not None:
        if out is not push_to.out_view or lse_out is not push_to.lse_view:
            raise ValueError("push_to: pass the exchange's out_view / lse_view as out / lse_out")
        p.exchange_bufs, p.exchange_world, p.exchange_rank = push_to._bufs, push_to.world, push_to.rank
        if collect_out is not None:
            if (collect_out.numel() != bsz * nq * hd or not collect_out.is_contiguous() or collect_out.device != dev
                    or collect_out.dtype not in _DT):
                raise ValueError("collect_out must be a contiguous (B, N, 1, 128) tensor on the inputs' device")
            p.exchange_out, p.exchange_out_dtype = collect_out.data_ptr(), _DT[collect_out.dtype]
    elif collect_out is not None:
        raise ValueError("collect_out needs push_to")
    p.qk_dtype, p.v_dtype, p.out_dtype = qdt, vdt, _DT[out_dtype]
    p.sm_scale = 0.0 if sm_scale is None else float(sm_scale)
    p.num_ctas = num_ctas
    p.mid_event = mid_event
    lib = _lib.load()
    with _on_device(dev):
        need = lib.pq_decode_workspace_bytes(bsz, nq, kvh, nb, grp, res, num_ctas)
        ws = workspace if workspace is not None else _workspace(dev, need)
        p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel() * ws.element_size()
        rc = lib.pq_decode_attention(ctypes.byref(p), _stream(dev))
    _lib.check(rc, "pq_decode_attention")
    del keep
    return (out, lse) if return_lse else out


def merge_lse(outs: torch.Tensor, lses: torch.Tensor, out_dtype: torch.dtype = torch.float32,
              return_lse: bool = False):
    """Merge P partial results: outs (P, ..., 128) fp32 normalised, lses (P, ...) fp32 natural log."""
    dev = _require_cuda(outs, lses)
    outs = outs.to(torch.float32).contiguous()
    lses = lses.to(torch.float32).contiguous()
    parts = outs.shape[0]
    hd = outs.shape[-1]
    rows = lses[0].numel()
    out = torch.empty(outs.shape[1:], dtype=out_dtype, device=dev)
    lse = torch.empty(lses.shape[1:], dtype=torch.float32, device=dev) if return_lse else None
    lib = _lib.load()
    with _on_device(dev):
        rc = lib.pq_merge_lse(outs.data_ptr(), lses.data_ptr(), parts, rows, hd, out.data_ptr(), _DT[out_dtype],
                              lse.data_ptr() if return_lse else None, _stream(dev))
    _lib.check(rc, "pq_merge_lse")
    return (out, lse) if return_lse else out


def merge_lse_gathered(gathered: torch.Tensor, parts: int, rows: int, out_dtype: torch.dtype = torch.float32,
                       out_shape=None) -> torch.Tensor:
    """Merge the buffer an all-gather fills: ``parts`` blocks of ``rows * 129`` fp32 back to back, each block
    [outs (rows, 128) | lses (rows)] - the layout ``distributed.sequence_parallel_decode`` exchanges - without
    slicing it apart first.  Returns (rows, 128) in ``out_dtype`` (reshaped to ``out_shape`` if given)."""
    dev = _require_cuda(gathered)
    if gathered.dtype != torch.float32 or not gathered.is_contiguous() or gathered.numel() != parts * rows * 129:
        raise ValueError("gathered must be a contiguous float32 buffer of parts * rows * 129 elements")
    out = torch.empty((rows, 128), dtype=out_dtype, device=dev)
    lib = _lib.load()
    base = gathered.data_ptr()
    with _on_device(dev):
        rc = lib.pq_merge_lse_strided(base, rows * 129, base + rows * 128 * 4, rows * 129, parts, rows, 128,
                                      out.data_ptr(), _DT[out_dtype], None, _stream(dev))
    _lib.check(rc, "pq_merge_lse_strided")
    return out.reshape(out_shape) if out_shape is not None else out


# ------------------------------------------------------------------------------------------------
# packed value cache
# ------------------------------------------------------------------------------------------------
_LAYOUTS = {"kivi": _lib.PQ_VALUES_KIVI, "tiled": _lib.PQ_VALUES_TILED}


def quantize_values(value_states: torch.Tensor, vbits: int = 4, layout: str = "kivi"):
    """Per-token 4-bit min/max quantisation of values (B, Nk, T, 128), strided views allowed.

    What ``triton_quantize_and_pack_along_last_dim(values, 128, 4)`` returns at
    models/modeling_llama_polar.py:242,285 (a KIVI routine): codes (B, Nk, T, 16) int32 and scale, mn
    (B, Nk, T, 1) in the value dtype.  ``layout="kivi"`` packs channel c at bits 4*(c%8) of word c//8;
    ``layout="tiled"`` is the order the fused attention kernel reads (see ``decode_attention``).
    """
    if value_states.dim() != 4:
        raise ValueError("value_states must be (batch, kv_heads, tokens, head_dim)")
    bsz, heads, tokens, hd = value_states.shape
    dev = _require_cuda(value_states)
    dt = _dtype_code(value_states, "quantize_values")
    if not _vec_ok(value_states, 8 if dt != _lib.PQ_F32 else 4):
        value_states = value_states.contiguous()
    codes = torch.empty((bsz, heads, tokens, hd * vbits // 32), dtype=torch.int32, device=dev)
    scale = torch.empty((bsz, heads, tokens, 1), dtype=value_states.dtype, device=dev)
    mn = torch.empty_like(scale)
    strides = (ctypes.c_int64 * 4)(*value_states.stride())
    lib = _lib.load()
    with _on_device(dev):
        rc = lib.pq_quantize_values(value_states.data_ptr(), strides, bsz, heads, tokens, hd, vbits, dt,
                                    _LAYOUTS[layout], codes.data_ptr(), scale.data_ptr(), mn.data_ptr(), None,
                                    _stream(dev))
    _lib.check(rc, "pq_quantize_values")
    return codes, scale, mn


def values_relayout(codes: torch.Tensor, to_layout: str) -> torch.Tensor:
    """Convert packed value codes (..., T, 16) int32 between the "kivi" and "tiled" layouts (new tensor)."""
    dev = _require_cuda(codes)
    if codes.dtype != torch.int32 or codes.shape[-1] != 16:
        raise ValueError("codes must be (..., 16) int32")
    codes = codes.contiguous()
    out = torch.empty_like(codes)
    lib = _lib.load()
    with _on_device(dev):
        rc = lib.pq_values_relayout(codes.data_ptr(), out.data_ptr(), codes.numel() // 16, _LAYOUTS[to_layout],
                                    _stream(dev))
    _lib.check(rc, "pq_values_relayout")
    return out


def values_matmul(probs: torch.Tensor, codes: torch.Tensor, scale: torch.Tensor, mn: torch.Tensor,
                  vbits: int = 4) -> torch.Tensor:
    """probs (B, H, M, T) times the dequantised values (B, H, T, 128) in the "kivi" layout -> (B, H, M, 128).

    What ``cuda_bmm_fA_qB_outer(128, probs, codes, scale, mn, 4)`` computes at
    models/modeling_llama_polar.py:230-237 (H = query heads there: the caller passes repeated kv tensors)."""
    dev = _require_cuda(probs, codes, scale, mn)
    dt = _dtype_code(probs, "values_matmul")
    bsz, heads, m, tokens = probs.shape
    if codes.shape[:3] != (bsz, heads, tokens) or codes.dtype != torch.int32:
        raise ValueError("codes must be (B, H, T, 16) int32 matching probs (B, H, M, T)")
    probs, codes = probs.contiguous(), codes.contiguous()
    scale = scale.to(probs.dtype).contiguous()
    mn = mn.to(probs.dtype).contiguous()
    out = torch.empty((bsz, heads, m, 128), dtype=probs.dtype, device=dev)
    lib = _lib.load()
    with _on_device(dev):
        rc = lib.pq_values_matmul(probs.data_ptr(), codes.data_ptr(), scale.data_ptr(), mn.data_ptr(),
                                  out.data_ptr(), bsz * heads, m, tokens, 128, vbits, dt, _stream(dev))
    _lib.check(rc, "pq_values_matmul")
    return out
