"""CPU oracle for the polar key-cache hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module.  Only the tests, the smoke
check and the CPU-baseline legs of the benchmark call it, and only as the
checker (or as the timed CPU arm), never as a fallback for the CUDA kernels.

It restates, in plain torch/numpy on whatever device the inputs live on, the
algorithm of the reference project (ericshwu/PolarQuant):

* ``quantize_ops``      - the op sequence of ``quantize_and_pack_nbit``
                          (models/modeling_llama_polar.py:135-157, same body at
                          models/modeling_qwen_polar.py:134-156).
* ``quantize_chain``    - the same quantizer written as an explicit chain of
                          "fp32 operation, then round to the key dtype" steps,
                          the form the CUDA kernel implements.  The constant
                          added to negative angles is a parameter because torch
                          rounds the Python scalar 2*pi to the tensor dtype on
                          CPU and keeps it in fp32 on CUDA.
* ``dequantize``        - models/kernel4group.py:151-153, evaluated in fp32 on
                          the stored scale values (what the reference Triton
                          kernel does at models/kernel4group.py:67,73).
* ``qk_logits_lut``     - the lookup-table form of the reference kernel
                          ``_kernel`` (models/kernel4group.py:37-80).
* ``qk_logits``         - dequantise-then-matmul, models/kernel4group.py:151-155.
* ``decode_attention``  - the decode branch of the patched attention forward
                          (models/modeling_llama_polar.py:77-99, Qwen copy at
                          models/modeling_qwen_polar.py:76-98) composed with the
                          fp32 logits above.
* ``pack_keys6`` / ``unpack_keys6`` - the 48-byte-per-token key container of this
                          library (no reference counterpart), restated from its definition.
* ``merge_lse``         - log-sum-exp merge of partial attention results; it has
                          no counterpart in the reference (the reference never
                          splits the sequence) and is defined by softmax algebra.

Parity pin: the reference ships no golden vectors or tests for this path.  The
functions here are pinned against the reference's own code executed on CPU (its
quantizer method, its Triton kernel under the Triton interpreter, and its
unmodified attention forward); the outputs of those runs are the fixtures under
tests/golden/, produced by tests/golden/make_golden.py.
"""
from __future__ import annotations

import math

import numpy as np
import torch

TWO_PI = 2.0 * math.pi


def _rn(x: torch.Tensor, dt: torch.dtype) -> torch.Tensor:
    """Round an fp32 tensor to ``dt`` (nearest even) and return it as fp32."""
    return x.to(dt).to(torch.float32)


def _sqrt_ieee(x: torch.Tensor) -> torch.Tensor:
    """Correctly rounded fp32 square root.  torch.sqrt on CPU goes through a vector
    math library that is not always correctly rounded; numpy's and CUDA's are."""
    if x.is_cuda:
        return torch.sqrt(x)
    return torch.from_numpy(np.sqrt(x.contiguous().numpy()))


# ----------------------------------------------------------------------------
# quantizer
# ----------------------------------------------------------------------------
def quantize_ops(key_states: torch.Tensor, rbits: int = 4, tbits: int = 4, group_size: int = 128):
    """Polar quantizer as the reference's sequence of tensor ops in the key dtype.

    Follows models/modeling_llama_polar.py:137-157 step for step: the
    (2, head_dim/2) view pairs channel d with channel d+head_dim/2 (:141), the
    angle is atan2 wrapped into [0, 2*pi) (:143-144), angle and radius are
    min/max quantised over each group of ``group_size`` tokens (:146-153) and
    packed as ``(rho << tbits) + theta`` in one byte per pair (:155).

    Runs on CPU or CUDA; on a given device it executes the same ATen kernels the
    reference would, so it is the bit-exact yardstick for that device.
    """
    bsz, heads, length, hd = key_states.shape
    if hd % 2 or length % group_size or rbits + tbits > 8:
        raise AssertionError("head_dim must be even, length a multiple of the group, rbits+tbits <= 8")
    half, grp = hd // 2, group_size
    pairs = key_states.view(bsz, heads, length // grp, grp, 2, half)
    first, second = pairs[..., 0, :], pairs[..., 1, :]

    angle = torch.atan2(second, first)
    angle = torch.where(angle < 0, angle + TWO_PI, angle)
    a_hi = angle.max(dim=-2, keepdim=True).values
    a_lo = angle.min(dim=-2, keepdim=True).values
    a_step = (a_hi - a_lo) / (2 ** tbits)
    a_code = torch.clamp(torch.floor((angle - a_lo) / a_step).to(torch.uint8), 0, 2 ** tbits - 1)

    radius = torch.norm(pairs, p=2, dim=-2)
    r_hi = radius.max(dim=-2, keepdim=True).values
    r_lo = radius.min(dim=-2, keepdim=True).values
    r_step = (r_hi - r_lo) / (2 ** rbits)
    r_code = torch.clamp(torch.floor((radius - r_lo) / r_step).to(torch.uint8), 0, 2 ** rbits - 1)

    codes = (r_code << tbits) + a_code
    return codes, r_step, r_lo, a_step, a_lo


def quantize_chain(key_states: torch.Tensor, rbits: int = 4, tbits: int = 4, group_size: int = 128,
                   wrap_constant: str = "dtype", atan2_fn=None):
    """The quantizer as explicit fp32 arithmetic with a rounding after every op.

    Every reference op (models/modeling_llama_polar.py:143-155) computes in fp32
    and rounds its result to the key dtype; this function spells that out, which
    is the arithmetic the CUDA kernel performs per (token, pair):

      phi   = RN(atan2f(y, x));  phi < 0 -> RN(phi + C)                    (:143-144)
      tstep = RN(RN(max phi - min phi) / 2^tbits)                           (:146-147)
      theta = min(u8(floor(RN(RN(phi - min phi) / tstep))), 2^tbits - 1)   (:148)
      r     = RN(sqrtf(x*x + y*y)),  same min/max/step/floor/clamp          (:150-153)
      code  = (rho << tbits) + theta                                        (:155)

    ``wrap_constant`` selects C: "dtype" rounds 2*pi to the key dtype first
    (torch on CPU), "fp32" keeps float32(2*pi) (torch on CUDA).
    ``atan2_fn(y, x)`` supplies the fp32 arctangent (default ``torch.atan2``);
    different math libraries differ in the last fp32 bit, which can move a
    rounded angle across a representable value.
    """
    dt = key_states.dtype
    bsz, heads, length, hd = key_states.shape
    if hd % 2 or length % group_size or rbits + tbits > 8:
        raise AssertionError("head_dim must be even, length a multiple of the group, rbits+tbits <= 8")
    half, grp = hd // 2, group_size
    k32 = key_states.to(torch.float32).view(bsz, heads, length // grp, grp, 2, half)
    x, y = k32[..., 0, :], k32[..., 1, :]
    atan2_fn = atan2_fn or torch.atan2

    if wrap_constant == "dtype":
        wrap = float(torch.tensor(TWO_PI, dtype=torch.float64).to(dt).to(torch.float32))
    elif wrap_constant == "fp32":
        wrap = float(torch.tensor(TWO_PI, dtype=torch.float64).to(torch.float32))
    else:
        raise ValueError("wrap_constant must be 'dtype' or 'fp32'")

    phi = _rn(atan2_fn(y, x), dt)
    phi = torch.where(phi < 0, _rn(phi + torch.tensor(wrap, dtype=torch.float32), dt), phi)

    def minmax_code(val: torch.Tensor, bits: int):
        hi = val.amax(dim=-2, keepdim=True)
        lo = val.amin(dim=-2, keepdim=True)
        step = _rn(_rn(hi - lo, dt) / float(2 ** bits), dt)
        quot = torch.floor(_rn(_rn(val - lo, dt) / step, dt))
        # float -> int64 -> uint8 like ATen's cast: NaN (0/0 in a constant group) gives 0
        as_int = torch.nan_to_num(quot, nan=0.0, posinf=255.0, neginf=0.0).to(torch.int64)
        code = torch.clamp(as_int & 0xFF, 0, 2 ** bits - 1).to(torch.uint8)
        return code, step, lo

    theta, tstep, tlo = minmax_code(phi, tbits)
    radius = _rn(_sqrt_ieee(x * x + y * y), dt)
    rho, rstep, rlo = minmax_code(radius, rbits)
    codes = ((rho.to(torch.int32) << tbits) + theta.to(torch.int32)).to(torch.uint8)
    return codes, rstep.to(dt), rlo.to(dt), tstep.to(dt), tlo.to(dt)


# ----------------------------------------------------------------------------
# dequantise / QK logits
# ----------------------------------------------------------------------------
def dequantize(codes, rscale, rmn, tscale, tmn, rbits: int = 4, tbits: int = 4) -> torch.Tensor:
    """Reconstructed keys (B, Nk, Nb*G, head_dim) in fp32.

    models/kernel4group.py:151-153: angle and radius are the bin centres
    ``code * step + step / 2 + min``; the key is ``[r cos(phi) | r sin(phi)]``
    with the cosines in channels 0..63 and the sines in channels 64..127.  The
    scales are upcast to fp32 before any arithmetic, as the reference kernel
    does (models/kernel4group.py:67,73).
    """
    bsz, kvh, nb, grp, half = codes.shape
    c = codes.to(torch.int32)
    theta = (c & ((1 << tbits) - 1)).to(torch.float32)
    rho = (c >> tbits).to(torch.float32)
    ts, tm = tscale.to(torch.float32), tmn.to(torch.float32)
    rs, rm = rscale.to(torch.float32), rmn.to(torch.float32)
    phi = ts * (theta + 0.5) + tm
    rad = rs * (rho + 0.5) + rm
    keys = torch.stack([rad * torch.cos(phi), rad * torch.sin(phi)], dim=-2)
    return keys.reshape(bsz, kvh, nb * grp, 2 * half)


def _expand_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """Query head i reads kv head i // n_rep (HF ``repeat_kv`` as used at
    models/modeling_llama_polar.py:79,99)."""
    if n_rep == 1:
        return x
    b, h, l, d = x.shape
    return x[:, :, None].expand(b, h, n_rep, l, d).reshape(b, h * n_rep, l, d)


def qk_logits(query, codes, rscale, rmn, tscale, tmn, rbits: int = 4, tbits: int = 4) -> torch.Tensor:
    """Un-scaled fp32 logits (B, N, 1, Nb*G): dequantise, then matmul
    (models/kernel4group.py:151-155)."""
    n_rep = query.shape[1] // codes.shape[1]
    keys = _expand_kv(dequantize(codes, rscale, rmn, tscale, tmn, rbits, tbits), n_rep)
    return torch.matmul(query.to(torch.float32), keys.transpose(2, 3))


def qk_logits_lut(query, codes, rscale, rmn, tscale, tmn, rbits: int = 4, tbits: int = 4) -> torch.Tensor:
    """The same logits in the lookup-table form of the reference Triton kernel.

    models/kernel4group.py:67-77: per (batch, kv head, group, pair) build the
    table ``T[h, d, a] = q_x[h, d] cos(phi_a) + q_y[h, d] sin(phi_a)`` over the
    angle levels a, gather it by the angle code, multiply by the radius level
    gathered by the radius code, and sum over the pairs d.  Query pair layout
    x = q[d], y = q[d + 64] (:64); query head kvh * (N / Nk) + h belongs to kv
    head kvh (:40,50).
    """
    bsz, kvh, nb, grp, half = codes.shape
    nq = query.shape[1]
    n_rep = nq // kvh
    q = query.to(torch.float32).reshape(bsz, kvh, n_rep, 2, half)
    qx, qy = q[..., 0, :], q[..., 1, :]                                   # (B, Nk, rep, D)
    levels_t = torch.arange(1 << tbits, dtype=torch.float32, device=codes.device) + 0.5
    levels_r = torch.arange(1 << rbits, dtype=torch.float32, device=codes.device) + 0.5
    ts, tm = tscale.to(torch.float32)[..., 0, :], tmn.to(torch.float32)[..., 0, :]   # (B, Nk, Nb, D)
    rs, rm = rscale.to(torch.float32)[..., 0, :], rmn.to(torch.float32)[..., 0, :]
    phi = ts[..., None] * levels_t + tm[..., None]                        # (B, Nk, Nb, D, A)
    table = (qx[:, :, :, None, :, None] * torch.cos(phi)[:, :, None]
             + qy[:, :, :, None, :, None] * torch.sin(phi)[:, :, None])   # (B, Nk, rep, Nb, D, A)
    radii = rs[..., None] * levels_r + rm[..., None]                      # (B, Nk, Nb, D, R)
    c = codes.to(torch.int64)
    a_idx = (c & ((1 << tbits) - 1)).transpose(-1, -2)                    # (B, Nk, Nb, D, G)
    r_idx = (c >> tbits).transpose(-1, -2)
    picked = torch.gather(table, -1, a_idx[:, :, None].expand(bsz, kvh, n_rep, nb, half, grp))
    rad = torch.gather(radii, -1, r_idx)                                  # (B, Nk, Nb, D, G)
    out = (picked * rad[:, :, None]).sum(dim=-2)                          # (B, Nk, rep, Nb, G)
    return out.reshape(bsz, nq, 1, nb * grp)


# ----------------------------------------------------------------------------
# fused decode attention (composition of the reference's decode branch)
# ----------------------------------------------------------------------------
def decode_attention(query, key_residual, codes, rscale, rmn, tscale, tmn, values,
                     attention_mask=None, rbits: int = 4, tbits: int = 4, sm_scale: float | None = None,
                     faithful_rounding: bool = True, return_lse: bool = False):
    """One decode step of polar attention, as the reference's eager ops compute it.

    models/modeling_llama_polar.py:77-99 with the quantised-part logits from
    ``qk_logits`` (fp32):

      w_res = fp32(RN_q(q @ K_res^T))          residual keys, incl. the new token  (:79)
      w     = [w_quant | w_res] / sqrt(head_dim)                                   (:80)
      w    += (1 - mask) * finfo(fp32).min     only when a mask is given           (:94-95)
      p     = RN_q(softmax_fp32(w))                                                (:97)
      out   = RN_q(p @ V)                      V incl. the new token               (:99)

    ``query`` (B, N, 1, hd); ``key_residual`` (B, Nk, R, hd) or None; ``codes``
    (B, Nk, Nb, G, hd/2) or None; ``values`` (B, Nk, Nb*G + R, hd).  With
    ``faithful_rounding=False`` the three RN_q roundings are skipped (all-fp32
    arithmetic), which is the noise-free target a fused kernel approximates.
    Returns (B, N, 1, hd) in the query dtype (fp32 when not faithful), plus the
    natural-log log-sum-exp (B, N) when ``return_lse``.
    """
    qdt = query.dtype
    bsz, nq, _, hd = query.shape
    kvh = values.shape[1]
    n_rep = nq // kvh
    scale = (1.0 / math.sqrt(hd)) if sm_scale is None else sm_scale
    parts = []
    if codes is not None and codes.shape[2] > 0:
        parts.append(qk_logits(query, codes, rscale, rmn, tscale, tmn, rbits, tbits))
    if key_residual is not None and key_residual.shape[2] > 0:
        kr = _expand_kv(key_residual, n_rep)
        if faithful_rounding:
            w_res = torch.matmul(query, kr.to(qdt).transpose(2, 3)).to(torch.float32)
        else:
            w_res = torch.matmul(query.to(torch.float32), kr.to(torch.float32).transpose(2, 3))
        parts.append(w_res)
    w = torch.cat(parts, dim=-1)
    # the reference divides by sqrt(head_dim); a caller-supplied scale multiplies
    w = w / math.sqrt(hd) if sm_scale is None else w * scale
    if attention_mask is not None:
        m = attention_mask.to(torch.float32)
        w = w + (1.0 - m[:, None, None, :]) * torch.finfo(torch.float32).min
    lse = torch.logsumexp(w, dim=-1)[:, :, 0]
    p = torch.softmax(w, dim=-1)
    vv = _expand_kv(values, n_rep)
    if faithful_rounding:
        out = torch.matmul(p.to(qdt), vv.to(qdt))
    else:
        out = torch.matmul(p, vv.to(torch.float32))
    return (out, lse) if return_lse else out


# ---------------------------------------------------------------------------------------------
# Quantised value cache (LlamaPolarMixedGroupAttention, models/modeling_llama_polar.py:160-292)
#
# PARITY UNPINNED for this part: the reference calls `triton_quantize_and_pack_along_last_dim` and
# `cuda_bmm_fA_qB_outer` from the KIVI project (github.com/jy-yuan/KIVI, `quant/new_pack.py` and
# `quant/matmul.py`; the reference imports them as models.kivi_quant.* and vendors neither, nor pins a
# version).  What follows restates KIVI's published algorithm as the reference's call sites use it
# (:242, :285: group 128 along the channel axis = one group per token, 4 bits; :230-237: dequantise
# and multiply); nothing here could be checked against an executed KIVI.
# ---------------------------------------------------------------------------------------------
def quantize_values(values: torch.Tensor, bits: int = 4, layout: str = "kivi", scalar_division: str = "reciprocal"):
    """Per-token asymmetric min/max quantisation of (B, Nk, T, 128) values, every op in the tensor dtype as
    torch executes it: ``mn, mx`` over the 128 channels; ``scale = (mx - mn) / (2^bits - 1)``;
    ``q = round_half_even(clamp((v - mn) / scale, 0, 2^bits - 1))`` (a constant token gives 0/0 = NaN, which the
    CUDA float-to-int cast turns into 0); 32/bits consecutive channels share an int32, channel ``c`` at bits
    ``bits * (c % (32/bits))`` of word ``c // (32/bits)``.  Returns codes (B, Nk, T, 128*bits/32) int32 and
    scale, mn (B, Nk, T, 1).  ``layout="tiled"`` applies ``kivi_to_tiled`` to the codes.

    ``scalar_division``: KIVI only runs on CUDA, where torch divides a tensor by a Python scalar by multiplying
    with the scalar's fp32 reciprocal - ``"reciprocal"`` states that explicitly (the default, on any device);
    ``"true"`` leaves ``/ (2^bits - 1)`` to torch, i.e. a true division on CPU and whatever the device does on
    CUDA (the GPU tests use it to pin "reciprocal" against torch executing there)."""
    levels = 2 ** bits - 1
    dt = values.dtype
    mn = values.min(dim=-1, keepdim=True)[0]
    mx = values.max(dim=-1, keepdim=True)[0]
    if scalar_division == "reciprocal":
        inv = torch.tensor(1.0, dtype=torch.float32, device=values.device) / levels
        scale = ((mx - mn).to(torch.float32) * inv).to(dt)
    elif scalar_division == "true":
        scale = (mx - mn) / levels
    else:
        raise ValueError(scalar_division)
    q = (values - mn) / scale
    q = torch.nan_to_num(q.clamp(0, levels).round().to(torch.float32), nan=0.0).to(torch.int32)
    per = 32 // bits
    q = q.reshape(*q.shape[:-1], q.shape[-1] // per, per)
    codes = torch.zeros(q.shape[:-1], dtype=torch.int32, device=values.device)
    for i in range(per):          # OR of disjoint bit fields; int32 wrap-around of the top field is intended
        codes |= q[..., i] << (bits * i)
    if layout == "tiled":
        codes = kivi_to_tiled(codes, bits)
    elif layout != "kivi":
        raise ValueError(layout)
    return codes, scale, mn


def unpack_values(codes: torch.Tensor, bits: int = 4, layout: str = "kivi") -> torch.Tensor:
    """Integer levels (B, Nk, T, 128) int32 from packed codes of either layout."""
    if layout == "tiled":
        codes = tiled_to_kivi(codes, bits)
    per = 32 // bits
    shifts = torch.arange(per, dtype=torch.int32, device=codes.device) * bits
    q = (codes[..., None] >> shifts) & (2 ** bits - 1)
    return q.reshape(*codes.shape[:-1], codes.shape[-1] * per)


def _tiled_perm(bits: int = 4) -> np.ndarray:
    """Channel held by each field of a token's packed row in the tiled layout, in field order.  4 bits: the row is
    eight 64-bit lane slots; slot g (words 2g, 2g+1) holds channels g + 8j at field j = 0..15 - what lane group
    g of the attention kernel needs for the rows (g, g + 8) of all eight 16-channel output tiles."""
    if bits != 4:
        raise NotImplementedError("tiled layout is defined for 4-bit values")
    perm = np.empty(128, dtype=np.int64)
    for g in range(8):
        for j in range(16):
            perm[16 * g + j] = g + 8 * j
    return perm


def kivi_to_tiled(codes: torch.Tensor, bits: int = 4) -> torch.Tensor:
    per = 32 // bits
    q = unpack_values(codes, bits)[..., torch.from_numpy(_tiled_perm(bits)).to(codes.device)]
    q = q.reshape(*q.shape[:-1], q.shape[-1] // per, per)
    out = torch.zeros(q.shape[:-1], dtype=torch.int32, device=codes.device)
    for i in range(per):
        out |= q[..., i] << (bits * i)
    return out


def tiled_to_kivi(codes: torch.Tensor, bits: int = 4) -> torch.Tensor:
    per = 32 // bits
    shifts = torch.arange(per, dtype=torch.int32, device=codes.device) * bits
    fields = ((codes[..., None] >> shifts) & (2 ** bits - 1)).reshape(*codes.shape[:-1], codes.shape[-1] * per)
    q = torch.empty_like(fields)
    q[..., torch.from_numpy(_tiled_perm(bits)).to(codes.device)] = fields
    q = q.reshape(*q.shape[:-1], q.shape[-1] // per, per)
    out = torch.zeros(q.shape[:-1], dtype=torch.int32, device=codes.device)
    for i in range(per):
        out |= q[..., i] << (bits * i)
    return out


def dequantize_values(codes, scale, mn, bits: int = 4, layout: str = "kivi") -> torch.Tensor:
    """fp32 values ``level * scale + mn`` (B, Nk, T, 128), scale and mn upcast first."""
    return unpack_values(codes, bits, layout).to(torch.float32) * scale.to(torch.float32) + mn.to(torch.float32)


def values_matmul(probs, codes, scale, mn, bits: int = 4) -> torch.Tensor:
    """``cuda_bmm_fA_qB_outer(128, probs, codes, scale, mn, bits)`` as the reference calls it
    (models/modeling_llama_polar.py:230-237): probs (B, H, M, T) times the dequantised values (B, H, T, 128),
    fp32 accumulation, result in the dtype of ``probs``."""
    v = dequantize_values(codes, scale, mn, bits)
    return torch.matmul(probs.to(torch.float32), v).to(probs.dtype)


def decode_attention_mixed(query, key_residual, codes, rscale, rmn, tscale, tmn, v_codes, v_scale, v_mn,
                           value_residual, attention_mask=None, rbits: int = 4, tbits: int = 4, vbits: int = 4,
                           sm_scale: float | None = None, faithful_rounding: bool = True,
                           return_lse: bool = False, layout: str = "kivi"):
    """Decode step with packed keys AND packed values (models/modeling_llama_polar.py:189-246): logits and
    softmax as in ``decode_attention``; ``out = RN_q(P[:, :Tq] @ dequant(V)) + RN_q(P[:, Tq:] @ V_res)`` where
    the first ``Tq = v_codes.shape[2]`` keys have packed values and the rest full-precision ones (:229-239)."""
    qdt = query.dtype
    bsz, nq, _, hd = query.shape
    kvh = (value_residual if value_residual is not None else v_codes).shape[1]
    n_rep = nq // kvh
    parts = []
    if codes is not None and codes.shape[2] > 0:
        parts.append(qk_logits(query, codes, rscale, rmn, tscale, tmn, rbits, tbits))
    if key_residual is not None and key_residual.shape[2] > 0:
        kr = _expand_kv(key_residual, n_rep)
        if faithful_rounding:
            parts.append(torch.matmul(query, kr.to(qdt).transpose(2, 3)).to(torch.float32))
        else:
            parts.append(torch.matmul(query.to(torch.float32), kr.to(torch.float32).transpose(2, 3)))
    w = torch.cat(parts, dim=-1)
    w = w / math.sqrt(hd) if sm_scale is None else w * sm_scale
    if attention_mask is not None:
        w = w + (1.0 - attention_mask.to(torch.float32)[:, None, None, :]) * torch.finfo(torch.float32).min
    lse = torch.logsumexp(w, dim=-1)[:, :, 0]
    p = torch.softmax(w, dim=-1)
    tq = 0 if v_codes is None else v_codes.shape[2]
    out = torch.zeros((bsz, nq, 1, hd), dtype=torch.float32, device=query.device)
    if faithful_rounding:
        p = p.to(qdt)
    if tq:
        vq = _expand_kv(dequantize_values(v_codes, v_scale, v_mn, vbits, layout), n_rep)
        o = torch.matmul(p[..., :tq].to(torch.float32), vq)
        out = out + (o.to(qdt).to(torch.float32) if faithful_rounding else o)
    if value_residual is not None and value_residual.shape[2] > 0:
        vr = _expand_kv(value_residual, n_rep)
        if faithful_rounding:
            o = torch.matmul(p[..., tq:], vr.to(qdt)).to(torch.float32)
        else:
            o = torch.matmul(p[..., tq:], vr.to(torch.float32))
        out = out + o
    out = out.to(qdt) if faithful_rounding else out
    return (out, lse) if return_lse else out


def merge_lse(outs: torch.Tensor, lses: torch.Tensor):
    """Merge partial attention results computed over disjoint key ranges.

    ``outs`` (P, ..., hd) are softmax-normalised partial outputs, ``lses``
    (P, ...) their natural-log log-sum-exps.  With L = logsumexp_p(lse_p) the
    result is ``sum_p exp(lse_p - L) * out_p`` and its log-sum-exp is L.
    """
    lses = lses.to(torch.float32)
    total = torch.logsumexp(lses, dim=0)
    w = torch.exp(lses - total[None])
    w = torch.where(torch.isfinite(w), w, torch.zeros_like(w))
    return (w[..., None] * outs.to(torch.float32)).sum(dim=0), total


# ----------------------------------------------------------------------------
# 6-bit packed key container (an opt-in format of this library; the reference keeps
# one byte per pair, models/modeling_llama_polar.py:155, and lists real packing as
# future work, models/kernel4group.py:1-3).  The layout is a definition, restated
# here field by field from the C header so that the kernels can be checked against
# an independent statement of it.
# ----------------------------------------------------------------------------
def pack_keys6(codes: torch.Tensor) -> torch.Tensor:
    """codes (..., T, 64) uint8 with T % 16 == 0 and values < 64 -> (..., T/16, 768) uint8.

    Per step of 16 tokens: lane l = 4 g + t owns pairs 16 t .. 16 t + 15 of tokens g and g + 8.  Bytes
    16 l .. 16 l + 15 hold the little-endian words A0, A1 of token g then of token g + 8; bytes 512 + 8 l .. hold
    the words H of token g and g + 8.  With c[p] the code of pair 16 t + p: nibble 2 i of A_k is c[8 k + i] & 15,
    nibble 2 i + 1 is c[8 k + 4 + i] & 15; bits 2 j, 2 j + 1 of H are c[4 W + E] >> 4 and bits 16 + 2 j, 17 + 2 j are
    c[4 W + E + 2] >> 4, j = 2 W + E."""
    c = codes.detach().cpu().numpy().astype(np.uint32)
    lead, T = c.shape[:-2], c.shape[-2]
    assert c.shape[-1] == 64 and T % 16 == 0
    c = c.reshape(-1, T // 16, 2, 8, 4, 16)                       # (unit, step, half, g, t, p)
    lo, hi = c & 15, (c >> 4) & 3
    A = np.zeros(c.shape[:-1] + (2,), dtype=np.uint32)            # (..., k)
    for k in range(2):
        for i in range(4):
            A[..., k] |= lo[..., 8 * k + i] << (4 * (2 * i)) | lo[..., 8 * k + 4 + i] << (4 * (2 * i + 1))
    H = np.zeros(c.shape[:-1], dtype=np.uint32)
    for W in range(4):
        for E in range(2):
            j = 2 * W + E
            H |= hi[..., 4 * W + E] << (2 * j) | hi[..., 4 * W + E + 2] << (16 + 2 * j)
    n = c.shape[0]
    tile = np.zeros((n, T // 16, 768), dtype=np.uint8)
    # words of lane l: [A0(g), A1(g), A0(g+8), A1(g+8)] at 16 l; [H(g), H(g+8)] at 512 + 8 l
    a_words = np.stack([A[:, :, 0, :, :, 0], A[:, :, 0, :, :, 1], A[:, :, 1, :, :, 0], A[:, :, 1, :, :, 1]], axis=-1)
    h_words = np.stack([H[:, :, 0], H[:, :, 1]], axis=-1)         # (unit, step, g, t, 2)
    tile[:, :, :512] = np.ascontiguousarray(a_words.reshape(n, T // 16, 32, 4)).astype("<u4").view(np.uint8) \
        .reshape(n, T // 16, 512)
    tile[:, :, 512:] = np.ascontiguousarray(h_words.reshape(n, T // 16, 32, 2)).astype("<u4").view(np.uint8) \
        .reshape(n, T // 16, 256)
    return torch.from_numpy(tile.reshape(*lead, T // 16, 768))


def unpack_keys6(tiles: torch.Tensor) -> torch.Tensor:
    """Inverse of ``pack_keys6``: (..., S, 768) uint8 -> (..., 16 S, 64) uint8."""
    t = tiles.detach().cpu().numpy()
    lead, S = t.shape[:-2], t.shape[-2]
    assert t.shape[-1] == 768
    t = t.reshape(-1, S, 768)
    n = t.shape[0]
    a = np.ascontiguousarray(t[:, :, :512]).view("<u4").reshape(n, S, 8, 4, 2, 2).astype(np.uint32)  # g, t, half, k
    h = np.ascontiguousarray(t[:, :, 512:]).view("<u4").reshape(n, S, 8, 4, 2).astype(np.uint32)     # g, t, half
    out = np.zeros((n, S, 2, 8, 4, 16), dtype=np.uint32)                                             # half, g, t, p
    for half in range(2):
        for k in range(2):
            for i in range(4):
                out[:, :, half, :, :, 8 * k + i] |= (a[:, :, :, :, half, k] >> (4 * (2 * i))) & 15
                out[:, :, half, :, :, 8 * k + 4 + i] |= (a[:, :, :, :, half, k] >> (4 * (2 * i + 1))) & 15
        for W in range(4):
            for E in range(2):
                j = 2 * W + E
                out[:, :, half, :, :, 4 * W + E] |= ((h[:, :, :, :, half] >> (2 * j)) & 3) << 4
                out[:, :, half, :, :, 4 * W + E + 2] |= ((h[:, :, :, :, half] >> (16 + 2 * j)) & 3) << 4
    return torch.from_numpy(out.astype(np.uint8).reshape(*lead, S * 16, 64))


# ----------------------------------------------------------------------------
# seeded synthetic inputs with the shapes and value distributions of the
# benchmark configurations
# ----------------------------------------------------------------------------
def synth_keys(bsz, kvh, length, hd, dtype, seed, kind="loguniform", device="cpu"):
    """Seeded synthetic keys.  kind="loguniform": randn times a per-(kv head,
    channel) scale drawn log-uniformly from [0.5, 8].  kind="outlier": randn with
    four seeded pair indices per head whose two channels are scaled by 10."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    k = torch.randn(bsz, kvh, length, hd, generator=g, dtype=torch.float32)
    if kind == "loguniform":
        s = torch.exp(torch.empty(kvh, hd).uniform_(math.log(0.5), math.log(8.0), generator=g))
        k = k * s[None, :, None, :]
    elif kind == "outlier":
        half = hd // 2
        for h in range(kvh):
            idx = torch.randperm(half, generator=g)[:4]
            k[:, h, :, idx] *= 10.0
            k[:, h, :, idx + half] *= 10.0
    elif kind != "randn":
        raise ValueError(kind)
    return k.to(dtype).to(device)


def as_numpy(t: torch.Tensor) -> np.ndarray:
    """Bit-preserving numpy view: bf16 tensors come back as uint16 words."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()
