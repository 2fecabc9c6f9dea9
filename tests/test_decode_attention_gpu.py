"""Fused CUDA decode attention (through the C ABI) against the composed oracle and the reference-forward fixtures.

Bar: max |diff| <= 2e-2 and mean |diff| <= 2e-3 on the (B, N, 1, 128) output, against the reference's
dequantise-then-matmul path in the tensors' own dtype.  One refinement, because both sides end in a rounding to
the output dtype: where an output element is so large that one unit in the last place of bf16/fp16 exceeds 2e-2
(|x| >= 4 in bf16), a difference of one such unit is a rounding flip, not an error, and is allowed.  Every
configuration is also run with fp32 output (no final rounding on the kernel's side)."""
import ctypes
import math

import pytest
import torch

from conftest import ATTN_MAX_ABS, ATTN_MEAN_ABS, golden_names, load_golden
from oracle import polar_oracle as oracle

pytestmark = pytest.mark.gpu


def _ulp(want):
    """Spacing of the output dtype at each element of ``want`` (0 for fp32)."""
    if want.dtype == torch.float32:
        return torch.zeros_like(want)
    mant = 7 if want.dtype == torch.bfloat16 else 10
    mag = want.float().abs().clamp_min(1e-30)
    return torch.exp2(torch.floor(torch.log2(mag)) - mant)


def _check(got, want, what=""):
    assert got.shape == want.shape, (got.shape, want.shape)
    diff = (got.float() - want.float()).abs()
    assert torch.isfinite(got.float()).all(), what
    allowed = torch.clamp_min(_ulp(want), ATTN_MAX_ABS)
    if got.dtype == torch.float32 and want.dtype != torch.float32:
        # an unrounded result against a reference that was rounded to bf16/fp16: the reference's own
        # rounding (half a unit in its last place) is not the kernel's error
        allowed = ATTN_MAX_ABS + 0.5 * _ulp(want)
    worst = float((diff - allowed).max())
    assert worst <= 0 and float(diff.mean()) <= ATTN_MEAN_ABS, (what, float(diff.max()), float(diff.mean()))


def _make(B, N, Nk, Nb, grp, R, dtype, rb, tb, seed, vdtype=None):
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(seed)
    ctx = Nb * grp + R
    keys = oracle.synth_keys(B, Nk, max(ctx, 1), 128, dtype, seed=seed + 1, device=dev)
    q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(dtype)
    v = torch.randn(B, Nk, ctx, 128, device=dev, generator=g).to(vdtype or dtype)
    quant = (None,) * 5
    if Nb:
        quant = oracle.quantize_ops(keys[:, :, :Nb * grp].contiguous(), rb, tb, grp)
    kres = keys[:, :, Nb * grp:ctx].contiguous() if R else None
    return q, kres, quant, v


@pytest.mark.parametrize("name", golden_names("attn_", exclude="attn_mixed_"))
def test_outputs_of_the_reference_forward(name):
    import polarquant_b200 as pq
    g = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in load_golden(name).items()}
    rb, tb, _ = g["meta"]
    mask = g["mask"] if g["mask"].numel() else None
    got = pq.decode_attention(g["q"], g["k_res"], g["indices"], g["rscale"], g["rmn"], g["tscale"], g["tmn"],
                              g["v"], attention_mask=mask, rbits=rb, tbits=tb)
    assert got.dtype == g["q"].dtype
    _check(got, g["out"], name)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,N,Nk,Nb,grp,R,rb,tb", [
    (2, 32, 8, 15, 128, 128, 4, 4),    # Llama-3.1-8B grouping, full residual window
    (2, 32, 8, 15, 128, 1, 4, 4),      # first step after a re-quantisation
    (2, 28, 4, 7, 128, 77, 4, 4),      # Qwen2.5-7B grouping: 7 heads per kv head
    (2, 28, 4, 28, 32, 100, 3, 3),
    (2, 28, 4, 28, 32, 16, 2, 4),
    (1, 28, 4, 7, 128, 17, 3, 3),
    (1, 28, 4, 7, 128, 128, 2, 4),
    (1, 32, 32, 31, 128, 128, 4, 4),   # MHA (Llama-2-7B shape, 4096 keys)
    (1, 64, 8, 4, 128, 33, 4, 4),      # 8 heads per kv head
    (1, 32, 2, 3, 64, 5, 4, 3),        # 16 heads per kv head: two head tiles
    (3, 8, 2, 0, 128, 50, 4, 4),       # nothing quantised yet
    (3, 8, 2, 5, 16, 0, 4, 4),         # no residual keys, smallest group
])
def test_seeded_configurations(dtype, B, N, Nk, Nb, grp, R, rb, tb):
    import polarquant_b200 as pq
    q, kres, quant, v = _make(B, N, Nk, Nb, grp, R, dtype, rb, tb, seed=90 + Nb + R)
    got, lse = pq.decode_attention(q, kres, *quant, v, rbits=rb, tbits=tb, return_lse=True)
    want, wlse = oracle.decode_attention(q, kres, *quant, v, rbits=rb, tbits=tb, return_lse=True)
    _check(got, want)
    assert float((lse - wlse).abs().max()) <= 2e-2
    got32 = pq.decode_attention(q, kres, *quant, v, rbits=rb, tbits=tb, out_dtype=torch.float32)
    _check(got32, want, "fp32 output")


def test_fp32_queries_and_keys_with_fp16_values():
    """The CPU-reference configuration: fp32 query, residual keys and scales, values stored in fp16."""
    import polarquant_b200 as pq
    q, kres, quant, v = _make(1, 32, 32, 8, 128, 128, torch.float32, 4, 4, seed=91, vdtype=torch.float16)
    got = pq.decode_attention(q, kres, *quant, v)
    assert got.dtype == torch.float32
    want = oracle.decode_attention(q, kres, *quant, v.float(), faithful_rounding=False)
    _check(got, want)


def test_key_mask_like_left_padding():
    import polarquant_b200 as pq
    q, kres, quant, v = _make(3, 8, 2, 4, 128, 60, torch.bfloat16, 4, 4, seed=92)
    ctx = 4 * 128 + 60
    mask = torch.ones(3, ctx, device="cuda")
    mask[0, :200] = 0
    mask[2, :513] = 0          # padding reaches into the residual window
    got = pq.decode_attention(q, kres, *quant, v, attention_mask=mask)
    want = oracle.decode_attention(q, kres, *quant, v, attention_mask=mask)
    _check(got, want)
    # an int64 0/1 mask (what HF hands over) behaves the same
    got2 = pq.decode_attention(q, kres, *quant, v, attention_mask=mask.long())
    assert torch.equal(got, got2)


def test_strided_values_and_keys_from_the_prefill_layout():
    """After prefill the value cache is a (B, L, Nk, hd)-strided view until the first torch.cat."""
    import polarquant_b200 as pq
    q, kres, quant, v = _make(2, 8, 2, 3, 128, 40, torch.bfloat16, 4, 4, seed=93)
    v_strided = v.transpose(1, 2).contiguous().transpose(1, 2)
    k_strided = kres.transpose(1, 2).contiguous().transpose(1, 2)
    assert not v_strided.is_contiguous()
    got = pq.decode_attention(q, k_strided, *quant, v_strided)
    _check(got, oracle.decode_attention(q, kres, *quant, v))
    assert torch.equal(got, pq.decode_attention(q, kres, *quant, v))


@pytest.mark.parametrize("num_ctas", [1, 2, 7, 148, 1000])
def test_result_does_not_depend_on_the_work_split(num_ctas):
    import polarquant_b200 as pq
    q, kres, quant, v = _make(2, 8, 2, 6, 128, 99, torch.bfloat16, 4, 4, seed=94)
    want = oracle.decode_attention(q, kres, *quant, v)
    got = pq.decode_attention(q, kres, *quant, v, num_ctas=num_ctas)
    _check(got, want, f"num_ctas={num_ctas}")


def test_results_are_bitwise_reproducible_from_call_to_call():
    """No atomics, no timing-dependent reduction order: the same inputs give the same bits every time."""
    import polarquant_b200 as pq
    for shape in ((4, 32, 8, 64, 128, 128), (5, 16, 4, 19, 16, 77), (3, 28, 4, 37, 32, 5)):
        q, kres, quant, v = _make(*shape, torch.bfloat16, 4, 4, seed=194)
        ref, lse = pq.decode_attention(q, kres, *quant, v, out_dtype=torch.float32, return_lse=True)
        for _ in range(40):
            got, lse2 = pq.decode_attention(q, kres, *quant, v, out_dtype=torch.float32, return_lse=True)
            assert torch.equal(got, ref) and torch.equal(lse2, lse)


def test_custom_softmax_scale_and_fp32_output():
    import polarquant_b200 as pq
    q, kres, quant, v = _make(1, 8, 2, 2, 128, 9, torch.float16, 4, 4, seed=95)
    got = pq.decode_attention(q, kres, *quant, v, sm_scale=0.05, out_dtype=torch.float32)
    want = oracle.decode_attention(q, kres, *quant, v, sm_scale=0.05, faithful_rounding=False)
    assert got.dtype == torch.float32
    _check(got, want)


def test_sequence_split_and_lse_merge_equal_the_unsplit_result():
    """Round trip: attention over two halves of the cache merged by log-sum-exp == attention over all of it."""
    import polarquant_b200 as pq
    q, kres, quant, v = _make(2, 16, 4, 8, 128, 70, torch.bfloat16, 4, 4, seed=96)
    full, lse = pq.decode_attention(q, kres, *quant, v, out_dtype=torch.float32, return_lse=True)
    half = 4
    first = [t[:, :, :half].contiguous() for t in quant]
    second = [t[:, :, half:].contiguous() for t in quant]
    o0, l0 = pq.decode_attention(q, None, *first, v[:, :, :half * 128], out_dtype=torch.float32, return_lse=True)
    o1, l1 = pq.decode_attention(q, kres, *second, v[:, :, half * 128:], out_dtype=torch.float32, return_lse=True)
    merged, mlse = pq.merge_lse(torch.stack([o0[:, :, 0], o1[:, :, 0]]), torch.stack([l0, l1]), return_lse=True)
    # the probabilities are rounded to bf16 relative to each run's own reference exponent, so the split and the
    # unsplit runs differ by that rounding noise (a few 1e-3), not bit for bit
    assert float((merged - full[:, :, 0]).abs().max()) <= 8e-3
    assert float((merged - full[:, :, 0]).abs().mean()) <= 5e-4
    assert float((mlse - lse).abs().max()) <= 1e-3
    want, wl = oracle.merge_lse(torch.stack([o0[:, :, 0], o1[:, :, 0]]), torch.stack([l0, l1]))
    assert float((merged - want).abs().max()) <= 1e-5 and float((mlse - wl).abs().max()) <= 1e-5


def test_host_buffer_entry_point():
    import polarquant_b200 as pq
    from polarquant_b200 import _lib
    lib = _lib.load()
    B, N, Nk, Nb, grp, R = 2, 8, 2, 3, 128, 21
    q, kres, quant, v = _make(B, N, Nk, Nb, grp, R, torch.bfloat16, 4, 4, seed=97)
    want = pq.decode_attention(q, kres, *quant, v)
    host = [t.cpu().contiguous().pin_memory() for t in (q, kres, *quant, v)]
    out = torch.empty(B, N, 1, 128, dtype=torch.bfloat16).pin_memory()
    p = _lib.DecodeParams()
    p.q, p.k_res, p.codes, p.rscale, p.rmn, p.tscale, p.tmn, p.v = (t.data_ptr() for t in host)
    p.out = out.data_ptr()
    p.B, p.N, p.Nk, p.Nb, p.G, p.R, p.hd = B, N, Nk, Nb, grp, R, 128
    p.rbits = p.tbits = 4
    p.qk_dtype = p.v_dtype = p.out_dtype = _lib.PQ_BF16
    need = lib.pq_decode_host_staging_bytes(B, N, Nk, Nb, grp, R, 128, _lib.PQ_BF16, _lib.PQ_BF16, _lib.PQ_BF16, 0)
    staging = torch.empty(need, dtype=torch.uint8, device="cuda")
    rc = lib.pq_decode_attention_host(ctypes.byref(p), staging.data_ptr(), need,
                                      ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.pq_strerror(rc)
    torch.cuda.synchronize()
    assert torch.equal(out.cuda(), want)
    # too small a staging area is refused, not overrun
    rc = lib.pq_decode_attention_host(ctypes.byref(p), staging.data_ptr(), need // 2,
                                      ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -3


def test_errors_are_reported_not_swallowed():
    import polarquant_b200 as pq
    q, kres, quant, v = _make(1, 8, 2, 1, 128, 4, torch.bfloat16, 4, 4, seed=98)
    with pytest.raises(ValueError):
        pq.decode_attention(q, kres, *quant, v[:, :, :-1])            # token count mismatch
    with pytest.raises(NotImplementedError):
        pq.decode_attention(q, kres, *quant, v, rbits=2, tbits=6)     # table wider than the kernel holds
    with pytest.raises(RuntimeError):
        pq.decode_attention(q.cpu(), kres.cpu(), *[t.cpu() for t in quant], v.cpu())


def test_decode_loop_with_requantisation_matches_the_eager_composition():
    """130 decode steps of one attention layer's cache logic, written as the reference's decode branch does it
    (models/modeling_llama_polar.py:61-101): append the new key to the residual window, attend, re-quantise the
    window when it reaches 128 tokens.  The CUDA path (fused attention + CUDA quantizer) must track the eager
    composition (oracle attention + the reference op sequence) at every step."""
    import polarquant_b200 as pq
    dev, dt = "cuda", torch.bfloat16
    B, N, Nk, grp = 2, 8, 2, 128
    g = torch.Generator(device=dev).manual_seed(99)
    prompt = 300                                        # 2 groups quantised at prefill, 44 keys left over
    keys = oracle.synth_keys(B, Nk, prompt, 128, dt, seed=100, device=dev)
    vals = torch.randn(B, Nk, prompt, 128, device=dev, generator=g).to(dt)
    nq = prompt - prompt % grp
    cache = list(pq.quantize_and_pack_nbit(keys[:, :, :nq].contiguous(), 4, 4, grp))
    ref_cache = list(oracle.quantize_ops(keys[:, :, :nq].contiguous(), 4, 4, grp))
    kres = keys[:, :, nq:]
    worst = 0.0
    for step in range(130):
        q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(dt)
        k_new = oracle.synth_keys(B, Nk, 1, 128, dt, seed=1000 + step, device=dev)
        v_new = torch.randn(B, Nk, 1, 128, device=dev, generator=g).to(dt)
        kres = torch.cat([kres, k_new], dim=2)
        vals = torch.cat([vals, v_new], dim=2)
        got = pq.decode_attention(q, kres, *cache, vals)
        want = oracle.decode_attention(q, kres, *ref_cache, vals)
        diff = (got.float() - want.float()).abs()
        worst = max(worst, float(diff.max()))
        assert float(diff.max()) <= ATTN_MAX_ABS and float(diff.mean()) <= ATTN_MEAN_ABS, step
        if kres.shape[2] % grp == 0:
            fresh = pq.quantize_and_pack_nbit(kres, 4, 4, grp)
            ref_fresh = oracle.quantize_ops(kres, 4, 4, grp)
            for a, b in zip(fresh, ref_fresh):
                assert torch.equal(a, b)
            cache = [torch.cat([a, b], dim=2) for a, b in zip(cache, fresh)]
            ref_cache = [torch.cat([a, b], dim=2) for a, b in zip(ref_cache, ref_fresh)]
            kres = kres[:, :, :0]
    assert cache[0].shape[2] == 3                        # one re-quantisation happened


def test_full_size_step():
    """Llama-3.1-8B decode shape: batch 16, 32 q / 8 kv heads, context 32768 (255 packed groups + 128 residual keys)."""
    import polarquant_b200 as pq
    B, N, Nk, Nb, grp, R = 16, 32, 8, 255, 128, 128
    g = torch.Generator(device="cuda").manual_seed(1002)
    scale = torch.exp(torch.empty(Nk, 128, device="cuda").uniform_(math.log(0.5), math.log(8.0), generator=g))
    q = torch.randn(B, N, 1, 128, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(B, Nk, Nb * grp + R, 128, device="cuda", generator=g).to(torch.bfloat16)
    kres = (torch.randn(B, Nk, R, 128, device="cuda", generator=g) * scale[None, :, None]).to(torch.bfloat16)
    quant = [[] for _ in range(5)]
    for b in range(B):                                   # quantise batch by batch to bound temporaries
        kb = (torch.randn(1, Nk, Nb * grp, 128, device="cuda", generator=g) * scale[None, :, None]).to(torch.bfloat16)
        for lst, t in zip(quant, pq.quantize_and_pack_nbit(kb, 4, 4, grp)):
            lst.append(t)
    quant = [torch.cat(lst, dim=0) for lst in quant]
    got = pq.decode_attention(q, kres, *quant, v)
    for b in range(0, B, 2):
        sl = slice(b, b + 2)
        want = oracle.decode_attention(q[sl], kres[sl], *[t[sl] for t in quant], v[sl])
        _check(got[sl], want, f"batch {b}")


def test_strided_merge_reads_an_all_gather_buffer_in_place():
    """pq_merge_lse_strided over [out | lse] blocks back to back equals pq_merge_lse over the tensors sliced apart."""
    import polarquant_b200 as pq
    from polarquant_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(55)
    parts, b, n = 3, 2, 8
    rows = b * n
    outs = torch.randn(parts, rows, 128, device="cuda", generator=g)
    lses = torch.randn(parts, rows, device="cuda", generator=g) * 3.0
    lses[1, 3] = float("-inf")                                   # a part without keys for that row
    gathered = torch.cat([torch.cat([outs[p].reshape(-1), lses[p]]) for p in range(parts)]).contiguous()
    want = pq.merge_lse(outs, lses, out_dtype=torch.bfloat16)
    got = ops.merge_lse_gathered(gathered, parts, rows, out_dtype=torch.bfloat16)
    assert torch.equal(got, want)
    ref, _ = oracle.merge_lse(outs.cpu(), lses.cpu())
    assert float((got.float().cpu() - ref).abs().max()) <= 2e-2
