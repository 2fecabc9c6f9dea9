"""Packed value cache on the GPU, through the C ABI: the per-token 4-bit quantiser bit-exact against the op chain
torch executes on the same device, both code layouts, the dequantise-and-multiply, and the fused decode attention
over packed keys AND packed values against the composed oracle and the fixtures made by the reference's
LlamaPolarMixedGroupAttention forward."""
import pytest
import torch

from conftest import ATTN_MAX_ABS, ATTN_MEAN_ABS, check_attn, check_mixed, golden_names, load_golden
from oracle import polar_oracle as oracle

pytestmark = pytest.mark.gpu


def _values(B, Nk, T, dtype, seed, kind="spread"):
    g = torch.Generator(device="cuda").manual_seed(seed)
    v = torch.randn(B, Nk, T, 128, device="cuda", generator=g)
    if kind == "spread":
        # per-token spread and offset, magnitudes of order one: with much larger values the reference's own
        # roundings of the probabilities (to bf16) move the output by more than the absolute bar of 2e-2
        v = v * (0.05 + 1.5 * torch.rand(B, Nk, T, 1, device="cuda", generator=g)) \
            + 0.3 * torch.randn(B, Nk, T, 1, device="cuda", generator=g)
    return v.to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("B,Nk,T", [(2, 3, 200), (1, 8, 4096), (3, 2, 1), (1, 1, 63)])
def test_quantiser_equals_the_torch_op_chain_on_this_device(dtype, B, Nk, T):
    import polarquant_b200 as pq
    v = _values(B, Nk, T, dtype, seed=11 + T)
    if T > 5:
        v[0, 0, 3] = 1.5                                  # constant token
        v[0, 0, 4, 7] = 300.0                             # outlier
    codes, scale, mn = pq.quantize_values(v)
    # torch on this device executes `/ 15` its own way ("true" leaves it to torch); the restated rule agrees
    want_c, want_s, want_m = oracle.quantize_values(v, scalar_division="true")
    rule_c, rule_s, _ = oracle.quantize_values(v, scalar_division="reciprocal")
    assert torch.equal(want_s, rule_s) and torch.equal(want_c, rule_c), "scalar-division rule does not hold here"
    assert torch.equal(mn, want_m) and torch.equal(scale, want_s)
    assert torch.equal(codes, want_c)
    # CPU execution of the same chain (what the committed fixtures were made with)
    cpu_c, cpu_s, cpu_m = oracle.quantize_values(v.cpu())
    assert torch.equal(cpu_s, scale.cpu()) and torch.equal(cpu_m, mn.cpu()) and torch.equal(cpu_c, codes.cpu())
    tiled, s2, m2 = pq.quantize_values(v, layout="tiled")
    assert torch.equal(s2, scale) and torch.equal(m2, mn)
    assert torch.equal(tiled, oracle.kivi_to_tiled(codes))
    assert torch.equal(pq.values_relayout(codes, "tiled"), tiled)
    assert torch.equal(pq.values_relayout(tiled, "kivi"), codes)


def test_quantiser_reads_strided_prefill_views_and_rejects_nothing_silently():
    import polarquant_b200 as pq
    base = _values(2, 300, 4, torch.bfloat16, seed=5)            # (B, L, Nk, hd) as the projection writes it
    v = base.transpose(1, 2)                                     # (B, Nk, L, hd) view
    codes, scale, mn = pq.quantize_values(v)
    want = oracle.quantize_values(v.contiguous())
    assert torch.equal(codes, want[0]) and torch.equal(scale, want[1]) and torch.equal(mn, want[2])
    with pytest.raises(NotImplementedError):
        pq.quantize_values(v, vbits=2)


def test_nan_and_inf_tokens_follow_torch():
    import polarquant_b200 as pq
    v = _values(1, 2, 16, torch.bfloat16, seed=6)
    v[0, 0, 1, 5] = float("nan")
    v[0, 0, 2, 9] = float("inf")
    v[0, 1, 3, 0] = float("-inf")
    got = pq.quantize_values(v)
    want = oracle.quantize_values(v, scalar_division="true")
    assert torch.equal(got[0], want[0])
    for a, b in zip(got[1:], want[1:]):
        assert torch.equal(torch.nan_to_num(a.float(), nan=123.0), torch.nan_to_num(b.float(), nan=123.0))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_values_matmul(dtype):
    import polarquant_b200 as pq
    B, H, T = 2, 6, 777
    v = _values(B, H, T, dtype, seed=21)
    codes, scale, mn = pq.quantize_values(v)
    p = torch.softmax(torch.randn(B, H, 1, T, device="cuda") * 3, -1).to(dtype)
    got = pq.values_matmul(p, codes, scale, mn)
    want = torch.matmul(p.float(), oracle.dequantize_values(codes, scale, mn))
    assert got.dtype == dtype and got.shape == (B, H, 1, 128)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((got.float() - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))
    # a non-contiguous slice of a longer probability row, as at models/modeling_llama_polar.py:232
    wide = torch.cat([p, torch.zeros(B, H, 1, 5, device="cuda", dtype=dtype)], -1)
    assert torch.equal(pq.values_matmul(wide[..., :-5], codes, scale, mn), got)


def _make(B, N, Nk, Nb, grp, R, dtype, rb, tb, seed):
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(seed)
    ctx = Nb * grp + R
    keys = oracle.synth_keys(B, Nk, max(ctx, 1), 128, dtype, seed=seed + 1, device=dev)
    q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(dtype)
    v = _values(B, Nk, ctx, dtype, seed + 2)
    quant = oracle.quantize_ops(keys[:, :, :Nb * grp].contiguous(), rb, tb, grp)
    kres = keys[:, :, Nb * grp:ctx].contiguous() if R else None
    return q, kres, quant, v


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,N,Nk,Nb,grp,R,rb,tb", [
    (2, 32, 8, 15, 128, 128, 4, 4),    # Llama-3.1-8B grouping, full residual window
    (2, 32, 8, 15, 128, 1, 4, 4),      # first step after a re-quantisation
    (2, 28, 4, 7, 128, 77, 4, 4),      # 7 heads per kv head
    (2, 28, 4, 28, 32, 100, 3, 3),
    (1, 32, 32, 31, 128, 128, 2, 4),   # MHA
    (1, 32, 2, 3, 64, 5, 4, 3),        # 16 heads per kv head: two head tiles
    (3, 8, 2, 5, 16, 0, 4, 4),         # no residual window at all
    (1, 8, 2, 260, 128, 128, 4, 4),    # 33k tokens: every warp range starts mid-unit
])
def test_fused_attention_with_packed_values(dtype, B, N, Nk, Nb, grp, R, rb, tb):
    import polarquant_b200 as pq
    q, kres, quant, v = _make(B, N, Nk, Nb, grp, R, dtype, rb, tb, seed=300 + Nb + R)
    tq = Nb * grp
    vc, vs, vm = pq.quantize_values(v[:, :, :tq], layout="tiled")
    v_res = v[:, :, tq:].contiguous() if R else None
    got, lse = pq.decode_attention(q, kres, *quant, v_res, rbits=rb, tbits=tb, return_lse=True,
                                   value_codes=vc, value_scale=vs, value_mn=vm)
    args = (q.cpu(), None if kres is None else kres.cpu(), *(t.cpu() for t in quant), vc.cpu(), vs.cpu(), vm.cpu(),
            None if v_res is None else v_res.cpu())
    # The reference rounds the probabilities to the tensor dtype and the packed part, the residual part and their
    # sum separately (models/modeling_llama_polar.py:225,237-239).  The fused kernel keeps fp32 (fp16 for the
    # packed product's probabilities), so the seeded cases compare with all-fp32 arithmetic over the same packed
    # cache, rounded once; the reference's own roundings are covered by the forward fixtures below.
    exact, wlse = oracle.decode_attention_mixed(*args, rbits=rb, tbits=tb, layout="tiled", faithful_rounding=False,
                                                return_lse=True)
    check_attn(got.cpu(), exact.to(dtype))
    assert float((lse.cpu() - wlse).abs().max()) <= 2e-2
    got32 = pq.decode_attention(q, kres, *quant, v_res, rbits=rb, tbits=tb, out_dtype=torch.float32,
                                value_codes=vc, value_scale=vs, value_mn=vm)
    diff = (got32.cpu() - exact).abs()
    assert float(diff.max()) <= ATTN_MAX_ABS and float(diff.mean()) <= ATTN_MEAN_ABS, (float(diff.max()), float(diff.mean()))
    # and packed values are what they claim to be: close to attention over the unpacked values
    full = pq.decode_attention(q, kres, *quant, v, rbits=rb, tbits=tb, out_dtype=torch.float32)
    step = float(vs.float().max())
    assert float((got32 - full).abs().max()) <= 0.6 * step + 2e-2


@pytest.mark.parametrize("name", golden_names("attn_mixed_"))
def test_outputs_of_the_reference_mixed_forward(name):
    import polarquant_b200 as pq
    g = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in load_golden(name).items()}
    rb, tb, _, vb = g["meta"]
    mask = g["mask"] if g["mask"].numel() else None
    tiled = pq.values_relayout(g["v_codes"], "tiled")
    got = pq.decode_attention(g["q"], g["k_res"], g["indices"], g["rscale"], g["rmn"], g["tscale"], g["tmn"],
                              g["v_res"], attention_mask=mask, rbits=rb, tbits=tb, value_codes=tiled,
                              value_scale=g["v_scale"], value_mn=g["v_mn"], vbits=vb)
    assert got.dtype == g["q"].dtype
    check_mixed(got, g["out"], name)


def test_packed_values_reproducible_and_masked():
    import polarquant_b200 as pq
    q, kres, quant, v = _make(3, 8, 2, 4, 128, 60, torch.bfloat16, 4, 4, seed=92)
    tq = 512
    vc, vs, vm = pq.quantize_values(v[:, :, :tq], layout="tiled")
    v_res = v[:, :, tq:].contiguous()
    mask = torch.ones(3, tq + 60, device="cuda")
    mask[0, :200] = 0
    mask[2, :513] = 0
    kw = dict(value_codes=vc, value_scale=vs, value_mn=vm, attention_mask=mask)
    a = pq.decode_attention(q, kres, *quant, v_res, **kw)
    b = pq.decode_attention(q, kres, *quant, v_res, **kw)
    assert torch.equal(a, b)
    want = oracle.decode_attention_mixed(q.cpu(), kres.cpu(), *(t.cpu() for t in quant), vc.cpu(), vs.cpu(), vm.cpu(),
                                         v_res.cpu(), attention_mask=mask.cpu(), layout="tiled")
    # two of the three sequences attend mostly to the residual window, whose logits the reference (and the kernel)
    # rounds to bf16: the composition with all of the reference's roundings is the comparison that applies
    check_mixed(a.cpu(), want)
    # dtype mismatch between keys and values is refused, not converted behind the caller's back
    with pytest.raises(NotImplementedError):
        pq.decode_attention(q.half(), kres.half(), quant[0], *(t.half() for t in quant[1:]), v_res,
                            value_codes=vc, value_scale=vs, value_mn=vm)


def test_full_size_step_with_packed_values():
    """The benchmark shape (batch 16, 32 q / 8 kv heads, context 32768): the packed-value kernel against the
    full-precision-value kernel fed with the dequantised values, reproducibility, and the sequence split + merge."""
    import math
    import polarquant_b200 as pq
    B, N, Nk, Nb, grp, R = 16, 32, 8, 255, 128, 128
    dev, dt = "cuda", torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(1002)
    scale = torch.exp(torch.empty(Nk, 128, device=dev).uniform_(math.log(0.5), math.log(8.0), generator=g))
    q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(dt)
    v = torch.randn(B, Nk, Nb * grp + R, 128, device=dev, generator=g).to(dt)
    kres = (torch.randn(B, Nk, R, 128, device=dev, generator=g) * scale[None, :, None]).to(dt)
    quant = [[] for _ in range(5)]
    for b in range(B):
        kb = (torch.randn(1, Nk, Nb * grp, 128, device=dev, generator=g) * scale[None, :, None]).to(dt)
        for lst, t in zip(quant, pq.quantize_and_pack_nbit(kb, 4, 4, grp)):
            lst.append(t)
    quant = [torch.cat(lst, dim=0) for lst in quant]
    tq = Nb * grp
    vc, vs, vm = pq.quantize_values(v[:, :, :tq], layout="tiled")
    kivi = pq.values_relayout(vc, "kivi")
    assert torch.equal(pq.values_relayout(kivi, "tiled"), vc)
    v_res = v[:, :, tq:].contiguous()
    kw = dict(value_codes=vc, value_scale=vs, value_mn=vm)
    got = pq.decode_attention(q, kres, *quant, v_res, out_dtype=torch.float32, **kw)
    assert torch.equal(got, pq.decode_attention(q, kres, *quant, v_res, out_dtype=torch.float32, **kw))
    # the same attention over the dequantised values (batch slices bound the fp32 temporaries)
    for b in range(0, B, 4):
        sl = slice(b, b + 4)
        v_hat = oracle.dequantize_values(kivi[sl], vs[sl], vm[sl])
        v_hat = torch.cat([v_hat.to(dt), v_res[sl]], dim=2)
        want = pq.decode_attention(q[sl], kres[sl], *[t[sl] for t in quant], v_hat, out_dtype=torch.float32)
        diff = (got[sl] - want).abs()
        assert float(diff.max()) <= ATTN_MAX_ABS and float(diff.mean()) <= ATTN_MEAN_ABS, (b, float(diff.max()))
    # split after 128 groups: two calls with log-sum-exp, merged
    h = 128
    o0, l0 = pq.decode_attention(q, None, *[t[:, :, :h] for t in quant], None, out_dtype=torch.float32,
                                 return_lse=True, value_codes=vc[:, :, :h * grp], value_scale=vs[:, :, :h * grp],
                                 value_mn=vm[:, :, :h * grp])
    o1, l1 = pq.decode_attention(q, kres, *[t[:, :, h:] for t in quant], v_res, out_dtype=torch.float32,
                                 return_lse=True, value_codes=vc[:, :, h * grp:], value_scale=vs[:, :, h * grp:],
                                 value_mn=vm[:, :, h * grp:])
    merged = pq.merge_lse(torch.stack([o0[:, :, 0], o1[:, :, 0]]), torch.stack([l0, l1]))
    assert float((merged - got[:, :, 0]).abs().max()) <= 8e-3
