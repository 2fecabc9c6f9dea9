"""CUDA QK-logits entry point (the drop-in for attention_decode_forward_triton_impl) against the oracle.

Tolerance: the kernel dequantises keys to fp16 before the tensor-core product, so each logit carries a
relative error of a few 2^-11 of the key magnitude.  Bar used here: max |diff| <= 2e-3 * max |logit| and
mean |diff| <= 4e-4 * max |logit| (after the 1/sqrt(128) scaling this is far inside the attention bar)."""
import pytest
import torch

from conftest import golden_names, load_golden
from oracle import polar_oracle as oracle

pytestmark = pytest.mark.gpu


def _check(got, want):
    assert got.shape == want.shape and got.dtype == torch.float32
    scale = max(1.0, float(want.abs().max()))
    diff = (got - want).abs()
    assert float(diff.max()) <= 2e-3 * scale, (float(diff.max()), scale)
    assert float(diff.mean()) <= 4e-4 * scale, (float(diff.mean()), scale)


@pytest.mark.parametrize("name", golden_names("qk_"))
def test_golden_logits_from_reference_kernel(name):
    import polarquant_b200 as pq
    g = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in load_golden(name).items()}
    rb, tb, _ = g["meta"]
    got = pq.attention_decode_forward_triton_impl(g["q"], g["indices"], g["rscale"], g["rmn"], g["tscale"],
                                                  g["tmn"], rbits=rb, tbits=tb)
    _check(got, g["logits"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("B,N,Nk,Nb,grp,rb,tb", [
    (2, 32, 8, 9, 128, 4, 4),      # Llama-3.1-8B grouping
    (2, 28, 4, 5, 128, 3, 3),      # Qwen2.5-7B grouping, 7 query heads per kv head
    (1, 28, 28, 3, 32, 2, 4),      # the Qwen patch passes repeated codes: Nk == N
    (3, 32, 32, 7, 32, 4, 4),      # benchmark_matmul.py: MHA, group 32
    (1, 64, 8, 3, 128, 4, 4),      # 8 query heads per kv head
    (1, 32, 2, 2, 64, 4, 3),       # 16 query heads per kv head: two head tiles
    (1, 8, 8, 1, 16, 3, 4),
])
def test_seeded_logits(dtype, B, N, Nk, Nb, grp, rb, tb):
    import polarquant_b200 as pq
    keys = oracle.synth_keys(B, Nk, Nb * grp, 128, dtype, seed=80 + Nb, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(81)
    q = torch.randn(B, N, 1, 128, device="cuda", generator=g).to(dtype)
    idx, rs, rm, ts, tm = oracle.quantize_ops(keys, rb, tb, grp)
    got = pq.attention_decode_forward_triton_impl(q, idx, rs, rm, ts, tm, rbits=rb, tbits=tb)
    _check(got, oracle.qk_logits(q, idx, rs, rm, ts, tm, rb, tb))


def test_arbitrary_codes_and_scales_like_the_reference_benchmark():
    """benchmark/benchmark_matmul.py:92-99 feeds random codes in [0, 250) and randn scales (negative too)."""
    import polarquant_b200 as pq
    g = torch.Generator(device="cuda").manual_seed(82)
    B, N, L, grp = 2, 32, 4096, 32
    q = torch.randn(B, N, 1, 128, device="cuda", generator=g).to(torch.float16)
    idx = torch.randint(0, 250, (B, N, L // grp, grp, 64), device="cuda", generator=g, dtype=torch.uint8)
    rs, rm, ts, tm = (torch.randn(B, N, L // grp, 1, 64, device="cuda", generator=g).to(torch.float16)
                      for _ in range(4))
    got = pq.attention_decode_forward_triton_impl(q, idx, rs, rm, ts, tm, rbits=4, tbits=4)
    _check(got, oracle.qk_logits(q, idx, rs, rm, ts, tm, 4, 4))


def test_keyword_call_as_the_attention_patch_makes_it():
    """models/modeling_llama_polar.py:66-75 passes tbits before rbits, both by keyword."""
    import polarquant_b200 as pq
    keys = oracle.synth_keys(1, 2, 256, 128, torch.bfloat16, seed=83, device="cuda")
    q = torch.randn(1, 8, 1, 128, device="cuda").to(torch.bfloat16)
    idx, rs, rm, ts, tm = oracle.quantize_ops(keys, 2, 4, 128)
    got = pq.attention_decode_forward_triton_impl(q, idx, rs, rm, ts, tm, tbits=4, rbits=2)
    _check(got, oracle.qk_logits(q, idx, rs, rm, ts, tm, 2, 4))
    # a query produced by the attention module: (B, 1, N, hd).transpose(1, 2)
    qt = q.reshape(1, 1, 8, 128).transpose(1, 2)
    got2 = pq.attention_decode_forward_triton_impl(qt, idx, rs, rm, ts, tm, tbits=4, rbits=2)
    assert torch.equal(got, got2)


def test_unsupported_bit_widths_fail_loudly():
    import polarquant_b200 as pq
    q = torch.randn(1, 2, 1, 128, device="cuda").to(torch.float16)
    idx = torch.zeros(1, 2, 1, 32, 64, dtype=torch.uint8, device="cuda")
    s = torch.ones(1, 2, 1, 1, 64, device="cuda").to(torch.float16)
    with pytest.raises(NotImplementedError):
        pq.attention_decode_forward_triton_impl(q, idx, s, s, s, s, rbits=2, tbits=6)


def test_full_size_logits():
    """Llama-3.1-8B shape: batch 16, 32 q / 8 kv heads, 32640 packed tokens, bf16, group 128."""
    import polarquant_b200 as pq
    g = torch.Generator(device="cuda").manual_seed(84)
    B, N, Nk, Nb, grp = 16, 32, 8, 255, 128
    q = torch.randn(B, N, 1, 128, device="cuda", generator=g).to(torch.bfloat16)
    idx = torch.randint(0, 256, (B, Nk, Nb, grp, 64), device="cuda", generator=g, dtype=torch.uint8)
    rs = (torch.rand(B, Nk, Nb, 1, 64, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    rm = torch.rand(B, Nk, Nb, 1, 64, device="cuda", generator=g).to(torch.bfloat16)
    ts = (torch.rand(B, Nk, Nb, 1, 64, device="cuda", generator=g) * 0.39).to(torch.bfloat16)
    tm = (torch.rand(B, Nk, Nb, 1, 64, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    got = pq.attention_decode_forward_triton_impl(q, idx, rs, rm, ts, tm)
    for b in range(0, B, 4):
        sl = slice(b, b + 4)
        _check(got[sl], oracle.qk_logits(q[sl], idx[sl], rs[sl], rm[sl], ts[sl], tm[sl], 4, 4))
