"""Parity at the full sizes of the benchmark configurations that the small-shape tests do not reach.

* Qwen2.5-7B-shaped sweep: batch 64, 28 query / 4 kv heads (7 query heads per kv head), context 8192, bf16,
  radius/angle bits {4/4, 3/3, 2/4} x token group {32, 128}.  Codes and scales must be bit-identical to the
  reference's op chain (models/modeling_llama_polar.py:135-157) executed by torch on the same GPU; attention
  outputs must be within max-abs 2e-2 / mean-abs 2e-3 of the reference's dequantise-then-matmul decode branch
  (models/modeling_llama_polar.py:77-99, restated by the oracle), checked in batch slices to bound temporaries.
* Llama-3.1-70B-shaped long context as one GPU of eight sees it: batch 8, 8 query heads on 1 kv head, context
  131072.  Only 8 (batch, kv head) units of 8192 steps each exist, so every unit is cut over ~55 CTAs: the extreme
  of the work-split arithmetic.  The result must not depend on the number of CTAs beyond the order of the merge.
"""
import math

import pytest
import torch

from conftest import check_attn
from oracle import polar_oracle as oracle

pytestmark = pytest.mark.gpu


def _synth(B, Nk, tokens, seed, dev="cuda"):
    """Keys: randn times a per-(kv head, channel) scale drawn log-uniform in [0.5, 8]."""
    g = torch.Generator(device=dev).manual_seed(seed)
    scale = torch.exp(torch.empty(Nk, 128, device=dev).uniform_(math.log(0.5), math.log(8.0), generator=g))
    return g, scale


@pytest.mark.parametrize("group", [32, 128])
@pytest.mark.parametrize("rbits,tbits", [(4, 4), (3, 3), (2, 4)])
def test_qwen_shaped_sweep_at_full_size(rbits, tbits, group):
    import polarquant_b200 as pq
    B, N, Nk, ctx, R = 64, 28, 4, 8192, 128
    Lq = ctx - R
    g, scale = _synth(B, Nk, ctx, 1003)
    q = torch.randn(B, N, 1, 128, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(B, Nk, ctx, 128, device="cuda", generator=g).to(torch.bfloat16)
    keys = (torch.randn(B, Nk, ctx, 128, device="cuda", generator=g) * scale[None, :, None]).to(torch.bfloat16)
    kq = keys[:, :, :Lq].contiguous()
    kres = keys[:, :, Lq:].contiguous()
    packed = pq.quantize_and_pack_nbit(kq, rbits, tbits, group)
    step = 8
    for b in range(0, B, step):                          # the eager op chain holds ~10 full-size temporaries
        want = oracle.quantize_ops(kq[b:b + step], rbits, tbits, group)
        for name, a, w in zip(("codes", "rscale", "rmn", "tscale", "tmn"), packed, want):
            assert torch.equal(a[b:b + step], w), (name, b)
    got = pq.decode_attention(q, kres, *packed, v, rbits=rbits, tbits=tbits)
    for b in range(0, B, step):
        sl = slice(b, b + step)
        want = oracle.decode_attention(q[sl], kres[sl], *[t[sl] for t in packed], v[sl], rbits=rbits, tbits=tbits)
        check_attn(got[sl], want, f"{rbits}/{tbits} G{group} batch {b}")


def test_long_context_one_kv_head_per_gpu_shape():
    import polarquant_b200 as pq
    B, N, Nk, ctx, R, G = 8, 8, 1, 131072, 128, 128
    Lq = ctx - R
    g, scale = _synth(B, Nk, ctx, 1005)
    q = torch.randn(B, N, 1, 128, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(B, Nk, ctx, 128, device="cuda", generator=g).to(torch.bfloat16)
    kres = (torch.randn(B, Nk, R, 128, device="cuda", generator=g) * scale[None, :, None]).to(torch.bfloat16)
    parts = [[] for _ in range(5)]
    for b in range(B):
        kb = (torch.randn(1, Nk, Lq, 128, device="cuda", generator=g) * scale[None, :, None]).to(torch.bfloat16)
        for lst, t in zip(parts, pq.quantize_and_pack_nbit(kb, 4, 4, G)):
            lst.append(t)
    packed = [torch.cat(lst, dim=0) for lst in parts]
    got = pq.decode_attention(q, kres, *packed, v)
    for b in range(0, B, 2):
        sl = slice(b, b + 2)
        want = oracle.decode_attention(q[sl], kres[sl], *[t[sl] for t in packed], v[sl])
        check_attn(got[sl], want, f"batch {b}")
    # the split over CTAs changes only the order in which partial sums are merged
    ref32 = pq.decode_attention(q, kres, *packed, v, out_dtype=torch.float32)
    for ctas in (1, 148, 444, 1000):
        o = pq.decode_attention(q, kres, *packed, v, out_dtype=torch.float32, num_ctas=ctas)
        d = (o - ref32).abs()
        assert float(d.max()) <= 2e-3 and float(d.mean()) <= 2e-4, (ctas, float(d.max()), float(d.mean()))
    # the same call twice gives the same bits
    assert torch.equal(ref32, pq.decode_attention(q, kres, *packed, v, out_dtype=torch.float32))
