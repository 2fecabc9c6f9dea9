"""The preallocated in-place cache against the reference-style growing cache (torch.cat + eager composition)."""
import pytest
import torch

from conftest import ATTN_MAX_ABS, ATTN_MEAN_ABS
from oracle import polar_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("prompt,steps,grp", [(300, 140, 128), (128, 130, 128), (7, 260, 128), (200, 70, 32)])
def test_in_place_cache_tracks_the_growing_cache(prompt, steps, grp):
    import polarquant_b200 as pq
    from polarquant_b200.cache import PolarKVCache
    dev, dt = "cuda", torch.bfloat16
    B, N, Nk = 2, 8, 2
    g = torch.Generator(device=dev).manual_seed(300 + prompt)
    # prompt keys / values in the (B, L, Nk, hd) layout of the projections
    k_blnh = oracle.synth_keys(B, prompt, Nk, 128, dt, seed=301, device=dev)
    v_blnh = torch.randn(B, prompt, Nk, 128, device=dev, generator=g).to(dt)
    keys, vals = k_blnh.transpose(1, 2), v_blnh.transpose(1, 2)

    cache = PolarKVCache(B, Nk, max_tokens=prompt + steps + 128, dtype=dt, group_size=grp)
    cache.prefill(keys, vals)

    # reference-style state: quantise the prompt's full windows, keep the rest, grow by concatenation
    nq = prompt - prompt % 128
    ref = list(oracle.quantize_ops(keys[:, :, :nq].contiguous(), 4, 4, grp)) if nq else None
    kres = keys[:, :, nq:].contiguous()
    v_all = vals.contiguous()
    for step in range(steps):
        q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(dt)
        k_new = oracle.synth_keys(B, Nk, 1, 128, dt, seed=2000 + step, device=dev)
        v_new = torch.randn(B, Nk, 1, 128, device=dev, generator=g).to(dt)
        got = cache.decode_step(q, k_new, v_new)
        kres = torch.cat([kres, k_new], dim=2)
        v_all = torch.cat([v_all, v_new], dim=2)
        want = oracle.decode_attention(q, kres, *(ref or (None,) * 5), v_all)
        diff = (got.float() - want.float()).abs()
        assert float(diff.max()) <= 3.2e-2 and float(diff.mean()) <= ATTN_MEAN_ABS, (step, float(diff.max()))
        # the same CUDA kernels on the growing cache give the same bits as on the in-place cache
        same = pq.decode_attention(q, kres, *(ref or (None,) * 5), v_all)
        assert torch.equal(got, same), step
        if kres.shape[2] % 128 == 0:
            fresh = oracle.quantize_ops(kres, 4, 4, grp)
            ref = [torch.cat([a, b], dim=2) for a, b in zip(ref, fresh)] if ref else list(fresh)
            kres = kres[:, :, :0]
        assert cache.seq_len == prompt + step + 1
    # codes and scales written in place equal the reference's concatenated ones, bit for bit
    tup = cache.as_reference_tuple()
    if ref:
        for a, b in zip(tup[1:6], ref):
            assert torch.equal(a, b)
    assert torch.equal(tup[6], v_all)


def test_cache_refuses_to_overflow():
    from polarquant_b200.cache import PolarKVCache
    cache = PolarKVCache(1, 1, max_tokens=128)
    k = torch.randn(1, 1, 128, 128, device="cuda").to(torch.bfloat16)
    cache.prefill(k, k)
    q = torch.randn(1, 4, 1, 128, device="cuda").to(torch.bfloat16)
    with pytest.raises(RuntimeError):
        cache.decode_step(q, k[:, :, :1], k[:, :, :1])
