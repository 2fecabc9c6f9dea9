"""The 6-bit packed key container (48 bytes per token instead of 64, bit splits 3/3 and 2/4).

The reference keeps one byte per pair (models/modeling_llama_polar.py:155) and names packing as future work
(models/kernel4group.py:1-3), so the byte container stays the bit-exact contract; the packed container is an
opt-in second format that must be LOSSLESS against it: the repack kernels agree with the oracle's restatement of
the layout, the quantizer's direct output equals the packed form of its byte output, and the fused attention kernel
gives the same bits on either container.
"""
import pytest
import torch

from conftest import check_attn
from oracle import polar_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_repack_kernels_agree_with_the_layout_definition_and_round_trip():
    import polarquant_b200 as pq
    g = torch.Generator().manual_seed(61)
    codes = torch.randint(0, 64, (2, 3, 2, 128, 64), generator=g, dtype=torch.uint8)
    packed = pq.keys_repack(codes.to(DEV), "packed6")
    assert packed.shape == (2, 3, 2, 8, 768)
    want = oracle.pack_keys6(codes.reshape(2, 3, 256, 64)).reshape(2, 3, 2, 8, 768)
    assert torch.equal(packed.cpu(), want)
    back = pq.keys_repack(packed, "byte")
    assert back.shape == codes.shape and torch.equal(back.cpu(), codes)
    # bits above the sixth are dropped by the packing
    dirty = codes | 0xC0
    assert torch.equal(pq.keys_repack(dirty.to(DEV), "packed6").cpu(), want)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("group", [32, 128, 48])
@pytest.mark.parametrize("rbits,tbits", [(3, 3), (2, 4)])
def test_quantizer_writes_the_packed_container_directly(rbits, tbits, group, dt):
    import polarquant_b200 as pq
    L = group * 3
    base = oracle.synth_keys(2, L, 3, 128, dt, seed=70 + group, device=DEV)      # (B, L, Nk, hd) storage
    keys = base.transpose(1, 2)
    byte = pq.quantize_and_pack_nbit(keys, rbits, tbits, group)
    packed = pq.quantize_and_pack_nbit(keys, rbits, tbits, group, key_format="packed6")
    assert packed[0].shape == (2, 3, 3, group // 16, 768)
    assert torch.equal(packed[0], pq.keys_repack(byte[0], "packed6"))
    for a, b in zip(packed[1:], byte[1:]):
        assert torch.equal(a, b)
    # and the byte form is the reference's
    want = oracle.quantize_ops(keys, rbits, tbits, group)
    assert torch.equal(byte[0], want[0])


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("N,Nk,Nb,G,R,vq", [(8, 2, 5, 128, 37, False), (7, 1, 9, 32, 0, False), (32, 4, 3, 128, 128, True),
                                            (16, 2, 40, 128, 1, False)])
@pytest.mark.parametrize("rbits,tbits", [(3, 3), (2, 4)])
def test_attention_is_bit_identical_on_either_container(rbits, tbits, N, Nk, Nb, G, R, vq, dt):
    import polarquant_b200 as pq
    B = 2
    g = torch.Generator(device=DEV).manual_seed(80 + N)
    keys = oracle.synth_keys(B, Nk, Nb * G + R, 128, dt, seed=81, device=DEV)
    q = torch.randn(B, N, 1, 128, device=DEV, generator=g).to(dt)
    v = torch.randn(B, Nk, Nb * G + R, 128, device=DEV, generator=g).to(dt)
    kq = keys[:, :, :Nb * G].contiguous()
    kres = keys[:, :, Nb * G:].contiguous() if R else None
    byte = pq.quantize_and_pack_nbit(kq, rbits, tbits, G)
    packed = pq.quantize_and_pack_nbit(kq, rbits, tbits, G, key_format="packed6")
    kw = dict(rbits=rbits, tbits=tbits, return_lse=True)
    vv = v
    if vq:
        vc, vs, vm = pq.quantize_values(v[:, :, :Nb * G], layout="tiled")
        kw.update(value_codes=vc, value_scale=vs, value_mn=vm)
        vv = v[:, :, Nb * G:].contiguous()
    out_b, lse_b = pq.decode_attention(q, kres, *byte, vv, **kw)
    out_p, lse_p = pq.decode_attention(q, kres, *packed, vv, key_format="packed6", **kw)
    assert torch.equal(out_p, out_b) and torch.equal(lse_p, lse_b)
    if not vq:
        check_attn(out_p, oracle.decode_attention(q, kres, *byte, v, rbits=rbits, tbits=tbits), "packed vs oracle")


def test_other_bit_splits_are_refused_for_the_packed_container():
    import polarquant_b200 as pq
    keys = oracle.synth_keys(1, 1, 128, 128, torch.bfloat16, seed=90, device=DEV)
    with pytest.raises(ValueError):
        pq.quantize_and_pack_nbit(keys, 4, 4, 128, key_format="packed6")
    byte = pq.quantize_and_pack_nbit(keys, 4, 2, 128)
    q = torch.randn(1, 4, 1, 128, device=DEV).to(torch.bfloat16)
    with pytest.raises(NotImplementedError):              # 6 bits, but not a split the packed kernels are built for
        pq.decode_attention(q, None, pq.keys_repack(byte[0], "packed6"), *byte[1:], keys, rbits=4, tbits=2,
                            key_format="packed6")


def test_packed_container_at_the_qwen_shaped_full_size():
    """Batch 64, 28 q / 4 kv heads, context 8192, 3/3, group 128: 48 instead of 64 key bytes per token."""
    import polarquant_b200 as pq
    B, N, Nk, ctx, R, G = 64, 28, 4, 8192, 128, 128
    Lq = ctx - R
    g = torch.Generator(device=DEV).manual_seed(1003)
    q = torch.randn(B, N, 1, 128, device=DEV, generator=g).to(torch.bfloat16)
    v = torch.randn(B, Nk, ctx, 128, device=DEV, generator=g).to(torch.bfloat16)
    keys = (torch.randn(B, Nk, ctx, 128, device=DEV, generator=g) * 2.0).to(torch.bfloat16)
    kq, kres = keys[:, :, :Lq].contiguous(), keys[:, :, Lq:].contiguous()
    byte = pq.quantize_and_pack_nbit(kq, 3, 3, G)
    packed = pq.quantize_and_pack_nbit(kq, 3, 3, G, key_format="packed6")
    assert packed[0].numel() * 4 == byte[0].numel() * 3
    assert torch.equal(pq.keys_repack(packed[0], "byte"), byte[0])
    a = pq.decode_attention(q, kres, *byte, v, rbits=3, tbits=3)
    b = pq.decode_attention(q, kres, *packed, v, rbits=3, tbits=3, key_format="packed6")
    assert torch.equal(a, b)


@pytest.mark.parametrize("vbits", [0, 4])
def test_in_place_cache_on_the_packed_container_tracks_the_byte_cache(vbits):
    """PolarKVCache(key_format='packed6'): prefill, eager decode steps across a window boundary and the replayed
    CUDA graph with device-side lengths all give the bits of the byte-container cache."""
    from polarquant_b200.cache import PolarKVCache
    dt = torch.bfloat16
    B, N, Nk, prompt, steps = 2, 8, 2, 300, 100
    g = torch.Generator(device=DEV).manual_seed(123)
    keys = oracle.synth_keys(B, prompt, Nk, 128, dt, seed=124, device=DEV).transpose(1, 2)
    vals = torch.randn(B, prompt, Nk, 128, device=DEV, generator=g).to(dt).transpose(1, 2)
    caches = []
    for fmt in ("byte", "packed6"):
        lengths = torch.zeros(2, dtype=torch.int32, device=DEV)
        c = PolarKVCache(B, Nk, max_tokens=prompt + steps + 128, dtype=dt, rbits=3, tbits=3, vbits=vbits,
                         lengths=lengths, key_format=fmt)
        c.prefill(keys, vals)
        caches.append(c)
    for step in range(steps):
        q = torch.randn(B, N, 1, 128, device=DEV, generator=g).to(dt)
        k_new = oracle.synth_keys(B, Nk, 1, 128, dt, seed=3000 + step, device=DEV)
        v_new = torch.randn(B, Nk, 1, 128, device=DEV, generator=g).to(dt)
        if step % 3 == 1:
            outs = [c.decode_step(q, k_new, v_new) for c in caches]
        elif step % 3 == 2:                        # everything on the device: append, attend, re-quantise, advance
            outs = []
            for c in caches:
                outs.append(c.decode_step_graph(q, k_new, v_new))
                c.requantize_graph()
                c.advance_graph()
                c.after_replay(device_requantized=True)
        else:                                      # the device-side-lengths path with the host re-quantising
            outs = []
            for c in caches:
                outs.append(c.decode_step_graph(q, k_new, v_new))
                c.lengths[1:2].add_(1)
                if c.after_replay():
                    c.sync_lengths()
        assert torch.equal(outs[0], outs[1]), step
    ta, tb = caches[0].as_reference_tuple(), caches[1].as_reference_tuple()
    assert caches[1].codes.shape[-1] == 768 and caches[1].codes.numel() * 4 == caches[0].codes.numel() * 3
    for x, y in zip(ta[1:6], tb[1:6]):
        assert torch.equal(x, y)
