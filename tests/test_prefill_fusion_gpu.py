"""Prefill-side fusion: rotary embedding and polar quantisation of the prompt's keys in one kernel.

The reference rotates the keys with the eager ``apply_rotary_pos_emb`` (models/modeling_llama_polar.py:57), attends,
and then quantises all but the last L % 128 keys (:116-126).  The fused entry must reproduce both steps bit for bit:
the rotated keys equal ``k * cos + rotate_half(k) * sin`` evaluated by torch on the same GPU, and codes and scales
equal the reference quantizer's op chain (``oracle.quantize_ops``, executed by torch on the GPU) applied to those
rotated keys.
"""
import pytest
import torch

from oracle import polar_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rotate_half(x):
    half = x.shape[-1] // 2
    return torch.cat([-x[..., half:], x[..., :half]], dim=-1)


def rope_tables(length, dtype, batch=None, theta=500000.0):
    inv = 1.0 / (theta ** (torch.arange(0, 128, 2, device=DEV, dtype=torch.float32) / 128))
    pos = torch.arange(length, device=DEV, dtype=torch.float32)
    if batch:
        pos = pos[None] + torch.arange(batch, device=DEV, dtype=torch.float32)[:, None] * 7.0
    ang = pos[..., None] * inv
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos().to(dtype), ang.sin().to(dtype)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("L,G,rb,tb,per_batch", [(300, 128, 4, 4, False), (256, 128, 4, 4, True), (100, 128, 4, 4, False),
                                                 (384, 32, 3, 3, False), (640, 64, 2, 4, True)])
def test_fused_rotation_and_quantisation_equal_the_two_eager_steps(dt, L, G, rb, tb, per_batch):
    import polarquant_b200 as pq
    B, Nk = 2, 3
    base = oracle.synth_keys(B, L, Nk, 128, dt, seed=L + G, device=DEV)        # (B, L, Nk, hd) projection layout
    keys = base.transpose(1, 2)
    cos, sin = rope_tables(L, dt, batch=B if per_batch else None)
    c4, s4 = (cos[:, None], sin[:, None]) if per_batch else (cos[None, None], sin[None, None])
    want_rot = keys * c4 + rotate_half(keys) * s4                              # the eager ops, rounded as torch rounds
    lq = L - L % 128
    rot, packed = pq.rope_quantize(keys, cos, sin, rb, tb, G)
    assert rot.shape == keys.shape and torch.equal(rot, want_rot)
    assert rot.stride() == keys.stride()                                       # same (strided) layout as the input
    if lq:
        want = oracle.quantize_ops(want_rot[:, :, :lq], rb, tb, G)
        for name, a, b in zip(("codes", "rscale", "rmn", "tscale", "tmn"), packed, want):
            assert torch.equal(a, b), name
    else:
        assert packed[0].shape[2] == 0
    # in place: the rotated keys overwrite the input
    work = base.clone().transpose(1, 2)
    rot2, packed2 = pq.rope_quantize(work, cos, sin, rb, tb, G, out=work)
    assert rot2.data_ptr() == work.data_ptr() and torch.equal(work, want_rot)
    assert all(torch.equal(a, b) for a, b in zip(packed2, packed))


def test_fused_prefill_fills_the_cache_like_the_two_step_prefill():
    import polarquant_b200 as pq
    from polarquant_b200.cache import PolarKVCache
    dt = torch.bfloat16
    B, Nk, L = 2, 2, 300
    base = oracle.synth_keys(B, L, Nk, 128, dt, seed=5, device=DEV)
    keys = base.transpose(1, 2)
    vals = torch.randn(B, L, Nk, 128, device=DEV).to(dt).transpose(1, 2)
    cos, sin = rope_tables(L, dt)
    rot_ref = keys * cos[None, None] + rotate_half(keys) * sin[None, None]
    a = PolarKVCache(B, Nk, max_tokens=512, dtype=dt)
    a.prefill(rot_ref, vals)
    b = PolarKVCache(B, Nk, max_tokens=512, dtype=dt)
    rot = b.prefill_rope(keys, vals, cos, sin)
    assert torch.equal(rot, rot_ref)
    for x, y in zip(a.as_reference_tuple()[:7], b.as_reference_tuple()[:7]):
        assert torch.equal(x, y)
    q = torch.randn(B, 8, 1, 128, device=DEV).to(dt)
    k1 = oracle.synth_keys(B, Nk, 1, 128, dt, seed=6, device=DEV)
    v1 = torch.randn(B, Nk, 1, 128, device=DEV).to(dt)
    assert torch.equal(a.decode_step(q, k1, v1), b.decode_step(q, k1, v1))


def test_packed_container_and_full_size_prefill():
    """3/3 codes straight into the 48-byte container, and the Llama-3.1-8B prefill shape (batch 16 x 8 kv heads x
    32768 tokens, strided) against the two-step path."""
    import polarquant_b200 as pq
    dt = torch.bfloat16
    keys = oracle.synth_keys(1, 256, 2, 128, dt, seed=9, device=DEV).transpose(1, 2)
    cos, sin = rope_tables(256, dt)
    rot, packed = pq.rope_quantize(keys, cos, sin, 3, 3, 128, key_format="packed6")
    want = pq.quantize_and_pack_nbit(rot, 3, 3, 128, key_format="packed6")
    assert all(torch.equal(a, b) for a, b in zip(packed, want))
    torch.manual_seed(3)
    base = torch.randn(16, 32768, 8, 128, device=DEV, dtype=torch.float32).to(dt)
    keys = base.transpose(1, 2)
    cos, sin = rope_tables(32768, dt)
    rot, packed = pq.rope_quantize(keys, cos, sin, 4, 4, 128)
    for b in range(0, 16, 4):
        want_rot = keys[b:b + 4] * cos[None, None] + rotate_half(keys[b:b + 4]) * sin[None, None]
        assert torch.equal(rot[b:b + 4], want_rot)
    want = pq.quantize_and_pack_nbit(rot, 4, 4, 128)
    assert all(torch.equal(a, b) for a, b in zip(packed, want))
