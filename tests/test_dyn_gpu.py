"""Device-side lengths through the C ABI: for a sweep of (groups, residual) states of one preallocated cache the
kernels that read the lengths on the device give the bits of the kernels that were handed the lengths by the host,
and lengths beyond the capacity are clamped instead of followed."""
import ctypes

import pytest
import torch

from oracle import polar_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("vbits", [0, 4])
@pytest.mark.parametrize("N,Nk", [(8, 2), (7, 1), (32, 2)])
def test_every_length_matches_the_host_planned_call(vbits, N, Nk):
    import polarquant_b200 as pq
    from polarquant_b200 import _lib, ops
    dev, dt = "cuda", torch.bfloat16
    B, G, cap_groups, RL = 2, 128, 6, 128
    g = torch.Generator(device=dev).manual_seed(31 + N)
    keys = oracle.synth_keys(B, Nk, cap_groups * G, 128, dt, seed=32, device=dev)
    packed = pq.quantize_and_pack_nbit(keys, 4, 4, G)
    kres = oracle.synth_keys(B, Nk, RL, 128, dt, seed=33, device=dev)
    v = torch.randn(B, Nk, cap_groups * G + RL, 128, device=dev, generator=g).to(dt)
    q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(dt)
    lib = _lib.load()
    ws = torch.empty(lib.pq_decode_workspace_bytes_dyn(B, N, Nk, 0) + 256, dtype=torch.uint8, device=dev)
    lengths = torch.zeros(2, dtype=torch.int32, device=dev)
    vq = pq.quantize_values(v[:, :, :cap_groups * G], layout="tiled") if vbits else None

    def dyn_call(nb, r):
        """All buffers at capacity; only the device-side lengths say how much of them is live."""
        p = _lib.DecodeParams()
        q3 = q.reshape(B, N, 128)
        out = torch.empty(B, N, 1, 128, dtype=dt, device=dev)
        p.q, p.q_stride_b, p.q_stride_h = q3.data_ptr(), q3.stride(0), q3.stride(1)
        p.codes, p.codes_stride_b, p.codes_stride_h = packed[0].data_ptr(), packed[0].stride(0), packed[0].stride(1)
        p.rscale, p.rmn, p.tscale, p.tmn = (t.data_ptr() for t in packed[1:])
        p.scale_stride_b, p.scale_stride_h = packed[1].stride(0), packed[1].stride(1)
        p.k_res, p.kres_stride_b, p.kres_stride_h, p.kres_stride_t = kres.data_ptr(), *kres.stride()[:3]
        if vbits:
            # the residual window's values follow the packed tokens of THIS state: stage them at the window's start
            win = v[:, :, nb * G: nb * G + RL].contiguous()
            p.v, p.v_stride_b, p.v_stride_h, p.v_stride_t = win.data_ptr(), *win.stride()[:3]
            p.v_codes, p.vcodes_stride_b, p.vcodes_stride_h = vq[0].data_ptr(), vq[0].stride(0) * 4, vq[0].stride(1) * 4
            p.v_scale, p.v_mn = vq[1].data_ptr(), vq[2].data_ptr()
            p.vscale_stride_b, p.vscale_stride_h = vq[1].stride(0), vq[1].stride(1)
            p.vbits = 4
        else:
            win = None
            p.v, p.v_stride_b, p.v_stride_h, p.v_stride_t = v.data_ptr(), *v.stride()[:3]
        p.out, p.out_stride_b, p.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
        p.workspace, p.workspace_bytes = ws.data_ptr() + (-ws.data_ptr()) % 256, ws.numel() - 256
        p.B, p.N, p.Nk, p.Nb, p.G, p.R, p.hd = B, N, Nk, cap_groups, G, RL, 128
        p.rbits, p.tbits = 4, 4
        p.qk_dtype = p.v_dtype = p.out_dtype = _lib.PQ_BF16
        p.dyn_lengths, p.dyn_r_add = lengths.data_ptr(), 0
        _lib.check(lib.pq_decode_attention(ctypes.byref(p), ops._stream(torch.device(dev))), "dyn")
        torch.cuda.synchronize()
        return out, win

    for nb, r in [(0, 1), (0, 17), (1, 0), (1, 128), (3, 5), (5, 128), (6, 77), (6, 128)]:
        lengths.copy_(torch.tensor([nb, r], dtype=torch.int32))
        got, win = dyn_call(nb, r)
        pk = tuple(t[:, :, :nb] for t in packed) if nb else (None,) * 5
        kr = kres[:, :, :r] if r else None
        if vbits and nb:
            want = pq.decode_attention(q, kr, *pk, win[:, :, :r] if r else None, value_codes=vq[0][:, :, :nb * G],
                                       value_scale=vq[1][:, :, :nb * G], value_mn=vq[2][:, :, :nb * G])
        elif vbits:
            want = pq.decode_attention(q, kr, *pk, win[:, :, :r])
        else:
            # values of the live tokens: the packed tokens' rows, then the window's rows right behind them
            want = pq.decode_attention(q, kr, *pk, v[:, :, :nb * G + r])
        assert torch.equal(got, want), (nb, r)

    # lengths past the capacity are clamped to it
    lengths.copy_(torch.tensor([cap_groups + 5, RL + 9], dtype=torch.int32))
    got, win = dyn_call(cap_groups, RL)
    lengths.copy_(torch.tensor([cap_groups, RL], dtype=torch.int32))
    want, _ = dyn_call(cap_groups, RL)
    assert torch.equal(got, want)


def test_empty_cache_lengths_give_a_defined_result_and_negative_offsets_are_refused():
    """Lengths {0, 0} with no token added describe attention over nothing: the kernels must not divide by the
    empty partition; the result is defined as zeros with log-sum-exp -inf.  A negative dyn_r_add is an argument
    error."""
    import polarquant_b200 as pq
    from polarquant_b200 import _lib, ops
    dev, dt = "cuda", torch.bfloat16
    B, N, Nk, G, cap_groups, RL = 2, 8, 2, 128, 2, 128
    keys = oracle.synth_keys(B, Nk, cap_groups * G, 128, dt, seed=41, device=dev)
    packed = pq.quantize_and_pack_nbit(keys, 4, 4, G)
    kres = oracle.synth_keys(B, Nk, RL, 128, dt, seed=42, device=dev)
    v = torch.randn(B, Nk, cap_groups * G + RL, 128, device=dev).to(dt)
    q = torch.randn(B, N, 128, device=dev).to(dt)
    lib = _lib.load()
    ws = torch.empty(lib.pq_decode_workspace_bytes_dyn(B, N, Nk, 0) + 256, dtype=torch.uint8, device=dev)
    lengths = torch.zeros(2, dtype=torch.int32, device=dev)
    out = torch.full((B, N, 128), float("nan"), dtype=dt, device=dev)
    lse = torch.full((B, N), float("nan"), dtype=torch.float32, device=dev)
    p = _lib.DecodeParams()
    p.q, p.q_stride_b, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    p.codes, p.codes_stride_b, p.codes_stride_h = packed[0].data_ptr(), packed[0].stride(0), packed[0].stride(1)
    p.rscale, p.rmn, p.tscale, p.tmn = (t.data_ptr() for t in packed[1:])
    p.scale_stride_b, p.scale_stride_h = packed[1].stride(0), packed[1].stride(1)
    p.k_res, p.kres_stride_b, p.kres_stride_h, p.kres_stride_t = kres.data_ptr(), *kres.stride()[:3]
    p.v, p.v_stride_b, p.v_stride_h, p.v_stride_t = v.data_ptr(), *v.stride()[:3]
    p.out, p.out_stride_b, p.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    p.lse = lse.data_ptr()
    p.workspace, p.workspace_bytes = ws.data_ptr() + (-ws.data_ptr()) % 256, ws.numel() - 256
    p.B, p.N, p.Nk, p.Nb, p.G, p.R, p.hd = B, N, Nk, cap_groups, G, RL, 128
    p.rbits, p.tbits = 4, 4
    p.qk_dtype = p.v_dtype = p.out_dtype = _lib.PQ_BF16
    p.dyn_lengths, p.dyn_r_add = lengths.data_ptr(), 0
    stream = ops._stream(torch.device(dev))
    assert lib.pq_decode_attention(ctypes.byref(p), stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(out, torch.zeros_like(out))
    assert bool(torch.isneginf(lse).all())
    p.dyn_r_add = -1
    assert lib.pq_decode_attention(ctypes.byref(p), stream) == -1
