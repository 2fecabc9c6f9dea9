"""The scratch-free entry point, pq_decode_attention_static, against pq_decode_attention.

Who needs it: a caller that may not allocate device memory when it runs attention - for example a serving
process that handed its whole device heap to its own pool at start-up, or a host application that forbids
allocator calls after initialisation.  Such a caller cannot give pq_decode_attention a workspace, so this entry
point keeps the partial results of the split-sequence kernel in a 16 MiB array that is part of the library image.

The test drives both entry points through the C ABI with the same inputs and outputs the caller owns, twice in a
row with different data (the built-in array still holds the first call's partials during the second), and requires
identical results.  It also checks that a problem too large for the built-in array is refused with its own status.
The file name sorts last so that a run stopping at the first failure has already executed every other test.
"""
import ctypes

import pytest
import torch

from conftest import check_attn
from oracle import polar_oracle as oracle

pytestmark = pytest.mark.gpu

B, N, NK, NB, G, R = 3, 16, 4, 9, 128, 77


def _inputs(seed):
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(seed)
    keys = oracle.synth_keys(B, NK, NB * G + R, 128, torch.bfloat16, seed=seed + 1, device=dev)
    q = torch.randn(B, N, 128, device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn(B, NK, NB * G + R, 128, device=dev, generator=g).to(torch.bfloat16)
    import polarquant_b200 as pq
    packed = pq.quantize_and_pack_nbit(keys[:, :, :NB * G].contiguous(), 4, 4, G)
    return q, keys[:, :, NB * G:].contiguous(), packed, v


def _params(q, kres, packed, v, out, lse):
    from polarquant_b200 import _lib
    codes, rs, rm, ts, tm = packed
    p = _lib.DecodeParams()
    p.q, p.q_stride_b, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    p.codes, p.codes_stride_b, p.codes_stride_h = codes.data_ptr(), codes.stride(0), codes.stride(1)
    p.rscale, p.rmn, p.tscale, p.tmn = rs.data_ptr(), rm.data_ptr(), ts.data_ptr(), tm.data_ptr()
    p.scale_stride_b, p.scale_stride_h = rs.stride(0), rs.stride(1)
    p.k_res = kres.data_ptr()
    p.kres_stride_b, p.kres_stride_h, p.kres_stride_t = kres.stride(0), kres.stride(1), kres.stride(2)
    p.v, p.v_stride_b, p.v_stride_h, p.v_stride_t = v.data_ptr(), v.stride(0), v.stride(1), v.stride(2)
    p.out, p.out_stride_b, p.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    p.lse = lse.data_ptr()
    p.B, p.N, p.Nk, p.Nb, p.G, p.R, p.hd = B, N, NK, NB, G, R, 128
    p.rbits = p.tbits = 4
    p.qk_dtype = p.v_dtype = p.out_dtype = _lib.PQ_BF16
    return p


def test_static_scratch_entry_point_matches_the_workspace_entry_point_twice_in_a_row():
    from polarquant_b200 import _lib
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    need = lib.pq_decode_workspace_bytes(B, N, NK, NB, G, R, 0)
    assert 0 < need <= lib.pq_decode_static_scratch_bytes() == 16 << 20
    ws = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
    # everything the calls write to is allocated up front, by the caller
    out_ws = torch.empty(B, N, 128, dtype=torch.bfloat16, device="cuda")
    out_st = torch.empty_like(out_ws)
    lse_ws = torch.empty(B, N, dtype=torch.float32, device="cuda")
    lse_st = torch.empty_like(lse_ws)
    for seed in (500, 600):                      # second round: the built-in array holds stale partials
        q, kres, packed, v = _inputs(seed)
        p = _params(q, kres, packed, v, out_ws, lse_ws)
        p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        rc = lib.pq_decode_attention(ctypes.byref(p), stream)
        assert rc == 0, lib.pq_strerror(rc)
        out_st.fill_(float("nan"))
        p2 = _params(q, kres, packed, v, out_st, lse_st)      # no workspace at all
        rc = lib.pq_decode_attention_static(ctypes.byref(p2), stream)
        assert rc == 0, lib.pq_strerror(rc)
        torch.cuda.synchronize()
        assert torch.isfinite(out_st.float()).all()
        # same kernels, same work split: the tolerance of the attention tests holds with room to spare,
        # and in fact the two results are identical
        diff = (out_st.float() - out_ws.float()).abs()
        assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3
        assert torch.equal(out_st, out_ws) and torch.equal(lse_st, lse_ws)
        # and against the reference's decode branch, at the bar every attention test uses
        check_attn(out_st[:, :, None], oracle.decode_attention(q[:, :, None], kres, *packed, v), f"seed {seed}")


def test_static_scratch_call_allocates_nothing_and_repeats_bit_for_bit():
    """Once the array's address is cached (first call on the device) a call must leave the amount of free device
    memory untouched, and the same inputs must give the same bits again."""
    from polarquant_b200 import _lib
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    q, kres, packed, v = _inputs(700)
    out_a = torch.empty(B, N, 128, dtype=torch.bfloat16, device="cuda")
    out_b = torch.empty_like(out_a)
    lse_a = torch.empty(B, N, dtype=torch.float32, device="cuda")
    lse_b = torch.empty_like(lse_a)
    pa, pb = _params(q, kres, packed, v, out_a, lse_a), _params(q, kres, packed, v, out_b, lse_b)
    assert lib.pq_decode_attention_static(ctypes.byref(pa), stream) == 0        # resolves the address if need be
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    assert lib.pq_decode_attention_static(ctypes.byref(pb), stream) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.equal(out_a, out_b) and torch.equal(lse_a, lse_b)


def test_static_scratch_with_device_side_lengths():
    """The graph-replay form (lengths read on the device) on the built-in array.  Its scratch bound grows with the
    CTA count: with num_ctas = 0 the entry point shrinks the grid until the bound fits 16 MiB, with an explicit
    count it runs exactly the plan pq_decode_attention runs (identical bits) or refuses with its own status."""
    from polarquant_b200 import _lib
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    q, kres, packed, v = _inputs(800)
    lengths = torch.tensor([NB - 2, R - 7], dtype=torch.int32, device="cuda")
    nb, r = NB - 2, R - 7 + 1                                  # dyn_r_add = 1: the appended token
    outs = {}
    for ctas in (64, 0):
        out_ws = torch.empty(B, N, 128, dtype=torch.bfloat16, device="cuda")
        out_st = torch.full_like(out_ws, float("nan"))
        lse = torch.empty(B, N, dtype=torch.float32, device="cuda")
        ws = torch.empty(lib.pq_decode_workspace_bytes_dyn(B, N, NK, ctas) + 256, dtype=torch.uint8, device="cuda")
        p = _params(q, kres, packed, v, out_ws, lse)
        p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        p.dyn_lengths, p.dyn_r_add, p.num_ctas = lengths.data_ptr(), 1, ctas
        assert lib.pq_decode_attention(ctypes.byref(p), stream) == 0
        p2 = _params(q, kres, packed, v, out_st, lse)
        p2.dyn_lengths, p2.dyn_r_add, p2.num_ctas = lengths.data_ptr(), 1, ctas
        rc = lib.pq_decode_attention_static(ctypes.byref(p2), stream)
        assert rc == 0, lib.pq_strerror(rc)
        torch.cuda.synchronize()
        if ctas:
            assert torch.equal(out_st, out_ws)
        outs[ctas] = out_st
        # what the lengths describe: nb groups and r residual keys, the window's values right behind the packed tokens'
        want = oracle.decode_attention(q[:, :, None], kres[:, :, :r], *[t[:, :, :nb] for t in packed],
                                       v[:, :, :nb * G + r])
        check_attn(out_st[:, :, None], want, f"num_ctas {ctas}")
    # both grids attend over the same keys
    d = (outs[0].float() - outs[64].float()).abs()
    assert float(d.max()) <= 2e-2 and float(d.mean()) <= 2e-3
    # an explicit grid whose bound exceeds the array is refused, with the array's own status
    p3 = _params(q, kres, packed, v, outs[0], torch.empty(B, N, dtype=torch.float32, device="cuda"))
    p3.dyn_lengths, p3.dyn_r_add, p3.num_ctas = lengths.data_ptr(), 1, 444
    assert lib.pq_decode_workspace_bytes_dyn(B, N, NK, 444) > lib.pq_decode_static_scratch_bytes()
    assert lib.pq_decode_attention_static(ctypes.byref(p3), stream) == -6


def test_problem_beyond_the_built_in_array_is_refused_before_any_work():
    from polarquant_b200 import _lib
    lib = _lib.load()
    p = _lib.DecodeParams()
    # many tiny units: one 16-token step each, so a warp touches many units and needs many partial slots
    p.B, p.N, p.Nk, p.Nb, p.G, p.R, p.hd = 2048, 8, 8, 1, 16, 0, 128
    p.rbits = p.tbits = 4
    p.qk_dtype = p.v_dtype = p.out_dtype = _lib.PQ_BF16
    assert lib.pq_decode_workspace_bytes(2048, 8, 8, 1, 16, 0, 0) > lib.pq_decode_static_scratch_bytes()
    rc = lib.pq_decode_attention_static(ctypes.byref(p), None)
    assert rc == -6
    assert b"16 MiB" in lib.pq_strerror(rc)
