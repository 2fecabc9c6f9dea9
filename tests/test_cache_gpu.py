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


def test_cache_serves_a_gqa_ratio_of_sixteen():
    """The scratch of the attention call grows with the 8-head tiles per kv head: a cache built with the default
    sizing (ratio 8) must regrow for 16 query heads per kv head, one built with num_q_heads must already fit, and
    a long context must not run out of partial slots either way."""
    import polarquant_b200 as pq
    from polarquant_b200.cache import PolarKVCache
    dev, dt = "cuda", torch.bfloat16
    B, N, Nk, prompt = 1, 128, 8, 32768 - 128
    g = torch.Generator(device=dev).manual_seed(77)
    keys = oracle.synth_keys(B, Nk, prompt, 128, dt, seed=78, device=dev)
    vals = torch.randn(B, Nk, prompt, 128, device=dev, generator=g).to(dt)
    q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(dt)
    k_new = oracle.synth_keys(B, Nk, 1, 128, dt, seed=79, device=dev)
    v_new = torch.randn(B, Nk, 1, 128, device=dev, generator=g).to(dt)
    outs = []
    for nq in (None, N):
        cache = PolarKVCache(B, Nk, max_tokens=prompt + 256, dtype=dt, num_q_heads=nq)
        cache.prefill(keys, vals)
        outs.append(cache.decode_step(q, k_new, v_new))
        lib_need = pq._lib.load().pq_decode_workspace_bytes(B, N, Nk, cache.max_groups, 128, 128, 0)
        assert cache.workspace.numel() >= lib_need
    assert torch.equal(outs[0], outs[1])
    packed = pq.quantize_and_pack_nbit(keys, 4, 4, 128)
    want = oracle.decode_attention(q, k_new, *packed, torch.cat([vals, v_new], dim=2))
    diff = (outs[0].float() - want.float()).abs()
    assert float(diff.max()) <= ATTN_MAX_ABS and float(diff.mean()) <= ATTN_MEAN_ABS


def test_cache_refuses_to_overflow():
    from polarquant_b200.cache import PolarKVCache
    cache = PolarKVCache(1, 1, max_tokens=128)
    k = torch.randn(1, 1, 128, 128, device="cuda").to(torch.bfloat16)
    cache.prefill(k, k)
    q = torch.randn(1, 4, 1, 128, device="cuda").to(torch.bfloat16)
    with pytest.raises(RuntimeError):
        cache.decode_step(q, k[:, :, :1], k[:, :, :1])


@pytest.mark.parametrize("prompt,steps", [(300, 140), (128, 130), (7, 260)])
def test_in_place_cache_with_packed_values_tracks_the_mixed_reference_state(prompt, steps):
    """vbits=4: the cache of LlamaPolarMixedGroupAttention (models/modeling_llama_polar.py:189-246) - values of
    the quantised tokens packed, those of the residual window in full precision, both re-quantised together."""
    import polarquant_b200 as pq
    from conftest import check_mixed
    from polarquant_b200.cache import PolarKVCache
    dev, dt = "cuda", torch.bfloat16
    B, N, Nk = 2, 8, 2
    g = torch.Generator(device=dev).manual_seed(400 + prompt)
    k_blnh = oracle.synth_keys(B, prompt, Nk, 128, dt, seed=401, device=dev)
    v_blnh = torch.randn(B, prompt, Nk, 128, device=dev, generator=g).to(dt)
    keys, vals = k_blnh.transpose(1, 2), v_blnh.transpose(1, 2)
    cache = PolarKVCache(B, Nk, max_tokens=prompt + steps + 128, dtype=dt, vbits=4)
    cache.prefill(keys, vals)

    nq = prompt - prompt % 128
    ref = list(oracle.quantize_ops(keys[:, :, :nq].contiguous(), 4, 4, 128)) if nq else None
    vref = list(oracle.quantize_values(vals[:, :, :nq].contiguous())) if nq else None
    kres, vres = keys[:, :, nq:].contiguous(), vals[:, :, nq:].contiguous()
    for step in range(steps):
        q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(dt)
        k_new = oracle.synth_keys(B, Nk, 1, 128, dt, seed=3000 + step, device=dev)
        v_new = torch.randn(B, Nk, 1, 128, device=dev, generator=g).to(dt)
        got = cache.decode_step(q, k_new, v_new)
        kres = torch.cat([kres, k_new], dim=2)
        vres = torch.cat([vres, v_new], dim=2)
        if step % 16 == 0 or kres.shape[2] % 128 in (0, 1):
            want = oracle.decode_attention_mixed(q, kres, *(ref or (None,) * 5), *(vref or (None,) * 3), vres)
            check_mixed(got, want, f"step {step}")
        if kres.shape[2] % 128 == 0:
            fresh, vfresh = oracle.quantize_ops(kres, 4, 4, 128), oracle.quantize_values(vres)
            ref = [torch.cat([a, b], dim=2) for a, b in zip(ref, fresh)] if ref else list(fresh)
            vref = [torch.cat([a, b], dim=2) for a, b in zip(vref, vfresh)] if vref else list(vfresh)
            kres, vres = kres[:, :, :0], vres[:, :, :0]
        assert cache.seq_len == prompt + step + 1
    tup = cache.as_reference_tuple()
    assert len(tup) == 11 and tup[10] == prompt + steps
    if ref:
        for a, b in zip(tup[1:6], ref):
            assert torch.equal(a, b)
        for a, b in zip(tup[7:10], vref):            # value codes (kivi layout), scales and minima, bit for bit
            assert torch.equal(a, b)
    if vres.shape[2]:
        assert torch.equal(tup[6], vres)
    else:
        assert tup[6] is None
    # the general (masked) path over the same cache state agrees with the lean path's kernels
    q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(dt)
    k_new = oracle.synth_keys(B, Nk, 1, 128, dt, seed=9, device=dev)
    mask = torch.ones(B, cache.seq_len + 1, device=dev)
    mask[0, :150] = 0                                   # left padding of the first sequence
    kres = torch.cat([kres, k_new], dim=2)
    vres = torch.cat([vres, k_new], dim=2)
    a = cache.decode_step(q, k_new, k_new, attention_mask=mask)
    want = oracle.decode_attention_mixed(q, kres, *(ref or (None,) * 5), *(vref or (None,) * 3), vres,
                                         attention_mask=mask)
    check_mixed(a, want, "masked step through the general path")


@pytest.mark.parametrize("vbits", [0, 4])
def test_one_captured_graph_replays_over_the_growing_cache(vbits):
    """Device-side lengths: the append + attention of a step are captured once in a CUDA graph and replayed for
    every token; results equal the eager cache's bit for bit, across a re-quantisation of the window."""
    from polarquant_b200.cache import PolarKVCache
    dev, dt = "cuda", torch.bfloat16
    B, N, Nk, prompt, steps = 2, 8, 2, 300, 100
    g = torch.Generator(device=dev).manual_seed(77)
    keys = oracle.synth_keys(B, Nk, prompt, 128, dt, seed=78, device=dev)
    vals = torch.randn(B, Nk, prompt, 128, device=dev, generator=g).to(dt)
    lengths = torch.zeros(2, dtype=torch.int32, device=dev)
    eager = PolarKVCache(B, Nk, max_tokens=prompt + steps + 128, dtype=dt, vbits=vbits)
    graph = PolarKVCache(B, Nk, max_tokens=prompt + steps + 128, dtype=dt, vbits=vbits, lengths=lengths)
    eager.prefill(keys, vals)
    graph.prefill(keys, vals)
    graph.sync_lengths()
    # static buffers the captured graph reads and writes
    q_buf = torch.empty(B, N, 1, 128, device=dev, dtype=dt)
    k_buf = torch.empty(B, Nk, 1, 128, device=dev, dtype=dt)
    v_buf = torch.empty(B, Nk, 1, 128, device=dev, dtype=dt)
    out_buf = torch.empty(B, N, 1, 128, device=dev, dtype=dt)

    def step_fn():
        graph.decode_step_graph(q_buf, k_buf, v_buf, out=out_buf)
        lengths[1:2].add_(1)

    q_buf.normal_(); k_buf.normal_(); v_buf.normal_()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        # warm-up outside capture, on a throw-away copy of the state: undo its effect on the lengths afterwards
        step_fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph.sync_lengths()                               # the warm-up step is discarded (its slot is overwritten)
    cg = torch.cuda.CUDAGraph()
    with torch.cuda.graph(cg):
        step_fn()
    graph.sync_lengths()                               # capture does not execute, but keep the state explicit
    crossed = False
    for step in range(steps):
        q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(dt)
        k_new = oracle.synth_keys(B, Nk, 1, 128, dt, seed=5000 + step, device=dev)
        v_new = torch.randn(B, Nk, 1, 128, device=dev, generator=g).to(dt)
        want = eager.decode_step(q, k_new, v_new)
        q_buf.copy_(q); k_buf.copy_(k_new); v_buf.copy_(v_new)
        cg.replay()
        assert torch.equal(out_buf, want), step
        if graph.after_replay():
            graph.sync_lengths()
            crossed = True
        assert graph.seq_len == eager.seq_len
        assert lengths.tolist() == [graph.num_groups, graph.res_len], step
    assert crossed
    for a, b in zip(graph.as_reference_tuple(), eager.as_reference_tuple()):
        assert (a is None and b is None) or (isinstance(a, int) and a == b) or torch.equal(a, b)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("vbits", [0, 4])
def test_fused_rope_append_equals_the_eager_ops(dt, vbits):
    """pq_rope_append: rotate-half RoPE of the step's query and key heads + append of key and value, in one kernel,
    bit-identical to `x * cos + rotate_half(x) * sin` followed by the plain append."""
    from polarquant_b200.cache import PolarKVCache
    dev = "cuda"
    B, N, Nk, prompt = 3, 8, 2, 200
    g = torch.Generator(device=dev).manual_seed(5)
    keys = oracle.synth_keys(B, Nk, prompt, 128, dt, seed=6, device=dev)
    vals = torch.randn(B, Nk, prompt, 128, device=dev, generator=g).to(dt)
    lengths = torch.zeros(2, dtype=torch.int32, device=dev)
    a = PolarKVCache(B, Nk, max_tokens=512, dtype=dt, vbits=vbits, lengths=lengths)
    b = PolarKVCache(B, Nk, max_tokens=512, dtype=dt, vbits=vbits, lengths=lengths)
    a.prefill(keys, vals); b.prefill(keys, vals); a.sync_lengths()
    for step in range(3):
        qkv = (torch.randn(B, 1, (N + 2 * Nk) * 128, device=dev, generator=g) * 2).to(dt)
        ang = torch.rand(128, device=dev, generator=g) * 6.28
        cos, sin = ang.cos().to(dt), ang.sin().to(dt)

        def rope(x):
            rot = torch.cat([-x[..., 64:], x[..., :64]], dim=-1)
            return x * cos + rot * sin

        q, k, v = qkv.split([N * 128, Nk * 128, Nk * 128], dim=-1)
        q = q.view(B, 1, N, 128).transpose(1, 2)
        k = k.view(B, 1, Nk, 128).transpose(1, 2)
        v = v.view(B, 1, Nk, 128).transpose(1, 2)
        want = a.decode_step_graph(rope(q).contiguous(), rope(k).contiguous(), v)
        q_rot = b.rope_append_graph(qkv, cos, sin)
        assert torch.equal(q_rot, rope(q))
        got = b.attend_graph(q_rot)
        assert torch.equal(got, want), step
        assert torch.equal(a.k_res[:, :, :a.res_len + 1], b.k_res[:, :, :a.res_len + 1])
        lengths[1:2].add_(1)
        a.after_replay(); b.after_replay()
    ta, tb = a.as_reference_tuple(), b.as_reference_tuple()
    assert torch.equal(ta[0], tb[0]) and torch.equal(ta[6], tb[6])


@pytest.mark.parametrize("vbits", [0, 4])
def test_chunked_prefill_fills_the_same_cache(vbits):
    from polarquant_b200.cache import PolarKVCache
    dev, dt = "cuda", torch.bfloat16
    B, Nk, L = 5, 2, 300
    g = torch.Generator(device=dev).manual_seed(3)
    k_blnh = oracle.synth_keys(B, L, Nk, 128, dt, seed=4, device=dev)
    v_blnh = torch.randn(B, L, Nk, 128, device=dev, generator=g).to(dt)
    keys, vals = k_blnh.transpose(1, 2), v_blnh.transpose(1, 2)
    whole = PolarKVCache(B, Nk, max_tokens=512, dtype=dt, vbits=vbits)
    parts = PolarKVCache(B, Nk, max_tokens=512, dtype=dt, vbits=vbits)
    whole.prefill(keys, vals)
    for b0 in range(0, B, 2):
        parts.prefill(keys[b0:b0 + 2], vals[b0:b0 + 2], batch_start=b0)
    assert (parts.num_groups, parts.res_len) == (whole.num_groups, whole.res_len) == (2, 44)
    for a, b in zip(whole.as_reference_tuple(), parts.as_reference_tuple()):
        assert (isinstance(a, int) and a == b) or torch.equal(a, b)
    with pytest.raises(ValueError):
        parts.prefill(keys[:2], vals[:2], batch_start=4)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("vbits", [0, 4])
def test_device_driven_requantisation_inside_the_graph(vbits, dt):
    """requantize_graph + advance_graph: the captured step also re-quantises the window when it fills and keeps the
    lengths, so 230 replays (crossing the window boundary twice) need nothing from the host; outputs and the final
    cache equal the eager cache's bit for bit."""
    from polarquant_b200.cache import PolarKVCache
    dev = "cuda"
    B, N, Nk, prompt, steps = 2, 8, 2, 300, 230         # residual 44: the window fills at steps 83 and 211
    g = torch.Generator(device=dev).manual_seed(78)
    keys = oracle.synth_keys(B, Nk, prompt, 128, dt, seed=79, device=dev)
    vals = torch.randn(B, Nk, prompt, 128, device=dev, generator=g).to(dt)
    lengths = torch.zeros(2, dtype=torch.int32, device=dev)
    eager = PolarKVCache(B, Nk, max_tokens=prompt + steps + 128, dtype=dt, vbits=vbits)
    graph = PolarKVCache(B, Nk, max_tokens=prompt + steps + 128, dtype=dt, vbits=vbits, lengths=lengths)
    eager.prefill(keys, vals)
    graph.prefill(keys, vals)
    q_buf = torch.empty(B, N, 1, 128, device=dev, dtype=dt)
    k_buf = torch.empty(B, Nk, 1, 128, device=dev, dtype=dt)
    v_buf = torch.empty(B, Nk, 1, 128, device=dev, dtype=dt)
    out_buf = torch.empty(B, N, 1, 128, device=dev, dtype=dt)

    def step_fn():
        graph.decode_step_graph(q_buf, k_buf, v_buf, out=out_buf)
        graph.requantize_graph()
        graph.advance_graph()

    q_buf.normal_(); k_buf.normal_(); v_buf.normal_()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step_fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph.sync_lengths()                               # discard the warm-up step
    cg = torch.cuda.CUDAGraph()
    with torch.cuda.graph(cg):
        step_fn()
    graph.sync_lengths()
    crossed = 0
    for step in range(steps):
        q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(dt)
        k_new = oracle.synth_keys(B, Nk, 1, 128, dt, seed=7000 + step, device=dev)
        v_new = torch.randn(B, Nk, 1, 128, device=dev, generator=g).to(dt)
        want = eager.decode_step(q, k_new, v_new)
        q_buf.copy_(q); k_buf.copy_(k_new); v_buf.copy_(v_new)
        cg.replay()
        assert torch.equal(out_buf, want), step
        crossed += graph.after_replay(device_requantized=True)
        if step % 37 == 0 or step == steps - 1:
            assert lengths.tolist() == [graph.num_groups, graph.res_len] == [eager.num_groups, eager.res_len], step
    assert crossed == 2
    for a, b in zip(graph.as_reference_tuple(), eager.as_reference_tuple()):
        assert (a is None and b is None) or (isinstance(a, int) and a == b) or torch.equal(a, b)
