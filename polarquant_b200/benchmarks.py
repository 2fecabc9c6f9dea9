"""Secondary timings of the polar key-cache kernels (the headline number is bench.py at the repository root).

    python -m polarquant_b200.benchmarks qk        # the reference's QK micro-benchmark grid
    python -m polarquant_b200.benchmarks sweep [name]   # fused decode attention over bit widths / group sizes / shapes
    python -m polarquant_b200.benchmarks quant     # quantizer at prefill sizes
    python -m polarquant_b200.benchmarks values    # packed (4-bit) value cache: fused attention and value quantiser
    python -m polarquant_b200.benchmarks packed_keys   # 6-bit key container (48 B/token) beside the byte container
    torchrun --nproc-per-node N -m polarquant_b200.benchmarks longctx   # 128k-context step sharded over N GPUs

`qk` reproduces the grid of the reference's benchmark/benchmark_matmul.py (`test4polar`, lines 89-120: 32 heads on
the code tensor, D = 64, fp16, random codes in [0, 250) and randn scales, batch 1/2/4/8, length 4096..131072), but
times with CUDA events over back-to-back launches instead of a host timer around each synchronised call.
Every line printed is one JSON object.
"""
from __future__ import annotations

import json
import sys

import torch

from . import ops


def _time_us(fn, reps: int = 20, warm: int = 3, graph: bool = True) -> float:
    """Mean microseconds per call over back-to-back launches; the call is replayed from a CUDA graph when it can
    be captured, so that small problems are not timed by the Python launcher."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    run = fn
    if graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            run = g.replay
            run()
        except Exception:
            torch.cuda.synchronize()
            run = fn
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        run()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps * 1e3


def qk_grid(group_size: int = 32, rbits: int = 4, tbits: int = 4, batches=(1, 2, 4, 8),
            lengths=(4096, 8192, 16384, 32768, 65536, 131072)):
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(2)
    for B in batches:
        for L in lengths:
            N = 32
            q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(torch.float16)
            idx = torch.randint(0, 250, (B, N, L // group_size, group_size, 64), device=dev, generator=g,
                                dtype=torch.uint8)
            sc = [torch.randn(B, N, L // group_size, 1, 64, device=dev, generator=g).to(torch.float16)
                  for _ in range(4)]
            us = _time_us(lambda: ops.qk_decode(q, idx, *sc, rbits=rbits, tbits=tbits))
            nbytes = idx.numel() + 4 * sc[0].numel() * 2 + q.numel() * 2 + B * N * L * 4
            print(json.dumps({"bench": "qk", "batch": B, "length": L, "group": group_size, "bits": f"{rbits}/{tbits}",
                              "ms": us / 1e3, "gbs": nbytes / us / 1e3}))
            del idx, sc


def decode_sweep(only: str | None = None):
    """`only`: run just the shapes whose name contains this string (e.g. "70b" for the long-context per-GPU share)."""
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(1003)
    shapes = [("llama3-8b B16 ctx32k", 16, 32, 8, 32768), ("qwen2.5-7b B64 ctx8k", 64, 28, 4, 8192),
              ("llama2-7b MHA B1 ctx4k", 1, 32, 32, 4096), ("70b-shaped 1 kv head/GPU B8 ctx128k", 8, 8, 1, 131072)]
    for name, B, N, Nk, ctx in shapes:
        if only and only not in name:
            continue
        for (rb, tb) in ((4, 4), (3, 3), (2, 4)):
            for G in (128, 32):
                R = 128
                Nb = (ctx - R) // G

                def one_set():
                    q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(torch.bfloat16)
                    v = torch.randn(B, Nk, ctx, 128, device=dev, generator=g).to(torch.bfloat16)
                    kres = torch.randn(B, Nk, R, 128, device=dev, generator=g).to(torch.bfloat16)
                    keys = torch.randn(B, Nk, Nb * G, 128, device=dev, generator=g).to(torch.bfloat16)
                    return q, kres, ops.quantize_and_pack_nbit(keys, rb, tb, G), v

                sets = [one_set()]
                q, kres, packed, v = sets[0]
                nbytes = (packed[0].numel() + 4 * packed[1].numel() * 2 + kres.numel() * 2 + v.numel() * 2
                          + q.numel() * 4)
                # a footprint below 512 MB is rotated over four input sets, so that no launch finds its
                # predecessor's lines in the 126 MB L2
                while nbytes < 512e6 and len(sets) < 4:
                    sets.append(one_set())

                def step():
                    for q_, kres_, packed_, v_ in sets:
                        ops.decode_attention(q_, kres_, *packed_, v_, rbits=rb, tbits=tb)

                us = _time_us(step, reps=20) / len(sets)
                print(json.dumps({"bench": "decode", "shape": name, "bits": f"{rb}/{tb}", "group": G, "us": us,
                                  "mb": nbytes / 1e6, "gbs": nbytes / us / 1e3, "input_sets_rotated": len(sets)}))
                del sets, packed, v, q, kres


def packed_keys():
    """The 48-byte-per-token key container beside the byte container, for the 6-bit splits: fused decode attention
    (same codes, both containers; the results are bit-identical) and the quantizer writing either."""
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(1007)
    shapes = [("llama3-8b B16 ctx32k", 16, 32, 8, 32768), ("qwen2.5-7b B64 ctx8k", 64, 28, 4, 8192)]
    for name, B, N, Nk, ctx in shapes:
        for (rb, tb) in ((3, 3), (2, 4)):
            G, R = 128, 128
            Nb = (ctx - R) // G
            q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(torch.bfloat16)
            v = torch.randn(B, Nk, ctx, 128, device=dev, generator=g).to(torch.bfloat16)
            kres = torch.randn(B, Nk, R, 128, device=dev, generator=g).to(torch.bfloat16)
            keys = torch.randn(B, Nk, Nb * G, 128, device=dev, generator=g).to(torch.bfloat16)
            us_qb = _time_us(lambda: ops.quantize_and_pack_nbit(keys, rb, tb, G), reps=10)
            us_qp = _time_us(lambda: ops.quantize_and_pack_nbit(keys, rb, tb, G, key_format="packed6"), reps=10)
            byte = ops.quantize_and_pack_nbit(keys, rb, tb, G)
            pack = ops.quantize_and_pack_nbit(keys, rb, tb, G, key_format="packed6")
            del keys
            us_b = _time_us(lambda: ops.decode_attention(q, kres, *byte, v, rbits=rb, tbits=tb), reps=20)
            us_p = _time_us(lambda: ops.decode_attention(q, kres, *pack, v, rbits=rb, tbits=tb, key_format="packed6"),
                            reps=20)
            same = torch.equal(ops.decode_attention(q, kres, *byte, v, rbits=rb, tbits=tb),
                               ops.decode_attention(q, kres, *pack, v, rbits=rb, tbits=tb, key_format="packed6"))
            rest = 4 * byte[1].numel() * 2 + kres.numel() * 2 + v.numel() * 2 + q.numel() * 4
            print(json.dumps({"bench": "packed_keys", "shape": name, "bits": f"{rb}/{tb}", "group": G,
                              "us_byte_container": us_b, "us_packed_container": us_p,
                              "key_bytes_per_token": {"byte": 64, "packed6": 48},
                              "cache_bytes_per_token_per_kv_head": {"byte": 64 + 4 + 256, "packed6": 48 + 4 + 256},
                              "gbs_byte": (rest + byte[0].numel()) / us_b / 1e3,
                              "gbs_packed": (rest + pack[0].numel()) / us_p / 1e3,
                              "quantizer_us_byte": us_qb, "quantizer_us_packed": us_qp, "bit_identical": same}))
            del byte, pack, v


def quant_sizes():
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(7)
    for (B, Nk, L, G, dt) in ((16, 8, 32768, 128, torch.bfloat16), (64, 4, 8192, 128, torch.bfloat16),
                              (64, 4, 8192, 32, torch.bfloat16), (16, 8, 32768, 128, torch.float16),
                              (16, 8, 128, 128, torch.bfloat16)):
        base = torch.randn(B, L, Nk, 128, device=dev, generator=g).to(dt)
        keys = base.transpose(1, 2)
        us = _time_us(lambda: ops.quantize_and_pack_nbit(keys, 4, 4, G), reps=10)
        es = base.element_size()
        nbytes = B * Nk * L * 128 * es + B * Nk * (L * 64 + (L // G) * 4 * 64 * es)
        print(json.dumps({"bench": "quantize", "batch": B, "kv_heads": Nk, "tokens": L, "group": G,
                          "dtype": str(dt).split(".")[-1], "us": us, "mb": nbytes / 1e6, "gbs": nbytes / us / 1e3}))
        del base, keys
    # prefill-side fusion: rotation + quantisation in one pass against the two separate passes
    B, Nk, L, G, dt = 16, 8, 32768, 128, torch.bfloat16
    base = torch.randn(B, L, Nk, 128, device=dev, generator=g).to(dt)
    keys = base.transpose(1, 2)
    inv = 1.0 / (500000.0 ** (torch.arange(0, 128, 2, device=dev, dtype=torch.float32) / 128))
    ang = torch.arange(L, device=dev, dtype=torch.float32)[:, None] * inv
    ang = torch.cat([ang, ang], dim=-1)
    cos, sin = ang.cos().to(dt), ang.sin().to(dt)
    out = torch.empty_like(keys)

    def two_step():
        half = 64
        rot = keys * cos[None, None] + torch.cat([-keys[..., half:], keys[..., :half]], dim=-1) * sin[None, None]
        return ops.quantize_and_pack_nbit(rot, 4, 4, G)

    us_fused = _time_us(lambda: ops.rope_quantize(keys, cos, sin, 4, 4, G, out=out), reps=10)
    us_quant = _time_us(lambda: ops.quantize_and_pack_nbit(keys, 4, 4, G), reps=10)
    us_two = _time_us(two_step, reps=5, graph=False)
    nbytes = B * Nk * L * 128 * 2 * 2 + B * Nk * (L * 64 + (L // G) * 4 * 64 * 2)
    print(json.dumps({"bench": "rope_quantize", "batch": B, "kv_heads": Nk, "tokens": L, "group": G, "dtype": "bfloat16",
                      "us_fused": us_fused, "mb_fused": nbytes / 1e6, "gbs_fused": nbytes / us_fused / 1e3,
                      "us_quantizer_alone": us_quant, "us_eager_rotation_then_quantizer": us_two}))


def packed_values():
    """Fused decode attention with packed keys AND packed 4-bit values (the mixed class of the reference,
    models/modeling_llama_polar.py:160-292) beside the same step with full-precision values, and the value
    quantiser at the prefill size.  Bytes are the algorithmic ones of each variant."""
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(1006)
    shapes = [("llama3-8b B16 ctx32k", 16, 32, 8, 32768), ("qwen2.5-7b B64 ctx8k", 64, 28, 4, 8192),
              ("70b-shaped 1 kv head/GPU B8 ctx128k", 8, 8, 1, 131072)]
    for name, B, N, Nk, ctx in shapes:
        G, R = 128, 128
        Nb = (ctx - R) // G
        q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(torch.bfloat16)
        v = torch.randn(B, Nk, ctx, 128, device=dev, generator=g).to(torch.bfloat16)
        kres = torch.randn(B, Nk, R, 128, device=dev, generator=g).to(torch.bfloat16)
        keys = torch.randn(B, Nk, Nb * G, 128, device=dev, generator=g).to(torch.bfloat16)
        packed = ops.quantize_and_pack_nbit(keys, 4, 4, G)
        del keys
        vq = v[:, :, :Nb * G]
        us_q = _time_us(lambda: ops.quantize_values(vq, layout="tiled"), reps=10)
        vc, vs, vm = ops.quantize_values(vq, layout="tiled")
        v_res = v[:, :, Nb * G:].contiguous()
        qbytes = vq.numel() * 2 + vc.numel() * 4 + 2 * vs.numel() * 2
        print(json.dumps({"bench": "quantize_values", "shape": name, "us": us_q, "mb": qbytes / 1e6,
                          "gbs": qbytes / us_q / 1e3}))
        us_full = _time_us(lambda: ops.decode_attention(q, kres, *packed, v), reps=20)
        us_pack = _time_us(lambda: ops.decode_attention(q, kres, *packed, v_res, value_codes=vc, value_scale=vs,
                                                        value_mn=vm), reps=20)
        kbytes = packed[0].numel() + 4 * packed[1].numel() * 2 + kres.numel() * 2 + q.numel() * 4
        full_b = kbytes + v.numel() * 2
        pack_b = kbytes + vc.numel() * 4 + 2 * vs.numel() * 2 + v_res.numel() * 2
        print(json.dumps({"bench": "decode_packed_values", "shape": name, "us_full_values": us_full,
                          "us_packed_values": us_pack, "speedup": us_full / us_pack, "mb_full": full_b / 1e6,
                          "mb_packed": pack_b / 1e6, "gbs_full": full_b / us_full / 1e3,
                          "gbs_packed": pack_b / us_pack / 1e3}))
        del packed, v, vc, vs, vm


def sequence_split_check(dev, rank: int, world: int) -> float:
    """Correctness of the one exchange the path has: a small seeded problem (every rank builds the same tensors),
    attended over all keys on this GPU and, split along the sequence, over the ranks with one NCCL all-gather of
    (output, log-sum-exp) and the CUDA merge.  Returns the largest absolute difference, maximised over ranks."""
    import torch.distributed as dist
    from . import distributed as pqd
    B, N, Nk, Nb, G, R = 2, 16, 4, 4 * max(world, 2) + 1, 128, 45
    g = torch.Generator(device=dev).manual_seed(2105)
    keys = (torch.randn(B, Nk, Nb * G + R, 128, device=dev, generator=g) * 3.0).to(torch.bfloat16)
    q = torch.randn(B, N, 1, 128, device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn(B, Nk, Nb * G + R, 128, device=dev, generator=g).to(torch.bfloat16)
    packed = ops.quantize_and_pack_nbit(keys[:, :, :Nb * G].contiguous(), 4, 4, G)
    kres = keys[:, :, Nb * G:].contiguous()
    full = ops.decode_attention(q, kres, *packed, v, out_dtype=torch.float32)
    g0, g1, owns = pqd.split_sequence(Nb, R, rank, world)
    mine = [t[:, :, g0:g1].contiguous() for t in packed] if g1 > g0 else None
    my_v = torch.cat([v[:, :, g0 * G:g1 * G]] + ([v[:, :, Nb * G:]] if owns else []), dim=2).contiguous()
    got = pqd.sequence_parallel_decode(q, kres if owns else None, mine, my_v, out_dtype=torch.float32)
    err = (got - full).abs().max().reshape(1)
    if world > 1:
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
    return float(err.item())


def long_context_legs(dev, rank: int, world: int, reps: int = 30) -> dict:
    """70B-shaped long-context decode attention over the GPUs of one node: 64 q / 8 kv heads, batch 8, context
    131072, polar 4/4, group 128, bf16.  Two shardings of the same step, each replayed from a CUDA graph and timed
    with CUDA events (max over ranks): `heads` - kv heads split over the ranks, no collective; `sequence` - every
    rank holds all heads but a slice of the context, one all-gather of (output, lse) per step and a local
    log-sum-exp merge.  With ``world > 1`` the default process group (NCCL) must be initialised."""
    import torch.distributed as dist
    from . import distributed as pqd
    B, N, Nk, ctx, G, R = 8, 64, 8, 131072, 128, 128
    Nb = (ctx - R) // G
    g = torch.Generator(device=dev).manual_seed(1005 + rank)

    def build(kv_heads, q_heads, groups, residual):
        tokens = groups * G + residual
        q = torch.randn(B, q_heads, 1, 128, device=dev, generator=g).to(torch.bfloat16)
        v = torch.randn(B, kv_heads, tokens, 128, device=dev, generator=g).to(torch.bfloat16)
        kres = torch.randn(B, kv_heads, residual, 128, device=dev, generator=g).to(torch.bfloat16) if residual else None
        packed = []
        for h in range(kv_heads):                      # head by head to bound temporaries
            keys = torch.randn(B, 1, groups * G, 128, device=dev, generator=g).to(torch.bfloat16)
            packed.append(ops.quantize_and_pack_nbit(keys, 4, 4, G))
        packed = [torch.cat([p[i] for p in packed], dim=1) for i in range(5)]
        nbytes = (packed[0].numel() + 4 * packed[1].numel() * 2 + v.numel() * 2 + q.numel() * 4
                  + (kres.numel() * 2 if residual else 0))
        return q, kres, packed, v, nbytes

    def timed(fn):
        if world > 1:
            dist.barrier()                             # ranks enter a leg together (the peer-memory waits are bounded)
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        graphed = True
        try:                                           # replay from a CUDA graph: the GPU's time, not the launcher's
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn()
            run = graph.replay
        except Exception:                              # capture not possible: time the eager calls
            torch.cuda.synchronize()
            run, graphed = fn, False
        if world > 1:
            dist.barrier()
        for _ in range(5):
            run()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        for _ in range(5):                             # the first launches behind a barrier run cold
            run()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            run()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / reps * 1e3], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), graphed

    def total(nbytes):
        tot = torch.tensor([float(nbytes)], device=dev)
        if world > 1:
            dist.all_reduce(tot)
        return float(tot.item())

    out = {"shape": f"batch {B}, {N} q / {Nk} kv heads, ctx {ctx}, polar 4/4, group {G}, bf16", "n_gpus": world}
    # A rank's share below 512 MB (8 GPUs: 340 MB) is rotated over four input sets, so that no launch finds its
    # predecessor's lines in the 126 MB L2; the criterion is the same on every rank.
    copies = 4 if B * Nk * ctx * 324 / world < 512e6 else 1
    out["input_sets_rotated"] = copies

    def over(sets, call):
        return lambda: [call(*s[:4]) for s in sets]

    # --- kv heads over ranks ---
    h0, h1 = pqd.shard_range(Nk, rank, world)
    sets = [build(h1 - h0, (h1 - h0) * (N // Nk), Nb, R) for _ in range(copies)]
    us, graphed = timed(over(sets, lambda q, kres, packed, v: ops.decode_attention(q, kres, *packed, v)))
    us /= copies
    agg = total(sets[0][4])
    out["heads"] = {"us": us, "aggregate_gbs": agg / us / 1e3, "aggregate_mb": agg / 1e6, "collective": "none",
                    "cuda_graph": graphed}
    del sets

    # --- sequence over ranks ---
    g0, g1, owns = pqd.split_sequence(Nb, R, rank, world)
    sets = [build(Nk, N, g1 - g0, R if owns else 0) for _ in range(copies)]
    if world > 1:
        for s_ in sets:
            dist.broadcast(s_[0], 0)                   # one query for all ranks
    q, kres, packed, v, nbytes = sets[0]
    us, graphed = timed(over(sets, (lambda q, kres, packed, v: pqd.sequence_parallel_decode(q, kres, packed, v))
                             if world > 1 else (lambda q, kres, packed, v: ops.decode_attention(q, kres, *packed, v))))
    us /= copies
    agg = total(nbytes)
    out["sequence"] = {"us": us, "aggregate_gbs": agg / us / 1e3, "aggregate_mb": agg / 1e6,
                       "collective": "one all_gather of (B*N, 129) fp32 per rank, merged in place by one kernel", "cuda_graph": graphed}
    if world > 1:
        # the parts of the sequence-split step, each replayed from a graph of its own: local attention, the
        # all-gather of the (B N, 129) fp32 blocks, the merge over the gathered buffer
        rows = B * N
        mine = torch.zeros(rows * 129, dtype=torch.float32, device=dev)
        gathered = torch.zeros(world * rows * 129, dtype=torch.float32, device=dev)
        o_view, l_view = mine[:rows * 128].view(B, N, 1, 128), mine[rows * 128:].view(B, N)
        us_local, _ = timed(over(sets, lambda q, kres, packed, v: ops.decode_attention(
            q, kres, *packed, v, out_dtype=torch.float32, out=o_view, lse_out=l_view)))
        us_local /= copies
        us_gather, _ = timed(lambda: dist.all_gather_into_tensor(gathered, mine))
        us_merge, _ = timed(lambda: ops.merge_lse_gathered(gathered, world, rows, out_dtype=torch.bfloat16))
        out["sequence"].update(local_attention_us=us_local, all_gather_us=us_gather, merge_us=us_merge,
                               exchange_bytes_per_rank=rows * 129 * 4)
        # the same step with the exchange done over NVLink peer memory instead of the all-gather + merge
        try:
            ex = pqd.PeerExchange(B, N, device=dev)
        except Exception as e:                         # raised on every rank alike (see PeerExchange)
            out["sequence_peer_memory"] = {"unavailable": str(e)[:200]}
        else:
            want = pqd.sequence_parallel_decode(q, kres, packed, v)
            us_p2p, graphed = timed(over(sets, lambda q, kres, packed, v: pqd.sequence_parallel_decode(
                q, kres, packed, v, exchange=ex)))
            us_p2p /= copies
            got = pqd.sequence_parallel_decode(q, kres, packed, v, exchange=ex)
            us_pp, _ = timed(over(sets, lambda q, kres, packed, v: pqd.sequence_parallel_decode(
                q, kres, packed, v, exchange=ex, collect_in_attention=False)))
            us_pp /= copies
            got_pp = pqd.sequence_parallel_decode(q, kres, packed, v, exchange=ex, collect_in_attention=False)
            us_kp, _ = timed(over(sets, lambda q, kres, packed, v: pqd.sequence_parallel_decode(
                q, kres, packed, v, exchange=ex, push_in_attention=False)))
            us_kp /= copies
            got_kp = pqd.sequence_parallel_decode(q, kres, packed, v, exchange=ex, push_in_attention=False)
            us_x, _ = timed(lambda: ex.merge(out_dtype=torch.bfloat16))
            flags = torch.tensor([float(torch.equal(got, want) and torch.equal(got_kp, want) and torch.equal(got_pp, want)),
                                  float(ex.status() == 0)], device=dev)
            dist.all_reduce(flags, op=dist.ReduceOp.MIN)
            out["sequence_peer_memory"] = {
                "us": us_p2p, "aggregate_gbs": agg / us_p2p / 1e3, "cuda_graph": graphed,
                "us_with_a_separate_collecting_kernel": us_pp,
                "us_with_the_push_in_that_kernel_too": us_kp, "exchange_kernel_us": us_x,
                "collective": "none: the attention's merge stores the (B*N, 129) fp32 block, paired with the step's "
                              "epoch, into every peer, collects the peers' blocks from local memory and merges",
                "bit_identical_to_all_gather_path": bool(flags[0].item()), "no_wait_timed_out": bool(flags[1].item())}
            ex.close()
    del sets, q, kres, packed, v
    return out


def long_context():
    """CLI form of `long_context_legs` (launch with torchrun for more than one GPU)."""
    import os
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    res = long_context_legs(dev, rank, world)
    if world > 1:
        res["seqsplit_max_abs_err"] = sequence_split_check(dev, rank, world)
    if rank == 0:
        print(json.dumps({"bench": "longctx", **res}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "sweep"
    if what == "sweep" and len(sys.argv) > 2:
        decode_sweep(sys.argv[2])
    else:
        {"qk": qk_grid, "sweep": decode_sweep, "quant": quant_sizes, "values": packed_values,
         "packed_keys": packed_keys, "longctx": long_context}[what]()
