"""End-to-end greedy decode of a random-init Llama-3.1-8B-shaped model on the in-place polar KV cache.

    python -m polarquant_b200.e2e_decode [--batch 32] [--prompt 8192] [--new-tokens 256] [--layers 32]
    torchrun --nproc-per-node N -m polarquant_b200.e2e_decode ...      # batch sharded over N replicas

This is the measurement harness for "e2e decode tokens/s": everything around the attention step is plain torch
(cuBLAS projections, fused torch attention for the prefill), the attention step itself is `PolarKVCache.decode_step`
(CUDA append + fused polar attention + in-place re-quantisation).  It stands in for the reference's
benchmark/benchmark_throughput.py protocol (prefill, then timed greedy decode with EOS disabled, :27-84,152), whose
model files cannot run without the reference checkout and real weights.  Weights are N(0, 0.02), prompts are uniform
random token ids; there is no tokenizer, sampling or stopping criterion.  Prints one JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import time

import torch
import torch.nn.functional as F

from .cache import PolarKVCache


class Layer:
    def __init__(self, hidden, heads, kv_heads, inter, device, gen):
        hd = hidden // heads
        def w(o, i):
            return (torch.randn(o, i, device=device, generator=gen, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        self.qkv = w((heads + 2 * kv_heads) * hd, hidden)
        self.o = w(hidden, heads * hd)
        self.gate_up = w(2 * inter, hidden)
        self.down = w(hidden, inter)
        self.n1 = torch.ones(hidden, device=device, dtype=torch.bfloat16)
        self.n2 = torch.ones(hidden, device=device, dtype=torch.bfloat16)


def rms_norm(x, w, eps=1e-5):
    return F.rms_norm(x, (x.shape[-1],), w, eps)


def rope_tables(positions, hd, theta, device):
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd))
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)


def apply_rope(x, cos, sin):
    """x (B, H, L, hd); the rotate-half convention, which pairs channel d with d + hd/2 like the polar quantizer."""
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos + rot * sin


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=8192)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--prefill-chunk", type=int, default=2, help="sequences prefilled at a time")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every decode step from Python instead of replaying one captured CUDA graph")
    ap.add_argument("--vbits", type=int, default=0, choices=(0, 4),
                    help="4: pack the values to 4 bits as well (the reference's mixed key/value class)")
    args = ap.parse_args()

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    result = run(args, rank, world, dev)
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run(args, rank: int, world: int, dev: torch.device) -> dict:
    """The measurement itself; ``args`` carries batch, prompt, new_tokens, layers, prefill_chunk, no_graph, vbits.
    With ``world > 1`` the default process group must be initialised.  Returns the result record (every rank)."""
    if world > 1:
        import torch.distributed as dist
    hidden, heads, kvh, inter, vocab, theta = 4096, 32, 8, 14336, 128256, 500000.0
    hd = hidden // heads
    lo, hi = (rank * args.batch) // world, ((rank + 1) * args.batch) // world
    B = hi - lo                                                    # this replica's sequences
    gen = torch.Generator(device=dev).manual_seed(1004)           # every replica holds the same weights
    embed = (torch.randn(vocab, hidden, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
    layers = [Layer(hidden, heads, kvh, inter, dev, gen) for _ in range(args.layers)]
    final_norm = torch.ones(hidden, device=dev, dtype=torch.bfloat16)
    lm_head = (torch.randn(vocab, hidden, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
    g2 = torch.Generator(device="cpu").manual_seed(1004)
    prompts = torch.randint(0, vocab, (args.batch, args.prompt), generator=g2)[lo:hi].to(dev)

    max_tokens = ((args.prompt + args.new_tokens + 127) // 128 + 1) * 128
    use_graph = not args.no_graph
    # all layers hold the same number of tokens: one device-side lengths pair serves every cache
    lengths = torch.zeros(2, dtype=torch.int32, device=dev) if use_graph else None
    caches = [PolarKVCache(B, kvh, max_tokens, dtype=torch.bfloat16, device=dev, vbits=args.vbits, lengths=lengths)
              for _ in range(args.layers)]

    def split_qkv(x, L):
        q, k, v = x.split([heads * hd, kvh * hd, kvh * hd], dim=-1)
        bsz = x.shape[0]
        return (q.view(bsz, L, heads, hd).transpose(1, 2), k.view(bsz, L, kvh, hd).transpose(1, 2),
                v.view(bsz, L, kvh, hd).transpose(1, 2))

    def mlp(layer, x):
        gu = F.linear(x, layer.gate_up)
        g, u = gu.chunk(2, dim=-1)
        return F.linear(F.silu(g) * u, layer.down)

    # ------------------------------------------------------------------ prefill
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    cos, sin = rope_tables(torch.arange(args.prompt, device=dev), hd, theta, dev)
    last_hidden = torch.empty(B, hidden, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        for c0 in range(0, B, args.prefill_chunk):
            sl = slice(c0, min(B, c0 + args.prefill_chunk))
            x = embed[prompts[sl]]
            for li, layer in enumerate(layers):
                h = rms_norm(x, layer.n1)
                q, k, v = split_qkv(F.linear(h, layer.qkv), args.prompt)
                q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
                att = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
                x = x + F.linear(att.transpose(1, 2).reshape(x.shape[0], args.prompt, heads * hd), layer.o)
                x = x + mlp(layer, rms_norm(x, layer.n2))
                # store this chunk's keys / values in the layer's cache (strided (B, L, Nk, hd) views, read in place)
                caches[li].prefill(k, v, batch_start=c0)
            last_hidden[sl] = x[:, -1]
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0

    # ------------------------------------------------------------------ greedy decode
    with torch.no_grad():
        tok = F.linear(rms_norm(last_hidden, final_norm), lm_head).argmax(-1)
        generated = [tok]
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        def model_step(tok_in, cos1, sin1, attend, fused_rope=False):
            x = embed[tok_in][:, None, :]
            for li, layer in enumerate(layers):
                h = rms_norm(x, layer.n1)
                if fused_rope:
                    # one kernel: rotate q and k, append k and v (positions from the device-side lengths)
                    q = caches[li].rope_append_graph(F.linear(h, layer.qkv), cos1, sin1)
                    att = caches[li].attend_graph(q)
                    caches[li].requantize_graph()         # does something only on the step that fills the window
                else:
                    q, k, v = split_qkv(F.linear(h, layer.qkv), 1)
                    q, k = apply_rope(q, cos1, sin1), apply_rope(k, cos1, sin1)
                    att = attend(caches[li], q, k, v)                       # (B, heads, 1, hd)
                x = x + F.linear(att.transpose(1, 2).reshape(B, 1, heads * hd), layer.o)
                x = x + mlp(layer, rms_norm(x, layer.n2))
            return F.linear(rms_norm(x[:, 0], final_norm), lm_head).argmax(-1)

        graph = None
        if use_graph:
            # The whole model step - 32 x (projections, RoPE, cache append, fused attention, MLP), the LM head, the
            # argmax and the advance of position and lengths - is captured once and replayed per token.  The cache
            # kernels read their lengths on the device, the window's re-quantisation included: nothing runs on the
            # host between tokens but the replay itself.
            caches[0].sync_lengths()
            tok_buf = tok.clone()
            pos_dev = torch.full((1,), args.prompt, device=dev, dtype=torch.int64)

            def graph_step():
                cos1, sin1 = rope_tables(pos_dev, hd, theta, dev)
                nxt = model_step(tok_buf, cos1, sin1, None, fused_rope=True)
                tok_buf.copy_(nxt)
                caches[0].advance_graph()                 # one lengths pair for all layers
                pos_dev.add_(1)

            # warm-up on a side stream, then restore what it changed: token, position, lengths (the slot it wrote
            # is overwritten by the first real step)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                graph_step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            tok_buf.copy_(tok); pos_dev.fill_(args.prompt); caches[0].sync_lengths()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                graph_step()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
        t0 = time.perf_counter()
        for step in range(args.new_tokens - 1):
            if graph is not None:
                graph.replay()
                generated.append(tok_buf.clone())
                for c in caches:                          # host counters only: the graph did the rest
                    c.after_replay(device_requantized=True)
                continue
            pos = args.prompt + step
            cos1, sin1 = rope_tables(torch.tensor([pos], device=dev), hd, theta, dev)
            tok = model_step(tok, cos1, sin1, lambda c, q, k, v: c.decode_step(q, k, v))
            generated.append(tok)
        torch.cuda.synchronize()
        decode_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([decode_s, prefill_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        decode_s, prefill_s = float(t[0]), float(t[1])
    steps = args.new_tokens - 1
    weight_bytes = sum(t.numel() * 2 for layer in layers for t in (layer.qkv, layer.o, layer.gate_up, layer.down)) \
        + lm_head.numel() * 2
    cache_bytes = args.layers * B * kvh * (args.prompt + args.new_tokens // 2) * (136 if args.vbits else 324)
    del layers, caches, embed, lm_head, graph
    torch.cuda.empty_cache()
    return {
        "bench": "e2e_decode", "model": f"Llama-3.1-8B-shaped, {args.layers} layers, random init, bf16",
        "n_gpus": world, "global_batch": args.batch, "prompt_tokens": args.prompt, "new_tokens": args.new_tokens,
        "decode_tokens_per_s": args.batch * steps / decode_s, "ms_per_decode_step": decode_s / steps * 1e3,
        "prefill_s": prefill_s, "keys": "polar 4/4, group 128, residual 128",
        "values": "4-bit per-token min/max, residual 128 in bf16" if args.vbits else "bf16",
        "cache_bytes_per_token_per_kv_head": 136 if args.vbits else 324,
        "bytes_per_step_per_gpu": weight_bytes + cache_bytes,
        "cuda_graph": use_graph,
        "note": ("one captured CUDA graph of the whole model step, replayed per token; cache lengths on the device"
                 if use_graph else
                 "eager torch around PolarKVCache.decode_step; the step is host-launch bound at this batch")}


if __name__ == "__main__":
    main()
