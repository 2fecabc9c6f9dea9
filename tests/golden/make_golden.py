"""Generate the golden fixtures in this directory by running the reference's own code on CPU.

    python tests/golden/make_golden.py /path/to/PolarQuant-checkout     (or set POLARQUANT_REFERENCE)

Needs the reference checkout, torch, transformers and triton (for its interpreter);
run it where those exist.  The tests only read the .npz files it writes.

What is executed (nothing of the reference is copied, its files are imported in place):
  * quantizer  - the method ``quantize_and_pack_nbit`` of ``LlamaPolarGroupAttention`` and
                 ``Qwen2PolarGroupAttention`` (models/modeling_llama_polar.py:135-157,
                 models/modeling_qwen_polar.py:134-156) on seeded keys in bf16 / fp16 / fp32.
  * QK logits  - the Triton kernel ``_kernel`` (models/kernel4group.py:14-80) under
                 TRITON_INTERPRET=1, launched with the grid of its wrapper (:99).
  * attention  - the decode branch of ``LlamaPolarGroupAttention.forward`` and
                 ``Qwen2PolarGroupAttention.forward`` (models/modeling_llama_polar.py:61-101,
                 models/modeling_qwen_polar.py:60-100), unmodified, with identity projections
                 and an identity rotary embedding so its inputs are the fixture's tensors; its
                 kernel call is served by the Triton kernel above through the interpreter.
  * mixed      - the decode branch of ``LlamaPolarMixedGroupAttention.forward``
                 (models/modeling_llama_polar.py:189-246), unmodified, the same way.  Its two KIVI routines are
                 not part of the reference checkout; the module globals ``cuda_bmm_fA_qB_outer`` and
                 ``triton_quantize_and_pack_along_last_dim`` are bound to the restatement in
                 oracle/polar_oracle.py, so these fixtures pin the reference's composition (which logits meet
                 which values, the roundings at :225, :237, :239), not KIVI's arithmetic.
"""
from __future__ import annotations

import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import polar_oracle as oracle  # noqa: E402
from polarquant_b200 import dropin  # noqa: E402

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("POLARQUANT_REFERENCE", os.path.join(os.sep, "root", "reference"))
DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


ONLY = os.environ.get("GOLDEN_ONLY")      # regenerate only the fixtures whose name starts with this


def save(name, **arrays):
    if ONLY and not name.startswith(ONLY):
        return
    out = {}
    for k, v in arrays.items():
        out[k] = oracle.as_numpy(v) if torch.is_tensor(v) else np.asarray(v)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: (v.shape, str(v.dtype)) for k, v in out.items()})


def reference_kernel_module():
    """The reference's models/kernel4group.py imported from its own path."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("ref_kernel4group", os.path.join(REF, "models", "kernel4group.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


REFK = reference_kernel_module()


def triton_logits_cpu(query_states, indices, rscale, rmn, tscale, tmn, rbits=4, tbits=4):
    """The reference wrapper (models/kernel4group.py:83-109) minus its CUDA device guard."""
    B, Nk, Nb, G, D = indices.shape
    N = query_states.shape[1]
    out = torch.empty((B, N, 1, Nb * G), dtype=torch.float32)
    REFK._kernel[(B * Nk, Nb)](query_states.contiguous(), indices.contiguous(), rscale.contiguous(),
                               rmn.contiguous(), tscale.contiguous(), tmn.contiguous(), out,
                               rbits, tbits, B, N, Nb, G, D, Nk)
    return out


def main():
    entry = types.ModuleType("models.kernel4group")
    entry.attention_decode_forward_triton_impl = triton_logits_cpu
    dropin.install(REF, entry_module=entry)
    import importlib
    llama = importlib.import_module("models.modeling_llama_polar")
    qwen = importlib.import_module("models.modeling_qwen_polar")

    # ---------------------------------------------------------------- quantizer
    quant_cases = [("bf16", 4, 4, 128), ("bf16", 3, 3, 32), ("bf16", 2, 4, 32), ("fp16", 4, 4, 128),
                   ("fp16", 3, 3, 32), ("fp16", 2, 4, 128), ("fp32", 4, 4, 128), ("fp32", 3, 3, 32)]
    for i, (dn, rb, tb, G) in enumerate(quant_cases):
        L = 256 if G == 128 else 96
        keys = oracle.synth_keys(1, 2, L, 128, DT[dn], seed=4000 + i, kind="loguniform" if i % 2 == 0 else "outlier")
        if i == 0:
            keys[0, 1, 128:256, 5] = keys[0, 1, 128, 5]       # a pair whose angle/radius are constant over a group
            keys[0, 1, 128:256, 69] = keys[0, 1, 128, 69]
        stub = types.SimpleNamespace(rbits=rb, tbits=tb, group_size=G)
        got = llama.LlamaPolarGroupAttention.quantize_and_pack_nbit(stub, keys)
        got_q = qwen.Qwen2PolarGroupAttention.quantize_and_pack_nbit(stub, keys)
        assert all(torch.equal(a, b) for a, b in zip(got, got_q)), "llama and qwen quantizers disagree"
        save(f"quant_{dn}_r{rb}t{tb}_g{G}", keys=keys, indices=got[0], rscale=got[1], rmn=got[2], tscale=got[3],
             tmn=got[4], meta=np.array([rb, tb, G]))

    # strided input, the (B, L, Nk, hd) layout the prefill hands to the quantizer
    base = oracle.synth_keys(2, 256, 2, 128, torch.bfloat16, seed=4100)        # (B, L, Nk, hd)
    keys = base.transpose(1, 2)                                                # (B, Nk, L, hd) view
    stub = types.SimpleNamespace(rbits=4, tbits=4, group_size=128)
    got = llama.LlamaPolarGroupAttention.quantize_and_pack_nbit(stub, keys)
    save("quant_bf16_strided", keys_blnh=base, indices=got[0], rscale=got[1], rmn=got[2], tscale=got[3], tmn=got[4],
         meta=np.array([4, 4, 128]))

    # ---------------------------------------------------------------- QK logits (Triton interpreter)
    qk_cases = [("bf16", 1, 8, 2, 2, 128, 4, 4), ("fp16", 2, 4, 4, 3, 32, 3, 3), ("fp32", 1, 4, 2, 2, 32, 2, 4),
                ("fp16", 1, 4, 1, 2, 128, 4, 4)]
    for i, (dn, B, N, Nk, Nb, G, rb, tb) in enumerate(qk_cases):
        g = torch.Generator().manual_seed(4200 + i)
        q = torch.randn(B, N, 1, 128, generator=g).to(DT[dn])
        keys = oracle.synth_keys(B, Nk, Nb * G, 128, DT[dn], seed=4300 + i)
        stub = types.SimpleNamespace(rbits=rb, tbits=tb, group_size=G)
        idx, rs, rm, ts, tm = llama.LlamaPolarGroupAttention.quantize_and_pack_nbit(stub, keys)
        logits = triton_logits_cpu(q, idx, rs, rm, ts, tm, rbits=rb, tbits=tb)
        save(f"qk_{dn}_n{N}k{Nk}_r{rb}t{tb}_g{G}", q=q, indices=idx, rscale=rs, rmn=rm, tscale=ts, tmn=tm,
             logits=logits, meta=np.array([rb, tb, G]))
    # arbitrary codes and scales, as benchmark/benchmark_matmul.py:94-99 feeds the entry point
    g = torch.Generator().manual_seed(4250)
    q = torch.randn(1, 4, 1, 128, generator=g).to(torch.float16)
    idx = torch.randint(0, 250, (1, 4, 2, 32, 64), generator=g, dtype=torch.uint8)
    rs, rm, ts, tm = (torch.randn(1, 4, 2, 1, 64, generator=g).to(torch.float16) for _ in range(4))
    save("qk_fp16_random_codes", q=q, indices=idx, rscale=rs, rmn=rm, tscale=ts, tmn=tm,
         logits=triton_logits_cpu(q, idx, rs, rm, ts, tm), meta=np.array([4, 4, 32]))

    # ---------------------------------------------------------------- decode branch of the real forward
    from transformers import LlamaConfig, Qwen2Config

    def run_forward(family, dn, B, N, Nk, Nb, R, with_mask, seed):
        """One decode step through the reference attention module.  Projections are 0/1
        selection matrices: hidden = [q (N*hd) | k_new (Nk*hd) | v_new (Nk*hd)]."""
        dt = DT[dn]
        hd, G = 128, 128
        hidden = (N + 2 * Nk) * hd
        if family == "llama":
            cfg = LlamaConfig(hidden_size=hidden, intermediate_size=64, num_hidden_layers=1,
                              num_attention_heads=N, num_key_value_heads=Nk, vocab_size=32, head_dim=hd)
            attn = llama.LlamaPolarGroupAttention(cfg, layer_idx=0)
        else:
            cfg = Qwen2Config(hidden_size=hidden, intermediate_size=64, num_hidden_layers=1,
                              num_attention_heads=N, num_key_value_heads=Nk, vocab_size=32, head_dim=hd)
            attn = qwen.Qwen2PolarGroupAttention(cfg, layer_idx=0)
        attn = attn.to(dt).eval()
        with torch.no_grad():
            def select(lin, start, rows):
                w = torch.zeros(rows, hidden)
                w[torch.arange(rows), start + torch.arange(rows)] = 1.0
                lin.weight.copy_(w.to(dt))
                if lin.bias is not None:
                    lin.bias.zero_()
            select(attn.q_proj, 0, N * hd)
            select(attn.k_proj, N * hd, Nk * hd)
            select(attn.v_proj, (N + Nk) * hd, Nk * hd)
            # o_proj maps N*hd -> hidden; keep the first N*hd outputs as the identity
            w = torch.zeros(hidden, N * hd)
            w[torch.arange(N * hd), torch.arange(N * hd)] = 1.0
            attn.o_proj.weight.copy_(w.to(dt))
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(B, N, 1, hd, generator=g).to(dt)
        k_new = oracle.synth_keys(B, Nk, 1, hd, dt, seed=seed + 1)
        v_all = torch.randn(B, Nk, Nb * G + R, hd, generator=g).to(dt)
        keys_q = oracle.synth_keys(B, Nk, Nb * G, hd, dt, seed=seed + 2)
        k_res_old = oracle.synth_keys(B, Nk, R - 1, hd, dt, seed=seed + 3) if R > 1 else None
        stub = types.SimpleNamespace(rbits=4, tbits=4, group_size=G)
        idx, rs, rm, ts, tm = llama.LlamaPolarGroupAttention.quantize_and_pack_nbit(stub, keys_q)
        hidden_states = torch.cat([q.transpose(1, 2).reshape(B, 1, N * hd),
                                   k_new.transpose(1, 2).reshape(B, 1, Nk * hd),
                                   v_all[:, :, -1:, :].transpose(1, 2).reshape(B, 1, Nk * hd)], dim=-1)
        cos = torch.ones(B, 1, hd, dtype=dt)
        sin = torch.zeros(B, 1, hd, dtype=dt)
        past = (k_res_old, idx, rs, rm, ts, tm, v_all[:, :, :-1, :], Nb * G + R - 1)
        mask = None
        if with_mask:
            mask = torch.ones(B, Nb * G + R, dtype=torch.float32)
            mask[0, :37] = 0.0                    # left padding of the first sequence
        with torch.no_grad():
            out, new_past = attn(hidden_states, attention_mask=mask, past_key_value=past,
                                 position_embeddings=(cos, sin))
        attn_out = out[:, 0, : N * hd].reshape(B, N, hd)[:, :, None, :]      # (B, N, 1, hd)
        k_res = k_new if k_res_old is None else torch.cat([k_res_old, k_new], dim=2)
        tag = f"attn_{family}_{dn}_n{N}k{Nk}_nb{Nb}_r{R}" + ("_mask" if with_mask else "")
        save(tag, q=q, k_res=k_res, indices=idx, rscale=rs, rmn=rm, tscale=ts, tmn=tm, v=v_all,
             mask=(mask if mask is not None else np.zeros(0, dtype=np.float32)), out=attn_out,
             meta=np.array([4, 4, G]))

    def run_forward_mixed(dn, B, N, Nk, Nb, R, with_mask, seed):
        """One decode step through LlamaPolarMixedGroupAttention: packed keys and packed values for the first
        Nb*128 tokens, R full-precision keys / values (incl. the new token) behind them."""
        dt = DT[dn]
        hd, G = 128, 128
        hidden = (N + 2 * Nk) * hd
        cfg = LlamaConfig(hidden_size=hidden, intermediate_size=64, num_hidden_layers=1,
                          num_attention_heads=N, num_key_value_heads=Nk, vocab_size=32, head_dim=hd)
        attn = llama.LlamaPolarMixedGroupAttention(cfg, layer_idx=0).to(dt).eval()
        with torch.no_grad():
            def select(lin, start, rows):
                w = torch.zeros(rows, hidden)
                w[torch.arange(rows), start + torch.arange(rows)] = 1.0
                lin.weight.copy_(w.to(dt))
            select(attn.q_proj, 0, N * hd)
            select(attn.k_proj, N * hd, Nk * hd)
            select(attn.v_proj, (N + Nk) * hd, Nk * hd)
            w = torch.zeros(hidden, N * hd)
            w[torch.arange(N * hd), torch.arange(N * hd)] = 1.0
            attn.o_proj.weight.copy_(w.to(dt))
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(B, N, 1, hd, generator=g).to(dt)
        k_new = oracle.synth_keys(B, Nk, 1, hd, dt, seed=seed + 1)
        v_q = (torch.randn(B, Nk, Nb * G, hd, generator=g) * (1.0 + torch.rand(B, Nk, Nb * G, 1, generator=g))).to(dt)
        v_res = torch.randn(B, Nk, R, hd, generator=g).to(dt)          # incl. the new token's value (last row)
        keys_q = oracle.synth_keys(B, Nk, Nb * G, hd, dt, seed=seed + 2)
        k_res_old = oracle.synth_keys(B, Nk, R - 1, hd, dt, seed=seed + 3) if R > 1 else None
        stub = types.SimpleNamespace(rbits=4, tbits=4, group_size=G)
        idx, rs, rm, ts, tm = llama.LlamaPolarGroupAttention.quantize_and_pack_nbit(stub, keys_q)
        vc, vs, vm = oracle.quantize_values(v_q, 4)
        hidden_states = torch.cat([q.transpose(1, 2).reshape(B, 1, N * hd),
                                   k_new.transpose(1, 2).reshape(B, 1, Nk * hd),
                                   v_res[:, :, -1:, :].transpose(1, 2).reshape(B, 1, Nk * hd)], dim=-1)
        cos = torch.ones(B, 1, hd, dtype=dt)
        sin = torch.zeros(B, 1, hd, dtype=dt)
        v_res_old = v_res[:, :, :-1, :] if R > 1 else None
        past = (k_res_old, idx, rs, rm, ts, tm, v_res_old, vc, vs, vm, Nb * G + R - 1)
        mask = None
        if with_mask:
            mask = torch.ones(B, Nb * G + R, dtype=torch.float32)
            mask[0, :37] = 0.0
        with torch.no_grad():
            out, new_past = attn(hidden_states, attention_mask=mask, past_key_value=past,
                                 position_embeddings=(cos, sin))
        attn_out = out[:, 0, : N * hd].reshape(B, N, hd)[:, :, None, :]
        k_res = k_new if k_res_old is None else torch.cat([k_res_old, k_new], dim=2)
        tag = f"attn_mixed_{dn}_n{N}k{Nk}_nb{Nb}_r{R}" + ("_mask" if with_mask else "")
        save(tag, q=q, k_res=k_res, indices=idx, rscale=rs, rmn=rm, tscale=ts, tmn=tm, v_codes=vc, v_scale=vs,
             v_mn=vm, v_res=v_res, mask=(mask if mask is not None else np.zeros(0, dtype=np.float32)),
             out=attn_out, meta=np.array([4, 4, G, 4]))

    llama.cuda_bmm_fA_qB_outer = lambda group, fA, qB, scales, zeros, bits: oracle.values_matmul(fA, qB, scales, zeros, bits)
    llama.triton_quantize_and_pack_along_last_dim = lambda data, group, bit: oracle.quantize_values(data, bit)
    run_forward_mixed("bf16", 2, 8, 2, 2, 37, False, 4500)
    run_forward_mixed("fp16", 1, 4, 4, 1, 1, False, 4510)
    run_forward_mixed("bf16", 2, 4, 2, 2, 100, True, 4520)

    run_forward("llama", "bf16", 2, 8, 2, 2, 37, False, 4400)
    run_forward("llama", "fp16", 1, 4, 4, 1, 1, False, 4410)
    run_forward("llama", "bf16", 2, 4, 2, 2, 100, True, 4420)
    run_forward("qwen", "bf16", 1, 7, 1, 2, 64, False, 4430)
    run_forward("llama", "fp32", 1, 4, 2, 1, 17, False, 4440)


if __name__ == "__main__":
    main()
