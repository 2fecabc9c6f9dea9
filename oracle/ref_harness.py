"""Drive the reference's OWN attention code (the copies under ``oracle/_ref``, see ``install_ref.py``) on given tensors.

Test infrastructure: used by ``tests/`` and by the reference arm of ``bench.py`` only.

The reference's decode branch lives inside ``LlamaPolarGroupAttention.forward`` / ``Qwen2PolarGroupAttention.forward``
(models/modeling_llama_polar.py:39-133, models/modeling_qwen_polar.py:30-156), behind the q/k/v/o projections and
the rotary embedding.  To feed it chosen query / key / value tensors, ``identity_attention`` builds the unmodified
module with 0/1 selection matrices as projections (hidden = [q heads | new key heads | new value heads]) and
``decode_step`` calls its ``forward`` with cos = 1, sin = 0.  Everything between the projections - the call of
``attention_decode_forward_triton_impl``, the residual-key logits, scaling, mask, softmax, P.V, the cache
concatenations and the re-quantisation of a full window - is the reference's code, executed as it is.
"""
from __future__ import annotations

import importlib.util
import os
import types

import torch

from . import install_ref
from . import polar_oracle as oracle


def ref_root() -> str | None:
    """Directory holding the reference's files for the path, or None when the recipe has not been run."""
    return install_ref.DEST if install_ref.installed() else None


def load_reference_kernel_module():
    """The reference's models/kernel4group.py (Triton kernel + wrapper) as a module of its own."""
    root = ref_root()
    if root is None:
        raise FileNotFoundError("oracle/_ref is absent: run `python oracle/install_ref.py` where the checkout exists")
    spec = importlib.util.spec_from_file_location("ref_kernel4group", os.path.join(root, "models", "kernel4group.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def dequantise_entry_module() -> types.ModuleType:
    """A stand-in for ``models.kernel4group`` that serves the logits by the reference's own dequantise-then-matmul
    formula (models/kernel4group.py:151-155, restated in ``polar_oracle.qk_logits``) - the form of the reference
    that runs on host cores, where its Triton kernel cannot."""
    mod = types.ModuleType("models.kernel4group")

    def attention_decode_forward_triton_impl(query_states, indices, rscale, rmn, tscale, tmn, rbits=4, tbits=4):
        return oracle.qk_logits(query_states, indices, rscale, rmn, tscale, tmn, rbits, tbits)

    mod.attention_decode_forward_triton_impl = attention_decode_forward_triton_impl
    return mod


def identity_attention(patch_module, family: str, N: int, Nk: int, dtype, device="cpu", cls_name: str | None = None):
    """The reference attention module (unmodified class) with selection-matrix projections."""
    from transformers import LlamaConfig, Qwen2Config
    hd = 128
    hidden = (N + 2 * Nk) * hd
    if family == "llama":
        cfg = LlamaConfig(hidden_size=hidden, intermediate_size=64, num_hidden_layers=1, num_attention_heads=N,
                          num_key_value_heads=Nk, vocab_size=32, head_dim=hd)
        cls = getattr(patch_module, cls_name or "LlamaPolarGroupAttention")
    else:
        cfg = Qwen2Config(hidden_size=hidden, intermediate_size=64, num_hidden_layers=1, num_attention_heads=N,
                          num_key_value_heads=Nk, vocab_size=32, head_dim=hd)
        cls = getattr(patch_module, cls_name or "Qwen2PolarGroupAttention")
    attn = cls(cfg, layer_idx=0).to(dtype).eval()
    with torch.no_grad():
        def select(lin, start, rows):
            w = torch.zeros(rows, hidden)
            w[torch.arange(rows), start + torch.arange(rows)] = 1.0
            lin.weight.copy_(w.to(dtype))
            if lin.bias is not None:
                lin.bias.zero_()
        select(attn.q_proj, 0, N * hd)
        select(attn.k_proj, N * hd, Nk * hd)
        select(attn.v_proj, (N + Nk) * hd, Nk * hd)
        w = torch.zeros(hidden, N * hd)
        w[torch.arange(N * hd), torch.arange(N * hd)] = 1.0
        attn.o_proj.weight.copy_(w.to(dtype))
    return attn.to(device)


def decode_step(attn, q, k_new, v_new, past, attention_mask=None):
    """One decode step of the reference forward.  q (B, N, 1, 128); k_new / v_new (B, Nk, 1, 128); ``past`` is the
    reference's cache tuple BEFORE the step.  Returns (attention output (B, N, 1, 128), new cache tuple)."""
    B, N, _, hd = q.shape
    Nk = k_new.shape[1]
    hidden_states = torch.cat([q.transpose(1, 2).reshape(B, 1, N * hd), k_new.transpose(1, 2).reshape(B, 1, Nk * hd),
                               v_new.transpose(1, 2).reshape(B, 1, Nk * hd)], dim=-1)
    cos = torch.ones(B, 1, hd, dtype=q.dtype, device=q.device)
    sin = torch.zeros(B, 1, hd, dtype=q.dtype, device=q.device)
    with torch.no_grad():
        out, new_past = attn(hidden_states, attention_mask=attention_mask, past_key_value=past,
                             position_embeddings=(cos, sin))
    return out[:, 0, : N * hd].reshape(B, N, hd)[:, :, None, :], new_past
