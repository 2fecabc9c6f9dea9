"""Run the reference's unmodified files on top of this package.

The reference (ericshwu/PolarQuant) reaches the hot path through a Python module
boundary: ``from .kernel4group import attention_decode_forward_triton_impl``
(models/modeling_llama_polar.py:20, models/modeling_qwen_polar.py:19,
benchmark/benchmark_matmul.py:10) and the bound method
``self.quantize_and_pack_nbit`` (models/modeling_llama_polar.py:84,126).  This
module interposes at exactly those two points and touches nothing else:

* ``install()`` registers this package's ``kernel4group`` as ``models.kernel4group``
  in ``sys.modules`` (plus raising stand-ins for the un-vendored ``models.kivi_quant``
  the patches import), so the binding holds whatever the ``sys.path`` order is -
  running ``benchmark/benchmark_matmul.py`` puts ``benchmark/`` first, where the
  reference's own copy of the kernel would otherwise win.
* ``bind_quantizer()`` replaces the quantizer method of the polar attention classes.
* ``apply_transformers_shim()`` restores the few transformers names the patches
  were written against (transformers 4.45-4.47) when a newer release is installed.
"""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys
import types

import torch

_OVERLAY = os.path.join(os.path.dirname(os.path.abspath(__file__)), "overlay")


def _sdpa_flash_attention_forward(query_states, key_states, value_states, attention_mask, query_length,
                                  is_causal=True, use_top_left_mask=False, **kwargs):
    """``_flash_attention_forward`` with the (B, L, H, D) layout the patches pass
    (models/modeling_llama_polar.py:106-114), served by torch's fused attention.
    Prefill is outside the key-cache hot path; this is a library call."""
    import torch.nn.functional as F
    q, k, v = (t.transpose(1, 2) for t in (query_states, key_states, value_states))
    n_rep = q.shape[1] // k.shape[1]
    if n_rep > 1:
        k = k.repeat_interleave(n_rep, dim=1)
        v = v.repeat_interleave(n_rep, dim=1)
    if attention_mask is None:
        out = F.scaled_dot_product_attention(q, k, v, is_causal=is_causal and q.shape[2] > 1)
    else:
        lq, lk = q.shape[2], k.shape[2]
        keep = attention_mask[:, None, None, :].to(torch.bool).expand(-1, 1, lq, lk)
        if is_causal:
            keep = keep & torch.ones(lq, lk, dtype=torch.bool, device=q.device).tril(lk - lq)
        out = F.scaled_dot_product_attention(q, k, v, attn_mask=keep)
    return out.transpose(1, 2)


def apply_transformers_shim() -> None:
    """Give ``transformers.models.{llama,qwen2}`` the names the reference imports.

    The patches import ``_flash_attention_forward`` from the model modules and read
    ``self.num_heads`` / ``self.num_key_value_heads`` (models/modeling_llama_polar.py:10,53-55);
    recent transformers releases moved or dropped them.
    """
    import transformers.models.llama.modeling_llama as llama
    import transformers.models.qwen2.modeling_qwen2 as qwen2
    for mod, cls in ((llama, llama.LlamaAttention), (qwen2, qwen2.Qwen2Attention)):
        if not hasattr(mod, "_flash_attention_forward"):
            mod._flash_attention_forward = _sdpa_flash_attention_forward
        if not hasattr(cls, "num_heads"):
            cls.num_heads = property(lambda self: self.config.num_attention_heads)
        if not hasattr(cls, "num_key_value_heads"):
            cls.num_key_value_heads = property(lambda self: self.config.num_key_value_heads)


def _load_file(name: str, path: str) -> types.ModuleType:
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def install(reference_root: str | None = None, entry_module=None) -> None:
    """Bind ``models.kernel4group`` (and the kivi stand-ins) to this package.

    ``reference_root``: a checkout of the reference; it (and nothing else) is
    appended to ``sys.path`` so ``models.modeling_*_polar`` resolve to the
    untouched reference files.  ``entry_module`` overrides the module registered
    as ``models.kernel4group`` (tests use it to inject an instrumented stand-in).
    """
    apply_transformers_shim()
    if reference_root and reference_root not in sys.path:
        sys.path.append(reference_root)
    for name in [n for n in sys.modules if n == "models" or n.startswith("models.")]:
        del sys.modules[name]
    pkg = types.ModuleType("models")
    search = [os.path.join(_OVERLAY, "models")]
    if reference_root:
        search.append(os.path.join(reference_root, "models"))
    pkg.__path__ = search
    sys.modules["models"] = pkg
    kq = types.ModuleType("models.kivi_quant")
    kq.__path__ = [os.path.join(_OVERLAY, "models", "kivi_quant")]
    sys.modules["models.kivi_quant"] = kq
    pkg.kivi_quant = kq
    for leaf in ("matmul", "new_pack"):
        mod = _load_file(f"models.kivi_quant.{leaf}", os.path.join(_OVERLAY, "models", "kivi_quant", leaf + ".py"))
        setattr(kq, leaf, mod)
    if entry_module is None:
        from . import kernel4group as entry_module
    sys.modules["models.kernel4group"] = entry_module
    pkg.kernel4group = entry_module


def bind_quantizer(*attention_classes, quantize_fn=None) -> None:
    """Replace ``quantize_and_pack_nbit`` on the given polar attention classes.

    The replacement reads ``self.rbits / self.tbits / self.group_size`` exactly as
    the reference method does (models/modeling_llama_polar.py:34-36,135-157).
    """
    if quantize_fn is None:
        from .ops import quantize_and_pack_nbit as quantize_fn

    def method(self, key_states):
        return quantize_fn(key_states, rbits=self.rbits, tbits=self.tbits, group_size=self.group_size)

    method.__name__ = "quantize_and_pack_nbit"
    for cls in attention_classes:
        cls.quantize_and_pack_nbit = method


def load_polar_patches(reference_root: str, entry_module=None, quantize_fn=None):
    """Import the reference's Llama and Qwen2 polar patches, untouched, bound to this package.

    Returns ``(modeling_llama_polar, modeling_qwen_polar)``.
    """
    install(reference_root, entry_module=entry_module)
    llama = importlib.import_module("models.modeling_llama_polar")
    qwen = importlib.import_module("models.modeling_qwen_polar")
    bind_quantizer(llama.LlamaPolarGroupAttention, qwen.Qwen2PolarGroupAttention, quantize_fn=quantize_fn)
    return llama, qwen


def load_benchmark_matmul(reference_root: str, entry_module=None):
    """Import the reference's ``benchmark/benchmark_matmul.py`` as a module bound to this package.

    Its ``__main__`` block only times the fp16 matmul; to time the polar entry set
    the module globals ``B`` and ``L`` and call ``test4polar()``
    (benchmark/benchmark_matmul.py:15,19,89).
    """
    install(None, entry_module=entry_module)
    bench_dir = os.path.join(reference_root, "benchmark")
    return _load_file("benchmark_matmul", os.path.join(bench_dir, "benchmark_matmul.py"))
