"""Drop-in mechanics: the reference's unmodified files bind to this package's entry points.

These tests import the reference checkout in place and therefore only run where it exists (the build
container); they are skipped elsewhere.  The compute itself is served by the CPU oracle through the
`entry_module` / `quantize_fn` hooks of `dropin`, so what is verified is the interface contract: names, argument
order, keyword use, shapes, dtypes and strides that cross the boundary during a real prefill + decode."""
import os
import sys
import types

import pytest
import torch

from oracle import polar_oracle as oracle

REF = os.environ.get("POLARQUANT_REFERENCE", os.path.join(os.sep, "root", "reference"))
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "models")),
                                reason="reference checkout not present")


class Recorder(types.ModuleType):
    def __init__(self):
        super().__init__("models.kernel4group")
        self.calls = []

    def attention_decode_forward_triton_impl(self, query_states, indices, rscale, rmn, tscale, tmn, rbits=4, tbits=4):
        self.calls.append(dict(q=(tuple(query_states.shape), query_states.dtype),
                               idx=(tuple(indices.shape), indices.dtype, indices.is_contiguous()),
                               scale=tuple(rscale.shape), rbits=rbits, tbits=tbits))
        return oracle.qk_logits(query_states, indices, rscale, rmn, tscale, tmn, rbits, tbits)


@pytest.fixture()
def patched():
    from polarquant_b200 import dropin
    saved = {k: v for k, v in sys.modules.items() if k == "models" or k.startswith("models.")}
    rec = Recorder()
    quant_calls = []

    def quant(key_states, rbits, tbits, group_size):
        quant_calls.append((tuple(key_states.shape), tuple(key_states.stride()), key_states.dtype))
        return oracle.quantize_ops(key_states, rbits, tbits, group_size)

    llama, qwen = dropin.load_polar_patches(REF, entry_module=rec, quantize_fn=quant)
    yield llama, qwen, rec, quant_calls
    for k in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
        del sys.modules[k]
    sys.modules.update(saved)


def test_reference_files_are_loaded_untouched_and_bound_to_our_entry(patched):
    llama, qwen, rec, _ = patched
    assert llama.__file__ == os.path.join(REF, "models", "modeling_llama_polar.py")
    assert qwen.__file__ == os.path.join(REF, "models", "modeling_qwen_polar.py")
    assert llama.attention_decode_forward_triton_impl.__self__ is rec
    assert qwen.attention_decode_forward_triton_impl.__self__ is rec


def test_default_binding_is_the_cuda_entry_point():
    from polarquant_b200 import dropin
    import polarquant_b200.kernel4group as ours
    saved = {k: v for k, v in sys.modules.items() if k == "models" or k.startswith("models.")}
    try:
        llama, _ = dropin.load_polar_patches(REF)
        assert llama.attention_decode_forward_triton_impl is ours.attention_decode_forward_triton_impl
        assert llama.LlamaPolarGroupAttention.quantize_and_pack_nbit.__name__ == "quantize_and_pack_nbit"
    finally:
        for k in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_llama_prefill_and_decode_cross_the_boundary_as_documented(patched):
    llama, _, rec, quant_calls = patched
    from transformers import LlamaConfig
    cfg = LlamaConfig(hidden_size=512, intermediate_size=256, num_hidden_layers=1, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=100, head_dim=128)
    torch.manual_seed(0)
    model = llama.LlamaPolarForCausalLM(cfg).to(torch.bfloat16).eval()
    ids = torch.randint(0, 100, (2, 300))
    with torch.no_grad():
        out = model(input_ids=ids, past_key_values=None, num_logits_to_keep=1)
        tok = out.logits.argmax(-1)
        for _ in range(3):
            out = model(input_ids=tok, past_key_values=out.past_key_values, num_logits_to_keep=1)
            tok = out.logits.argmax(-1)
    # prefill hands the quantizer a (B, Nk, 256, 128) view of (B, L, Nk, hd) storage
    shape, stride, dtype = quant_calls[0]
    assert shape == (2, 2, 256, 128) and dtype == torch.bfloat16
    assert stride[3] == 1 and stride[2] == 2 * 128 and stride[1] == 128
    # decode passes GQA-grouped codes natively (Nk = 2 < N = 4) and tbits/rbits by keyword
    c = rec.calls[0]
    assert c["q"] == ((2, 4, 1, 128), torch.bfloat16)
    assert c["idx"] == ((2, 2, 2, 128, 64), torch.uint8, True)
    assert c["scale"] == (2, 2, 2, 1, 64) and c["rbits"] == 4 and c["tbits"] == 4
    assert len(rec.calls) == 3


def test_qwen_patch_passes_repeated_codes(patched):
    _, qwen, rec, _ = patched
    from transformers import Qwen2Config
    cfg = Qwen2Config(hidden_size=7 * 128, intermediate_size=128, num_hidden_layers=1, num_attention_heads=7,
                      num_key_value_heads=1, vocab_size=100)
    torch.manual_seed(0)
    model = qwen.Qwen2PolarForCausalLM(cfg).to(torch.bfloat16).eval()
    with torch.no_grad():
        out = model(input_ids=torch.randint(0, 100, (1, 256)), num_logits_to_keep=1)
        model(input_ids=out.logits.argmax(-1), past_key_values=out.past_key_values, num_logits_to_keep=1)
    c = rec.calls[0]
    assert c["q"][0] == (1, 7, 1, 128)
    assert c["idx"][0] == (1, 7, 2, 128, 64)       # codes repeated to one kv head per query head


def test_benchmark_script_binds_to_our_entry(patched):
    from polarquant_b200 import dropin
    _, _, rec, _ = patched
    bm = dropin.load_benchmark_matmul(REF, entry_module=rec)
    assert bm.attention_decode_forward_triton_impl.__self__ is rec
    assert callable(bm.test4polar) and bm.N == 32 and bm.D == 64


def test_mixed_class_reaches_the_value_cache_entry_points(patched, monkeypatch):
    """LlamaPolarMixedGroupAttention (models/modeling_llama_polar.py:160-292), unmodified: its two KIVI names
    resolve to the overlay, which forwards the value-cache calls to `ops.quantize_values` / `ops.values_matmul`
    (served here by the oracle) and refuses everything else KIVI offers."""
    llama, _, rec, _ = patched
    from polarquant_b200 import ops
    from transformers import LlamaConfig
    calls = []

    def fake_quantize_values(v, vbits=4, layout="kivi"):
        calls.append(("pack", tuple(v.shape), v.dtype, vbits, layout))
        return oracle.quantize_values(v.contiguous(), vbits)

    def fake_values_matmul(p, codes, scale, mn, vbits=4):
        calls.append(("matmul", tuple(p.shape), tuple(codes.shape), codes.dtype, tuple(scale.shape), vbits))
        return oracle.values_matmul(p, codes, scale, mn, vbits)

    monkeypatch.setattr(ops, "quantize_values", fake_quantize_values)
    monkeypatch.setattr(ops, "values_matmul", fake_values_matmul)
    assert llama.cuda_bmm_fA_qB_outer.__module__ == "models.kivi_quant.matmul"
    with pytest.raises(NotImplementedError):                      # a KIVI key-cache call: not part of the polar path
        llama.cuda_bmm_fA_qB_outer(32, torch.zeros(1, 1, 1, 64), torch.zeros(1, 1, 64, 8, dtype=torch.int32),
                                   torch.zeros(1, 1, 64, 4), torch.zeros(1, 1, 64, 4), 2)
    with pytest.raises(NotImplementedError):
        llama.triton_quantize_and_pack_along_last_dim(torch.zeros(1, 1, 128, 64), 32, 2)

    cfg = LlamaConfig(hidden_size=512, intermediate_size=256, num_hidden_layers=1, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=100, head_dim=128)
    torch.manual_seed(0)
    attn = llama.LlamaPolarMixedGroupAttention(cfg, layer_idx=0).to(torch.bfloat16).eval()
    B, L = 2, 300
    hidden = torch.randn(B, L, 512).to(torch.bfloat16)
    cos, sin = torch.ones(B, L, 128, dtype=torch.bfloat16), torch.zeros(B, L, 128, dtype=torch.bfloat16)
    with torch.no_grad():
        out, past = attn(hidden, attention_mask=None, past_key_value=None, position_embeddings=(cos, sin))
        assert len(past) == 11 and past[7].shape == (B, 2, 256, 16) and past[6].shape == (B, 2, 44, 128)
        for _ in range(2):
            step = torch.randn(B, 1, 512).to(torch.bfloat16)
            out, past = attn(step, attention_mask=None, past_key_value=past,
                             position_embeddings=(cos[:, :1], sin[:, :1]))
    assert out.shape == (B, 1, 512) and torch.isfinite(out.float()).all()
    # prefill packs the 256 quantised tokens' values, one group of 128 channels per token, 4 bits
    assert calls[0] == ("pack", (B, 2, 256, 128), torch.bfloat16, 4, "kivi")
    # decode multiplies the probabilities of the packed tokens with per-query-head copies of the codes
    kind, pshape, cshape, cdtype, sshape, bits = calls[1]
    assert kind == "matmul" and pshape == (B, 4, 1, 256) and cshape == (B, 4, 256, 16) and cdtype == torch.int32
    assert sshape == (B, 4, 256, 1) and bits == 4
    assert [c[0] for c in calls] == ["pack", "matmul", "matmul"]


def test_snapkv_class_runs_on_the_same_two_entry_points(patched):
    """LlamaSnapKVAttention (models/modeling_llama_polar.py:295-443), unmodified: its prompt-side token selection is
    plain torch; what reaches this package is the quantizer call on the selected keys (1024 + 128 of them) and the
    same decode entry point as the base class."""
    llama, _, rec, quant_calls = patched
    from transformers import LlamaConfig
    cfg = LlamaConfig(hidden_size=512, intermediate_size=256, num_hidden_layers=1, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=100, head_dim=128)
    torch.manual_seed(0)
    attn = llama.LlamaSnapKVAttention(cfg, layer_idx=0).to(torch.bfloat16).eval()
    L = 1300                                              # longer than max_capacity_prompt = 1024 + 128
    hidden = torch.randn(1, L, 512).to(torch.bfloat16)
    cos, sin = torch.ones(1, L, 128, dtype=torch.bfloat16), torch.zeros(1, L, 128, dtype=torch.bfloat16)
    n_calls = len(rec.calls)
    with torch.no_grad():
        out, past = attn(hidden, attention_mask=None, past_key_value=None, position_embeddings=(cos, sin))
        # 1152 keys survive the selection: all of them are whole groups, nothing stays in full precision
        assert past[0] is None and past[1].shape == (1, 2, 9, 128, 64) and past[6].shape == (1, 2, 1152, 128)
        step = torch.randn(1, 1, 512).to(torch.bfloat16)
        out, past = attn(step, attention_mask=None, past_key_value=past, position_embeddings=(cos[:, :1], sin[:, :1]))
    assert quant_calls[-1][0] == (1, 2, 1152, 128)
    assert len(rec.calls) == n_calls + 1 and rec.calls[-1]["idx"][0] == (1, 2, 9, 128, 64)
    assert out.shape == (1, 1, 512) and torch.isfinite(out.float()).all()
