"""The reference's own, unmodified files running on top of the CUDA kernels on a GPU.

``oracle/install_ref.py`` places byte-for-byte copies of the reference's attention patches, its Triton kernel module
and its micro-benchmark under the git-ignored ``oracle/_ref``; these tests are skipped when that directory is
absent.  ``polarquant_b200.dropin`` binds the patches to this package exactly as a user would (the module
``models.kernel4group`` and the method ``quantize_and_pack_nbit``, models/modeling_llama_polar.py:20,84,126), with
the DEFAULT binding: the CUDA library.  The yardstick is the same model, same weights, same tokens, run through the
reference's own Triton kernel (models/kernel4group.py:14-109) and its own eager quantizer (:135-157) on the same
GPU - or, where Triton cannot build that kernel for this GPU, through the reference's dequantise-then-matmul
formula (models/kernel4group.py:151-155).
"""
import importlib
import os
import sys
import types

import pytest
import torch

from conftest import ATTN_MAX_ABS, ATTN_MEAN_ABS
from oracle import polar_oracle as oracle
from oracle import ref_harness

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(ref_harness.ref_root() is None, reason="oracle/_ref not installed (oracle/install_ref.py)")]

DEV = "cuda"


@pytest.fixture()
def clean_models_namespace():
    saved = {k: v for k, v in sys.modules.items() if k == "models" or k.startswith("models.")}
    yield
    for k in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
        del sys.modules[k]
    sys.modules.update(saved)


_TRITON_STATE = {}


def reference_entry_module():
    """The reference's kernel module when Triton can compile its kernel here, else the dequantise formula; the
    second element says which."""
    if "mod" not in _TRITON_STATE:
        try:
            refk = ref_harness.load_reference_kernel_module()
            q = torch.randn(1, 4, 1, 128, device=DEV, dtype=torch.float16)
            idx = torch.randint(0, 250, (1, 4, 1, 32, 64), device=DEV, dtype=torch.uint8)
            sc = [torch.randn(1, 4, 1, 1, 64, device=DEV, dtype=torch.float16) for _ in range(4)]
            refk.attention_decode_forward_triton_impl(q, idx, *sc)
            torch.cuda.synchronize()
            _TRITON_STATE.update(mod=refk, kind="triton", error=None)
        except Exception as e:  # Triton cannot build the kernel for this GPU / release
            _TRITON_STATE.update(mod=ref_harness.dequantise_entry_module(), kind="dequantise formula",
                                 error=f"{type(e).__name__}: {e}"[:300])
    return _TRITON_STATE["mod"], _TRITON_STATE["kind"]


def load_patches(entry_module=None, bind_cuda_quantizer=True):
    """The reference patches from oracle/_ref; with ``bind_cuda_quantizer=False`` the quantizer stays the
    reference's own method."""
    from polarquant_b200 import dropin
    root = ref_harness.ref_root()
    if bind_cuda_quantizer:
        return dropin.load_polar_patches(root, entry_module=entry_module)
    dropin.install(root, entry_module=entry_module)
    return importlib.import_module("models.modeling_llama_polar"), importlib.import_module("models.modeling_qwen_polar")


def run_teacher_forced(model, prompt_ids, forced, hook_layer0):
    """Prefill + one decode step per column of ``forced``; returns (per-step logits, layer-0 attention outputs,
    final cache)."""
    captured = []
    handle = model.model.layers[0].self_attn.register_forward_hook(lambda m, i, o: captured.append(o[0].detach().clone()))
    logits = []
    with torch.no_grad():
        out = model(input_ids=prompt_ids, past_key_values=None, num_logits_to_keep=1)
        logits.append(out.logits[:, -1].float())
        for s in range(forced.shape[1]):
            out = model(input_ids=forced[:, s:s + 1], past_key_values=out.past_key_values, num_logits_to_keep=1)
            logits.append(out.logits[:, -1].float())
    handle.remove()
    return logits, captured, out.past_key_values


def compare_runs(build_model, family_loader, prompt_len=300, steps=140, batch=2, vocab=128):
    """Model A: reference files on the CUDA kernels.  Model B: reference files on the reference's own kernel and
    quantizer.  Same weights, same tokens."""
    entry_b, kind = reference_entry_module()
    patch_a = family_loader(load_patches(None, True))
    torch.manual_seed(0)
    model_a = build_model(patch_a).to(torch.bfloat16).to(DEV).eval()
    state = {k: v.clone() for k, v in model_a.state_dict().items()}
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, vocab, (batch, prompt_len), generator=g).to(DEV)
    forced = torch.randint(0, vocab, (batch, steps), generator=g).to(DEV)
    logits_a, attn_a, past_a = run_teacher_forced(model_a, prompt, forced, True)

    patch_b = family_loader(load_patches(entry_b, False))
    assert patch_b is not patch_a
    model_b = build_model(patch_b).to(torch.bfloat16).to(DEV).eval()
    model_b.load_state_dict(state)
    logits_b, attn_b, past_b = run_teacher_forced(model_b, prompt, forced, True)

    # layer 0 sees identical inputs in both runs (embeddings of the same tokens), so its cache must hold the same
    # bits: codes and scales from the CUDA quantizer vs the reference's eager quantizer, at the prefill call (a
    # strided view) and at the decode-branch call (a full window)
    for i in range(1, 6):
        assert torch.equal(past_a[0][i], past_b[0][i]), f"layer-0 cache element {i} differs (yardstick: {kind})"
    assert past_a[0][-1] == past_b[0][-1] == prompt_len + steps
    # layer-0 attention outputs (after o_proj, whose gain is below one for these weights): the attention bar
    for s, (a, b) in enumerate(zip(attn_a[1:], attn_b[1:])):                 # [0] is the prefill
        d = (a.float() - b.float()).abs()
        assert float(d.max()) <= ATTN_MAX_ABS and float(d.mean()) <= ATTN_MEAN_ABS, (s, float(d.max()), kind)
    # logits after the remaining layers: errors of the first layer's attention pass through norms and projections
    for s, (a, b) in enumerate(zip(logits_a, logits_b)):
        scale = float(b.abs().max())
        d = (a - b).abs()
        assert float(d.max()) <= 5e-2 * scale and float(d.mean()) <= 5e-3 * scale, (s, float(d.max()), scale, kind)
    return kind


def test_llama_patch_prefill_and_decode_on_the_cuda_kernels(clean_models_namespace):
    from transformers import LlamaConfig
    cfg = LlamaConfig(hidden_size=1024, intermediate_size=512, num_hidden_layers=2, num_attention_heads=8,
                      num_key_value_heads=2, vocab_size=128, head_dim=128)
    kind = compare_runs(lambda llama: llama.LlamaPolarForCausalLM(cfg), lambda pair: pair[0])
    print("yardstick:", kind, _TRITON_STATE.get("error"))


def test_qwen_patch_prefill_and_decode_on_the_cuda_kernels(clean_models_namespace):
    """7 query heads per kv head; the Qwen patch hands the kernel codes and scales repeated per query head
    (models/modeling_qwen_polar.py:64-76).  Two kv heads, not one: with a single kv head ``repeat_kv_quant``
    returns a stride-0 view instead of a copy, and the reference's Triton wrapper, which does raw pointer
    arithmetic on what it assumes to be contiguous tensors (models/kernel4group.py:40-53), then reads memory that
    is not the tensor's.  This library's entry point honours the strides (covered with one kv head by
    test_decode_branch_of_the_reference_forward_matches_the_fused_kernel); the yardstick needs a case where the
    reference itself is well defined."""
    from transformers import Qwen2Config
    cfg = Qwen2Config(hidden_size=14 * 128, intermediate_size=512, num_hidden_layers=2, num_attention_heads=14,
                      num_key_value_heads=2, vocab_size=128)
    compare_runs(lambda qwen: qwen.Qwen2PolarForCausalLM(cfg), lambda pair: pair[1])


def test_reference_generate_loop_runs_on_the_cuda_kernels(clean_models_namespace):
    """The reference's own greedy ``generate`` (models/modeling_llama_polar.py:622-666) over the patched model:
    it must produce max_new_tokens ids, crossing a window boundary, with the CUDA binding."""
    from transformers import LlamaConfig
    llama, _ = load_patches(None, True)
    cfg = LlamaConfig(hidden_size=1024, intermediate_size=512, num_hidden_layers=2, num_attention_heads=8,
                      num_key_value_heads=2, vocab_size=128, head_dim=128)
    torch.manual_seed(1)
    model = llama.LlamaPolarForCausalLM(cfg).to(torch.bfloat16).to(DEV).eval()
    ids = torch.randint(0, 128, (2, 250), device=DEV)
    gen_cfg = types.SimpleNamespace(eos_token_id=[-1], top_k=0, top_p=1.0, temperature=1.0)
    out = llama.generate(model, ids, None, gen_cfg, do_sample=False, max_new_tokens=20)
    assert out.shape == (2, 20) and int(out.min()) >= 0 and int(out.max()) < 128


def test_mixed_and_snapkv_classes_decode_on_the_cuda_kernels(clean_models_namespace):
    """LlamaPolarMixedGroupAttention (models/modeling_llama_polar.py:160-292) and LlamaSnapKVAttention (:295-443),
    unmodified, one prefill and a few decode steps each on CUDA.  Yardstick: the base class on the same inputs -
    the mixed class differs from it only by the 4-bit values (bar of the packed-value tests), the SnapKV class
    with a prompt shorter than its budget keeps every token and must match closely."""
    from transformers import LlamaConfig
    from conftest import check_mixed
    llama, _ = load_patches(None, True)
    cfg = LlamaConfig(hidden_size=512, intermediate_size=256, num_hidden_layers=1, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=100, head_dim=128)
    B, L = 2, 300
    g = torch.Generator().manual_seed(3)
    hidden = torch.randn(B, L, 512, generator=g).to(torch.bfloat16).to(DEV)
    steps = [torch.randn(B, 1, 512, generator=g).to(torch.bfloat16).to(DEV) for _ in range(3)]
    cos = torch.ones(B, L, 128, dtype=torch.bfloat16, device=DEV)
    sin = torch.zeros(B, L, 128, dtype=torch.bfloat16, device=DEV)

    def run(cls_name, nb=B):
        torch.manual_seed(0)
        attn = getattr(llama, cls_name)(cfg, layer_idx=0).to(torch.bfloat16).to(DEV).eval()
        outs = []
        with torch.no_grad():
            out, past = attn(hidden[:nb], attention_mask=None, past_key_value=None,
                             position_embeddings=(cos[:nb], sin[:nb]))
            for st in steps:
                out, past = attn(st[:nb], attention_mask=None, past_key_value=past,
                                 position_embeddings=(cos[:nb, :1], sin[:nb, :1]))
                outs.append(out)
        return outs, past

    base, past_base = run("LlamaPolarGroupAttention")
    mixed, past_mixed = run("LlamaPolarMixedGroupAttention")
    assert len(past_mixed) == 11 and past_mixed[7].dtype == torch.int32
    for a, b in zip(mixed, base):
        assert torch.isfinite(a.float()).all()
        d = (a.float() - b.float()).abs()
        # 4-bit values: error of the value reconstruction (step / 2 per channel, |V| ~ 0.6 here) behind o_proj
        assert float(d.max()) <= 0.15 and float(d.mean()) <= 2e-2, (float(d.max()), float(d.mean()))
    # the SnapKV class decodes one sequence at a time (it asserts bsz == 1, :330); below its prompt budget it keeps
    # every token, so it must reproduce the base class
    base1, past_base1 = run("LlamaPolarGroupAttention", 1)
    snap, past_snap = run("LlamaSnapKVAttention", 1)
    for a, b in zip(snap, base1):
        d = (a.float() - b.float()).abs()
        assert float(d.max()) <= ATTN_MAX_ABS and float(d.mean()) <= ATTN_MEAN_ABS
    for i in range(1, 6):
        assert torch.equal(past_snap[i], past_base1[i])
    # and with a prompt beyond its budget of 1024 + 128 tokens the selection feeds the same quantizer
    Ll = 1300
    hid = torch.randn(1, Ll, 512, generator=g).to(torch.bfloat16).to(DEV)
    c1 = torch.ones(1, Ll, 128, dtype=torch.bfloat16, device=DEV)
    s1 = torch.zeros(1, Ll, 128, dtype=torch.bfloat16, device=DEV)
    torch.manual_seed(0)
    attn = llama.LlamaSnapKVAttention(cfg, layer_idx=0).to(torch.bfloat16).to(DEV).eval()
    with torch.no_grad():
        out, past = attn(hid, attention_mask=None, past_key_value=None, position_embeddings=(c1, s1))
        assert past[0] is None and past[1].shape == (1, 2, 9, 128, 64) and past[6].shape == (1, 2, 1152, 128)
        out, past = attn(steps[0][:1], attention_mask=None, past_key_value=past,
                         position_embeddings=(c1[:, :1], s1[:, :1]))
    assert out.shape == (1, 1, 512) and torch.isfinite(out.float()).all()


def test_decode_branch_of_the_reference_forward_matches_the_fused_kernel(clean_models_namespace):
    """The decode branch itself (models/modeling_llama_polar.py:61-101), executed on CUDA by the reference's code
    with the logits from this library's drop-in entry, against the one-call fused kernel on the same tensors."""
    import polarquant_b200 as pq
    llama, qwen = load_patches(None, True)
    for family, patch, N, Nk in (("llama", llama, 8, 2), ("qwen", qwen, 7, 1)):
        dt = torch.bfloat16
        attn = ref_harness.identity_attention(patch, family, N, Nk, dt, device=DEV)
        B, Nb, G, R = 2, 3, 128, 57
        g = torch.Generator(device=DEV).manual_seed(12)
        keys = oracle.synth_keys(B, Nk, Nb * G + R, 128, dt, seed=13, device=DEV)
        q = torch.randn(B, N, 1, 128, device=DEV, generator=g).to(dt)
        v = torch.randn(B, Nk, Nb * G + R, 128, device=DEV, generator=g).to(dt)
        packed = pq.quantize_and_pack_nbit(keys[:, :, :Nb * G].contiguous(), 4, 4, G)
        past = (keys[:, :, Nb * G:-1].contiguous(), *packed, v[:, :, :-1].contiguous(), Nb * G + R - 1)
        ref_out, _ = ref_harness.decode_step(attn, q, keys[:, :, -1:], v[:, :, -1:], past)
        got = pq.decode_attention(q, keys[:, :, Nb * G:].contiguous(), *packed, v)
        d = (got.float() - ref_out.float()).abs()
        assert float(d.max()) <= ATTN_MAX_ABS and float(d.mean()) <= ATTN_MEAN_ABS, (family, float(d.max()))


def test_reference_micro_benchmark_runs_on_the_cuda_entry(clean_models_namespace, capsys):
    """benchmark/benchmark_matmul.py::test4polar (:89-120), unmodified, at its largest grid point (batch 8,
    131072 keys): 1000 warm-up and 10000 timed calls of the entry point it imports by name."""
    from polarquant_b200 import dropin
    import polarquant_b200.kernel4group as ours
    bm = dropin.load_benchmark_matmul(ref_harness.ref_root())
    assert bm.attention_decode_forward_triton_impl is ours.attention_decode_forward_triton_impl
    bm.B, bm.L = 8, 131072
    t = bm.test4polar()
    text = capsys.readouterr().out
    assert "Polar CUDA Test" in text and t > 0
    ms_per_call = t * 10.0 / 10000 * 1000                   # test4polar returns total seconds * 0.1
    print(f"test4polar on the CUDA entry: {ms_per_call:.3f} ms per call")
    assert ms_per_call < 5.79                               # the figure the reference publishes for this point
