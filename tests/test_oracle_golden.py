"""The CPU oracle against the fixtures produced by the reference's own code (tests/golden/make_golden.py)."""
import pytest
import torch

from conftest import ATTN_MAX_ABS, ATTN_MEAN_ABS, golden_names, load_golden
from oracle import polar_oracle as oracle


def _equal_values(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b)


@pytest.mark.parametrize("name", [n for n in golden_names("quant_") if "strided" not in n])
def test_quantizer_ops_and_chain_match_reference_bit_for_bit(name):
    g = load_golden(name)
    rb, tb, grp = g["meta"]
    want = (g["indices"], g["rscale"], g["rmn"], g["tscale"], g["tmn"])
    for fn, kw in ((oracle.quantize_ops, {}), (oracle.quantize_chain, {"wrap_constant": "dtype"})):
        got = fn(g["keys"], rb, tb, grp, **kw)
        for a, b, what in zip(got, want, ("indices", "rscale", "rmn", "tscale", "tmn")):
            assert _equal_values(a, b), f"{fn.__name__}: {what} differs from the reference"


def test_quantizer_strided_input_matches_reference():
    g = load_golden("quant_bf16_strided")
    keys = g["keys_blnh"].transpose(1, 2)          # (B, Nk, L, hd) view of (B, L, Nk, hd) storage
    assert not keys.is_contiguous()
    got = oracle.quantize_ops(keys, 4, 4, 128)
    for a, b in zip(got, (g["indices"], g["rscale"], g["rmn"], g["tscale"], g["tmn"])):
        assert _equal_values(a, b)


def test_constant_group_quantises_to_code_zero():
    g = load_golden("quant_bf16_r4t4_g128")
    # pair 5 of head 1 is constant over the second group: both steps are 0 and 0/0 casts to code 0
    assert float(g["tscale"][0, 1, 1, 0, 5]) == 0.0 and float(g["rscale"][0, 1, 1, 0, 5]) == 0.0
    assert int(g["indices"][0, 1, 1, :, 5].max()) == 0
    got = oracle.quantize_chain(g["keys"], 4, 4, 128)
    assert int(got[0][0, 1, 1, :, 5].max()) == 0


def test_wrap_constant_conventions_differ_only_for_reduced_precision():
    keys = oracle.synth_keys(1, 2, 256, 128, torch.float32, seed=11)
    a = oracle.quantize_chain(keys, 4, 4, 128, wrap_constant="dtype")
    b = oracle.quantize_chain(keys, 4, 4, 128, wrap_constant="fp32")
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    keys = keys.to(torch.bfloat16)
    a = oracle.quantize_chain(keys, 4, 4, 128, wrap_constant="dtype")
    b = oracle.quantize_chain(keys, 4, 4, 128, wrap_constant="fp32")
    assert not torch.equal(a[3], b[3])             # angle steps move when 2*pi is rounded to bf16 first


@pytest.mark.parametrize("name", golden_names("qk_"))
def test_qk_logits_match_reference_kernel(name):
    g = load_golden(name)
    rb, tb, _ = g["meta"]
    args = (g["q"], g["indices"], g["rscale"], g["rmn"], g["tscale"], g["tmn"], rb, tb)
    scale = float(g["logits"].abs().max())
    for fn in (oracle.qk_logits, oracle.qk_logits_lut):
        got = fn(*args)
        assert got.shape == g["logits"].shape and got.dtype == torch.float32
        assert float((got - g["logits"]).abs().max()) <= 2e-5 * max(1.0, scale), fn.__name__


@pytest.mark.parametrize("name", golden_names("attn_"))
def test_decode_attention_matches_reference_forward(name):
    g = load_golden(name)
    rb, tb, _ = g["meta"]
    mask = g["mask"] if g["mask"].numel() else None
    got = oracle.decode_attention(g["q"], g["k_res"], g["indices"], g["rscale"], g["rmn"], g["tscale"], g["tmn"],
                                  g["v"], attention_mask=mask, rbits=rb, tbits=tb)
    diff = (got.float() - g["out"].float()).abs()
    # same op sequence as the reference forward: agreement to the last rounding of the output dtype
    assert float(diff.max()) <= 4e-3 and float(diff.mean()) <= 2e-4, (float(diff.max()), float(diff.mean()))
    exact = oracle.decode_attention(g["q"], g["k_res"], g["indices"], g["rscale"], g["rmn"], g["tscale"], g["tmn"],
                                    g["v"], attention_mask=mask, rbits=rb, tbits=tb, faithful_rounding=False)
    diff = (exact - g["out"].float()).abs()
    assert float(diff.max()) <= ATTN_MAX_ABS and float(diff.mean()) <= ATTN_MEAN_ABS


def test_merge_lse_recombines_a_split_sequence():
    g = load_golden("attn_llama_bf16_n8k2_nb2_r37")
    rb, tb, grp = g["meta"]
    full, lse = oracle.decode_attention(g["q"], g["k_res"], g["indices"], g["rscale"], g["rmn"], g["tscale"],
                                        g["tmn"], g["v"], rbits=rb, tbits=tb, faithful_rounding=False,
                                        return_lse=True)
    # part 0: first group only; part 1: second group + residual
    sl = lambda t, a, b: t[:, :, a:b]
    o0, l0 = oracle.decode_attention(g["q"], None, sl(g["indices"], 0, 1), sl(g["rscale"], 0, 1), sl(g["rmn"], 0, 1),
                                     sl(g["tscale"], 0, 1), sl(g["tmn"], 0, 1), g["v"][:, :, :grp], rbits=rb,
                                     tbits=tb, faithful_rounding=False, return_lse=True)
    o1, l1 = oracle.decode_attention(g["q"], g["k_res"], sl(g["indices"], 1, 2), sl(g["rscale"], 1, 2),
                                     sl(g["rmn"], 1, 2), sl(g["tscale"], 1, 2), sl(g["tmn"], 1, 2),
                                     g["v"][:, :, grp:], rbits=rb, tbits=tb, faithful_rounding=False,
                                     return_lse=True)
    merged, mlse = oracle.merge_lse(torch.stack([o0[:, :, 0], o1[:, :, 0]]), torch.stack([l0, l1]))
    assert float((merged - full[:, :, 0]).abs().max()) < 1e-5
    assert float((mlse - lse).abs().max()) < 1e-5
