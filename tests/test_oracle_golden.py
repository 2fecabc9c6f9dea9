"""The CPU oracle against the fixtures produced by the reference's own code (tests/golden/make_golden.py)."""
import pytest
import torch

from conftest import ATTN_MAX_ABS, ATTN_MEAN_ABS, check_mixed, golden_names, load_golden
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


@pytest.mark.parametrize("name", golden_names("attn_", exclude="attn_mixed_"))
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


@pytest.mark.parametrize("name", golden_names("attn_mixed_"))
def test_mixed_decode_attention_matches_reference_forward(name):
    """The reference's LlamaPolarMixedGroupAttention forward (its KIVI calls served by the oracle's restatement)
    against the oracle's own composition of packed keys + packed values + residual window."""
    g = load_golden(name)
    rb, tb, _, vb = g["meta"]
    mask = g["mask"] if g["mask"].numel() else None
    args = (g["q"], g["k_res"], g["indices"], g["rscale"], g["rmn"], g["tscale"], g["tmn"], g["v_codes"],
            g["v_scale"], g["v_mn"], g["v_res"])
    got = oracle.decode_attention_mixed(*args, attention_mask=mask, rbits=rb, tbits=tb, vbits=vb)
    diff = (got.float() - g["out"].float()).abs()
    assert float(diff.max()) <= 8e-3 and float(diff.mean()) <= 4e-4, (float(diff.max()), float(diff.mean()))
    exact = oracle.decode_attention_mixed(*args, attention_mask=mask, rbits=rb, tbits=tb, vbits=vb,
                                          faithful_rounding=False)
    check_mixed(exact, g["out"], name)
    # the tiled layout holds the same levels
    tiled = oracle.kivi_to_tiled(g["v_codes"])
    assert torch.equal(oracle.tiled_to_kivi(tiled), g["v_codes"])
    again = oracle.decode_attention_mixed(*args[:7], tiled, *args[8:], attention_mask=mask, rbits=rb, tbits=tb,
                                          vbits=vb, faithful_rounding=False, layout="tiled")
    assert torch.equal(again, exact)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_value_quantiser_properties(dtype):
    torch.manual_seed(7)
    v = (torch.randn(2, 3, 50, 128) * (0.2 + 3 * torch.rand(2, 3, 50, 1))).to(dtype)
    v[0, 0, 3] = 1.5                                    # constant token: 0 / 0 -> level 0, exact reconstruction
    v[1, 2, 7, 5] = 40.0                                # outlier stretches one token's scale
    codes, scale, mn = oracle.quantize_values(v)
    assert codes.shape == (2, 3, 50, 16) and codes.dtype == torch.int32 and scale.shape == (2, 3, 50, 1)
    levels = oracle.unpack_values(codes)
    assert int(levels.min()) >= 0 and int(levels.max()) <= 15
    assert torch.equal(levels[0, 0, 3], torch.zeros(128, dtype=torch.int32)) and float(scale[0, 0, 3]) == 0.0
    back = oracle.dequantize_values(codes, scale, mn)
    assert torch.equal(back[0, 0, 3], torch.full((128,), 1.5))
    # every channel within (a little over, for the 16-bit roundings) half a step of its value
    err = (back - v.float()).abs()
    slack = 0.5 if dtype == torch.float32 else 0.65
    assert bool((err <= slack * scale.float() + 1e-6).all())
    # the minimum maps to level 0 and the maximum to level 15
    am, ax = v.float().argmin(-1, keepdim=True), v.float().argmax(-1, keepdim=True)
    nz = scale.float()[..., 0] > 0
    assert bool((levels.gather(-1, am)[..., 0][nz] == 0).all()) and bool((levels.gather(-1, ax)[..., 0][nz] == 15).all())
    # the two scale formulas differ only in the last place of the scale
    _, s_true, _ = oracle.quantize_values(v, scalar_division="true")
    assert float(((s_true.float() - scale.float()).abs() / scale.float().clamp_min(1e-30)).max()) <= 2.0 ** -7
    # product with probabilities
    p = torch.softmax(torch.randn(2, 3, 1, 50), -1).to(dtype)
    ref = torch.matmul(p.float(), back)
    got = oracle.values_matmul(p, codes, scale, mn)
    assert float((got.float() - ref).abs().max()) <= 2e-2


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


def test_packed_key_container_round_trips_in_the_oracle():
    """pack_keys6 / unpack_keys6 restate the 48-byte-per-token layout; they must invert each other and place
    individual codes where the definition says."""
    import numpy as np
    g = torch.Generator().manual_seed(17)
    c = torch.randint(0, 64, (3, 48, 64), generator=g, dtype=torch.uint8)
    p = oracle.pack_keys6(c)
    assert p.shape == (3, 3, 768) and torch.equal(oracle.unpack_keys6(p), c)
    tile = p[1, 2].numpy()                                     # unit 1, tokens 32..47
    lane = 4 * 5 + 2                                           # token row g = 5, pair block t = 2
    a1 = int(np.frombuffer(tile[16 * lane + 4: 16 * lane + 8].tobytes(), dtype="<u4")[0])     # A1 of token 32 + 5
    assert (a1 >> 8) & 15 == int(c[1, 37, 32 + 8 + 1]) & 15    # nibble 2: code p = 9 (k = 1, i = 1)
    h_hi = int(np.frombuffer(tile[512 + 8 * lane + 4: 512 + 8 * lane + 8].tobytes(), dtype="<u4")[0])   # token 45
    assert (h_hi >> (16 + 2 * 5)) & 3 == int(c[1, 45, 32 + 4 * 2 + 1 + 2]) >> 4                # W = 2, E = 1 partner
