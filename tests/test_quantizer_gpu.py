"""CUDA polar quantizer (through the C ABI) against the reference op sequence executed by torch on the same GPU.

Bar: bit-exact codes and scales (torch.equal on all five outputs)."""
import pytest
import torch

from conftest import golden_names, load_golden
from oracle import polar_oracle as oracle

pytestmark = pytest.mark.gpu

NAMES = ("indices", "rscale", "rmn", "tscale", "tmn")


def _assert_same(got, want):
    for a, b, what in zip(got, want, NAMES):
        assert a.shape == b.shape and a.dtype == b.dtype, what
        if not torch.equal(a, b):
            bad = (a != b)
            raise AssertionError(f"{what}: {int(bad.sum())} of {a.numel()} elements differ")


@pytest.mark.parametrize("name", [n for n in golden_names("quant_") if "strided" not in n])
def test_golden_inputs_bit_exact_vs_torch_cuda(name):
    import polarquant_b200 as pq
    g = load_golden(name)
    rb, tb, grp = g["meta"]
    keys = g["keys"].cuda()
    got = pq.quantize_and_pack_nbit(keys, rb, tb, grp)
    _assert_same(got, oracle.quantize_ops(keys, rb, tb, grp))


@pytest.mark.parametrize("name", [n for n in golden_names("quant_") if "strided" not in n])
def test_cpu_convention_flag_reproduces_reference_cpu_fixtures(name):
    """With the wrap constant rounded to the key dtype (torch's CPU behaviour) the kernel reproduces the
    fixtures the reference produced on CPU, up to last-bit differences between the two atan2f libraries."""
    import polarquant_b200 as pq
    from polarquant_b200 import _lib
    g = load_golden(name)
    rb, tb, grp = g["meta"]
    flags = _lib.PQ_QUANT_WRAP_DTYPE
    got = pq.quantize_and_pack_nbit(g["keys"].cuda(), rb, tb, grp, flags=flags)
    mism = float((got[0].cpu() != g["indices"]).float().mean())
    assert mism <= 2e-3, f"{mism:.2e} of the codes differ from the CPU fixture"


def test_strided_prefill_layout_is_read_in_place():
    import polarquant_b200 as pq
    g = load_golden("quant_bf16_strided")
    keys = g["keys_blnh"].cuda().transpose(1, 2)
    assert not keys.is_contiguous()
    got = pq.quantize_and_pack_nbit(keys, 4, 4, 128)
    _assert_same(got, oracle.quantize_ops(keys, 4, 4, 128))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rb,tb,grp", [(4, 4, 128), (3, 3, 32), (2, 4, 32), (4, 4, 32), (3, 3, 128), (2, 4, 128),
                                       (4, 4, 64), (4, 4, 16), (3, 5, 48), (8, 0, 128), (1, 1, 24)])
def test_seeded_keys_bit_exact(dtype, rb, tb, grp):
    import polarquant_b200 as pq
    length = grp * 6
    for kind, seed in (("loguniform", 70), ("outlier", 71)):
        keys = oracle.synth_keys(3, 4, length, 128, dtype, seed=seed, kind=kind, device="cuda")
        got = pq.quantize_and_pack_nbit(keys, rb, tb, grp)
        _assert_same(got, oracle.quantize_ops(keys, rb, tb, grp))


def test_edge_values_bit_exact():
    """Zeros, signed zeros, axis-aligned pairs, tiny and huge magnitudes, constant groups."""
    import polarquant_b200 as pq
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        keys = oracle.synth_keys(1, 2, 256, 128, dtype, seed=72, device="cuda")
        keys[0, 0, :, 0] = 0.0                     # x == 0 for a whole pair
        keys[0, 0, :, 1] = -0.0
        keys[0, 0, :, 65] = 0.0                    # y == 0
        keys[0, 0, ::2, 2] = 0.0
        keys[0, 0, ::2, 66] = 0.0                  # (0, 0) every other token
        keys[0, 0, :, 3] = 1.0
        keys[0, 0, :, 67] = -1.0                   # constant pair: zero angle and radius range
        keys[0, 1, :, 4] *= 1e-3
        keys[0, 1, :, 68] *= 1e-3
        big = 100.0 if dtype == torch.float16 else 1e4
        keys[0, 1, :, 5] *= big
        keys[0, 1, :, 69] *= big
        keys[0, 1, :128, 6] = keys[0, 1, :128, 6].abs()     # angles only in quadrants 1 and 4
        got = pq.quantize_and_pack_nbit(keys, 4, 4, 128)
        _assert_same(got, oracle.quantize_ops(keys, 4, 4, 128))


@pytest.mark.parametrize("dtype_name", ["bf16", "fp16"])
@pytest.mark.parametrize("which", [0, 1, 2])
def test_fast_paths_agree_with_exact_paths_for_every_16_bit_input_pair(dtype_name, which):
    """Exhaustive: all 2^32 (x, y) patterns.  which 0 = angle and radius of a key pair, 1 = quantisation level from
    the refined division, 2 = the packed 16-bit subtraction."""
    from polarquant_b200 import _lib
    lib = _lib.load()
    counter = torch.zeros(1, dtype=torch.int64, device="cuda")
    dt = _lib.PQ_BF16 if dtype_name == "bf16" else _lib.PQ_F16
    rc = lib.pq_selftest_quantizer(dt, which, counter.data_ptr(), None)
    assert rc == 0, lib.pq_strerror(rc)
    torch.cuda.synchronize()
    assert int(counter.item()) == 0


def test_empty_and_invalid_inputs():
    import polarquant_b200 as pq
    out = pq.quantize_and_pack_nbit(torch.empty(2, 4, 0, 128, dtype=torch.bfloat16, device="cuda"), 4, 4, 128)
    assert out[0].shape == (2, 4, 0, 128, 64) and out[1].shape == (2, 4, 0, 1, 64)
    keys = torch.randn(1, 2, 100, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(AssertionError):            # the reference asserts L % group_size == 0
        pq.quantize_and_pack_nbit(keys, 4, 4, 128)
    with pytest.raises(AssertionError):            # and rbits + tbits <= 8
        pq.quantize_and_pack_nbit(keys[:, :, :64], 5, 4, 32)
    with pytest.raises(RuntimeError):              # no CPU path
        pq.quantize_and_pack_nbit(keys.cpu()[:, :, :64], 4, 4, 32)


def test_full_size_prefill_bit_exact():
    """Llama-3.1-8B-shaped prefill: batch 16, 8 kv heads, 32768 tokens, bf16, in the strided (B, L, Nk, hd) layout."""
    import polarquant_b200 as pq
    torch.manual_seed(1002)
    base = torch.randn(16, 32768, 8, 128, device="cuda", dtype=torch.float32)
    scale = torch.exp(torch.empty(8, 128, device="cuda").uniform_(-0.6931, 2.0794))
    base = (base * scale).to(torch.bfloat16)
    keys = base.transpose(1, 2)
    got = pq.quantize_and_pack_nbit(keys, 4, 4, 128)
    for b in range(0, 16, 4):                      # the eager ops need several full-size temporaries
        want = oracle.quantize_ops(keys[b:b + 4], 4, 4, 128)
        _assert_same([t[b:b + 4] for t in got], want)


def test_host_buffer_entry_point_matches_device_entry_point():
    import ctypes
    import polarquant_b200 as pq
    from polarquant_b200 import _lib
    lib = _lib.load()
    keys = oracle.synth_keys(2, 2, 256, 128, torch.bfloat16, seed=73).contiguous().pin_memory()
    want = pq.quantize_and_pack_nbit(keys.cuda(), 4, 4, 128)
    codes = torch.empty(2, 2, 2, 128, 64, dtype=torch.uint8).pin_memory()
    sc = [torch.empty(2, 2, 2, 1, 64, dtype=torch.bfloat16).pin_memory() for _ in range(4)]
    need = lib.pq_quantize_host_staging_bytes(2, 2, 256, 128, 128, _lib.PQ_BF16)
    staging = torch.empty(need, dtype=torch.uint8, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.pq_quantize_host(keys.data_ptr(), 2, 2, 256, 128, 128, 4, 4, _lib.PQ_BF16, 0, codes.data_ptr(),
                              sc[0].data_ptr(), sc[1].data_ptr(), sc[2].data_ptr(), sc[3].data_ptr(),
                              staging.data_ptr(), need, stream)
    assert rc == 0, lib.pq_strerror(rc)
    torch.cuda.synchronize()
    _assert_same([codes, *sc], [t.cpu() for t in want])


def test_key_range_check_flags_scales_beyond_the_fp16_range():
    """The decode kernels dequantise in fp16; pq_key_range_check tells a caller when a cache's radii cannot be
    represented there (bf16 keys can reach 3e38)."""
    import polarquant_b200 as pq
    keys = oracle.synth_keys(1, 2, 256, 128, torch.bfloat16, seed=91, device="cuda")
    _, rs, rm, _, _ = pq.quantize_and_pack_nbit(keys, 4, 4, 128)
    assert int(pq.key_range_check(rs, rm, 4)) == 0
    big = keys.clone()
    big[0, 1, 200, 5] = 7.0e4                       # one channel beyond 65504
    _, rs, rm, _, _ = pq.quantize_and_pack_nbit(big, 4, 4, 128)
    assert int(pq.key_range_check(rs, rm, 4)) == 1
    nan = keys.clone()
    nan[0, 0, 3, 70] = float("nan")
    _, rs, rm, _, _ = pq.quantize_and_pack_nbit(nan, 4, 4, 128)
    assert int(pq.key_range_check(rs, rm, 4)) == 1
