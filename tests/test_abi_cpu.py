"""The C-ABI library loads without a GPU and exports every symbol include/polarquant_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "polarquant_b200.h")


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared_functions()
    for must in ("pq_quantize", "pq_qk_decode", "pq_decode_attention", "pq_decode_workspace_bytes", "pq_merge_lse",
                 "pq_quantize_host", "pq_decode_attention_host", "pq_strerror"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from polarquant_b200 import _lib
    lib = _lib.load()
    for name in _declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    for name in _lib.EXPORTED_SYMBOLS:
        assert name in _declared_functions(), f"{name} is bound in Python but missing from the header"


def test_struct_mirror_and_status_strings():
    from polarquant_b200 import _lib
    lib = _lib.load()
    assert lib.pq_abi_version() == 8
    assert lib.pq_decode_params_size() == ctypes.sizeof(_lib.DecodeParams)
    for code in (0, -1, -2, -3, -4, -5):
        assert lib.pq_strerror(code)
    assert b"unknown" in lib.pq_strerror(-99)


def test_argument_validation_needs_no_gpu():
    """Bad arguments are rejected before any CUDA call, so these run on a CPU-only box."""
    from polarquant_b200 import _lib
    lib = _lib.load()
    st = (ctypes.c_int64 * 4)(128 * 256, 256 * 128, 128, 1)
    assert lib.pq_quantize(None, st, 1, 1, 256, 128, 128, 5, 4, _lib.PQ_BF16, 0, None, None, None, None, None, None) == -1
    assert lib.pq_quantize(None, st, 1, 1, 200, 128, 128, 4, 4, _lib.PQ_BF16, 0, None, None, None, None, None, None) == -1
    assert lib.pq_quantize(None, st, 1, 1, 256, 64, 128, 4, 4, _lib.PQ_BF16, 0, None, None, None, None, None, None) == -2
    assert lib.pq_quantize(None, st, 0, 1, 256, 128, 128, 4, 4, _lib.PQ_BF16, 0, None, None, None, None, None, None) == 0
    assert lib.pq_qk_decode(None, 0, 0, None, None, None, None, None, None, 1, 6, 4, 1, 128, 64, 4, 4, 0, None) == -1
    p = _lib.DecodeParams()
    p.B, p.N, p.Nk, p.Nb, p.G, p.R, p.hd = 1, 8, 2, 1, 128, 0, 128
    p.rbits, p.tbits = 4, 5
    assert lib.pq_decode_attention(ctypes.byref(p), None) == -1           # rbits + tbits > 8
    p.tbits = 4
    p.v_dtype = _lib.PQ_F32
    assert lib.pq_decode_attention(ctypes.byref(p), None) == -2           # fp32 values are not built
    p.v_dtype = _lib.PQ_BF16
    p.vbits = 2
    assert lib.pq_decode_attention(ctypes.byref(p), None) == -2           # only 4-bit packed values are built
    # packed value cache
    vst = (ctypes.c_int64 * 4)(128 * 64, 128 * 64, 128, 1)
    assert lib.pq_quantize_values(None, vst, 1, 1, 64, 128, 4, _lib.PQ_BF16, 7, None, None, None, None, None) == -1
    assert lib.pq_quantize_values(None, vst, 1, 1, 64, 128, 2, _lib.PQ_BF16, 0, None, None, None, None, None) == -2
    assert lib.pq_quantize_values(None, vst, 1, 1, 64, 64, 4, _lib.PQ_BF16, 0, None, None, None, None, None) == -2
    assert lib.pq_quantize_values(None, vst, 1, 1, 0, 128, 4, _lib.PQ_BF16, 0, None, None, None, None, None) == 0
    assert lib.pq_quantize_values(None, vst, 1, 1, 64, 128, 4, _lib.PQ_BF16, 0, None, None, None, None, None) == -1
    assert lib.pq_lengths_advance(None, 128, 128, None) == -1
    assert lib.pq_quantize_values_dyn(None, vst, 1, 1, 64, 128, 4, _lib.PQ_BF16, 0, None, None, None, None, 128, 256,
                                      None, 1, None) == -1
    assert lib.pq_values_relayout(None, None, 0, 1, None) == 0
    assert lib.pq_values_relayout(None, None, 5, 1, None) == -1
    assert lib.pq_values_matmul(None, None, None, None, None, 0, 1, 10, 128, 4, 0, None) == 0
    assert lib.pq_values_matmul(None, None, None, None, None, 2, 1, 10, 128, 8, 0, None) == -2
    assert lib.pq_decode_workspace_bytes(16, 32, 8, 255, 128, 128, 0) > 0
    assert lib.pq_decode_workspace_bytes(16, 32, 6, 255, 128, 128, 0) == 0
    # packed key container, fused rotary + quantizer, strided merge, range check
    assert lib.pq_quantize(None, st, 1, 1, 256, 128, 128, 4, 4, _lib.PQ_BF16, _lib.PQ_QUANT_PACK6, None, None, None, None,
                           None, None) == -1                              # the packed container holds 6-bit codes only
    assert lib.pq_quantize(None, st, 1, 1, 240, 128, 24, 3, 3, _lib.PQ_BF16, _lib.PQ_QUANT_PACK6, None, None, None, None,
                           None, None) == -1                              # groups of 16 k tokens
    assert lib.pq_keys_repack(None, None, 0, _lib.PQ_KEYS_PACKED6, None) == 0
    assert lib.pq_keys_repack(None, None, 4, _lib.PQ_KEYS_PACKED6, None) == -1
    assert lib.pq_keys_repack(None, None, 4, 7, None) == -1
    p2 = _lib.DecodeParams()
    p2.B, p2.N, p2.Nk, p2.Nb, p2.G, p2.R, p2.hd = 1, 8, 2, 1, 128, 0, 128
    p2.rbits, p2.tbits, p2.v_dtype, p2.key_format = 4, 4, _lib.PQ_BF16, _lib.PQ_KEYS_PACKED6
    assert lib.pq_decode_attention(ctypes.byref(p2), None) == -1          # 4/4 codes do not fit the 6-bit container
    p2.key_format = 9
    assert lib.pq_decode_attention(ctypes.byref(p2), None) == -1
    cs = (ctypes.c_int64 * 2)(0, 128)
    assert lib.pq_rope_quantize(None, st, None, None, cs, None, st, 1, 1, 256, 200, 128, 128, 4, 4, _lib.PQ_BF16, 0, None,
                                None, None, None, None, None, None) == -1  # Lq must be whole groups
    assert lib.pq_rope_quantize(None, st, None, None, cs, None, st, 1, 1, 256, 256, 128, 128, 4, 4, _lib.PQ_F32, 0, None,
                                None, None, None, None, None, None) == -2  # 16-bit keys only
    assert lib.pq_rope_quantize(None, st, None, None, cs, None, st, 0, 1, 256, 256, 128, 128, 4, 4, _lib.PQ_BF16, 0, None,
                                None, None, None, None, None, None) == 0
    assert lib.pq_merge_lse_strided(None, 0, None, 0, 0, 4, 128, None, 0, None, None) == -1
    assert lib.pq_merge_lse_strided(None, 0, None, 0, 2, 0, 128, None, 0, None, None) == 0
    assert lib.pq_key_range_check(None, None, 0, 4, _lib.PQ_BF16, None, None) == 0
    assert lib.pq_key_range_check(None, None, 8, 4, _lib.PQ_BF16, None, None) == -1
    # the built-in scratch array: a device-side-lengths call whose explicit grid cannot fit is refused up front
    p3 = _lib.DecodeParams()
    p3.B, p3.N, p3.Nk, p3.Nb, p3.G, p3.R, p3.hd = 16, 32, 8, 255, 128, 128, 128
    p3.rbits, p3.tbits, p3.num_ctas = 4, 4, 444
    p3.dyn_lengths = 8                                                     # any non-null address: never dereferenced here
    assert lib.pq_decode_attention_static(ctypes.byref(p3), None) == -6


def test_ops_refuse_cpu_tensors():
    import torch
    import polarquant_b200 as pq
    with pytest.raises(RuntimeError, match="no CPU path"):
        pq.quantize_and_pack_nbit(torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16), 4, 4, 128)
    q = torch.zeros(1, 2, 1, 128, dtype=torch.float16)
    idx = torch.zeros(1, 2, 1, 32, 64, dtype=torch.uint8)
    s = torch.zeros(1, 2, 1, 1, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        pq.attention_decode_forward_triton_impl(q, idx, s, s, s, s)


def test_missing_library_fails_loudly(monkeypatch):
    from polarquant_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libpolarquant_b200.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()
