"""ctypes binding of libpolarquant_b200.so (C ABI declared in include/polarquant_b200.h).

The CUDA library is the only compute path of this package: if it has not been
built, importing this module raises instead of falling back to anything else.
Build it with ``python -c "import __graft_entry__ as g; g.build()"`` or
``make -C polarquant_b200/csrc``.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# POLARQUANT_B200_LIB points at an alternative build of the same library (kernel tuning experiments)
LIB_PATH = os.environ.get("POLARQUANT_B200_LIB") or os.path.join(_HERE, "csrc", "libpolarquant_b200.so")

PQ_F16, PQ_BF16, PQ_F32 = 0, 1, 2
PQ_OK = 0
PQ_QUANT_WRAP_DTYPE = 1
PQ_QUANT_NORM_FMA = 2
PQ_VALUES_KIVI, PQ_VALUES_TILED = 0, 1
PQ_IPC_HANDLE_BYTES = 64
PQ_EXCHANGE_MAX_RANKS = 8
PQ_EXCHANGE_AFTER_ATTENTION = 1
PQ_EXCHANGE_PUSHED = 2
PQ_KEYS_BYTE, PQ_KEYS_PACKED6 = 0, 1
PQ_QUANT_PACK6 = 4

EXPORTED_SYMBOLS = (
    "pq_quantize", "pq_qk_decode", "pq_decode_attention", "pq_decode_workspace_bytes", "pq_merge_lse",
    "pq_quantize_host", "pq_quantize_host_staging_bytes", "pq_decode_attention_host",
    "pq_decode_host_staging_bytes", "pq_strerror", "pq_last_cuda_error", "pq_abi_version", "pq_decode_params_size",
    "pq_event_create", "pq_event_destroy", "pq_event_record", "pq_event_elapsed_ms",
    "pq_decode_attention_static", "pq_decode_static_scratch_bytes", "pq_selftest_quantizer", "pq_quantize_into", "pq_cache_append",
    "pq_quantize_values", "pq_values_relayout", "pq_values_matmul",
    "pq_cache_append_dyn", "pq_decode_workspace_bytes_dyn", "pq_rope_append",
    "pq_quantize_into_dyn", "pq_quantize_values_dyn", "pq_lengths_advance", "pq_key_range_check",
    "pq_keys_repack", "pq_rope_quantize", "pq_merge_lse_strided",
)

_i64, _int, _vp, _sz, _f32 = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float


class DecodeParams(ctypes.Structure):
    """Mirror of ``struct pq_decode_params`` (field order and types must match the header)."""
    _fields_ = [
        ("q", _vp), ("q_stride_b", _i64), ("q_stride_h", _i64),
        ("codes", _vp), ("codes_stride_b", _i64), ("codes_stride_h", _i64),
        ("rscale", _vp), ("rmn", _vp), ("tscale", _vp), ("tmn", _vp),
        ("scale_stride_b", _i64), ("scale_stride_h", _i64),
        ("k_res", _vp), ("kres_stride_b", _i64), ("kres_stride_h", _i64), ("kres_stride_t", _i64),
        ("v", _vp), ("v_stride_b", _i64), ("v_stride_h", _i64), ("v_stride_t", _i64),
        ("mask", _vp), ("mask_stride_b", _i64),
        ("out", _vp), ("out_stride_b", _i64), ("out_stride_h", _i64),
        ("lse", _vp),
        ("workspace", _vp), ("workspace_bytes", _sz),
        ("B", _int), ("N", _int), ("Nk", _int), ("Nb", _int), ("G", _int), ("R", _int), ("hd", _int),
        ("rbits", _int), ("tbits", _int),
        ("qk_dtype", _int), ("v_dtype", _int), ("out_dtype", _int),
        ("sm_scale", _f32),
        ("num_ctas", _int),
        ("mid_event", _vp),
        ("v_codes", _vp), ("vcodes_stride_b", _i64), ("vcodes_stride_h", _i64),
        ("v_scale", _vp), ("v_mn", _vp), ("vscale_stride_b", _i64), ("vscale_stride_h", _i64),
        ("vbits", _int),
        ("dyn_lengths", _vp), ("dyn_r_add", _int),
        ("key_format", _int),
        ("exchange_bufs", ctypes.POINTER(_vp)), ("exchange_world", _int), ("exchange_rank", _int),
        ("exchange_out", _vp), ("exchange_out_dtype", _int), ("exchange_lse_out", _vp),
    ]


def _declare(lib: ctypes.CDLL) -> None:
    lib.pq_quantize.restype = _int
    lib.pq_quantize.argtypes = [_vp, ctypes.POINTER(_i64), _int, _int, _int, _int, _int, _int, _int, _int,
                                ctypes.c_uint, _vp, _vp, _vp, _vp, _vp, _vp]
    lib.pq_rope_quantize.restype = _int
    lib.pq_rope_quantize.argtypes = [_vp, ctypes.POINTER(_i64), _vp, _vp, ctypes.POINTER(_i64), _vp, ctypes.POINTER(_i64),
                                     _int, _int, _int, _int, _int, _int, _int, _int, _int, ctypes.c_uint,
                                     _vp, _vp, _vp, _vp, _vp, ctypes.POINTER(_i64), _vp]
    lib.pq_keys_repack.restype = _int
    lib.pq_keys_repack.argtypes = [_vp, _vp, _i64, _int, _vp]
    lib.pq_key_range_check.restype = _int
    lib.pq_key_range_check.argtypes = [_vp, _vp, _i64, _int, _int, _vp, _vp]
    lib.pq_selftest_quantizer.restype = _int
    lib.pq_selftest_quantizer.argtypes = [_int, _int, _vp, _vp]
    lib.pq_quantize_into.restype = _int
    lib.pq_quantize_into.argtypes = [_vp, ctypes.POINTER(_i64), _int, _int, _int, _int, _int, _int, _int, _int,
                                     ctypes.c_uint, _vp, _vp, _vp, _vp, _vp, ctypes.POINTER(_i64), _vp]
    lib.pq_cache_append.restype = _int
    lib.pq_cache_append.argtypes = [_vp, _vp, ctypes.POINTER(_i64), _vp, ctypes.POINTER(_i64), _vp,
                                    ctypes.POINTER(_i64), _int, _int, _int, _int, _int, _int, _vp]
    lib.pq_quantize_values.restype = _int
    lib.pq_quantize_values.argtypes = [_vp, ctypes.POINTER(_i64), _int, _int, _int, _int, _int, _int, _int,
                                       _vp, _vp, _vp, ctypes.POINTER(_i64), _vp]
    lib.pq_values_relayout.restype = _int
    lib.pq_values_relayout.argtypes = [_vp, _vp, _i64, _int, _vp]
    lib.pq_values_matmul.restype = _int
    lib.pq_values_matmul.argtypes = [_vp, _vp, _vp, _vp, _vp, _i64, _int, _int, _int, _int, _int, _vp]
    lib.pq_cache_append_dyn.restype = _int
    lib.pq_cache_append_dyn.argtypes = [_vp, _vp, ctypes.POINTER(_i64), _vp, ctypes.POINTER(_i64), _vp,
                                        ctypes.POINTER(_i64), _int, _int, _int, _int, _vp, _int, _int, _int, _int, _vp]
    lib.pq_quantize_into_dyn.restype = _int
    lib.pq_quantize_into_dyn.argtypes = [_vp, ctypes.POINTER(_i64), _int, _int, _int, _int, _int, _int, _int, _int,
                                         ctypes.c_uint, _vp, _vp, _vp, _vp, _vp, ctypes.POINTER(_i64), _int, _vp,
                                         _int, _vp]
    lib.pq_quantize_values_dyn.restype = _int
    lib.pq_quantize_values_dyn.argtypes = [_vp, ctypes.POINTER(_i64), _int, _int, _int, _int, _int, _int, _int,
                                           _vp, _vp, _vp, ctypes.POINTER(_i64), _int, _int, _vp, _int, _vp]
    lib.pq_lengths_advance.restype = _int
    lib.pq_lengths_advance.argtypes = [_vp, _int, _int, _vp]
    lib.pq_rope_append.restype = _int
    lib.pq_rope_append.argtypes = [_vp, _i64, _vp, _vp, _i64, _vp, _vp, ctypes.POINTER(_i64), _vp,
                                   ctypes.POINTER(_i64), _int, _int, _int, _int, _int, _vp, _int, _int, _int, _int,
                                   _int, _int, _vp]
    lib.pq_decode_workspace_bytes_dyn.restype = _sz
    lib.pq_decode_workspace_bytes_dyn.argtypes = [_int] * 4
    lib.pq_qk_decode.restype = _int
    lib.pq_qk_decode.argtypes = [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp,
                                 _int, _int, _int, _int, _int, _int, _int, _int, _int, _vp]
    lib.pq_decode_attention.restype = _int
    lib.pq_decode_attention.argtypes = [ctypes.POINTER(DecodeParams), _vp]
    lib.pq_decode_attention_static.restype = _int
    lib.pq_decode_attention_static.argtypes = [ctypes.POINTER(DecodeParams), _vp]
    lib.pq_decode_static_scratch_bytes.restype = _sz
    lib.pq_decode_static_scratch_bytes.argtypes = []
    lib.pq_decode_workspace_bytes.restype = _sz
    lib.pq_decode_workspace_bytes.argtypes = [_int] * 7
    lib.pq_merge_lse.restype = _int
    lib.pq_merge_lse.argtypes = [_vp, _vp, _int, _i64, _int, _vp, _int, _vp, _vp]
    lib.pq_merge_lse_strided.restype = _int
    lib.pq_merge_lse_strided.argtypes = [_vp, _i64, _vp, _i64, _int, _i64, _int, _vp, _int, _vp, _vp]
    lib.pq_exchange_bytes.restype = _i64
    lib.pq_exchange_bytes.argtypes = [_int, _i64, _int]
    lib.pq_exchange_slot_offset.restype = _i64
    lib.pq_exchange_slot_offset.argtypes = [_int, _i64, _int, _int]
    lib.pq_peer_alloc.restype = _int
    lib.pq_peer_alloc.argtypes = [_i64, ctypes.POINTER(_vp), ctypes.c_char_p]
    lib.pq_peer_open.restype = _int
    lib.pq_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(_vp)]
    lib.pq_peer_close.restype = _int
    lib.pq_peer_close.argtypes = [_vp]
    lib.pq_peer_free.restype = _int
    lib.pq_peer_free.argtypes = [_vp]
    lib.pq_exchange_merge.restype = _int
    lib.pq_exchange_merge.argtypes = [ctypes.POINTER(_vp), _int, _int, _i64, _int, _vp, _int, _vp, ctypes.c_uint, _vp]
    lib.pq_exchange_merge_emulated.restype = _int
    lib.pq_exchange_merge_emulated.argtypes = [ctypes.POINTER(_vp), _int, _i64, _int, ctypes.POINTER(_vp), _int,
                                               ctypes.POINTER(_vp), ctypes.c_uint, _vp]
    lib.pq_exchange_status.restype = _int
    lib.pq_exchange_status.argtypes = [_vp, _int, _i64, _int, ctypes.POINTER(ctypes.c_uint), _vp]
    lib.pq_quantize_host.restype = _int
    lib.pq_quantize_host.argtypes = [_vp, _int, _int, _int, _int, _int, _int, _int, _int, ctypes.c_uint,
                                     _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]
    lib.pq_quantize_host_staging_bytes.restype = _sz
    lib.pq_quantize_host_staging_bytes.argtypes = [_int] * 6
    lib.pq_decode_attention_host.restype = _int
    lib.pq_decode_attention_host.argtypes = [ctypes.POINTER(DecodeParams), _vp, _sz, _vp]
    lib.pq_decode_host_staging_bytes.restype = _sz
    lib.pq_decode_host_staging_bytes.argtypes = [_int] * 11
    lib.pq_event_create.restype = _int
    lib.pq_event_create.argtypes = [ctypes.POINTER(_vp)]
    lib.pq_event_destroy.restype = _int
    lib.pq_event_destroy.argtypes = [_vp]
    lib.pq_event_record.restype = _int
    lib.pq_event_record.argtypes = [_vp, _vp]
    lib.pq_event_elapsed_ms.restype = _int
    lib.pq_event_elapsed_ms.argtypes = [_vp, _vp, ctypes.POINTER(_f32)]
    lib.pq_strerror.restype = ctypes.c_char_p
    lib.pq_strerror.argtypes = [_int]
    lib.pq_last_cuda_error.restype = _int
    lib.pq_last_cuda_error.argtypes = []
    lib.pq_abi_version.restype = _int
    lib.pq_abi_version.argtypes = []
    lib.pq_decode_params_size.restype = _sz
    lib.pq_decode_params_size.argtypes = []


_lib = None


def load() -> ctypes.CDLL:
    """Load the CUDA library once; raise a clear error when it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"polarquant_b200: CUDA library not built ({LIB_PATH} missing). "
                "Run `make -C polarquant_b200/csrc` (needs nvcc); there is no CPU fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        _declare(lib)
        if lib.pq_abi_version() != 8:
            raise RuntimeError("polarquant_b200: library ABI version does not match this package")
        if lib.pq_decode_params_size() != ctypes.sizeof(DecodeParams):
            raise RuntimeError("polarquant_b200: pq_decode_params layout differs between library and binding")
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    """Turn a negative pq_status into the exception the reference's callers would see."""
    if status == PQ_OK:
        return
    lib = load()
    msg = lib.pq_strerror(status).decode()
    if status == -4:
        msg += f" [cudaError {lib.pq_last_cuda_error()}]"
    if status in (-1, -5):
        raise ValueError(f"{what}: {msg}")
    if status == -2:
        raise NotImplementedError(f"{what}: {msg}")
    raise RuntimeError(f"{what}: {msg}")
