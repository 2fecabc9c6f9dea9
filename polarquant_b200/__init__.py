"""polarquant_b200: the polar key-cache hot path of ericshwu/PolarQuant as hand-written sm_100a CUDA.

* ``quantize_and_pack_nbit`` - polar key quantizer (reference: models/modeling_llama_polar.py:135-157)
* ``attention_decode_forward_triton_impl`` - fp32 QK logits over packed keys (models/kernel4group.py:83-109)
* ``decode_attention`` - fused decode attention over the polar cache (models/modeling_llama_polar.py:66-99)
* ``merge_lse`` - log-sum-exp merge for sequence-split attention
* ``rope_quantize`` - prefill-side fusion: rotary embedding and key quantisation in one pass
* ``keys_repack`` / ``key_format="packed6"`` - opt-in 48-byte-per-token container for the 6-bit bit splits
* ``quantize_values`` / ``values_matmul`` / ``values_relayout`` - 4-bit value cache of the mixed key/value class
  (models/modeling_llama_polar.py:160-292); ``decode_attention(value_codes=...)`` fuses it
* ``dropin`` - run the reference's unmodified attention patches and benchmark on top of this package

All compute goes through ``polarquant_b200/csrc/libpolarquant_b200.so``; there is no CPU path.
"""
from .kernel4group import attention_decode_forward_triton_impl
from .ops import (decode_attention, key_range_check, keys_repack, merge_lse, qk_decode, quantize_and_pack_nbit, quantize_values, rope_quantize,
                  values_matmul, values_relayout)

__all__ = [
    "attention_decode_forward_triton_impl",
    "decode_attention",
    "key_range_check",
    "keys_repack",
    "merge_lse",
    "qk_decode",
    "quantize_and_pack_nbit",
    "quantize_values",
    "rope_quantize",
    "values_matmul",
    "values_relayout",
]
