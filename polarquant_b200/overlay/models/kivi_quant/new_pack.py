"""The KIVI packer the reference imports unconditionally (models/modeling_llama_polar.py:18) but does not ship.
The polar classes call it on values with one group per token and 4 bits (:242, :285); that case runs on this
package's CUDA library, anything else raises."""
from polarquant_b200 import ops as _ops


def triton_quantize_and_pack_along_last_dim(data, group_size, bit):
    """data (B, Nk, T, 128) -> (codes (B, Nk, T, 16) int32, scale (B, Nk, T, 1), mn (B, Nk, T, 1))."""
    if data.dim() != 4 or data.shape[-1] != group_size or group_size != 128 or bit != 4:
        raise NotImplementedError("only the value-cache packing of the polar classes is provided: one group of 128 "
                                  "channels per token, 4 bits (KIVI itself is a third-party package the reference "
                                  "does not vendor)")
    return _ops.quantize_values(data, bit, layout="kivi")
