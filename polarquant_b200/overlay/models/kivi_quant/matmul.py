"""The KIVI products the reference imports unconditionally (models/modeling_llama_polar.py:19,
benchmark/benchmark_matmul.py:9) but does not ship.  The one use the polar classes make of them - probabilities times
the 4-bit value cache, group 128 (models/modeling_llama_polar.py:230-237) - runs on this package's CUDA library; the
KIVI key-cache uses (other group sizes and bit widths) are not part of the polar path and raise."""
from polarquant_b200 import ops as _ops


def cuda_bmm_fA_qB_outer(group_size, fA, qB, scales, zeros, bits, mqa=False):
    """fA (B, H, M, T) x dequantised qB (B, H, T, 128 * bits / 32 int32) -> (B, H, M, 128)."""
    if group_size != 128 or bits != 4 or qB.shape[-1] != 16 or scales.shape[-1] != 1 or mqa:
        raise NotImplementedError("only the value-cache product of the polar classes is provided: group 128 along "
                                  "the channels, 4 bits (KIVI itself is a third-party package the reference does "
                                  "not vendor)")
    return _ops.values_matmul(fA, qB, scales, zeros, bits)


triton_bmm_fA_qB_outer = cuda_bmm_fA_qB_outer
