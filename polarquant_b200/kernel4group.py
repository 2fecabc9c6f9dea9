"""Drop-in for the reference module ``models/kernel4group.py``.

Keeps the reference's entry-point name and signature
(``attention_decode_forward_triton_impl``, models/kernel4group.py:83-92) so the
reference's attention patches and its QK micro-benchmark bind to the CUDA
library without modification.  The name mentions Triton only because callers
import it by that name; nothing here uses Triton.
"""
from __future__ import annotations

import torch

from .ops import qk_decode


def attention_decode_forward_triton_impl(
    query_states: torch.Tensor,   # (b, n, 1, 2 * d)
    indices: torch.Tensor,        # (b, nk, nb, g, d) uint8
    rscale: torch.Tensor,         # (b, nk, nb, 1, d)
    rmn: torch.Tensor,
    tscale: torch.Tensor,
    tmn: torch.Tensor,
    rbits: int = 4,
    tbits: int = 4,
) -> torch.Tensor:
    """fp32 logits (b, n, 1, nb * g), un-scaled, on the query's device and current stream."""
    return qk_decode(query_states, indices, rscale, rmn, tscale, tmn, rbits=rbits, tbits=tbits)


__all__ = ["attention_decode_forward_triton_impl"]
