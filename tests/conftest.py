import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str) -> dict:
    """Read a fixture; uint16 arrays are bf16 bit patterns (numpy has no bf16)."""
    out = {}
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        for k in z.files:
            a = z[k]
            if a.dtype == np.uint16:
                out[k] = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
            elif k == "meta":
                out[k] = [int(x) for x in a]
            else:
                out[k] = torch.from_numpy(a.copy())
    return out


def golden_names(prefix: str, exclude: str | None = None):
    return sorted(f[:-4] for f in os.listdir(GOLDEN)
                  if f.startswith(prefix) and f.endswith(".npz") and not (exclude and f.startswith(exclude)))


# tolerance of attention outputs against the reference's dequantise-then-matmul path
ATTN_MAX_ABS = 2e-2
ATTN_MEAN_ABS = 2e-3


def out_ulp(want: torch.Tensor) -> torch.Tensor:
    """Spacing of the output dtype at each element of ``want`` (0 for fp32)."""
    if want.dtype == torch.float32:
        return torch.zeros_like(want)
    mant = 7 if want.dtype == torch.bfloat16 else 10
    mag = want.float().abs().clamp_min(1e-30)
    return torch.exp2(torch.floor(torch.log2(mag)) - mant)


def check_mixed(got: torch.Tensor, want: torch.Tensor, what: str = "") -> None:
    """Bar for the packed-value decode step against the reference's mixed forward.  That forward rounds to the
    output dtype three times (the packed part at models/modeling_llama_polar.py:237, the residual part and their
    sum at :239), so against an unrounded or once-rounded result its own rounding noise is about half a unit in
    the last place per element on average: the mean bound is 2e-3 plus half the mean spacing of the output dtype.
    The max bound is 2e-2 or two and a half spacings, whichever is larger: three half-spacings from the reference's
    roundings (whose intermediate parts can be larger than their sum), one more from the rounding of the result
    under test."""
    diff = (got.float() - want.float()).abs()
    assert torch.isfinite(got.float()).all(), what
    ulp = out_ulp(want)
    worst = float((diff - torch.clamp_min(2.5 * ulp, ATTN_MAX_ABS)).max())
    mean_bar = ATTN_MEAN_ABS + 0.5 * float(ulp.mean())
    assert worst <= 0 and float(diff.mean()) <= mean_bar, (what, float(diff.max()), float(diff.mean()), mean_bar)


def check_attn(got: torch.Tensor, want: torch.Tensor, what: str = "") -> None:
    """The attention bar (max 2e-2, mean 2e-3) with its one refinement: where one spacing of the output dtype
    exceeds 2e-2 a difference of one spacing is a rounding flip, not an error."""
    assert got.shape == want.shape, (got.shape, want.shape)
    diff = (got.float() - want.float()).abs()
    assert torch.isfinite(got.float()).all(), what
    allowed = torch.clamp_min(out_ulp(want), ATTN_MAX_ABS)
    worst = float((diff - allowed).max())
    assert worst <= 0 and float(diff.mean()) <= ATTN_MEAN_ABS, (what, float(diff.max()), float(diff.mean()))
