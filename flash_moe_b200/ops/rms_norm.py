"""RMS pre-norm for a decoder block built around the FlashMoE layer (the reference leaves it to its caller)."""

from __future__ import annotations

from typing import Optional

import torch

from .. import _lib
from .utils import contiguous


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor] = None, eps: float = 1e-6) -> torch.Tensor:
    """``x * rsqrt(mean(x^2, -1) + eps) * weight`` over the last dimension, float32 inside, one rounding."""
    dev = _lib.require_cuda(x, weight)
    xc = contiguous(x)
    H = xc.shape[-1]
    if weight is not None and (weight.shape != (H,) or weight.dtype != xc.dtype):
        raise _lib.FmoeError("weight must be a [hidden] tensor in the dtype of x")
    w = None if weight is None else contiguous(weight)
    out = torch.empty_like(xc)
    rows = xc.numel() // H if H else 0
    with torch.cuda.device(dev):
        rc = _lib.lib().fmoe_rms_norm(xc.data_ptr(), _lib.ptr(w), out.data_ptr(), _lib.dtype_code(xc), rows, H, float(eps),
                                      _lib.current_stream_ptr(dev))
    _lib.check(rc, "fmoe_rms_norm")
    return out
