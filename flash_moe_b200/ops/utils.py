"""Small host-side helpers shared by the ops (counterpart of flash_moe/ops/utils.py)."""

from __future__ import annotations

import torch

FORWARD_ONLY_MSG = (
    "flash_moe_b200 implements the forward pass only; call it under torch.no_grad() "
    "or detach the outputs (the reference's backward kernels have no counterpart here)"
)


def contiguous(t):
    """The reference makes every tensor argument contiguous before a kernel sees it (ops/utils.py:35-45)."""
    return t.contiguous() if isinstance(t, torch.Tensor) else t


class ForwardOnly(torch.autograd.Function):
    """Base class: forward works in any grad mode, backward fails loudly."""

    @staticmethod
    def backward(ctx, *grads):
        raise NotImplementedError(FORWARD_ONLY_MSG)
