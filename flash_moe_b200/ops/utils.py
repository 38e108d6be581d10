"""Small host-side helpers shared by the ops (counterpart of flash_moe/ops/utils.py)."""

from __future__ import annotations

import torch


def contiguous(t):
    """The reference makes every tensor argument contiguous before a kernel sees it (ops/utils.py:35-45)."""
    return t.contiguous() if isinstance(t, torch.Tensor) else t
