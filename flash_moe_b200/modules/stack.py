"""A residual stack of FlashMoE layers used as the MLP path of a decoder: x <- x + layer(x).

The reference ships the single layer only; this is the caller-side composition of the
multi-layer benchmark configuration (layer l seeded with torch.manual_seed(l)).  The skip connection is
handed to the layer (`residual=`), which adds it in the epilogue of its last GEMM: one kernel fewer per
layer and one rounding of `x + layer(x)` instead of two.  With `pre_norm=True` each layer sees
`rms_norm(x)` (a learnable weight per layer) while the skip connection carries the un-normalised x - the
usual pre-norm decoder block.  `GraphedFlashMoE(stack, x)` captures the whole stack in one CUDA graph."""

from __future__ import annotations

from typing import List, Tuple

import torch
import torch.nn as nn

from .flash_moe import FlashMoE, FlashMoEConfig


class FlashMoEStack(nn.Module):
    def __init__(self, config: FlashMoEConfig, num_layers: int, seeds=None, pre_norm: bool = False, norm_eps: float = 1e-6):
        super().__init__()
        self.norm_eps = norm_eps
        self.norms = (nn.ParameterList([nn.Parameter(torch.ones(config.hidden_size)) for _ in range(num_layers)])
                      if pre_norm else None)
        layers = []
        for i in range(num_layers):
            if seeds is not None:
                torch.manual_seed(seeds[i])
            layers.append(FlashMoE(config))
        self.layers = nn.ModuleList(layers)
        # the layers run one after another on one stream, so they can share one scratch allocation
        for layer in layers[1:]:
            layer._workspaces = layers[0]._workspaces

    def forward(self, hidden_states: torch.Tensor) -> Tuple[torch.Tensor, List[torch.Tensor]]:
        """Returns the final hidden states and every layer's router logits."""
        all_logits = []
        x = hidden_states
        for i, layer in enumerate(self.layers):
            if self.norms is not None:
                if torch.is_grad_enabled() and (x.requires_grad or self.norms[i].requires_grad):
                    xn = torch.nn.functional.rms_norm(x, (x.shape[-1],), self.norms[i], self.norm_eps)
                else:
                    from ..ops.rms_norm import rms_norm

                    xn = rms_norm(x, self.norms[i].detach(), self.norm_eps)
                x, logits = layer(xn, residual=x)
            else:
                x, logits = layer(x, residual=x)
            all_logits.append(logits)
        return x, all_logits
