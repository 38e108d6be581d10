"""A residual stack of FlashMoE layers used as the MLP path of a decoder: x <- x + layer(x).

The reference ships the single layer only; this is the caller-side composition of the
multi-layer benchmark configuration (layer l seeded with torch.manual_seed(l)).  The skip connection is
handed to the layer (`residual=`), which adds it in the epilogue of its last GEMM: one kernel fewer per
layer and one rounding of `x + layer(x)` instead of two.  `GraphedFlashMoE(stack, x)` captures the
whole stack in one CUDA graph."""

from __future__ import annotations

from typing import List, Tuple

import torch
import torch.nn as nn

from .flash_moe import FlashMoE, FlashMoEConfig


class FlashMoEStack(nn.Module):
    def __init__(self, config: FlashMoEConfig, num_layers: int, seeds=None):
        super().__init__()
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
        for layer in self.layers:
            x, logits = layer(x, residual=x)
            all_logits.append(logits)
        return x, all_logits
