"""PEER retrieval baseline (drop-in for flash_moe/ops/triton/peer.py:246-255): the expert sum with an exact GELU."""

from __future__ import annotations

import torch

from .. import _lib
from .utils import contiguous


class PEERFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden_states, down_embed, up_embed, routing_weights, indices):
        dev = _lib.require_cuda(hidden_states, down_embed, up_embed, routing_weights, indices)
        x, d, u, w, idx = (contiguous(t) for t in (hidden_states, down_embed, up_embed, routing_weights, indices))
        if x.dim() != 2 or d.dim() != 2 or d.shape != u.shape or d.shape[1] != x.shape[1] or idx.shape != w.shape:
            raise _lib.FmoeError("expected hidden_states[T,H], down/up_embed[N,H], routing_weights/indices[T,k]")
        if not (d.dtype == u.dtype == x.dtype):
            raise _lib.FmoeError("hidden_states and the embeddings must share one dtype")
        T, H = x.shape
        N, k = d.shape[0], idx.shape[1]
        idx = idx.to(torch.int64)
        w = w.to(x.dtype)
        out = torch.empty_like(x)
        L = _lib.lib()
        ws_bytes = L.fmoe_expert_workspace_bytes(T, H, N, k)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            rc = L.fmoe_peer_forward(x.data_ptr(), d.data_ptr(), u.data_ptr(), w.data_ptr(), idx.data_ptr(), out.data_ptr(),
                                     _lib.dtype_code(x), T, H, N, k, ws.data_ptr(), ws_bytes,
                                     _lib.status_word(dev).data_ptr(), _lib.current_stream_ptr(dev))
        _lib.check(rc, "fmoe_peer_forward")
        return out

    @staticmethod
    def backward(ctx, grad_output):
        # as in the reference (flash_moe/ops/triton/peer.py:241-243)
        raise NotImplementedError("PEERFunc backward is not implemented.")


def peer_func(hidden_states, down_embed, up_embed, routing_weights, indices):
    """out[t] = sum_j gelu(<x[t], down_embed[idx]>) * routing_weights[t,j] * up_embed[idx]."""
    return PEERFunc.apply(hidden_states, down_embed, up_embed, routing_weights, indices)


triton_peer_func = peer_func
