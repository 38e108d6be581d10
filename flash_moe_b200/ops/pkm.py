"""Product-key-memory value lookup (drop-in for flash_moe/ops/triton/pkm.py:195-200)."""

from __future__ import annotations

import torch

from .. import _lib
from .utils import contiguous


class PKMFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, values, routing_weights, indices):
        dev = _lib.require_cuda(values, routing_weights, indices)
        v, w, idx = (contiguous(t) for t in (values, routing_weights, indices))
        if v.dim() != 2 or idx.dim() != 2 or idx.shape != w.shape:
            raise _lib.FmoeError("expected values[N,H], routing_weights/indices[T,k]")
        N, H = v.shape
        T, k = idx.shape
        idx = idx.to(torch.int64)
        w = w.to(v.dtype)
        out = torch.empty((T, H), device=dev, dtype=v.dtype)
        L = _lib.lib()
        ws_bytes = L.fmoe_pkm_workspace_bytes(T, k)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            rc = L.fmoe_pkm_forward(v.data_ptr(), w.data_ptr(), idx.data_ptr(), out.data_ptr(), _lib.dtype_code(v), T, H, N,
                                    k, ws.data_ptr(), ws_bytes, _lib.status_word(dev).data_ptr(),
                                    _lib.current_stream_ptr(dev))
        _lib.check(rc, "fmoe_pkm_forward")
        return out

    @staticmethod
    def backward(ctx, grad_output):
        # as in the reference (flash_moe/ops/triton/pkm.py:190-192)
        raise NotImplementedError("PKMFunc backward is not implemented.")


def pkm_func(values, routing_weights, indices):
    """out[t] = sum_j routing_weights[t,j] * values[indices[t,j]]."""
    return PKMFunc.apply(values, routing_weights, indices)


triton_pkm_func = pkm_func
