"""Fine-grained expert forward (drop-in for flash_moe/ops/triton/flash_expert.py:831-836)."""

from __future__ import annotations

import torch

from .. import _lib
from .utils import contiguous


def _expert_forward(hidden_states, down_weights, up_weights, indices, routing_weights, out_dtype=None, save_scores=False):
    dev = _lib.require_cuda(hidden_states, down_weights, up_weights, indices, routing_weights)
    x, d, u, idx, g = (contiguous(t) for t in (hidden_states, down_weights, up_weights, indices, routing_weights))
    if x.dim() != 2 or d.dim() != 2 or u.dim() != 2 or idx.dim() != 2:
        raise _lib.FmoeError("expected hidden_states[T,H], down/up_weights[N,H], indices[T,k]")
    T, H = x.shape
    N = d.shape[0]
    k = idx.shape[1]
    if d.shape != u.shape or d.shape[1] != H or idx.shape[0] != T or tuple(g.shape) != (T, k):
        raise _lib.FmoeError("shape mismatch between hidden_states, expert tables, indices and routing_weights")
    if not (d.dtype == u.dtype == x.dtype):
        raise _lib.FmoeError("hidden_states and the expert tables must share one dtype")
    if idx.dtype != torch.int64:
        idx = idx.to(torch.int64)
    if g.dtype != x.dtype:
        g = g.to(x.dtype)
    out_dtype = x.dtype if out_dtype is None else out_dtype
    out = torch.empty((T, H), device=dev, dtype=out_dtype)
    L = _lib.lib()
    ws_bytes = L.fmoe_expert_workspace_bytes(T, H, N, k)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
    saved = torch.empty((T, k), device=dev, dtype=torch.float32) if save_scores else None
    with torch.cuda.device(dev):
        if save_scores:
            rc = L.fmoe_expert_forward_saving_scores(
                x.data_ptr(), d.data_ptr(), u.data_ptr(), idx.data_ptr(), g.data_ptr(), out.data_ptr(), saved.data_ptr(),
                _lib.dtype_code(x), _lib.DTYPE_CODE[out_dtype], T, H, N, k, ws.data_ptr(), ws_bytes,
                _lib.status_word(dev).data_ptr(), _lib.current_stream_ptr(dev),
            )
        else:
            rc = L.fmoe_expert_forward(
                x.data_ptr(), d.data_ptr(), u.data_ptr(), idx.data_ptr(), g.data_ptr(), out.data_ptr(),
                _lib.dtype_code(x), _lib.DTYPE_CODE[out_dtype], T, H, N, k, ws.data_ptr(), ws_bytes,
                _lib.status_word(dev).data_ptr(), _lib.current_stream_ptr(dev),
            )
    _lib.check(rc, "fmoe_expert_forward")
    return (out, saved) if save_scores else out


def _expert_backward(dout, hidden_states, down_weights, up_weights, indices, routing_weights, saved_scores=None):
    """(dx, ddown, dup, dgates) of the expert sum (flash_moe/ops/triton/flash_expert.py:653-745)."""
    dev = _lib.require_cuda(dout, hidden_states, down_weights, up_weights, indices, routing_weights)
    do, x, d, u, idx, g = (contiguous(t) for t in (dout, hidden_states, down_weights, up_weights, indices, routing_weights))
    T, H = x.shape
    N, k = d.shape[0], idx.shape[1]
    if do.dtype != x.dtype:
        do = do.to(x.dtype)
    if idx.dtype != torch.int64:
        idx = idx.to(torch.int64)
    if g.dtype != x.dtype:
        g = g.to(x.dtype)
    dx, dd, du, dg = torch.empty_like(x), torch.empty_like(d), torch.empty_like(u), torch.empty_like(g)
    L = _lib.lib()
    ws_bytes = L.fmoe_expert_backward_workspace_bytes(T, H, N, k)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = L.fmoe_expert_backward(
            do.data_ptr(), x.data_ptr(), d.data_ptr(), u.data_ptr(), idx.data_ptr(), g.data_ptr(),
            _lib.ptr(saved_scores), dx.data_ptr(),
            dd.data_ptr(), du.data_ptr(), dg.data_ptr(), _lib.dtype_code(x), T, H, N, k, ws.data_ptr(), ws_bytes,
            _lib.status_word(dev).data_ptr(), _lib.current_stream_ptr(dev),
        )
    _lib.check(rc, "fmoe_expert_backward")
    return dx, dd, du, dg


class FlashExpertFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden_states, down_weights, up_weights, indices, routing_weights):
        if not any(ctx.needs_input_grad):
            return _expert_forward(hidden_states, down_weights, up_weights, indices, routing_weights)
        # like the reference (flash_expert.py:784-794) keep the pre-activation scores for the backward
        out, scores = _expert_forward(hidden_states, down_weights, up_weights, indices, routing_weights, save_scores=True)
        ctx.save_for_backward(hidden_states, down_weights, up_weights, indices, routing_weights, scores)
        return out

    @staticmethod
    def backward(ctx, dexperts_states):
        x, d, u, idx, g, scores = ctx.saved_tensors
        dx, dd, du, dg = _expert_backward(dexperts_states, x, d, u, idx, g, scores)
        return dx, dd, du, None, dg.to(g.dtype)


def flash_expert_func(hidden_states, down_weights, up_weights, indices, routing_weights):
    """experts_states[T,H] = sum_j silu(<x, down[idx_j]>) * routing_weights_j * up[idx_j], in hidden_states.dtype."""
    return FlashExpertFunc.apply(hidden_states, down_weights, up_weights, indices, routing_weights)


def flash_expert_fp32(hidden_states, down_weights, up_weights, indices, routing_weights):
    """Same sum returned as the unrounded float32 accumulator."""
    return _expert_forward(hidden_states, down_weights, up_weights, indices, routing_weights, torch.float32)


def combine_partial_rows(rows, slot, num_tokens):
    """out[t] = sum_g rows[slot[g, t]] (slot < 0 skipped), float32; the combine step of the expert-sharded layout.

    rows [R, H] float32 (partial sums received from the ranks that own the experts), slot [G, num_tokens] int32.
    """
    dev = _lib.require_cuda(rows, slot)
    rows, slot = contiguous(rows), contiguous(slot)
    if rows.dtype != torch.float32 or slot.dtype != torch.int32 or rows.dim() != 2 or slot.dim() != 2:
        raise _lib.FmoeError("expected rows[R,H] float32 and slot[G,T] int32")
    if slot.shape[1] != num_tokens:
        raise _lib.FmoeError("slot must have one column per token")
    out = torch.empty((num_tokens, rows.shape[1]), device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        rc = _lib.lib().fmoe_combine_partial_rows(
            rows.data_ptr(), rows.shape[0], slot.data_ptr(), slot.shape[0], num_tokens, rows.shape[1], out.data_ptr(),
            _lib.status_word(dev).data_ptr(), _lib.current_stream_ptr(dev))
    _lib.check(rc, "fmoe_combine_partial_rows")
    return out


triton_flash_expert_func = flash_expert_func
