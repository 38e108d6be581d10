"""Shared SwiGLU MLP (drop-in for flash_moe/ops/triton/flash_mlp.py:169-181)."""

from __future__ import annotations

import torch

from .. import _lib
from .utils import contiguous


def _mlp_forward(x, gate_weight, up_weight, down_weight, addend=None, save_preacts=False):
    dev = _lib.require_cuda(x, gate_weight, up_weight, down_weight, addend)
    lead = x.shape[:-1]
    H = x.shape[-1]
    x2, wg, wu, wd = (contiguous(t) for t in (x.reshape(-1, H), gate_weight, up_weight, down_weight))
    T = x2.shape[0]
    I = wg.shape[0]
    if wg.shape != (I, H) or wu.shape != (I, H) or wd.shape != (H, I):
        raise _lib.FmoeError("expected gate/up_weight[I,H] and down_weight[H,I]")
    if not (wg.dtype == wu.dtype == wd.dtype == x2.dtype):
        raise _lib.FmoeError("x and the MLP weights must share one dtype")
    if addend is not None:
        addend = contiguous(addend.reshape(-1, H))
        if addend.dtype != torch.float32 or addend.shape != (T, H):
            raise _lib.FmoeError("addend must be float32 [T,H]")
    out = torch.empty((T, H), device=dev, dtype=x2.dtype)
    L = _lib.lib()
    code = _lib.dtype_code(x2)
    ws_bytes = L.fmoe_mlp_workspace_bytes(T, H, I, code)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
    if save_preacts and addend is None and T > 0:
        # the fused gate/up GEMM can also store the two pre-activations (its CTA-pair form only)
        a = torch.empty((T, I), device=dev, dtype=x2.dtype)
        b = torch.empty((T, I), device=dev, dtype=x2.dtype)
        with torch.cuda.device(dev):
            rc = L.fmoe_mlp_forward_saving_preacts(
                x2.data_ptr(), wg.data_ptr(), wu.data_ptr(), wd.data_ptr(), out.data_ptr(), a.data_ptr(), b.data_ptr(), code,
                T, H, I, ws.data_ptr(), ws_bytes, _lib.status_word(dev).data_ptr(), _lib.current_stream_ptr(dev),
            )
        if rc == 0:
            return out.view(*lead, H), a, b
        if rc != _lib.ERR_UNSUPPORTED:
            _lib.check(rc, "fmoe_mlp_forward_saving_preacts")
    with torch.cuda.device(dev):
        rc = L.fmoe_mlp_forward(
            x2.data_ptr(), wg.data_ptr(), wu.data_ptr(), wd.data_ptr(), _lib.ptr(addend), out.data_ptr(), code, T, H, I,
            ws.data_ptr(), ws_bytes, _lib.status_word(dev).data_ptr(), _lib.current_stream_ptr(dev),
        )
    _lib.check(rc, "fmoe_mlp_forward")
    return (out.view(*lead, H), None, None) if save_preacts else out.view(*lead, H)


def swiglu_backward(dh, a, b, want_h=False):
    """(da, db[, h]) for h = silu(a) * b (flash_moe/ops/triton/flash_mlp.py:52-102,:125-147)."""
    dev = _lib.require_cuda(dh, a, b)
    dh, a, b = (contiguous(t) for t in (dh, a, b))
    if not (dh.shape == a.shape == b.shape and dh.dtype == a.dtype == b.dtype):
        raise _lib.FmoeError("dh, a and b must share shape and dtype")
    da, db = torch.empty_like(a), torch.empty_like(b)
    h = torch.empty_like(a) if want_h else None
    with torch.cuda.device(dev):
        rc = _lib.lib().fmoe_swiglu_backward(dh.data_ptr(), a.data_ptr(), b.data_ptr(), da.data_ptr(), db.data_ptr(),
                                             _lib.ptr(h), _lib.dtype_code(a), a.numel(), _lib.current_stream_ptr(dev))
    _lib.check(rc, "fmoe_swiglu_backward")
    return (da, db, h) if want_h else (da, db)


class FlashMLPFunc(torch.autograd.Function):
    """Forward: the fused kernels.  Backward: like the reference (flash_mlp.py:150-181) the contractions are plain
    library GEMMs (torch.matmul) and the SwiGLU derivative is this library's kernel.  The two pre-activations are
    kept by the forward when the fused GEMM can store them (as the reference's TritonSwiGLUFunc does) and
    recomputed otherwise."""

    @staticmethod
    def forward(ctx, x, gate_weight, up_weight, down_weight):
        if not any(ctx.needs_input_grad):
            return _mlp_forward(x, gate_weight, up_weight, down_weight)
        out, a, b = _mlp_forward(x, gate_weight, up_weight, down_weight, save_preacts=True)
        ctx.have_preacts = a is not None
        if ctx.have_preacts:
            ctx.save_for_backward(x, gate_weight, up_weight, down_weight, a, b)
        else:
            ctx.save_for_backward(x, gate_weight, up_weight, down_weight)
        return out

    @staticmethod
    def backward(ctx, dy):
        if ctx.have_preacts:
            x, wg, wu, wd, a, b = ctx.saved_tensors
        else:
            x, wg, wu, wd = ctx.saved_tensors
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        dy2 = dy.reshape(-1, H).to(x2.dtype)
        if not ctx.have_preacts:
            a = torch.matmul(x2, wg.t())
            b = torch.matmul(x2, wu.t())
        dh = torch.matmul(dy2, wd)
        da, db, h = swiglu_backward(dh, a, b, want_h=True)
        dwd = torch.matmul(dy2.t(), h)
        dwg = torch.matmul(da.t(), x2)
        dwu = torch.matmul(db.t(), x2)
        dx = torch.addmm(torch.matmul(da, wg), db, wu)
        return dx.reshape(x.shape), dwg, dwu, dwd


def flash_mlp_func(x, gate_weight, up_weight, down_weight):
    """(silu(x Wg^T) * (x Wu^T)) Wd^T with the activation fused into the first GEMM's epilogue."""
    return FlashMLPFunc.apply(x, gate_weight, up_weight, down_weight)


def flash_mlp_add(x, gate_weight, up_weight, down_weight, addend_fp32):
    """Same with a float32 [T,H] addend summed into the accumulator before the single rounding."""
    return _mlp_forward(x, gate_weight, up_weight, down_weight, addend_fp32)


triton_flash_mlp_func = flash_mlp_func
