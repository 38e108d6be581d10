"""Router front end: BatchNorm1d(affine=False) -> router_gate Linear -> per-half log-softmax
(flash_moe/modules/flash_moe.py:65-72) as one library call."""

from __future__ import annotations

import torch

from .. import _lib
from .utils import contiguous


def router_front(x2d, router_weight, running_mean, running_var, training=False, momentum=0.1, eps=1e-5):
    """Returns (logits[T, 2nk], log_probs[2, T, nk]) in x2d.dtype; updates the running buffers when training."""
    dev = _lib.require_cuda(x2d, router_weight, running_mean, running_var)
    x2d, w = contiguous(x2d), contiguous(router_weight)
    T, H = x2d.shape
    nk = w.shape[0] // 2
    if w.shape != (2 * nk, H) or w.dtype != x2d.dtype:
        raise _lib.FmoeError("router_weight must be [2*num_keys, H] in the dtype of x")
    for b in (running_mean, running_var):
        if b is not None and (b.dtype != x2d.dtype or b.shape != (H,) or not b.is_contiguous()):
            raise _lib.FmoeError("running buffers must be contiguous [H] tensors in the dtype of x")
    logits = torch.empty((T, 2 * nk), device=dev, dtype=x2d.dtype)
    logp = torch.empty((2, T, nk), device=dev, dtype=x2d.dtype)
    L = _lib.lib()
    code = _lib.dtype_code(x2d)
    ws_bytes = L.fmoe_router_front_workspace_bytes(T, H, nk, code)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = L.fmoe_router_front(
            x2d.data_ptr(), w.data_ptr(), _lib.ptr(running_mean), _lib.ptr(running_var), int(bool(training)),
            float(momentum), float(eps), logits.data_ptr(), logp.data_ptr(), code, T, H, nk, ws.data_ptr(), ws_bytes,
            _lib.status_word(dev).data_ptr(), _lib.current_stream_ptr(dev),
        )
    _lib.check(rc, "fmoe_router_front")
    return logits, logp
