"""Product-key router top-k (drop-in for flash_moe/ops/triton/flash_router.py:381-382)."""

from __future__ import annotations

import torch

from .. import _lib
from .utils import contiguous


def _router_forward(router_logits: torch.Tensor, num_expert_keys: int, num_experts_per_tok: int, want_gates=False,
                    norm_topk_prob=False):
    # same argument checks and messages as flash_router.py:257-263
    assert router_logits.dim() == 3, (
        "router_logits must be a 3D tensor of shape (2, batch_size * seq_len, num_expert_keys)"
    )
    assert router_logits.size(0) == 2, "The first dimension of router_logits must be 2"
    assert 0 <= num_experts_per_tok <= num_expert_keys, (
        f"num_experts_per_tok should be in [0, {num_expert_keys}], but got {num_experts_per_tok}"
    )
    dev = _lib.require_cuda(router_logits)
    lp = contiguous(router_logits)
    if lp.size(2) != num_expert_keys:
        lp = lp[:, :, :num_expert_keys].contiguous()
    T = lp.size(1)
    scores = torch.empty((T, num_experts_per_tok), device=dev, dtype=lp.dtype)
    indices = torch.empty((T, num_experts_per_tok), device=dev, dtype=torch.int64)
    gates = torch.empty_like(scores) if want_gates else None
    with torch.cuda.device(dev):
        rc = _lib.lib().fmoe_router_topk(
            lp.data_ptr(), _lib.dtype_code(lp), T, num_expert_keys, num_experts_per_tok, scores.data_ptr(),
            indices.data_ptr(), _lib.ptr(gates), int(bool(norm_topk_prob)), _lib.current_stream_ptr(dev),
        )
    _lib.check(rc, "fmoe_router_topk")
    return (scores, indices, gates) if want_gates else (scores, indices)


def _router_backward(dscores, indices, num_expert_keys):
    """dlog_probs[2,T,nk] of the selected sums (flash_moe/ops/triton/flash_router.py:316-345)."""
    dev = _lib.require_cuda(dscores, indices)
    ds, idx = contiguous(dscores), contiguous(indices)
    T, k = ds.shape
    out = torch.empty((2, T, num_expert_keys), device=dev, dtype=ds.dtype)
    with torch.cuda.device(dev):
        rc = _lib.lib().fmoe_router_topk_backward(ds.data_ptr(), idx.data_ptr(), _lib.dtype_code(ds), T, num_expert_keys, k,
                                                  out.data_ptr(), _lib.current_stream_ptr(dev))
    _lib.check(rc, "fmoe_router_topk_backward")
    return out


class FlashRouterFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, router_logits, num_expert_keys, num_experts_per_tok):
        scores, indices = _router_forward(router_logits, num_expert_keys, num_experts_per_tok)
        ctx.mark_non_differentiable(indices)
        ctx.save_for_backward(indices)
        ctx.num_expert_keys = num_expert_keys
        ctx.in_keys = router_logits.size(2)
        return scores, indices

    @staticmethod
    def backward(ctx, dscores, dindices):
        (indices,) = ctx.saved_tensors
        d = _router_backward(dscores, indices, ctx.num_expert_keys)
        if ctx.in_keys != ctx.num_expert_keys:  # the forward read only the first num_expert_keys columns
            d = torch.nn.functional.pad(d, (0, ctx.in_keys - ctx.num_expert_keys))
        return d, None, None


def flash_router_func(router_logits, num_expert_keys, num_experts_per_tok):
    """(scores[T,k] in the input dtype, indices[T,k] int64) for log-probs ``router_logits[2,T,nk]``."""
    return FlashRouterFunc.apply(router_logits, num_expert_keys, num_experts_per_tok)


def flash_router_with_gates(router_logits, num_expert_keys, num_experts_per_tok, norm_topk_prob=False):
    """Same, plus gates = exp(scores) (renormalised per token when asked) from the same kernel."""
    return _router_forward(router_logits, num_expert_keys, num_experts_per_tok, True, norm_topk_prob)


# name the reference module exports (flash_moe/ops/triton/flash_router.py:381)
triton_flash_router_func = flash_router_func
