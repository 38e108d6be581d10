"""CPU restatement of the FlashMoE forward path (router -> fine-grained experts -> shared SwiGLU MLP).

TEST INFRASTRUCTURE ONLY: used by the tests, the smoke check and the CPU-baseline
legs of the benchmark.  The product package never imports it.

Parity pin: the functions below are checked against the reference's own code
(its eager ``FlashMoE_Pytorch`` module and its Triton router run under the Triton
CPU interpreter) by ``tests/golden/make_golden.py``; the outputs of those runs are
committed under ``tests/golden/`` and re-checked by ``tests/test_oracle_golden.py``.

Every function cites the reference lines it restates (paths are relative to the
reference project root).  Dense GEMMs, batch-norm, log-softmax, exp and SiLU are
torch's own CPU kernels, exactly the third-party arithmetic the reference calls.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

BN_EPS = 1e-5  # nn.BatchNorm1d default, flash_moe/modules/flash_moe.py:49
BN_MOMENTUM = 0.1


# --------------------------------------------------------------------------------------
# Router
# --------------------------------------------------------------------------------------
def router_front(
    x2d: torch.Tensor,
    router_weight: torch.Tensor,
    running_mean: Optional[torch.Tensor],
    running_var: Optional[torch.Tensor],
    training: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """BatchNorm1d(affine=False) -> Linear(H, 2*nk) -> per-half log-softmax.

    Restates flash_moe/modules/flash_moe.py:65-72.  Returns ``(logits[T, 2nk],
    log_probs[2, T, nk])`` in the dtype of ``x2d``; half ``h`` of the logits is
    columns ``h*nk .. (h+1)*nk``.  In training mode the running statistics are
    updated in place like ``nn.BatchNorm1d`` does.
    """
    T = x2d.shape[0]
    nk = router_weight.shape[0] // 2
    xn = F.batch_norm(x2d, running_mean, running_var, None, None, training, BN_MOMENTUM, BN_EPS)
    logits = F.linear(xn, router_weight)
    halves = logits.view(T, 2, nk).transpose(0, 1)
    return logits, F.log_softmax(halves, dim=-1).contiguous()


def router_topk(log_probs: torch.Tensor, num_keys: int, top_k: int, chunk: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Exact top-k over the Cartesian sums ``lp[0,t,i] + lp[1,t,j]`` with flat id ``i*nk + j``.

    Restates the result of the reference router kernels
    (flash_moe/ops/triton/flash_router.py:8-63 and :66-194): the pair sum is
    formed in the *input dtype* (:51-53), the k winners are emitted by repeated
    arg-max, i.e. in descending score order with ties going to the lowest flat
    index (``tl.argmax`` breaks ties to the left).  A stable descending sort of
    the flattened sums gives the same sequence.  ``indices`` are int64 (:270-275).
    """
    assert log_probs.dim() == 3 and log_probs.size(0) == 2  # flash_router.py:257-260
    assert 0 <= top_k <= num_keys  # flash_router.py:261-263
    T = log_probs.size(1)
    nk = num_keys
    if chunk <= 0:
        chunk = max(1, (1 << 24) // max(1, nk * nk))
    scores = torch.empty(T, top_k, dtype=log_probs.dtype)
    indices = torch.empty(T, top_k, dtype=torch.int64)
    for t0 in range(0, T, chunk):
        a = log_probs[0, t0 : t0 + chunk, :nk]
        b = log_probs[1, t0 : t0 + chunk, :nk]
        s = (a.unsqueeze(-1) + b.unsqueeze(-2)).reshape(a.shape[0], nk * nk)
        order = torch.sort(s.float(), dim=-1, descending=True, stable=True).indices[:, :top_k]
        scores[t0 : t0 + chunk] = s.gather(-1, order)
        indices[t0 : t0 + chunk] = order
    return scores, indices


def router_all_scores(log_probs: torch.Tensor, num_keys: int, t0: int, t1: int) -> torch.Tensor:
    """Reference score (input-dtype pair sum, as float32) of every candidate for tokens t0..t1."""
    a = log_probs[0, t0:t1, :num_keys]
    b = log_probs[1, t0:t1, :num_keys]
    return (a.unsqueeze(-1) + b.unsqueeze(-2)).reshape(a.shape[0], -1).float()


def routing_weights(scores: torch.Tensor, norm_topk_prob: bool) -> torch.Tensor:
    """exp(score) in the score dtype, optional renormalisation (flash_moe/modules/flash_moe.py:80-85)."""
    g = torch.exp(scores)
    if norm_topk_prob:
        g = g / g.sum(dim=-1, keepdim=True)
    return g


# --------------------------------------------------------------------------------------
# Experts and shared MLP
# --------------------------------------------------------------------------------------
def expert_forward(
    x2d: torch.Tensor,
    down_table: torch.Tensor,
    up_table: torch.Tensor,
    indices: torch.Tensor,
    gates: torch.Tensor,
    compute_dtype: torch.dtype = torch.float32,
    chunk: int = 256,
) -> torch.Tensor:
    """``out[t] = sum_j silu(<x[t], D[idx[t,j]]>) * g[t,j] * U[idx[t,j]]``.

    Restates the arithmetic of flash_moe/ops/triton/flash_expert.py:13-211
    (scores kernel + states kernel; duplicates of an expert id inside a token
    accumulate) and of the eager path flash_moe/modules/flash_moe.py:178-186.
    Evaluated in ``compute_dtype`` (float32 by default) on the given, possibly
    bf16-rounded, operands; the result is returned in ``compute_dtype``.
    """
    T, H = x2d.shape
    out = torch.empty(T, H, dtype=compute_dtype)
    for t0 in range(0, T, chunk):
        ids = indices[t0 : t0 + chunk]
        xs = x2d[t0 : t0 + chunk].to(compute_dtype)
        d = down_table[ids].to(compute_dtype)  # (t, k, H)
        s = torch.einsum("tkh,th->tk", d, xs)
        gs = F.silu(s) * gates[t0 : t0 + chunk].to(compute_dtype)
        u = up_table[ids].to(compute_dtype)
        out[t0 : t0 + chunk] = torch.einsum("tk,tkh->th", gs, u)
    return out


def expert_forward_eager(x2d, down_table, up_table, indices, gates) -> torch.Tensor:
    """The reference eager formulation in the operands' own dtype (flash_moe/modules/flash_moe.py:178-186)."""
    T = x2d.shape[0]
    d = down_table[indices]
    u = up_table[indices]
    w = torch.matmul(d, x2d.view(T, -1, 1)).view(T, -1)
    w = F.silu(w) * gates
    return torch.matmul(w.view(T, 1, -1), u).view(T, -1)


def mlp_forward(x2d, gate_w, up_w, down_w, compute_dtype: torch.dtype = torch.float32, round_h_to=None) -> torch.Tensor:
    """``(silu(x Wg^T) * (x Wu^T)) Wd^T`` (flash_moe/ops/triton/flash_mlp.py:169-181) evaluated in compute_dtype.

    ``round_h_to``: round the intermediate ``h = silu(.) * (.)`` once to that dtype before the down
    projection, as every implementation that stores h in 16 bits between the two GEMMs does (the
    reference stores it in the module dtype, flash_mlp.py:46-48,:119).
    """
    xs = x2d.to(compute_dtype)
    h = F.silu(xs @ gate_w.to(compute_dtype).t()) * (xs @ up_w.to(compute_dtype).t())
    if round_h_to is not None:
        h = h.to(round_h_to).to(compute_dtype)
    return h @ down_w.to(compute_dtype).t()


def mlp_forward_eager(x2d, gate_w, up_w, down_w) -> torch.Tensor:
    """Same formula in the operands' dtype (flash_moe/modules/flash_moe.py:187-189)."""
    return F.linear(F.silu(F.linear(x2d, gate_w)) * F.linear(x2d, up_w), down_w)


def peer_forward(x2d, down_table, up_table, weights, indices) -> torch.Tensor:
    """PEER baseline: ``sum_j gelu(<x, D[idx]>) * w * U[idx]`` with the exact (erf) GELU, float32
    (flash_moe/ops/triton/peer.py:23-148; eager statement tests/test_peer.py:9-24)."""
    d, u = down_table[indices].float(), up_table[indices].float()
    s = torch.einsum("tkh,th->tk", d, x2d.float())
    return torch.einsum("tk,tkh->th", F.gelu(s) * weights.float(), u)


def pkm_forward(values, weights, indices) -> torch.Tensor:
    """PKM baseline: ``sum_j w[t,j] * values[idx[t,j]]`` in float32 (flash_moe/ops/triton/pkm.py:25-120)."""
    return torch.einsum("tk,tkh->th", weights.float(), values[indices].float())


# --------------------------------------------------------------------------------------
# Backward of the three ops (float32 restatements)
# --------------------------------------------------------------------------------------
def router_backward(dscores: torch.Tensor, indices: torch.Tensor, num_keys: int) -> torch.Tensor:
    """``dlog_probs[2,T,nk]``: every selected pair (i, j) passes its score gradient to sub-key i of half 0 and
    sub-key j of half 1 (flash_moe/ops/triton/flash_router.py:197-249,:316-345).  float32 sums."""
    T = dscores.shape[0]
    d = torch.zeros(2, T, num_keys, dtype=torch.float32)
    ds = dscores.float()
    d[0].scatter_add_(1, indices // num_keys, ds)
    d[1].scatter_add_(1, indices % num_keys, ds)
    return d


def expert_backward(dout, x2d, down_table, up_table, indices, gates, chunk: int = 256):
    """``(dx, ddown, dup, dgates)`` of `expert_forward` in float32.

    Restates flash_moe/ops/triton/flash_expert.py:214-525 (host side :653-745): with s = <x, D[e]>,
    q = <dout, U[e]>: dgate = q*silu(s), ds = q*gate*silu'(s), dx = sum ds*D[e], dD[e] += ds*x, dU[e] += silu(s)*gate*dout.
    """
    T, H = x2d.shape
    N = down_table.shape[0]
    dx = torch.empty(T, H)
    dd = torch.zeros(N, H)
    du = torch.zeros(N, H)
    dg = torch.empty(indices.shape, dtype=torch.float32)
    for t0 in range(0, T, chunk):
        ids = indices[t0 : t0 + chunk]
        xs, do = x2d[t0 : t0 + chunk].float(), dout[t0 : t0 + chunk].float()
        d, u = down_table[ids].float(), up_table[ids].float()
        g = gates[t0 : t0 + chunk].float()
        s = torch.einsum("tkh,th->tk", d, xs)
        q = torch.einsum("tkh,th->tk", u, do)
        sig = torch.sigmoid(s)
        act = s * sig
        ds = q * g * sig * (1 + s * (1 - sig))
        dg[t0 : t0 + chunk] = q * act
        dx[t0 : t0 + chunk] = torch.einsum("tk,tkh->th", ds, d)
        dd.index_add_(0, ids.reshape(-1), (ds.unsqueeze(-1) * xs.unsqueeze(1)).reshape(-1, H))
        du.index_add_(0, ids.reshape(-1), ((act * g).unsqueeze(-1) * do.unsqueeze(1)).reshape(-1, H))
    return dx, dd, du, dg


def swiglu_backward(dh, a, b):
    """``(da, db)`` of h = silu(a) * b in float32 (flash_moe/ops/triton/flash_mlp.py:52-102)."""
    dh, a, b = dh.float(), a.float(), b.float()
    sig = torch.sigmoid(a)
    return dh * b * sig * (1 + a * (1 - sig)), dh * a * sig


def mlp_backward(dy, x2d, gate_w, up_w, down_w):
    """``(dx, dgate_w, dup_w, ddown_w)`` of `mlp_forward` in float32: the chain the reference's autograd builds
    from its matmuls and `TritonSwiGLUFunc` (flash_moe/ops/triton/flash_mlp.py:150-181)."""
    dy, xs, wg, wu, wd = dy.float(), x2d.float(), gate_w.float(), up_w.float(), down_w.float()
    a, b = xs @ wg.t(), xs @ wu.t()
    h = F.silu(a) * b
    da, db = swiglu_backward(dy @ wd, a, b)
    return da @ wg + db @ wu, da.t() @ xs, db.t() @ xs, dy.t() @ h


class _RouterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, log_probs, num_keys, top_k):
        scores, indices = router_topk(log_probs, num_keys, top_k)
        ctx.save_for_backward(indices)
        ctx.num_keys = num_keys
        ctx.mark_non_differentiable(indices)
        return scores, indices

    @staticmethod
    def backward(ctx, dscores, _):
        (indices,) = ctx.saved_tensors
        return router_backward(dscores, indices, ctx.num_keys).to(dscores.dtype), None, None


class _ExpertFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, down_table, up_table, indices, gates):
        ctx.save_for_backward(x2d, down_table, up_table, indices, gates)
        return expert_forward(x2d, down_table, up_table, indices, gates).to(x2d.dtype)

    @staticmethod
    def backward(ctx, dout):
        x2d, down_table, up_table, indices, gates = ctx.saved_tensors
        dx, dd, du, dg = expert_backward(dout, x2d, down_table, up_table, indices, gates)
        return dx.to(x2d.dtype), dd.to(down_table.dtype), du.to(up_table.dtype), None, dg.to(gates.dtype)


class _MlpFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, gate_w, up_w, down_w):
        ctx.save_for_backward(x2d, gate_w, up_w, down_w)
        return mlp_forward(x2d, gate_w, up_w, down_w).to(x2d.dtype)

    @staticmethod
    def backward(ctx, dy):
        x2d, gate_w, up_w, down_w = ctx.saved_tensors
        dx, dg, du, dd = mlp_backward(dy, x2d, gate_w, up_w, down_w)
        return dx.to(x2d.dtype), dg.to(gate_w.dtype), du.to(up_w.dtype), dd.to(down_w.dtype)


# --------------------------------------------------------------------------------------
# The whole layer
# --------------------------------------------------------------------------------------
class OracleFlashMoE(nn.Module):
    """Eager CPU layer with the reference's parameter names, shapes and construction order.

    Mirrors ``FlashMoE_Pytorch`` (flash_moe/modules/flash_moe.py:108-191) with
    ``mlp_bias=False``; built under the same ``torch.manual_seed`` it holds
    bit-identical parameters to the reference modules (checked by the golden
    generator).  Only ``hidden_act == "silu"`` is meaningful because the
    reference kernels hard-code SiLU (flash_expert.py:8-10, flash_mlp.py:8-10).
    """

    def __init__(self, hidden_size, intermediate_size, num_experts, num_experts_per_tok, norm_topk_prob=False):
        super().__init__()
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.num_experts = num_experts
        self.num_keys = math.floor(math.sqrt(num_experts))  # flash_moe.py:38
        self.top_k = num_experts_per_tok
        self.norm_topk_prob = norm_topk_prob
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)
        self.router_gate = nn.Linear(hidden_size, self.num_keys * 2, bias=False)
        self.router_norm = nn.BatchNorm1d(hidden_size, affine=False)
        self.down_embed = nn.Embedding(num_experts, hidden_size)
        self.up_embed = nn.Embedding(num_experts, hidden_size)

    # stage-by-stage so that tests can chain / teacher-force
    def route(self, x2d):
        logits, logp = router_front(
            x2d, self.router_gate.weight, self.router_norm.running_mean, self.router_norm.running_var, self.training
        )
        if self.training and self.router_norm.num_batches_tracked is not None:
            self.router_norm.num_batches_tracked += 1
        scores, indices = router_topk(logp, self.num_keys, self.top_k)
        return logits, logp, scores, indices

    def forward(self, hidden_states: torch.Tensor):
        """Free-running eager forward in the module dtype; returns (y[B,S,H], router_logits[2,T,nk])."""
        B, S, H = hidden_states.shape
        x2d = hidden_states.reshape(-1, H)
        logits, _, scores, indices = self.route(x2d)
        gates = routing_weights(scores, self.norm_topk_prob)
        experts = expert_forward_eager(x2d, self.down_embed.weight, self.up_embed.weight, indices, gates)
        mlp = mlp_forward_eager(x2d, self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight)
        y = (mlp + experts).view(B, S, H)
        return y, logits.view(B * S, 2, self.num_keys).transpose(0, 1)

    def forward_differentiable(self, hidden_states: torch.Tensor):
        """The forward as a chain of autograd nodes whose three custom ops use the explicit backward
        restatements above; everything else (batch-norm, linear, log-softmax, exp, add) is torch autograd, as in
        the reference module (flash_moe/modules/flash_moe.py:55-105)."""
        B, S, H = hidden_states.shape
        x2d = hidden_states.reshape(-1, H)
        logits = self.router_gate(self.router_norm(x2d))
        halves = logits.view(B * S, 2, -1).transpose(0, 1)
        scores, indices = _RouterFn.apply(F.log_softmax(halves, dim=-1), self.num_keys, self.top_k)
        gates = routing_weights(scores, self.norm_topk_prob)
        experts = _ExpertFn.apply(x2d, self.down_embed.weight, self.up_embed.weight, indices, gates)
        mlp = _MlpFn.apply(x2d, self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight)
        return (mlp + experts).view(B, S, H), halves

    def forward_fp32_given_routing(self, hidden_states, indices, gates, round_h_to=None) -> torch.Tensor:
        """float32 evaluation of experts + MLP + add on the stored (possibly bf16) operands for a *given* routing.
        ``round_h_to`` rounds the MLP intermediate once to that dtype (see `mlp_forward`)."""
        H = hidden_states.shape[-1]
        x2d = hidden_states.reshape(-1, H)
        e = expert_forward(x2d, self.down_embed.weight, self.up_embed.weight, indices, gates)
        m = mlp_forward(x2d, self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight, round_h_to=round_h_to)
        return (e + m).view(*hidden_states.shape)


# --------------------------------------------------------------------------------------
# Parity helpers shared by tests / smoke / bench
# --------------------------------------------------------------------------------------
def check_router_threshold(log_probs, num_keys, top_k, got_indices, rel=1e-3, chunk=64):
    """Index-set parity up to score ties.

    With r = the reference score of every candidate and tau = its k-th largest:
    every returned index must have r >= tau - rel*|tau|, every candidate with
    r > tau + rel*|tau| must be returned, no duplicates, all ids in [0, nk^2).
    Returns a dict of violation counts (all zero = pass).
    """
    T = log_probs.size(1)
    bad_low = missing = dups = oob = 0
    for t0 in range(0, T, chunk):
        r = router_all_scores(log_probs, num_keys, t0, min(T, t0 + chunk))
        got = got_indices[t0 : t0 + chunk]
        oob += int(((got < 0) | (got >= num_keys * num_keys)).sum())
        got_c = got.clamp(0, num_keys * num_keys - 1)
        tau = torch.sort(r, dim=-1, descending=True).values[:, top_k - 1 : top_k] if top_k > 0 else None
        if tau is None:
            continue
        tol = rel * tau.abs()
        bad_low += int((r.gather(-1, got_c) < tau - tol).sum())
        sel = torch.zeros_like(r, dtype=torch.bool)
        sel.scatter_(-1, got_c, True)
        dups += int((sel.sum(-1) != top_k).sum())
        missing += int(((r > tau + tol) & ~sel).sum())
    return {"below_threshold": bad_low, "missing": missing, "duplicate_rows": dups, "out_of_range": oob}


def rel_rms_error(got: torch.Tensor, want: torch.Tensor) -> float:
    """max |got - want| / RMS(want), the layer-output parity figure (budget 2e-2 for bf16)."""
    want = want.double()
    rms = want.pow(2).mean().sqrt().item()
    return (got.double() - want).abs().max().item() / max(rms, 1e-30)


def output_parity(got: torch.Tensor, want: torch.Tensor, dtype: torch.dtype):
    """Parity figures for a 16-bit result `got` against the float32 evaluation `want`.

    Returns ``(raw, floor, excess)``, all as multiples of RMS(want):
    ``raw``    max|got - want| (the budget for bf16 layer outputs is 2e-2);
    ``floor``  the same figure for `want` itself rounded once to `dtype` - what a perfect
               implementation that must return `dtype` would score (max|y| * 2^-8 / RMS in the worst
               case for bf16, so a heavy-tailed output can exceed the budget by rounding alone);
    ``excess`` the largest error left after discounting, per element, that half-ulp rounding error.
    """
    want = want.double()
    rms = max(want.pow(2).mean().sqrt().item(), 1e-30)
    err = (got.double() - want).abs()
    raw = err.max().item() / rms
    floor = (want.to(dtype).double() - want).abs().max().item() / rms
    half_ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    excess = (err - want.abs() * half_ulp).clamp_min(0).max().item() / rms
    return raw, floor, excess


def assert_output_parity(got, want, dtype, raw_budget=2e-2, slack=8e-3, strict=False):
    """float32: raw < 1e-4.  16-bit: raw < raw_budget, or - when the rounding floor of the output
    format is itself near or above the budget - raw < floor + slack with nothing but `slack` left
    beyond the final rounding.  `strict` always applies the floor test, with the slack tightened to 3e-3."""
    if dtype == torch.float32:
        raw = rel_rms_error(got, want)
        assert raw < 1e-4, raw
        return raw
    raw, floor, excess = output_parity(got.float(), want, dtype)
    if strict:
        slack = 3e-3
    if raw >= raw_budget or strict:
        assert raw < floor + slack and excess < slack, (
            f"raw {raw:.3e} x RMS (budget {raw_budget}, rounding floor {floor:.3e}, beyond rounding {excess:.3e})"
        )
    return raw
