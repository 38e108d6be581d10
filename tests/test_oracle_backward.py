"""The oracle's backward restatements: against torch autograd of the eager formulas (float64) and against the
gradients the reference's own eager module produced under autograd (tests/golden/*_grads*.npz)."""

import os

import numpy as np
import pytest
import torch

from oracle import flashmoe_oracle as O


def test_expert_backward_formulas_match_autograd():
    g = torch.Generator().manual_seed(0)
    T, H, N, k = 9, 16, 12, 5
    x = torch.randn(T, H, generator=g, dtype=torch.float64, requires_grad=True)
    d = torch.randn(N, H, generator=g, dtype=torch.float64, requires_grad=True)
    u = torch.randn(N, H, generator=g, dtype=torch.float64, requires_grad=True)
    idx = torch.randint(0, N, (T, k), generator=g)
    idx[0, 1] = idx[0, 0]  # a duplicate inside one token
    gates = torch.rand(T, k, generator=g, dtype=torch.float64, requires_grad=True)
    dout = torch.randn(T, H, generator=g, dtype=torch.float64)
    O.expert_forward_eager(x, d, u, idx, gates).backward(dout)
    dx, dd, du, dg = O.expert_backward(dout, x.detach(), d.detach(), u.detach(), idx, gates.detach())
    for got, want in ((dx, x.grad), (dd, d.grad), (du, u.grad), (dg, gates.grad)):
        assert torch.allclose(got.double(), want, rtol=1e-4, atol=1e-5)


def test_mlp_and_router_backward_formulas_match_autograd():
    g = torch.Generator().manual_seed(1)
    T, H, I = 7, 12, 20
    x = torch.randn(T, H, generator=g, dtype=torch.float64, requires_grad=True)
    wg = torch.randn(I, H, generator=g, dtype=torch.float64, requires_grad=True)
    wu = torch.randn(I, H, generator=g, dtype=torch.float64, requires_grad=True)
    wd = torch.randn(H, I, generator=g, dtype=torch.float64, requires_grad=True)
    dy = torch.randn(T, H, generator=g, dtype=torch.float64)
    O.mlp_forward_eager(x, wg, wu, wd).backward(dy)
    got = O.mlp_backward(dy, x.detach(), wg.detach(), wu.detach(), wd.detach())
    for a, b in zip(got, (x.grad, wg.grad, wu.grad, wd.grad)):
        assert torch.allclose(a.double(), b, rtol=1e-4, atol=1e-4)
    nk, k = 6, 4
    lp = torch.log_softmax(torch.randn(2, T, nk, generator=g, dtype=torch.float64), -1).requires_grad_()
    scores, idx = O.router_topk(lp.detach().float(), nk, k)
    ds = torch.randn(T, k, generator=g, dtype=torch.float64)
    picked = lp[0].gather(1, idx // nk) + lp[1].gather(1, idx % nk)
    picked.backward(ds)
    assert torch.allclose(O.router_backward(ds, idx, nk).double(), lp.grad, atol=1e-6)


@pytest.mark.parametrize("name", ["eager_mini_fp32_grads", "eager_mini_fp32_grads_norm_train"])
def test_differentiable_oracle_layer_reproduces_reference_gradients(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    H, I, N, k, norm, B, S, train = (int(v) for v in z["cfg"])
    layer = O.OracleFlashMoE(H, I, N, k, bool(norm))
    layer.load_state_dict({n[len("param."):]: torch.from_numpy(z[n]) for n in z.files if n.startswith("param.")})
    layer.train(bool(train))
    x = torch.from_numpy(z["x"]).requires_grad_()
    y, _ = layer.forward_differentiable(x)
    assert torch.allclose(y, torch.from_numpy(z["y"]), rtol=1e-4, atol=1e-5)
    (y * torch.from_numpy(z["w"])).sum().backward()
    grads = dict({"x": x.grad}, **{n: p.grad for n, p in layer.named_parameters()})
    for n, got in grads.items():
        want = torch.from_numpy(z["grad." + n])
        scale = want.abs().max().clamp_min(1e-6)
        assert float((got - want).abs().max() / scale) < 2e-4, n
