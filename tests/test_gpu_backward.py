"""Backward of the three ops and of the layer through the C ABI, against the oracle's float32 restatements and the
gradients of the reference's own eager module (golden fixtures)."""

import os

import numpy as np
import pytest
import torch

from oracle import flashmoe_oracle as O
from tests.helpers import randn

pytestmark = pytest.mark.gpu


def rel_err(got, want):
    want = want.float()
    return float((got.detach().float().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-12))


def tol(dtype):
    return {torch.float32: 2e-5, torch.bfloat16: 1.2e-2, torch.float16: 2e-3}[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,nk,k", [(1, 4, 1), (33, 16, 4), (257, 128, 64), (64, 100, 100)])
def test_router_backward(dtype, T, nk, k):
    from flash_moe_b200.ops.flash_router import flash_router_func

    lp = torch.log_softmax(randn((2, T, nk), T + nk, torch.float32), -1).to(dtype).cuda().requires_grad_()
    scores, idx = flash_router_func(lp, nk, k)
    ds = randn((T, k), 5, torch.float32).to(dtype).cuda()
    scores.backward(ds)
    want = O.router_backward(ds.cpu(), idx.cpu(), nk)
    assert lp.grad.shape == (2, T, nk) and lp.grad.dtype == dtype
    assert rel_err(lp.grad, want) <= (1e-6 if dtype == torch.float32 else tol(dtype))
    # every slot's gradient arrives exactly twice (once per half)
    assert abs(float(lp.grad.float().sum()) - 2 * float(ds.float().sum())) <= 1e-2 * (1 + float(ds.float().abs().sum()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_swiglu_backward(dtype):
    from flash_moe_b200.ops.flash_mlp import swiglu_backward

    a, b, dh = (randn((37, 256), s, torch.float32).mul(2).to(dtype).cuda() for s in (1, 2, 3))
    da, db, h = swiglu_backward(dh, a, b, want_h=True)
    wa, wb = O.swiglu_backward(dh.cpu(), a.cpu(), b.cpu())
    wh = torch.nn.functional.silu(a.cpu().float()) * b.cpu().float()
    for got, want in ((da, wa), (db, wb), (h, wh)):
        assert rel_err(got, want) <= tol(dtype)


def expert_case(T, H, N, k, dtype, zipf=False, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(T, H, generator=g) * 0.5).to(dtype)
    d = (torch.randn(N, H, generator=g) * 0.2).to(dtype)
    u = (torch.randn(N, H, generator=g) * 0.2).to(dtype)
    if zipf:
        p = torch.arange(1, N + 1, dtype=torch.float64).pow(-1.1)
        idx = torch.multinomial((p / p.sum()).float(), T * k, replacement=True, generator=g).view(T, k)
    else:
        idx = torch.randint(0, N, (T, k), generator=g)
    if k > 1:
        idx[0, 1] = idx[0, 0]
    gates = torch.softmax(torch.randn(T, k, generator=g), -1).to(dtype)
    dout = torch.randn(T, H, generator=g).to(dtype)
    return x, d, u, idx, gates, dout


def run_expert_backward(x, d, u, idx, gates, dout):
    from flash_moe_b200.ops.flash_expert import flash_expert_func

    xs, ds_, us, gs = (t.cuda().requires_grad_() for t in (x, d, u, gates))
    out = flash_expert_func(xs, ds_, us, idx.cuda(), gs)
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    return xs.grad, ds_.grad, us.grad, gs.grad


@pytest.mark.parametrize(
    "T,H,N,k,dtype,zipf",
    [
        (5, 8, 7, 1, torch.float32, False),
        (64, 72, 50, 3, torch.float32, False),      # sorted schedule, ragged column block
        (300, 256, 64, 8, torch.float32, True),     # hot experts: rows assembled from several chunk partials
        (128, 64, 4096, 4, torch.bfloat16, False),  # token-centric schedule, most experts untouched
        (512, 1280, 96, 16, torch.bfloat16, True),  # two column blocks, hot experts
        (200, 128, 33, 6, torch.float16, True),
        (2048, 1024, 16384, 16, torch.bfloat16, False),
    ],
)
def test_expert_backward(T, H, N, k, dtype, zipf):
    from flash_moe_b200 import check_status

    x, d, u, idx, gates, dout = expert_case(T, H, N, k, dtype, zipf, seed=T + N)
    got = run_expert_backward(x, d, u, idx, gates, dout)
    check_status()
    want = O.expert_backward(dout, x, d, u, idx, gates)
    for name, g_, w_ in zip(("dx", "ddown", "dup", "dgates"), got, want):
        assert g_.dtype == dtype
        assert rel_err(g_, w_) <= tol(dtype), name
    untouched = torch.ones(N, dtype=torch.bool)
    untouched[idx.unique()] = False
    if untouched.any():  # experts nobody selected get exact zero rows
        assert float(got[1][untouched.cuda()].abs().max()) == 0.0 and float(got[2][untouched.cuda()].abs().max()) == 0.0
    again = run_expert_backward(x, d, u, idx, gates, dout)
    assert all(torch.equal(a, b) for a, b in zip(got, again))  # fixed summation order: bit-equal reruns


def test_expert_backward_skips_out_of_range_ids():
    from flash_moe_b200 import read_status, _lib

    x, d, u, idx, gates, dout = expert_case(40, 64, 20, 4, torch.float32, seed=3)
    idx[3, 2] = -2
    idx[7, 0] = 20
    read_status()
    got = run_expert_backward(x, d, u, idx, gates, dout)
    assert read_status() & _lib.STATUS_BAD_EXPERT_ID
    g0 = gates.clone()
    g0[3, 2] = 0
    g0[7, 0] = 0
    want = O.expert_backward(dout, x, d, u, idx.clamp(0, 19), g0)
    for g_, w_ in zip(got[:3], want[:3]):
        assert rel_err(g_, w_) <= 2e-5
    assert float(got[3][3, 2]) == 0.0 and float(got[3][7, 0]) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mlp_backward(dtype):
    from flash_moe_b200.ops.flash_mlp import flash_mlp_func

    T, H, I = 200, 128, 384
    x = (randn((T, H), 1, torch.float32) * 0.5).to(dtype)
    wg, wu = ((randn((I, H), s, torch.float32) * 0.1).to(dtype) for s in (2, 3))
    wd = (randn((H, I), 4, torch.float32) * 0.1).to(dtype)
    dy = randn((T, H), 5, torch.float32).to(dtype)
    leaves = [t.cuda().requires_grad_() for t in (x, wg, wu, wd)]
    flash_mlp_func(*leaves).backward(dy.cuda())
    want = O.mlp_backward(dy, x, wg, wu, wd)
    for leaf, w_ in zip(leaves, want):
        assert leaf.grad.dtype == dtype
        assert rel_err(leaf.grad, w_) <= (1e-4 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("name", ["eager_mini_fp32_grads", "eager_mini_fp32_grads_norm_train"])
def test_layer_gradients_match_reference_eager_module(golden_dir, name):
    """float32 layer with the fixture's parameters: gradients of sum(y * w) equal the reference's autograd result."""
    from flash_moe_b200 import FlashMoE, FlashMoEConfig, check_status

    z = np.load(os.path.join(golden_dir, name + ".npz"))
    H, I, N, k, norm, B, S, train = (int(v) for v in z["cfg"])
    layer = FlashMoE(FlashMoEConfig(H, I, "silu", N, k, bool(norm)))
    layer.load_state_dict({n[len("param."):]: torch.from_numpy(z[n]) for n in z.files if n.startswith("param.")})
    layer = layer.cuda().train(bool(train))
    x = torch.from_numpy(z["x"]).cuda().requires_grad_()
    y, _ = layer(x)
    assert rel_err(y, torch.from_numpy(z["y"])) < 1e-4
    (y * torch.from_numpy(z["w"]).cuda()).sum().backward()
    torch.cuda.synchronize()
    check_status()
    grads = dict({"x": x.grad}, **{n: p.grad for n, p in layer.named_parameters()})
    for n, got in grads.items():
        assert rel_err(got, torch.from_numpy(z["grad." + n])) < 5e-4, n


def test_layer_backward_bf16_runs_and_no_grad_path_is_unchanged():
    from flash_moe_b200 import FlashMoE, FlashMoEConfig, check_status

    torch.manual_seed(0)
    layer = FlashMoE(FlashMoEConfig(256, 512, "silu", 1024, 8, True)).to(torch.bfloat16).cuda().train()
    x = randn((2, 64, 256), 3, torch.bfloat16).cuda().requires_grad_()
    y, logits = layer(x)
    assert y.requires_grad and logits.requires_grad
    y.float().pow(2).mean().backward()
    torch.cuda.synchronize()
    check_status()
    for n, p in layer.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad.float()).all(), n
        assert float(p.grad.float().abs().max()) > 0, n
    assert torch.isfinite(x.grad.float()).all()
    layer.eval()
    with torch.no_grad():
        y2, _ = layer(x)
    assert not y2.requires_grad


def test_training_step_replays_from_a_cuda_graph():
    """Forward + backward of the layer captured as one CUDA graph (every launch of the library, the stable sort
    included, is capturable): replayed gradients are bit-equal to the eager step's."""
    from flash_moe_b200 import FlashMoE, FlashMoEConfig, check_status

    torch.manual_seed(0)
    layer = FlashMoE(FlashMoEConfig(256, 512, "silu", 1024, 8, True)).to(torch.bfloat16).cuda().eval()
    x = randn((2, 64, 256), 3, torch.bfloat16).cuda().requires_grad_()
    dy = randn((2, 64, 256), 4, torch.bfloat16).cuda()

    def step():
        for p in layer.parameters():
            p.grad = None
        x.grad = None
        y, _ = layer(x)
        y.backward(dy)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    want = {n: p.grad.clone() for n, p in layer.named_parameters()}
    want_x = x.grad.clone()
    for p in layer.parameters():
        p.grad = None
    x.grad = None
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y, _ = layer(x)
        y.backward(dy)
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    check_status()
    assert torch.equal(x.grad, want_x)
    for n, p in layer.named_parameters():
        assert torch.equal(p.grad, want[n]), n


def test_backward_with_no_pairs():
    """k = 0: the expert op's gradients are all zero (and every table row is written)."""
    from flash_moe_b200.ops.flash_expert import _expert_backward

    dt = torch.float32
    x, dout = randn((6, 32), 1, dt).cuda(), randn((6, 32), 2, dt).cuda()
    d, u = randn((10, 32), 3, dt).cuda(), randn((10, 32), 4, dt).cuda()
    idx = torch.empty(6, 0, dtype=torch.int64, device="cuda")
    gates = torch.empty(6, 0, dtype=dt, device="cuda")
    dx, dd, du, dg = _expert_backward(dout, x, d, u, idx, gates)
    torch.cuda.synchronize()
    assert float(dx.abs().max()) == 0.0 and float(dd.abs().max()) == 0.0 and float(du.abs().max()) == 0.0
    assert dg.shape == (6, 0)


def test_mlp_backward_with_kept_preactivations():
    """A shape the CTA-pair GEMM covers: the forward keeps x Wg^T and x Wu^T, the backward uses them."""
    from flash_moe_b200.ops.flash_mlp import FlashMLPFunc, _mlp_forward

    dtype = torch.bfloat16
    T, H, I = 1024, 256, 512
    x = (randn((T, H), 1, torch.float32) * 0.5).to(dtype)
    wg, wu = ((randn((I, H), s, torch.float32) * 0.1).to(dtype) for s in (2, 3))
    wd = (randn((H, I), 4, torch.float32) * 0.1).to(dtype)
    dy = randn((T, H), 5, torch.float32).to(dtype)
    out, a, b = _mlp_forward(x.cuda(), wg.cuda(), wu.cuda(), wd.cuda(), save_preacts=True)
    assert a is not None and rel_err(a, x.float() @ wg.float().t()) < 1e-2 and rel_err(b, x.float() @ wu.float().t()) < 1e-2
    assert torch.equal(out, _mlp_forward(x.cuda(), wg.cuda(), wu.cuda(), wd.cuda()))  # same kernels, same output
    leaves = [t.cuda().requires_grad_() for t in (x, wg, wu, wd)]
    FlashMLPFunc.apply(*leaves).backward(dy.cuda())
    want = O.mlp_backward(dy, x, wg, wu, wd)
    for leaf, w_ in zip(leaves, want):
        assert rel_err(leaf.grad, w_) <= 2e-2
