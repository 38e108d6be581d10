"""Router parity on the GPU, through the C ABI (fmoe_router_topk / fmoe_router_front)."""

import os

import numpy as np
import pytest
import torch

from oracle import flashmoe_oracle as O
from tests.helpers import bf16_ulp_close, log_probs, randn

pytestmark = pytest.mark.gpu


def run_router(lp, nk, k):
    from flash_moe_b200.ops.flash_router import flash_router_func

    s, i = flash_router_func(lp.cuda(), nk, k)
    torch.cuda.synchronize()
    return s.cpu(), i.cpu()


@pytest.mark.parametrize(
    "T,nk,k",
    [(64, 32, 8), (256, 128, 64), (33, 100, 7), (5, 16, 1), (9, 16, 16), (17, 1, 1), (40, 256, 32), (12, 512, 128),
     (7, 48, 48), (3, 1000, 10)],
)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_router_topk_exact(T, nk, k, dtype):
    """Scores, indices and their order are bit-identical to the reference semantics, ties included
    (16-bit inputs produce many exactly equal pair sums)."""
    lp = log_probs(T, nk, seed=T * 1000 + nk, dtype=dtype)
    want_s, want_i = O.router_topk(lp, nk, k)
    got_s, got_i = run_router(lp, nk, k)
    assert got_i.dtype == torch.int64 and got_s.dtype == dtype
    assert torch.equal(got_s.float(), want_s.float())
    assert torch.equal(got_i, want_i)
    assert all(v == 0 for v in O.check_router_threshold(lp, nk, k, got_i).values())


@pytest.mark.parametrize(
    "name", ["triton_router_nk16_k4", "triton_router_nk16_k4_tied", "triton_router_nk32_k8_tied", "triton_router_nk128_k16"]
)
def test_router_topk_matches_reference_kernel_fixture(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    got_s, got_i = run_router(torch.from_numpy(z["log_probs"]), int(z["nk"]), int(z["k"]))
    assert np.array_equal(got_s.numpy(), z["scores"])
    assert np.array_equal(got_i.numpy(), z["indices"])


@pytest.mark.parametrize("T,nk,k", [(16, 64, 32), (8, 128, 64), (8, 256, 32), (6, 512, 16)])
def test_router_heavy_ties_and_infinities(T, nk, k):
    """Log-probabilities on a grid of 0.5: hundreds of candidates tie with the threshold (short tie lists ranked by
    shuffles, long ones by the bitwise search, overflowing ones by the per-row search), at shapes that keep the
    candidates in shared memory (64 keys) and in registers (128 and more keys)."""
    lp = torch.round(randn((2, T, nk), 3) * 2) / 2 - 3.0
    lp[0, 0, :] = -1.0  # a whole half tied
    lp[1, 1, :] = float("-inf")  # every sum is -inf for this token
    lp[0, 2, 5] = float("-inf")
    for dtype in (torch.float32, torch.bfloat16):
        x = lp.to(dtype)
        want_s, want_i = O.router_topk(x, nk, k)
        got_s, got_i = run_router(x, nk, k)
        assert torch.equal(got_s.float(), want_s.float())
        assert torch.equal(got_i, want_i)


def test_router_empty_and_argument_errors():
    from flash_moe_b200.ops.flash_router import flash_router_func

    lp = log_probs(4, 16, 1, torch.float32).cuda()
    s, i = flash_router_func(lp, 16, 0)
    assert s.shape == (4, 0) and i.shape == (4, 0)
    s, i = flash_router_func(lp[:, :0], 16, 4)
    assert s.shape == (0, 4)
    with pytest.raises(AssertionError):
        flash_router_func(lp, 16, 17)
    with pytest.raises(AssertionError):
        flash_router_func(lp[0], 16, 4)
    with pytest.raises(Exception):
        flash_router_func(lp.cpu(), 16, 4)


@pytest.mark.parametrize("norm", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_gates(norm, dtype):
    from flash_moe_b200.ops.flash_router import flash_router_with_gates

    T, nk, k = 128, 64, 16
    lp = log_probs(T, nk, 11, dtype)
    s, i, g = flash_router_with_gates(lp.cuda(), nk, k, norm)
    want = O.routing_weights(s.cpu(), norm)
    if dtype == torch.float32:
        torch.testing.assert_close(g.cpu(), want, rtol=2e-6, atol=0)
    else:
        assert bf16_ulp_close(g.cpu(), want, 1).all()
        assert (g.cpu() == want).float().mean() > 0.98


@pytest.mark.parametrize("T,H,nk", [(256, 256, 32), (300, 1024, 128), (130, 512, 256), (64, 128, 24), (200, 64, 512)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("training", [False, True])
def test_router_front(T, H, nk, dtype, training):
    """logits against a float32 evaluation of BN -> Linear on the same stored operands (2e-2 x RMS for
    16-bit), log-probs against torch's log-softmax of OUR logits (one rounding step), and the
    batch-norm running-statistics side effect."""
    from flash_moe_b200.ops.router_front import router_front

    x = randn((T, H), 5, dtype) + (0.25 if training else 0.0)
    w = randn((2 * nk, H), 6, dtype, scale=1.0 / H**0.5)
    rm = randn((H,), 7, dtype, scale=0.1)
    rv = (randn((H,), 8).abs() + 0.5).to(dtype)
    rm_g, rv_g = rm.clone().cuda(), rv.clone().cuda()
    logits, logp = router_front(x.cuda(), w.cuda(), rm_g, rv_g, training=training)
    torch.cuda.synchronize()
    rm32, rv32 = rm.float().clone(), rv.float().clone()
    want_logits, _ = O.router_front(x.float(), w.float(), rm32, rv32, training)
    tol = 2e-2 if dtype != torch.float32 else 1e-4
    assert O.rel_rms_error(logits.cpu().float(), want_logits) < tol
    chained = torch.log_softmax(logits.cpu().view(T, 2, nk).transpose(0, 1).float(), dim=-1).to(dtype)
    if dtype == torch.float32:
        torch.testing.assert_close(logp.cpu(), chained.contiguous(), rtol=1e-5, atol=2e-6)
    else:
        assert bf16_ulp_close(logp.cpu(), chained.contiguous(), 1).all()
        assert (logp.cpu() == chained).float().mean() > 0.99
    if training:
        torch.testing.assert_close(rm_g.cpu().float(), rm32, rtol=1e-2, atol=1e-2 if dtype != torch.float32 else 1e-5)
        torch.testing.assert_close(rv_g.cpu().float(), rv32, rtol=1e-2, atol=1e-2 if dtype != torch.float32 else 1e-5)
    else:
        assert torch.equal(rm_g.cpu(), rm) and torch.equal(rv_g.cpu(), rv)


def test_router_full_size_properties():
    """Config-3 shape (16384 tokens, nk=512, k=128, bf16): properties that need no brute force -
    sorted output, no duplicates, ids in range, scores equal the in-dtype pair sum of their id;
    plus exact parity on a 64-token sample."""
    T, nk, k = 16384, 512, 128
    lp = log_probs(T, nk, 21, torch.bfloat16)
    s, i = run_router(lp, nk, k)
    assert ((i >= 0) & (i < nk * nk)).all()
    sf = s.float()
    assert (sf[:, :-1] >= sf[:, 1:]).all()
    assert (torch.sort(i, dim=-1).values.diff(dim=-1) > 0).all()
    a = lp[0].gather(-1, i // nk)
    b = lp[1].gather(-1, i % nk)
    assert torch.equal((a + b).float(), sf)
    tie = sf[:, :-1] == sf[:, 1:]
    assert (i[:, :-1][tie] < i[:, 1:][tie]).all()
    sel = torch.arange(0, T, T // 64)
    want_s, want_i = O.router_topk(lp[:, sel], nk, k)
    assert torch.equal(s[sel].float(), want_s.float()) and torch.equal(i[sel], want_i)
