"""The PEER and PKM comparison ops through the C ABI against the oracle and the reference's golden outputs."""

import os

import numpy as np
import pytest
import torch

from oracle import flashmoe_oracle as O
from tests.helpers import randn

pytestmark = pytest.mark.gpu


def case(T, H, N, k, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(T, H, generator=g) * 0.5).to(dtype)
    d = (torch.randn(N, H, generator=g) * 0.3).to(dtype)
    u = (torch.randn(N, H, generator=g) * 0.3).to(dtype)
    idx = torch.randint(0, N, (T, k), generator=g)
    if k > 1:
        idx[0, 1] = idx[0, 0]
    w = torch.softmax(torch.randn(T, k, generator=g), -1).to(dtype)
    return x, d, u, w, idx


@pytest.mark.parametrize(
    "T,H,N,k,dtype",
    [
        (1, 8, 4, 1, torch.float32),
        (50, 72, 33, 5, torch.float32),
        (256, 256, 4096, 16, torch.bfloat16),
        (64, 1280, 300, 7, torch.float16),
        (2048, 1024, 16384, 32, torch.bfloat16),
    ],
)
def test_peer_and_pkm_forward(T, H, N, k, dtype):
    from flash_moe_b200 import check_status
    from flash_moe_b200.ops.peer import triton_peer_func
    from flash_moe_b200.ops.pkm import triton_pkm_func

    x, d, u, w, idx = case(T, H, N, k, dtype, T + k)
    args = [t.cuda() for t in (x, d, u, w, idx)]
    y_peer = triton_peer_func(*args)
    y_pkm = triton_pkm_func(args[2], args[3], args[4])
    torch.cuda.synchronize()
    check_status()
    for got, want in ((y_peer, O.peer_forward(x, d, u, w, idx)), (y_pkm, O.pkm_forward(u, w, idx))):
        assert got.dtype == dtype and got.shape == (T, H)
        if dtype == torch.float32:
            assert torch.allclose(got.cpu(), want, rtol=2e-5, atol=2e-6)
        else:
            O.assert_output_parity(got.float().cpu(), want, dtype)
    assert torch.equal(y_pkm, triton_pkm_func(args[2], args[3], args[4]))


def test_peer_and_pkm_golden_from_reference_kernels(golden_dir):
    from flash_moe_b200.ops.peer import triton_peer_func
    from flash_moe_b200.ops.pkm import triton_pkm_func

    z = np.load(os.path.join(golden_dir, "triton_peer_pkm_small.npz"))
    x, d, u, w, idx = (torch.from_numpy(z[n]).cuda() for n in ("x", "down", "up", "weights", "indices"))
    assert torch.allclose(triton_peer_func(x, d, u, w, idx).cpu(), torch.from_numpy(z["y_peer"]), rtol=1e-4, atol=1e-5)
    assert torch.allclose(triton_pkm_func(u, w, idx).cpu(), torch.from_numpy(z["y_pkm"]), rtol=1e-5, atol=1e-6)


def test_peer_and_pkm_have_no_backward_like_the_reference():
    from flash_moe_b200.ops.pkm import triton_pkm_func

    x, d, u, w, idx = case(8, 16, 12, 2, torch.float32, 1)
    y = triton_pkm_func(u.cuda().requires_grad_(), w.cuda(), idx.cuda())
    with pytest.raises(NotImplementedError):
        y.sum().backward()
