"""Shared builders for the parity tests: seeded inputs generated on CPU, then copied to the GPU,
so the CPU oracle and the CUDA path see identical bits."""

import math

import torch

from oracle import flashmoe_oracle as O


def bf16_ulp_close(a: torch.Tensor, b: torch.Tensor, ulps: int = 1):
    """True where two bf16 tensors differ by at most `ulps` representable steps."""
    ia = a.contiguous().view(torch.int16).to(torch.int32)
    ib = b.contiguous().view(torch.int16).to(torch.int32)
    # map sign-magnitude to a monotone integer line
    ia = torch.where(ia < 0, -(ia & 0x7FFF), ia)
    ib = torch.where(ib < 0, -(ib & 0x7FFF), ib)
    return (ia - ib).abs() <= ulps


def make_layer_pair(H, I, N, k, norm, dtype, seed=0):
    """(oracle layer on CPU, our layer on cuda:0) holding identical parameters."""
    from flash_moe_b200 import FlashMoE, FlashMoEConfig

    torch.manual_seed(seed)
    ref = O.OracleFlashMoE(H, I, N, k, norm).to(dtype)
    torch.manual_seed(seed)
    ours = FlashMoE(FlashMoEConfig(H, I, "silu", N, k, norm)).to(dtype)
    for (n1, p1), (n2, p2) in zip(sorted(ref.state_dict().items()), sorted(ours.state_dict().items())):
        assert n1 == n2 and torch.equal(p1, p2), f"parameter {n1} differs between oracle and module"
    return ref, ours.cuda()


def randn(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def log_probs(T, nk, seed, dtype):
    return torch.log_softmax(randn((2, T, nk), seed), dim=-1).to(dtype)


def num_keys(N):
    return math.floor(math.sqrt(N))
