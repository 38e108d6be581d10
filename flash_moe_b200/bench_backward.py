"""Timing of the backward pass at the benchmark shape (4096 tokens, H 1024, I 4096, 16384 experts, k 64, bf16):

    python -m flash_moe_b200.bench_backward [--steps 20] [--no-graph]

Prints one JSON line: the expert op's backward alone, the expert op forward + backward, and one full layer
forward + backward step (eager autograd, and replayed from a CUDA graph of the whole step unless --no-graph).
Times are CUDA-event means over --steps iterations after 3 warm-ups; inputs stay resident on the GPU.
"""

from __future__ import annotations

import argparse
import json

import torch

from . import FlashMoE, FlashMoEConfig, check_status
from .ops.flash_expert import _expert_backward, flash_expert_func


def timed(fn, steps):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    T, H, I, N, k = 4096, 1024, 4096, 16384, 64
    torch.manual_seed(0)
    layer = FlashMoE(FlashMoEConfig(H, I, "silu", N, k, False)).to(torch.bfloat16).to(dev).eval()
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(1, T, H, device=dev, generator=g).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(1, T, H, device=dev, generator=g).to(torch.bfloat16)
    idx = torch.randint(0, N, (T, k), device=dev, generator=g)
    gates = torch.softmax(torch.randn(T, k, device=dev, generator=g), -1).to(torch.bfloat16)
    xf, do = x.detach().view(T, H), dy.view(T, H)
    down, up = layer.down_embed.weight.detach(), layer.up_embed.weight.detach()
    out = {"config": {"tokens": T, "hidden": H, "intermediate": I, "experts": N, "top_k": k, "dtype": "bf16"},
           "steps": args.steps}
    out["expert_backward_ms"] = timed(lambda: _expert_backward(do, xf, down, up, idx, gates), args.steps)

    def expert_step():
        leaves = [t.detach().requires_grad_() for t in (xf, down, up, gates)]
        flash_expert_func(leaves[0], leaves[1], leaves[2], idx, leaves[3]).backward(do)

    out["expert_forward_backward_ms"] = timed(expert_step, args.steps)

    def layer_step():
        for p in layer.parameters():
            p.grad = None
        x.grad = None
        y, _ = layer(x)
        y.backward(dy)

    out["layer_forward_backward_ms"] = timed(layer_step, args.steps)
    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            layer_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        for p in layer.parameters():
            p.grad = None
        x.grad = None
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y, _ = layer(x)
            y.backward(dy)
        out["layer_forward_backward_graph_ms"] = timed(graph.replay, args.steps)
    check_status()
    out["tokens_per_s_training_step"] = T / (min(out["layer_forward_backward_ms"],
                                                 out.get("layer_forward_backward_graph_ms", 1e9)) * 1e-3)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
