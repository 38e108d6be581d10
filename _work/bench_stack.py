"""Timing of a residual stack of FlashMoE layers with the tokens sharded over N GPUs of one node (weights
replicated, no collective in eval mode), at the shape of the multi-layer benchmark configuration:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m flash_moe_b200.bench_stack [--layers 8 --tokens 131072 --hidden 2048 --intermediate 5632 \
                                       --experts 65536 --top-k 32 --steps 5]

--tokens is the TOTAL over all ranks (strong scaling).  Rank 0 prints one JSON line: tokens/s over all ranks from the
maximum over ranks of the CUDA-event time per step, and the dense bf16 rate of the two shared-MLP GEMMs implied by it.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from . import FlashMoEConfig, check_status
from .modules.stack import FlashMoEStack
from .parallel import token_shard


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=131072)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--intermediate", type=int, default=5632)
    ap.add_argument("--experts", type=int, default=65536)
    ap.add_argument("--top-k", type=int, default=32)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    cfg = FlashMoEConfig(args.hidden, args.intermediate, "silu", args.experts, args.top_k, True)
    with torch.device(dev):
        stack = FlashMoEStack(cfg, args.layers, seeds=list(range(args.layers))).to(torch.bfloat16).eval()
    s, e = token_shard(args.tokens, rank, world)
    x = torch.randn(1, e - s, args.hidden, device=dev, generator=torch.Generator(device=dev).manual_seed(100 + rank))
    x = x.to(torch.bfloat16)
    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            stack(x)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.steps):
            y, _ = stack(x)
        end.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    check_status()
    ms = torch.tensor([start.elapsed_time(end) / args.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = float(ms)
        mlp_flops = 6.0 * args.tokens * args.hidden * args.intermediate * args.layers
        print(json.dumps({
            "metric": "FlashMoE stack fwd tokens/s", "value": args.tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "ms_per_step": ms, "ms_per_layer": ms / args.layers, "scaling": "strong", "dtype": "bf16", "data": "synthetic",
            "config": {"layers": args.layers, "tokens_total": args.tokens, "hidden": args.hidden,
                       "intermediate": args.intermediate, "experts": args.experts, "top_k": args.top_k,
                       "norm_topk_prob": True, "mode": "eval", "parallelism": f"tokens sharded x{world}, weights replicated"},
            "shared_mlp_tflops_per_gpu_if_all_time_were_gemm": mlp_flops / world / (ms * 1e-3) / 1e12,
            "finite": bool(torch.isfinite(y.float()).all()),
        }))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
