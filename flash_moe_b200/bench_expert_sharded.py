"""Timing of the expert-sharded paths (tables sharded by expert id) on N GPUs of one node, at the shape of the
2^20-expert configuration:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m flash_moe_b200.bench_expert_sharded [--mode a2a|peer] [--tokens 32768 --hidden 2048 --experts 1048576 --top-k 16]

--mode a2a: all-to-all dispatch of token rows and combine of partial rows (ExpertShardedExperts).
--mode peer: shards in symmetric memory, remote rows read in place over NVLink by the gather kernels
             (PeerShardedExperts): no exchange at all.

Tokens are split evenly over the ranks, expert ids are Zipf(1.1) distributed, gates are a softmax of
normal logits.  Rank 0 prints one JSON line: tokens/s over all ranks (max over ranks of the CUDA-event
time per step), the rows each rank sends and receives (load imbalance) and the all-to-all payload.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .parallel import ExpertShardedExperts, PeerShardedExperts, token_shard


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=1 << 20)
    ap.add_argument("--top-k", type=int, default=16)
    ap.add_argument("--mode", default="a2a", choices=["a2a", "peer"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    dist.init_process_group("nccl", device_id=dev, rank=rank, world_size=world)
    T, H, N, k = args.tokens, args.hidden, args.experts, args.top_k
    dt = torch.bfloat16
    rows = (N - rank + world - 1) // world  # experts with id % world == rank
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    down = torch.empty(rows, H, dtype=dt, device=dev).normal_(0, 0.1, generator=g)
    up = torch.empty(rows, H, dtype=dt, device=dev).normal_(0, 0.1, generator=g)
    s, e = token_shard(T, rank, world)
    x = (torch.randn(e - s, H, generator=g, device=dev) * 0.5).to(dt)
    p = torch.arange(1, N + 1, dtype=torch.float64, device=dev).pow(-1.1)
    cdf = torch.cumsum(p / p.sum(), 0)
    idx = torch.searchsorted(cdf, torch.rand(e - s, k, generator=g, dtype=torch.float64, device=dev)).clamp_(max=N - 1)
    gates = torch.softmax(torch.randn(e - s, k, generator=g, device=dev), -1).to(dt)
    if args.mode == "peer":
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        layer = PeerShardedExperts(N, H, dt, dev)
        layer.down_shard.copy_(down)
        layer.up_shard.copy_(up)
        del down, up
        layer.publish()
        layer.last_stats = {"sent_rows": 0, "received_rows": 0}
    else:
        layer = ExpertShardedExperts(down, up, N)
    for _ in range(max(args.warmup, 3)):
        layer.forward(x, idx, gates)
    dist.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        layer.forward(x, idx, gates)
    end.record()
    dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([start.elapsed_time(end) / args.steps], device=dev, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    stats = torch.tensor([layer.last_stats["sent_rows"], layer.last_stats["received_rows"]], device=dev, dtype=torch.int64)
    allstats = [torch.zeros_like(stats) for _ in range(world)]
    dist.all_gather(allstats, stats)
    if rank == 0:
        sent = [int(t[0]) for t in allstats]
        recv = [int(t[1]) for t in allstats]
        print(json.dumps({
            "metric": "expert-sharded experts fwd tokens/s", "mode": args.mode, "value": T / (float(ms) * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "ms_per_step": float(ms), "dtype": "bf16", "data": "synthetic",
            "config": {"tokens": T, "hidden": H, "experts": N, "top_k": k, "ids": "Zipf(1.1)", "tables": "id % world"},
            "rows_sent_per_rank": sent, "rows_received_per_rank": recv,
            "dispatch_bytes_per_rank_max": max(sent) * H * 2, "combine_bytes_per_rank_max": max(recv) * H * 4,
            "peer_row_bytes_per_rank": (2 * (e - s) * k * H * 2 * (world - 1) // world) if args.mode == "peer" else 0,
        }))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
