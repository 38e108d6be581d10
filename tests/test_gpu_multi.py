"""Two-GPU checks (NCCL): token-sharded layers agree with the single-GPU result, and the
expert-sharded dispatch/combine reproduces the unsharded expert op.  Skipped on one GPU."""

import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent(
    """
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, os.environ["FMOE_ROOT"])
    from flash_moe_b200 import FlashMoE, FlashMoEConfig, check_status
    from flash_moe_b200.parallel import ExpertShardedExperts, shard_expert_table, token_shard
    from flash_moe_b200.ops.flash_expert import flash_expert_fp32
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    dt = torch.bfloat16
    # --- tokens sharded, weights replicated: each rank's rows equal the single-GPU rows
    torch.manual_seed(0)
    layer = FlashMoE(FlashMoEConfig(256, 512, "silu", 1024, 8)).to(dt).eval().to(dev)
    x = torch.randn(1, 300, 256, generator=torch.Generator().manual_seed(1)).to(dt).to(dev)
    with torch.no_grad():
        full, _ = layer(x)
        s, e = token_shard(300, rank, world)
        part, _ = layer(x[:, s:e].contiguous())
    assert torch.equal(part, full[:, s:e]), "token shard differs from the unsharded forward"
    # --- training mode: batch-norm statistics of the WHOLE batch under token sharding
    torch.manual_seed(0)
    tl_full = FlashMoE(FlashMoEConfig(256, 512, "silu", 1024, 8)).to(dev).train()
    torch.manual_seed(0)
    tl_shard = FlashMoE(FlashMoEConfig(256, 512, "silu", 1024, 8)).to(dev).train()
    xf = (torch.randn(1, 300, 256, generator=torch.Generator().manual_seed(2)) * 1.7 + 0.4).to(dev)
    with torch.no_grad():
        _, logits_full = tl_full(xf)
        s, e = token_shard(300, rank, world)
        _, logits_part = tl_shard(xf[:, s:e].contiguous(), bn_sync_group=dist.group.WORLD)
    torch.testing.assert_close(logits_part, logits_full[:, s:e], rtol=2e-4, atol=2e-5)
    torch.testing.assert_close(tl_shard.router_norm.running_mean, tl_full.router_norm.running_mean, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(tl_shard.router_norm.running_var, tl_full.router_norm.running_var, rtol=1e-5, atol=1e-6)
    # --- experts sharded by id % world, all-to-all dispatch / combine
    g = torch.Generator().manual_seed(3)
    T, H, N, k = 512, 256, 4096, 8
    xs = (torch.randn(T, H, generator=g) * 0.5).to(dt).to(dev)
    down = (torch.randn(N, H, generator=g) * 0.1).to(dt).to(dev)
    up = (torch.randn(N, H, generator=g) * 0.1).to(dt).to(dev)
    p = torch.arange(1, N + 1, dtype=torch.float64).pow(-1.1)
    idx = torch.multinomial((p / p.sum()).float(), T * k, replacement=True, generator=g).view(T, k).to(dev)
    gates = torch.softmax(torch.randn(T, k, generator=g), -1).to(dt).to(dev)
    want = flash_expert_fp32(xs, down, up, idx, gates)
    s, e = token_shard(T, rank, world)
    sharded = ExpertShardedExperts(shard_expert_table(down, rank, world), shard_expert_table(up, rank, world), N)
    got = sharded.forward(xs[s:e], idx[s:e], gates[s:e])
    torch.cuda.synchronize(); check_status()
    err = (got - want[s:e]).abs().max().item() / want.abs().max().item()
    assert err < 1e-5, err
    from flash_moe_b200.parallel import choose_hot_experts
    sharded.replicate_hot_experts(choose_hot_experts(idx[s:e], N, 64))
    got = sharded.forward(xs[s:e], idx[s:e], gates[s:e])
    torch.cuda.synchronize(); check_status()
    err = max(err, (got - want[s:e]).abs().max().item() / want.abs().max().item())
    assert err < 1e-5, err
    dist.barrier(); dist.destroy_process_group()
    print("rank", rank, "ok", err, sharded.last_stats)
    """
)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_token_and_expert_sharding(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, FMOE_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29741", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("ok") == 2


PEER_WORKER = textwrap.dedent(
    """
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, os.environ["FMOE_ROOT"])
    from flash_moe_b200 import check_status
    from flash_moe_b200.parallel import PeerShardedExperts, choose_hot_experts, shard_expert_table, token_shard
    from flash_moe_b200.ops.flash_expert import flash_expert_fp32, flash_expert_func
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(3)
    T, H, N, k = 512, 256, 4099, 8            # an expert count the world size does not divide
    xs = (torch.randn(T, H, generator=g) * 0.5).to(dt).to(dev)
    down = (torch.randn(N, H, generator=g) * 0.1).to(dt).to(dev)
    up = (torch.randn(N, H, generator=g) * 0.1).to(dt).to(dev)
    idx = torch.randint(0, N, (T, k), generator=g).to(dev)
    idx[0, 0] = N - 1
    idx[1, 1] = -1                            # an empty slot
    gates = torch.softmax(torch.randn(T, k, generator=g), -1).to(dt).to(dev)
    want32 = flash_expert_fp32(xs, down, up, idx, gates)
    want16 = flash_expert_func(xs, down, up, idx, gates)
    layer = PeerShardedExperts(N, H, dt, dev)
    layer.down_shard.copy_(shard_expert_table(down, rank, world))
    layer.up_shard.copy_(shard_expert_table(up, rank, world))
    layer.publish()
    s, e = token_shard(T, rank, world)
    got32 = layer.forward(xs[s:e], idx[s:e], gates[s:e], out_dtype=torch.float32)
    got16 = layer.forward(xs[s:e], idx[s:e], gates[s:e])
    torch.cuda.synchronize(); check_status()
    assert torch.equal(got32, want32[s:e]) and torch.equal(got16, want16[s:e]), "peer-sharded result differs"
    # the most popular experts copied to every GPU: same bits, their rows no longer cross NVLink
    layer.replicate_hot_experts(choose_hot_experts(idx[s:e], N, 64))
    got16 = layer.forward(xs[s:e], idx[s:e], gates[s:e])
    torch.cuda.synchronize(); check_status()
    assert torch.equal(got16, want16[s:e]), "peer-sharded result with replicated hot experts differs"
    dist.barrier(); dist.destroy_process_group()
    print("rank", rank, "peer ok")
    """
)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_peer_memory_expert_sharding(tmp_path):
    """Tables sharded over two GPUs and read in place through peer pointers: bit-equal to the unsharded op."""
    script = tmp_path / "peer_worker.py"
    script.write_text(PEER_WORKER)
    env = dict(os.environ, FMOE_ROOT=ROOT, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29743", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("peer ok") == 2
