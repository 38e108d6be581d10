"""Host-side multi-GPU logic on CPU: token sharding arithmetic and the expert-sharded
dispatch/combine run as two gloo ranks with the oracle standing in for the CUDA expert op."""

import os
import subprocess
import sys
import textwrap

import pytest
import torch

from flash_moe_b200.parallel import plan_dispatch_device, shard_expert_table, token_shard

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_token_shard_covers_all_rows_once():
    for T in (0, 1, 7, 4096, 4097):
        for world in (1, 2, 3, 8):
            spans = [token_shard(T, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == T
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - s for s, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        token_shard(10, 2, 2)


def test_device_plan_marks_each_token_once_per_owner():
    g = torch.Generator().manual_seed(0)
    T, k, N, world = 50, 6, 40, 4
    idx = torch.randint(0, N, (T, k), generator=g)
    idx[3, 2] = -1
    idx[4, 0] = N  # out of range: dropped
    skip = torch.zeros(T, k, dtype=torch.bool)
    skip[5, 1] = True  # a slot served from replicated rows does not travel
    member, dest, local, live = plan_dispatch_device(idx, N, world, skip)
    assert member.shape == (T, world) and not live[3, 2] and not live[4, 0] and not live[5, 1]
    for t in range(T):
        owners = {int(e) % world for j, e in enumerate(idx[t]) if 0 <= e < N and not skip[t, j]}
        assert {g_ for g_ in range(world) if member[t, g_]} == owners
        for j in range(k):
            if live[t, j]:
                assert int(dest[t, j]) == int(idx[t, j]) % world and int(local[t, j]) == int(idx[t, j]) // world
    assert int(live.sum()) == int(((idx >= 0) & (idx < N)).sum()) - 1
    table = torch.arange(N).unsqueeze(1).float()
    assert torch.equal(shard_expert_table(table, 1, world)[:, 0], torch.arange(1, N, world).float())


WORKER = textwrap.dedent(
    """
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, os.environ["FMOE_ROOT"])
    from flash_moe_b200.parallel import ExpertShardedExperts, shard_expert_table, token_shard
    from oracle import flashmoe_oracle as O
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    g = torch.Generator().manual_seed(5)
    T, H, N, k = 37, 32, 64, 5
    x = torch.randn(T, H, generator=g)
    down = torch.randn(N, H, generator=g) * 0.3
    up = torch.randn(N, H, generator=g) * 0.3
    p = torch.arange(1, N + 1, dtype=torch.float64).pow(-1.1)
    idx = torch.multinomial((p / p.sum()).float(), T * k, replacement=True, generator=g).view(T, k)
    gates = torch.softmax(torch.randn(T, k, generator=g), -1)
    want = O.expert_forward(x, down, up, idx, gates)
    s, e = token_shard(T, rank, world)

    def combine(rows, slot, ntok):  # CPU stand-in of combine_partial_rows
        out = torch.zeros(ntok, rows.shape[1])
        for g_ in range(slot.shape[0]):
            m = slot[g_] >= 0
            out[m] += rows[slot[g_][m].long()]
        return out

    layer = ExpertShardedExperts(shard_expert_table(down, rank, world), shard_expert_table(up, rank, world), N,
                                 expert_fn=O.expert_forward, combine_fn=combine)
    got = layer.forward(x[s:e], idx[s:e], gates[s:e])
    err = (got - want[s:e]).abs().max().item()
    assert err < 1e-5, err
    assert layer.last_stats["sent_rows"] <= (e - s) * min(k, world)
    sent_before = layer.last_stats["sent_rows"]
    # the hottest experts replicated on every rank: same result, fewer rows on the wire
    from flash_moe_b200.parallel import choose_hot_experts
    hot = choose_hot_experts(idx[s:e], N, 8)
    assert hot.numel() == 8 and 0 in hot.tolist()  # Zipf: id 0 is the most popular expert
    layer.replicate_hot_experts(hot)
    got = layer.forward(x[s:e], idx[s:e], gates[s:e])
    err = max(err, (got - want[s:e]).abs().max().item())
    assert err < 1e-5, err
    assert layer.last_stats["sent_rows"] <= sent_before and layer.last_stats["hot_experts"] == 8
    dist.barrier()
    dist.destroy_process_group()
    print("rank", rank, "ok", err)
    """
)


def test_expert_sharded_dispatch_combine_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, FMOE_ROOT=ROOT, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29733", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert res.stdout.count("ok") == 2


FAILURE_WORKER = textwrap.dedent(
    """
    import datetime, os, sys, time, torch, torch.distributed as dist
    sys.path.insert(0, os.environ["FMOE_ROOT"])
    import flash_moe_b200.parallel as P
    from oracle import flashmoe_oracle as O
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=8))
    rank, world = dist.get_rank(), dist.get_world_size()
    store = dist.distributed_c10d._get_default_store()
    mode = os.environ["FMOE_FAILURE"]

    def say(*parts):  # one write per line, so the two ranks' lines cannot interleave
        os.write(1, (" ".join(str(p_) for p_ in parts) + "\\n").encode())

    g = torch.Generator().manual_seed(5)
    T, H, N, k = 16, 8, 32, 3
    x = torch.randn(T, H, generator=g)
    down, up = torch.randn(N, H, generator=g), torch.randn(N, H, generator=g)
    idx = torch.randint(0, N, (T, k), generator=g)
    gates = torch.softmax(torch.randn(T, k, generator=g), -1)
    s, e = P.token_shard(T, rank, world)

    def combine(rows, slot, ntok):
        out = torch.zeros(ntok, rows.shape[1])
        for g_ in range(slot.shape[0]):
            m = slot[g_] >= 0
            out[m] += rows[slot[g_][m].long()]
        return out

    layer = P.ExpertShardedExperts(P.shard_expert_table(down, rank, world), P.shard_expert_table(up, rank, world), N,
                                   expert_fn=O.expert_forward, combine_fn=combine)
    guard = P.StepGuard(store, rank, world)
    guard.begin_step()
    layer.forward(x[s:e], idx[s:e], gates[s:e])  # step 0 works on every rank
    dist.barrier()
    if mode == "bad_split_table":
        # rank 1 comes with rows of another layout (fewer slots per token): every rank sees it in the gathered
        # table and refuses on the host; no payload is posted, nobody waits
        kk = k - 1 if rank == 1 else k
        try:
            guard.begin_step()
            layer.forward(x[s:e], idx[s:e, :kk], gates[s:e, :kk])
            say("rank", rank, "UNEXPECTED success")
        except ValueError as err:
            say("rank", rank, "refused the exchange:", str(err)[:40])
        os._exit(0)
    if mode == "rank_dies":
        # rank 1 dies without a word before the step's first collective: the short timeout of the process group
        # ends rank 0's collective with an error instead of blocking it for ever
        if rank == 1:
            os._exit(0)
        t0 = time.time()
        try:
            layer.forward(x[s:e], idx[s:e], gates[s:e])
            say("rank", rank, "UNEXPECTED success")
        except Exception as err:
            say("rank", rank, "collective failed after %.0f s: %s" % (time.time() - t0, type(err).__name__))
        os._exit(0)
    if mode == "rank_leaves":
        if rank == 1:
            guard.leave()  # between steps, nothing in flight
            say("rank", rank, "left")
            os._exit(0)
        store.wait([guard._left_key(1)], datetime.timedelta(seconds=8))
        try:
            guard.begin_step()
            say("rank", rank, "UNEXPECTED launch")
        except P.PeerLeftError as err:
            say("rank", rank, "did not launch:", str(err)[:50])
        os._exit(0)
    """
)


@pytest.mark.parametrize("mode", ["bad_split_table", "rank_dies", "rank_leaves"])
def test_failures_are_reported_on_the_host_instead_of_waited_for(tmp_path, mode):
    """Two gloo ranks: (a) a rank that announces rows of another layout is refused by every rank on the host, before
    any payload is posted; (b) a rank that dies silently makes the other's collective end with an error after the
    group's short timeout instead of blocking for ever; (c) a rank that leaves between steps is noticed by the other
    on the host, before it launches the next step."""
    script = tmp_path / "failure_worker.py"
    script.write_text(FAILURE_WORKER)
    env = dict(os.environ, FMOE_ROOT=ROOT, OMP_NUM_THREADS="1", FMOE_FAILURE=mode)
    port = {"bad_split_table": "29735", "rank_dies": "29736", "rank_leaves": "29737"}[mode]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", port, str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    out = res.stdout + res.stderr
    assert "UNEXPECTED" not in out, out[-3000:]
    if mode == "bad_split_table":
        assert "rank 0 refused the exchange" in out and "rank 1 refused the exchange" in out, out[-3000:]
    elif mode == "rank_dies":
        assert "rank 0 collective failed" in out, out[-3000:]
    else:
        assert "rank 1 left" in out and "rank 0 did not launch" in out, out[-3000:]
