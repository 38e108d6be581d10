"""Host-side multi-GPU logic on CPU: token sharding arithmetic and the expert-sharded
dispatch/combine run as two gloo ranks with the oracle standing in for the CUDA expert op."""

import os
import subprocess
import sys
import textwrap

import pytest
import torch

from flash_moe_b200.parallel import plan_dispatch, shard_expert_table, token_shard

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


def test_plan_dispatch_sends_each_token_once_per_owner():
    g = torch.Generator().manual_seed(0)
    T, k, N, world = 50, 6, 40, 4
    idx = torch.randint(0, N, (T, k), generator=g)
    idx[3, 2] = -1
    idx[4, 0] = N  # out of range: dropped
    gates = torch.rand(T, k, generator=g)
    counts, tok, ids, gts = plan_dispatch(idx, gates, N, world)
    assert sum(counts) == tok.numel() == ids.shape[0] == gts.shape[0]
    off = 0
    total_pairs = 0
    for dest, c in enumerate(counts):
        t = tok[off : off + c]
        assert t.unique().numel() == c  # one row per (token, destination)
        for row, token in enumerate(t.tolist()):
            mine = [(int(e) // world, float(w)) for e, w in zip(idx[token], gates[token]) if 0 <= e < N and e % world == dest]
            got = [(int(e), float(w)) for e, w in zip(ids[off + row], gts[off + row]) if w != 0]
            assert sorted(mine) == sorted(got)
            # the other slots are empty: id -1, gate 0
            assert {int(e) for e in ids[off + row]} - {-1} == {e for e, _ in mine}
            assert all(float(w) == 0 for e, w in zip(ids[off + row], gts[off + row]) if int(e) == -1)
            total_pairs += len(mine)
        off += c
    assert total_pairs == int(((idx >= 0) & (idx < N)).sum())
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
        if rank == 1:
            real = P.plan_dispatch
            def broken(*a, **kw):  # announces one row more than it holds
                counts, tok, ids, gts = real(*a, **kw)
                counts[0] += 1
                return counts, tok, ids, gts
            P.plan_dispatch = broken
        t0 = time.time()
        try:
            guard.begin_step()
            layer.forward(x[s:e], idx[s:e], gates[s:e])
            print("rank", rank, "UNEXPECTED success")
        except ValueError as err:
            print("rank", rank, "refused its own plan:", str(err)[:60])
        except Exception as err:  # the healthy rank: its collective ends with an error after the group's timeout
            print("rank", rank, "collective failed after %.0f s: %s" % (time.time() - t0, type(err).__name__))
        os._exit(0)
    if mode == "rank_leaves":
        if rank == 1:
            guard.leave()  # between steps, nothing in flight
            print("rank", rank, "left")
            os._exit(0)
        store.wait([guard._left_key(1)], datetime.timedelta(seconds=8))
        try:
            guard.begin_step()
            print("rank", rank, "UNEXPECTED launch")
        except P.PeerLeftError as err:
            print("rank", rank, "did not launch:", str(err)[:50])
        os._exit(0)
    """
)


@pytest.mark.parametrize("mode", ["bad_split_table", "rank_leaves"])
def test_failures_are_reported_on_the_host_instead_of_waited_for(tmp_path, mode):
    """Two gloo ranks: (a) a rank whose split table does not describe its payload refuses to post it, and the
    healthy rank's collective ends with an error after the group's short timeout instead of blocking for ever;
    (b) a rank that leaves between steps is noticed by the other on the host, before it launches the next step."""
    script = tmp_path / "failure_worker.py"
    script.write_text(FAILURE_WORKER)
    env = dict(os.environ, FMOE_ROOT=ROOT, OMP_NUM_THREADS="1", FMOE_FAILURE=mode)
    port = "29735" if mode == "bad_split_table" else "29737"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", port, str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    out = res.stdout + res.stderr
    assert "UNEXPECTED" not in out, out[-3000:]
    if mode == "bad_split_table":
        assert "rank 1 refused its own plan" in out, out[-3000:]
        assert "rank 0 collective failed" in out, out[-3000:]
    else:
        assert "rank 1 left" in out and "rank 0 did not launch" in out, out[-3000:]
