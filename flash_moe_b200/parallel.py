"""Multi-GPU host logic for the FlashMoE forward: one process per GPU over `torch.distributed`.

Two ways the path shards (the reference itself has no distributed code):

* **tokens** - every token's work is independent given the weights, so `[T, H]` splits into
  contiguous row blocks with replicated weights and no collective in eval mode
  (`token_shard`);
* **experts** - when the two `[N, H]` tables are too large to replicate, rank r owns the experts
  with `id % world == r` (strided, so a skewed popularity spreads over ranks) and tokens travel:
  each token row is sent ONCE to every rank that owns at least one of its experts together with
  its k (local id, gate) slots, the owner evaluates its local experts, and the partial `[H]`
  rows come back and are summed in float32 (`ExpertShardedExperts`).  Exchanges are
  `all_to_all_single` calls (NCCL on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def token_shard(num_tokens: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous row range [start, end) of rank `rank`; sizes differ by at most one row."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, extra = divmod(num_tokens, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_expert_table(table: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rows of the experts rank `rank` owns (global id = local id * world + rank)."""
    return table[rank::world].contiguous()


def plan_dispatch(indices: torch.Tensor, gates: torch.Tensor, num_experts: int, world: int):
    """Group the (token, slot) pairs by owning rank.

    Returns `(counts, token_ids, local_ids, local_gates)`: `counts[g]` tokens go to rank g;
    `token_ids` lists them destination by destination; `local_ids/local_gates [sum(counts), k]` hold,
    per sent token, its slots owned by that destination (local expert id, gate); the other slots are empty:
    id -1 (which the expert kernels skip) and gate 0.  Ids outside [0, num_experts) are dropped.
    """
    valid = (indices >= 0) & (indices < num_experts)
    dest = torch.where(valid, indices % world, torch.full_like(indices, -1))
    local = torch.where(valid, indices // world, torch.zeros_like(indices))
    tok_l, id_l, gate_l, counts = [], [], [], []
    zero_g = torch.zeros_like(gates)
    for g in range(world):
        m = dest == g
        tok = m.any(dim=1).nonzero(as_tuple=True)[0]
        counts.append(int(tok.numel()))
        tok_l.append(tok)
        id_l.append(torch.where(m, local, torch.full_like(local, -1))[tok])
        gate_l.append(torch.where(m, gates, zero_g)[tok])
    return counts, torch.cat(tok_l), torch.cat(id_l), torch.cat(gate_l)


def _all_to_all(t: torch.Tensor, recv_rows: int, out_splits: List[int], in_splits: List[int], group) -> torch.Tensor:
    out = torch.empty((recv_rows,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    dist.all_to_all_single(out, t.contiguous(), out_splits, in_splits, group=group)
    return out


class ExpertShardedExperts:
    """Fine-grained experts with the tables sharded over the ranks of `group` (see module docstring).

    `expert_fn(x, down, up, indices, gates) -> float32 [rows, H]` evaluates local experts and
    `combine_fn(rows, slot, num_tokens) -> float32 [num_tokens, H]` sums the returned partial rows
    (`slot[g, t]` = row that rank g returned for token t, -1 if none); the defaults are the CUDA ops of this
    package; CPU tests pass stand-ins with the same signatures.
    """

    def __init__(self, down_shard: torch.Tensor, up_shard: torch.Tensor, num_experts: int, group=None,
                 expert_fn: Optional[Callable] = None, combine_fn: Optional[Callable] = None):
        self.down, self.up = down_shard, up_shard
        self.num_experts = num_experts
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if expert_fn is None:
            from .ops.flash_expert import flash_expert_fp32 as expert_fn
        if combine_fn is None:
            from .ops.flash_expert import combine_partial_rows as combine_fn
        self.expert_fn = expert_fn
        self.combine_fn = combine_fn
        self.last_stats = {}

    def forward(self, x: torch.Tensor, indices: torch.Tensor, gates: torch.Tensor) -> torch.Tensor:
        """x [T_local, H], indices [T_local, k] (global ids), gates [T_local, k] -> float32 [T_local, H]."""
        world, group = self.world, self.group
        counts, tok, ids, gts = plan_dispatch(indices, gates, self.num_experts, world)
        send_counts = torch.tensor(counts, dtype=torch.int64, device=x.device)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
        recv = [int(v) for v in recv_counts.tolist()]
        rows = sum(recv)
        x_in = _all_to_all(x[tok], rows, recv, counts, group)
        ids_in = _all_to_all(ids, rows, recv, counts, group)
        gts_in = _all_to_all(gts, rows, recv, counts, group)
        if rows > 0:
            partial = self.expert_fn(x_in, self.down, self.up, ids_in, gts_in).to(torch.float32)
        else:
            partial = torch.zeros((0, x.shape[1]), dtype=torch.float32, device=x.device)
        back = _all_to_all(partial, sum(counts), counts, recv, group)
        # slot[g, t] = position in `back` of the row rank g returned for token t (rows come back in the order sent)
        sent = sum(counts)
        owner = torch.repeat_interleave(torch.arange(world, device=x.device),
                                        torch.tensor(counts, device=x.device), output_size=sent)
        slot = torch.full((world, x.shape[0]), -1, dtype=torch.int32, device=x.device)
        slot[owner, tok] = torch.arange(sent, dtype=torch.int32, device=x.device)
        out = self.combine_fn(back, slot, x.shape[0])
        self.last_stats = {"sent_rows": sum(counts), "received_rows": rows,
                           "dispatch_bytes": sum(counts) * x.shape[1] * x.element_size(),
                           "combine_bytes": rows * x.shape[1] * 4}
        return out
