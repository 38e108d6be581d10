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
  `all_to_all_single` calls (NCCL on GPUs, gloo in the CPU tests).  On the GPUs of ONE node the same
  layout needs no exchange at all: `PeerShardedExperts` keeps the shards in symmetric memory and the
  gather kernels read the rows of the other GPUs through peer pointers over NVLink.
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


class PeerLeftError(RuntimeError):
    """Another rank of the group has announced that it left; no multi-GPU step may be launched any more."""


class StepGuard:
    """Host-side agreement that every rank is still there, checked BEFORE a multi-GPU step is launched.

    A rank leaves only between steps, with none of its kernels or collectives in flight, and says so through the
    key-value store of the process group (`leave()`); the others learn of it at their next `begin_step()` - on the
    host, before any kernel or collective of that step exists - and raise `PeerLeftError` instead of waiting for a
    peer that will never come.  A rank that dies without saying so is caught one level down, by the process group's
    timeout on its next collective (give `init_process_group` a short `timeout`).
    """

    def __init__(self, store, rank: int, world: int, prefix: str = "fmoe_step_guard"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix
        self.step = -1

    def _left_key(self, r: int) -> str:
        return f"{self.prefix}/left/{r}"

    def begin_step(self) -> int:
        gone = [r for r in range(self.world) if r != self.rank and self.store.check([self._left_key(r)])]
        if gone:
            raise PeerLeftError(f"rank(s) {gone} left the group after step {self.step}; not launching step {self.step + 1}")
        self.step += 1
        self.store.set(f"{self.prefix}/step/{self.rank}", str(self.step))
        return self.step

    def leave(self) -> None:
        """Call between steps, after synchronising this rank's device: announces that this rank is gone."""
        self.store.set(self._left_key(self.rank), str(self.step))


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
        # a split table that does not describe the payload would make the peers wait for rows that never come:
        # refuse it here, on the host, before anything is posted
        if len(counts) != world or min(counts) < 0 or sum(counts) != int(tok.numel()) or ids.shape[0] != sum(counts) \
                or gts.shape[0] != sum(counts):
            raise ValueError(f"dispatch plan is inconsistent: counts {counts} for {int(tok.numel())} token rows")
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


class PeerShardedExperts:
    """Fine-grained experts with the tables sharded by `id % world` over the GPUs of one node and read in place:
    every rank maps the other ranks' shards (torch symmetric memory, no multicast) and the two gather kernels
    address row `id // world` of shard `id % world` directly, so a token never leaves its GPU and there is no
    dispatch, no all-to-all and no host-side planning.  The result equals the unsharded op bit for bit.

    Build it collectively (every rank of `group`), fill `down_shard` / `up_shard` (views of this rank's symmetric
    buffers, `[rows_per_rank, H]`) with `shard_expert_table(table, rank, world)`, then call `publish()` once.
    """

    def __init__(self, num_experts: int, hidden: int, dtype: torch.dtype, device, group=None):
        import os

        import torch.distributed._symmetric_memory as symm_mem

        if dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("peer-sharded experts support bfloat16 and float16 tables")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer loads only
        group = dist.group.WORLD if group is None else group
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.num_experts, self.hidden, self.dtype = num_experts, hidden, dtype
        self.device = torch.device(device)
        self.rows_per_rank = (num_experts + self.world - 1) // self.world
        self.my_rows = (num_experts - self.rank + self.world - 1) // self.world
        self._buffers, self._handles, self._ptr_arrays = [], [], []
        for _ in range(2):
            buf = symm_mem.empty(self.rows_per_rank, hidden, dtype=dtype, device=self.device)
            hdl = symm_mem.rendezvous(buf, group)
            self._buffers.append(buf)
            self._handles.append(hdl)
            self._ptr_arrays.append(torch.tensor([int(p) for p in hdl.buffer_ptrs], dtype=torch.int64, device=self.device))
        self.down_shard = self._buffers[0][: self.my_rows]
        self.up_shard = self._buffers[1][: self.my_rows]

    def publish(self) -> None:
        """Make this rank's shard contents visible to the others: finish the copies, then meet at a barrier."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def forward(self, x: torch.Tensor, indices: torch.Tensor, gates: torch.Tensor, out_dtype=None) -> torch.Tensor:
        """x [T_local, H], indices [T_local, k] (global ids), gates [T_local, k] -> [T_local, H] (x.dtype or float32)."""
        from . import _lib

        dev = _lib.require_cuda(x, indices, gates)
        x, idx, g = x.contiguous(), indices.contiguous().to(torch.int64), gates.contiguous().to(x.dtype)
        if x.dtype != self.dtype or x.shape[1] != self.hidden:
            raise _lib.FmoeError("x must match the tables' dtype and hidden size")
        T, k = idx.shape
        out_dtype = x.dtype if out_dtype is None else out_dtype
        out = torch.empty((T, self.hidden), device=dev, dtype=out_dtype)
        L = _lib.lib()
        ws_bytes = L.fmoe_expert_workspace_bytes(T, self.hidden, self.num_experts, k)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            rc = L.fmoe_expert_forward_sharded(
                x.data_ptr(), self._ptr_arrays[0].data_ptr(), self._ptr_arrays[1].data_ptr(), self.world, idx.data_ptr(),
                g.data_ptr(), out.data_ptr(), _lib.dtype_code(x), _lib.DTYPE_CODE[out_dtype], T, self.hidden,
                self.num_experts, k, ws.data_ptr(), ws_bytes, _lib.status_word(dev).data_ptr(), _lib.current_stream_ptr(dev))
        _lib.check(rc, "fmoe_expert_forward_sharded")
        return out
