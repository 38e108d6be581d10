"""Multi-GPU host logic for the FlashMoE forward: one process per GPU over `torch.distributed`.

Two ways the path shards (the reference itself has no distributed code):

* **tokens** - every token's work is independent given the weights, so `[T, H]` splits into
  contiguous row blocks with replicated weights and no collective in eval mode
  (`token_shard`);
* **experts** - when the two `[N, H]` tables are too large to replicate, rank r owns the experts
  with `id % world == r` (strided, so a skewed popularity spreads over ranks) and tokens travel:
  each token row is sent ONCE to every rank that owns at least one of its experts together with
  its k (local id, gate) slots, the owner evaluates its local experts, and the partial `[H]`
  rows come back and are summed in float32 (`ExpertShardedExperts`).  The plan is built on the
  device, the only host read is the world x world matrix of row counts, and there are two payload
  exchanges (`all_to_all_single`: NCCL on GPUs, gloo in the CPU tests).  The hottest experts can be
  replicated on every rank (`choose_hot_experts`, `replicate_hot_experts`): their pairs never travel.  On the GPUs of ONE node the same
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


def choose_hot_experts(indices: torch.Tensor, num_experts: int, count: int, group=None) -> torch.Tensor:
    """The `count` most frequently selected expert ids over all ranks' `indices` (a calibration batch), ascending by
    id.  Under a skewed popularity a few hundred experts hold most pairs; copying their rows to every GPU keeps
    those pairs off the wire.  Collective: every rank of `group` calls it."""
    valid = (indices >= 0) & (indices < num_experts)
    hist = torch.bincount(indices[valid].reshape(-1), minlength=num_experts).to(torch.int64)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(hist, group=group)
    count = min(count, num_experts)
    return torch.sort(torch.topk(hist, count).indices).values


def gather_hot_rows(shard: torch.Tensor, hot_ids: torch.Tensor, rank: int, world: int, group=None) -> torch.Tensor:
    """Rows of the experts `hot_ids` (global ids) from a table sharded by id % world, assembled on every rank: each
    owner fills its rows, the rest stays zero, and a sum over the ranks puts the pieces together (exact: one
    non-zero term per element).  Collective."""
    out = torch.zeros((hot_ids.numel(), shard.shape[1]), dtype=shard.dtype, device=shard.device)
    mine = (hot_ids % world) == rank
    out[mine] = shard[(hot_ids[mine] // world)]
    if dist.is_initialized() and world > 1:
        dist.all_reduce(out, group=group)
    return out


def plan_dispatch_device(indices: torch.Tensor, num_experts: int, world: int, skip: Optional[torch.Tensor] = None):
    """Device-side half of the dispatch plan, no host synchronisation: which (token, destination) pairs exist.

    Returns `(member, dest, local, live)`: `member[t, g]` - token t has a live slot owned by rank g; `dest/local
    [T, k]` - owner and local row of every slot; `live [T, k]` - slots that travel (in range and not in `skip`,
    the mask of slots served from replicated rows)."""
    live = (indices >= 0) & (indices < num_experts)
    if skip is not None:
        live = live & ~skip
    dest = torch.where(live, indices % world, torch.zeros_like(indices))
    local = torch.where(live, indices // world, torch.zeros_like(indices))
    owners = torch.arange(world, device=indices.device).view(1, 1, world)
    member = ((dest.unsqueeze(-1) == owners) & live.unsqueeze(-1)).any(dim=1)
    return member, dest, local, live


class ExpertShardedExperts:
    """Fine-grained experts with the tables sharded over the ranks of `group` (see module docstring).

    One forward = a plan built on the device (membership matrix, one stable sort), ONE device-to-host read (the
    world x world matrix of row counts, which the exchange needs as host-side split sizes), and two payload
    exchanges: token rows out - each row packed with its k (local id, gate) slots into one buffer - and float32
    partial rows back.  `replicate_hot_experts` additionally keeps the most popular experts on every rank; their
    pairs are evaluated where the token lives and never travel.

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
        self.hot_ids = None
        self.hot_slot = None  # [num_experts] int64: position in the replicated tables, -1 for the others
        self.hot_down = self.hot_up = None
        self.last_stats = {}

    def replicate_hot_experts(self, hot_ids: torch.Tensor) -> None:
        """Keep a copy of the experts `hot_ids` (global ids, identical on every rank) on this rank.  Collective."""
        hot_ids = hot_ids.to(self.down.device, torch.int64)
        self.hot_down = gather_hot_rows(self.down, hot_ids, self.rank, self.world, self.group)
        self.hot_up = gather_hot_rows(self.up, hot_ids, self.rank, self.world, self.group)
        self.hot_slot = torch.full((self.num_experts,), -1, dtype=torch.int64, device=self.down.device)
        self.hot_slot[hot_ids] = torch.arange(hot_ids.numel(), device=self.down.device)
        self.hot_ids = hot_ids

    def forward(self, x: torch.Tensor, indices: torch.Tensor, gates: torch.Tensor) -> torch.Tensor:
        """x [T_local, H], indices [T_local, k] (global ids), gates [T_local, k] -> float32 [T_local, H]."""
        world, group, dev = self.world, self.group, x.device
        T, k = indices.shape
        H, es = x.shape[1], x.element_size()
        hot = None
        if self.hot_slot is not None:
            inside = (indices >= 0) & (indices < self.num_experts)
            hot_pos = torch.where(inside, self.hot_slot[indices.clamp(0, self.num_experts - 1)], torch.full_like(indices, -1))
            hot = hot_pos >= 0
        member, dest, local, live = plan_dispatch_device(indices, self.num_experts, world, hot)
        # what every rank tells the others: its row counts per destination and the layout of one packed row
        layout = torch.tensor([k, H, es, gates.element_size()], dtype=torch.int64, device=dev)
        counts_dev = torch.cat([member.sum(0).to(torch.int64), layout])
        gathered = [torch.empty_like(counts_dev) for _ in range(world)]
        dist.all_gather(gathered, counts_dev, group=group)
        table = torch.stack(gathered).cpu()  # the one host read of the forward
        # every rank sees the same table, so a rank whose rows would not fit the others' split sizes is refused by
        # ALL ranks here, on the host, before any payload is posted - nobody is left waiting for bytes
        odd = [r for r in range(world) if not torch.equal(table[r, world:], table[self.rank, world:])]
        if odd:
            raise ValueError(f"rank(s) {odd} announce a different row layout [k, H, bytes per value] than rank {self.rank}: "
                             f"{table[:, world:].tolist()}")
        matrix = table[:, :world]  # matrix[r][g] rows go from r to g
        counts = [int(v) for v in matrix[self.rank].tolist()]
        recv = [int(v) for v in matrix[:, self.rank].tolist()]
        sent, rows = sum(counts), sum(recv)
        # sent rows ordered by destination, then token: positions of the set bits of member^T
        flat = member.t().reshape(-1)
        order = torch.argsort(flat.logical_not(), stable=True)[:sent]
        owner, tok = order // T, order % T
        mine = (dest[tok] == owner.unsqueeze(1)) & live[tok]
        ids = torch.where(mine, local[tok], torch.full_like(local[tok], -1)).to(torch.int32)
        gts = torch.where(mine, gates[tok], torch.zeros_like(gates[tok]))
        # one packed buffer per exchange: [x row | k local ids (int32) | k gates], padded to 16 bytes
        xb, ib, gb = H * es, k * 4, k * gts.element_size()
        row_bytes = (xb + ib + gb + 15) // 16 * 16
        if xb % 4 != 0:
            raise ValueError("hidden size must make the row a multiple of 4 bytes")
        buf = torch.zeros((sent, row_bytes), dtype=torch.uint8, device=dev)
        buf[:, :xb].view(x.dtype).copy_(x[tok])
        buf[:, xb:xb + ib].view(torch.int32).copy_(ids)
        buf[:, xb + ib:xb + ib + gb].view(gts.dtype).copy_(gts)
        got = _all_to_all(buf, rows, recv, counts, group)
        if rows > 0:
            x_in = got[:, :xb].view(x.dtype).contiguous()
            ids_in = got[:, xb:xb + ib].view(torch.int32).to(torch.int64)
            gts_in = got[:, xb + ib:xb + ib + gb].view(gts.dtype).contiguous()
            partial = self.expert_fn(x_in, self.down, self.up, ids_in, gts_in).to(torch.float32)
        else:
            partial = torch.zeros((0, H), dtype=torch.float32, device=dev)
        back = _all_to_all(partial, sent, counts, recv, group)
        # slot[g, t] = position in `back` of the row rank g returned for token t (rows come back in the order sent)
        slot = torch.full((world, T), -1, dtype=torch.int32, device=dev)
        slot[owner, tok] = torch.arange(sent, dtype=torch.int32, device=dev)
        out = self.combine_fn(back, slot, T)
        if hot is not None:
            hot_ids = torch.where(hot, hot_pos, torch.full_like(hot_pos, -1))  # other slots: empty (id -1, gate 0)
            hot_gates = torch.where(hot, gates, torch.zeros_like(gates))
            out = out + self.expert_fn(x, self.hot_down, self.hot_up, hot_ids, hot_gates).to(torch.float32)
        self.last_stats = {"sent_rows": sent, "received_rows": rows, "dispatch_bytes": sent * row_bytes,
                           "combine_bytes": rows * H * 4, "collectives": "counts all-gather + 2 payload exchanges",
                           "hot_experts": 0 if self.hot_ids is None else int(self.hot_ids.numel())}
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
        self.hot_ids = None
        self.hot_slot = None
        self.hot_down = self.hot_up = None

    def replicate_hot_experts(self, hot_ids: torch.Tensor) -> None:
        """Keep a copy of the experts `hot_ids` (global ids, identical on every rank) in this GPU's own memory; the
        gather kernels then read those rows locally instead of over NVLink.  Call after `publish()`.  Collective."""
        hot_ids = hot_ids.to(self.device, torch.int64)
        self.hot_down = gather_hot_rows(self.down_shard, hot_ids, self.rank, self.world, self.group)
        self.hot_up = gather_hot_rows(self.up_shard, hot_ids, self.rank, self.world, self.group)
        self.hot_slot = torch.full((self.num_experts,), -1, dtype=torch.int64, device=self.device)
        self.hot_slot[hot_ids] = torch.arange(hot_ids.numel(), device=self.device)
        self.hot_ids = hot_ids

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
        num_hot = 0
        if self.hot_slot is not None:  # hot expert j is addressed as num_experts + j
            inside = (idx >= 0) & (idx < self.num_experts)
            pos = torch.where(inside, self.hot_slot[idx.clamp(0, self.num_experts - 1)], torch.full_like(idx, -1))
            idx = torch.where(pos >= 0, pos + self.num_experts, idx)
            num_hot = int(self.hot_ids.numel())
        out_dtype = x.dtype if out_dtype is None else out_dtype
        out = torch.empty((T, self.hidden), device=dev, dtype=out_dtype)
        L = _lib.lib()
        ws_bytes = L.fmoe_expert_workspace_bytes(T, self.hidden, self.num_experts, k)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            rc = L.fmoe_expert_forward_sharded(
                x.data_ptr(), self._ptr_arrays[0].data_ptr(), self._ptr_arrays[1].data_ptr(), self.world, idx.data_ptr(),
                g.data_ptr(), out.data_ptr(), _lib.dtype_code(x), _lib.DTYPE_CODE[out_dtype], T, self.hidden,
                self.num_experts, k, ws.data_ptr(), ws_bytes, _lib.status_word(dev).data_ptr(), _lib.current_stream_ptr(dev),
                _lib.ptr(self.hot_down), _lib.ptr(self.hot_up), num_hot)
        _lib.check(rc, "fmoe_expert_forward_sharded")
        return out
