"""`FlashMoE` / `FlashMoEConfig` with the reference's API (flash_moe/modules/flash_moe.py:12-105),
forward running on the sm_100a kernels of libfmoe_sm100a.so.

Parameter and buffer names, shapes and construction order are the reference's, so a reference
``state_dict`` loads unchanged and a common ``torch.manual_seed`` yields identical weights.
"""

from __future__ import annotations

import ctypes
import math
import warnings
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _lib


class FlashMoEConfig:
    """Same six fields and defaults as the reference (flash_moe/modules/flash_moe.py:12-27)."""

    def __init__(
        self,
        hidden_size: int,
        intermediate_size: int,
        hidden_act: str,
        num_experts: int,
        num_experts_per_tok: int,
        norm_topk_prob: bool = False,
    ):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.hidden_act = hidden_act
        self.num_experts = num_experts
        self.num_experts_per_tok = num_experts_per_tok
        self.norm_topk_prob = norm_topk_prob


class StageTimer:
    """CUDA events recorded by the library around each stage of one layer forward."""

    def __init__(self):
        self.events = [torch.cuda.Event(enable_timing=True) for _ in range(2 * _lib.NUM_STAGES)]
        self._arr = (ctypes.c_void_p * (2 * _lib.NUM_STAGES))()
        self._bound = False

    def c_array(self):
        if not self._bound:
            # torch creates the underlying cudaEvent lazily on first record
            s = torch.cuda.current_stream()
            for e in self.events:
                e.record(s)
            for i, e in enumerate(self.events):
                self._arr[i] = e.cuda_event
            self._bound = True
        return ctypes.cast(self._arr, ctypes.POINTER(ctypes.c_void_p))

    def elapsed_ms(self) -> Dict[str, float]:
        """Call after synchronising; duration of every stage of the last timed forward."""
        return {
            name: self.events[2 * i].elapsed_time(self.events[2 * i + 1]) for i, name in enumerate(_lib.STAGE_NAMES)
        }


class FlashMoE(nn.Module):
    def __init__(self, config: FlashMoEConfig, overlap_shared_mlp: bool = False):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.intermediate_size = config.intermediate_size
        if config.hidden_act != "silu":
            # the reference builds act_fn from hidden_act but its kernels always apply SiLU
            # (flash_expert.py:8-10, flash_mlp.py:8-10); same here, but say so
            warnings.warn(f"hidden_act={config.hidden_act!r} is ignored: the FlashMoE kernels apply SiLU")
        self.hidden_act = config.hidden_act

        self.num_experts = config.num_experts
        self.num_keys = math.floor(math.sqrt(self.num_experts))
        self.top_k = config.num_experts_per_tok
        self.norm_topk_prob = config.norm_topk_prob

        # shared expert
        self.gate_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
        self.up_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
        self.down_proj = nn.Linear(self.intermediate_size, self.hidden_size, bias=False)
        # router
        self.router_gate = nn.Linear(self.hidden_size, self.num_keys * 2, bias=False)
        self.router_norm = nn.BatchNorm1d(self.hidden_size, affine=False)
        # routed experts
        self.down_embed = nn.Embedding(self.num_experts, self.hidden_size)
        self.up_embed = nn.Embedding(self.num_experts, self.hidden_size)

        self.overlap_shared_mlp = overlap_shared_mlp
        self._aux_streams: Dict[int, torch.cuda.Stream] = {}
        self._workspaces: Dict[int, torch.Tensor] = {}
        self.last_indices: Optional[torch.Tensor] = None
        self.last_gates: Optional[torch.Tensor] = None

    def _aux_stream(self, dev: torch.device) -> torch.cuda.Stream:
        key = dev.index if dev.index is not None else torch.cuda.current_device()
        if key not in self._aux_streams:
            self._aux_streams[key] = torch.cuda.Stream(device=dev)
        return self._aux_streams[key]

    def _workspace(self, dev: torch.device, nbytes: int) -> torch.Tensor:
        """Scratch memory kept by the module and reused by every forward (grown on demand).  Successive
        forwards issued from one stream are ordered by that stream; callers that drive ONE module
        instance from several streams at once must synchronise them themselves."""
        key = dev.index if dev.index is not None else torch.cuda.current_device()
        ws = self._workspaces.get(key)
        if ws is None or ws.numel() < nbytes:
            ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
            self._workspaces[key] = ws
        return ws

    def kernels_per_forward(self) -> int:
        """Kernels of this library launched by one fused forward: router GEMM (16-bit modules: the batch-norm is applied
        inside it; float32: a separate normalisation pass), top-k (with the log-softmax inside for num_keys <= 1024),
        experts (16-bit tables: scores + accumulate, or one fused kernel once a table reaches 1 GiB; float32: histogram,
        scan, scatter, scores, accumulate), MLP up GEMM, MLP down GEMM; training adds the batch statistics passes."""
        sixteen = self.down_embed.weight.element_size() == 2
        n = 1 + 1 + 1 + 1  # router GEMM, top-k, MLP up, MLP down
        if not sixteen or self.hidden_size % 8 != 0 or self.hidden_size > 3072 or (2 * self.num_keys) % 8 != 0:
            n += 1  # stand-alone normalisation pass
        if self.num_keys > 1024 or not sixteen:
            n += 1  # separate log-softmax pass
        if sixteen:
            big = self.num_experts * self.hidden_size * 2 >= (1 << 30) and self.hidden_size <= 2048
            n += 1 if big else 2
        else:
            n += 5
            if (self.num_experts + 2047) // 2048 > 16:
                n += 1  # two-level scan
        if self.training:
            n += 2  # batch statistics pass + finalize
        return n

    def _forward_differentiable(self, hidden_states, return_routing=False):
        """The layer as a chain of autograd nodes (same order of operations as the reference module)."""
        from ..ops.flash_expert import flash_expert_func
        from ..ops.flash_mlp import flash_mlp_func
        from ..ops.flash_router import flash_router_func

        bsz, seq_len, _ = hidden_states.shape
        x = hidden_states.reshape(-1, self.hidden_size)
        router_logits = self.router_gate(self.router_norm(x))
        router_logits = router_logits.view(bsz * seq_len, 2, -1).transpose(0, 1)
        log_probs = F.log_softmax(router_logits, dim=-1)
        scores, indices = flash_router_func(log_probs, self.num_keys, self.top_k)
        gates = torch.exp(scores)
        if self.norm_topk_prob:
            gates = gates / gates.sum(dim=-1, keepdim=True)
        experts = flash_expert_func(x, self.down_embed.weight, self.up_embed.weight, indices, gates)
        shared = flash_mlp_func(x, self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight)
        if return_routing:
            self.last_indices, self.last_gates = indices, gates.detach()
        return (shared + experts).view(bsz, seq_len, -1), router_logits

    def forward(
        self,
        hidden_states: torch.Tensor,
        return_routing: bool = False,
        stage_timer: Optional[StageTimer] = None,
        bn_sync_group=None,
        residual: Optional[torch.Tensor] = None,
        **kwargs,
    ) -> Tuple[torch.Tensor, torch.Tensor]:
        """(y[B,S,H], router_logits[2, B*S, num_keys]) like the reference.

        With autograd off (``torch.no_grad()`` / inference mode, or nothing that requires grad) one fused library
        call runs the whole layer.  When a graph is being recorded the layer is composed of the three
        differentiable ops with torch's batch-norm, linear and log-softmax around them, exactly like the
        reference's forward (flash_moe/modules/flash_moe.py:55-105), so ``backward()`` works.

        ``bn_sync_group``: a torch.distributed process group over which the tokens are sharded.  In
        training mode the router batch-norm then uses the statistics of the whole (global) batch: the
        ranks all-reduce 2*H float32 sums before the router GEMM.

        ``return_routing=True`` additionally keeps the selected expert ids and gates in
        ``self.last_indices`` / ``self.last_gates``.

        ``residual`` (same shape and dtype as ``hidden_states``): the skip connection of the surrounding decoder
        block.  The fused path adds it in the epilogue of the last GEMM, so ``residual + layer(x)`` is formed in
        float32 and rounded once; the differentiable path adds it as a separate autograd node.
        """
        bsz, seq_len, _ = hidden_states.shape
        dev = _lib.require_cuda(hidden_states)
        if torch.is_grad_enabled() and (hidden_states.requires_grad or any(p.requires_grad for p in self.parameters())):
            if bn_sync_group is not None or stage_timer is not None:
                raise _lib.FmoeError("bn_sync_group and stage_timer belong to the fused path: call under torch.no_grad()")
            y, router_logits = self._forward_differentiable(hidden_states, return_routing)
            return (y if residual is None else residual + y), router_logits
        x = hidden_states.reshape(-1, self.hidden_size)
        if not x.is_contiguous():
            x = x.contiguous()
        dtype = x.dtype
        w = self.gate_proj.weight
        if w.dtype != dtype or w.device != dev:
            raise _lib.FmoeError(f"module is {w.dtype} on {w.device}, input is {dtype} on {dev}")
        T = x.shape[0]
        H, I, N, nk, k = self.hidden_size, self.intermediate_size, self.num_experts, self.num_keys, self.top_k
        res = None
        if residual is not None:
            if residual.shape != hidden_states.shape or residual.dtype != dtype or residual.device != dev:
                raise _lib.FmoeError("residual must match hidden_states in shape, dtype and device")
            res = residual.reshape(-1, H)
            if not res.is_contiguous():
                res = res.contiguous()
        bn = self.router_norm
        training = bool(self.training) or bn.running_mean is None
        if training and T == 1:
            # nn.BatchNorm1d refuses a one-row training batch (its variance is undefined); so does this layer
            raise ValueError("Expected more than 1 value per channel when training, got input size " + str(list(x.shape)))
        if bn.momentum is None:
            # torch's cumulative moving average: the factor is 1 / (batches seen, this one included)
            seen = int(bn.num_batches_tracked.item()) if bn.num_batches_tracked is not None else 0
            momentum = 1.0 / float(seen + 1)
        else:
            momentum = float(bn.momentum)

        y = torch.empty((T, H), device=dev, dtype=dtype)
        logits = torch.empty((T, 2 * nk), device=dev, dtype=dtype)
        idx = torch.empty((T, k), device=dev, dtype=torch.int64) if return_routing else None
        gates = torch.empty((T, k), device=dev, dtype=dtype) if return_routing else None
        L = _lib.lib()
        code = _lib.dtype_code(x)
        ws_bytes = L.fmoe_layer_workspace_bytes(T, H, I, N, nk, k, code)
        ws = self._workspace(dev, ws_bytes)

        bn_sums, bn_count = None, 0
        if training and bn_sync_group is not None:
            import torch.distributed as dist

            bn_sums = torch.empty(2 * H, dtype=torch.float32, device=dev)
            bws_bytes = L.fmoe_bn_batch_sums_workspace_bytes(H)
            bws = torch.empty(bws_bytes, dtype=torch.uint8, device=dev)
            with torch.cuda.device(dev):
                _lib.check(L.fmoe_bn_batch_sums(x.data_ptr(), code, T, H, bn_sums.data_ptr(), bws.data_ptr(), bws_bytes,
                                                _lib.current_stream_ptr(dev)), "fmoe_bn_batch_sums")
            count = torch.tensor([float(T)], dtype=torch.float64, device=dev)
            dist.all_reduce(bn_sums, group=bn_sync_group)
            dist.all_reduce(count, group=bn_sync_group)
            bn_count = int(count.item())

        with torch.cuda.device(dev):
            main = torch.cuda.current_stream(dev)
            aux = self._aux_stream(dev) if self.overlap_shared_mlp else None
            a = _lib.LayerArgs()
            a.x = x.data_ptr()
            a.gate_proj = self.gate_proj.weight.data_ptr()
            a.up_proj = self.up_proj.weight.data_ptr()
            a.down_proj = self.down_proj.weight.data_ptr()
            a.router_gate = self.router_gate.weight.data_ptr()
            a.down_embed = self.down_embed.weight.data_ptr()
            a.up_embed = self.up_embed.weight.data_ptr()
            a.running_mean = _lib.ptr(bn.running_mean)
            a.running_var = _lib.ptr(bn.running_var)
            a.y = y.data_ptr()
            a.router_logits = logits.data_ptr()
            a.indices_out = _lib.ptr(idx)
            a.gates_out = _lib.ptr(gates)
            a.workspace = ws.data_ptr()
            a.workspace_bytes = ws_bytes
            a.status = _lib.status_word(dev).data_ptr()
            a.stream = main.cuda_stream
            a.aux_stream = aux.cuda_stream if aux is not None else None
            a.stage_events = stage_timer.c_array() if stage_timer is not None else None
            a.num_tokens, a.num_experts = T, N
            a.hidden, a.intermediate, a.num_keys, a.top_k = H, I, nk, k
            a.dtype = code
            a.training = int(training)
            a.norm_topk_prob = int(bool(self.norm_topk_prob))
            a.bn_momentum = momentum
            a.bn_eps = float(bn.eps)
            a.bn_global_sums = _lib.ptr(bn_sums)
            a.bn_global_count = bn_count
            a.residual = _lib.ptr(res)
            rc = L.fmoe_layer_forward(ctypes.byref(a))
        _lib.check(rc, "fmoe_layer_forward")
        # The side stream is joined back into the calling stream inside the library call, so the
        # input, the outputs and the workspace need no cross-stream bookkeeping afterwards.
        if training and bn.num_batches_tracked is not None and self.training:
            bn.num_batches_tracked += 1
        if return_routing:
            self.last_indices, self.last_gates = idx, gates
        router_logits = logits.view(T, 2, nk).transpose(0, 1)
        return y.view(bsz, seq_len, H), router_logits


class GraphedFlashMoE:
    """A forward captured in a CUDA graph for a fixed input shape: the kernels replay back to back without
    per-launch host work.  `module` is one `FlashMoE` layer or any eval-mode module built from such layers whose
    forward maps hidden states to ``(output, router_logits)`` - e.g. a `FlashMoEStack`, whose eight layers then
    replay as one graph.  Write the input into ``static_input`` (or pass it to ``__call__``, which copies it there),
    then read ``static_output`` / ``static_router_logits``; they are overwritten by the next replay.

    The graph has the addresses of the layers' scratch memory baked in, so it keeps those allocations alive: a later
    eager forward with more tokens makes a layer allocate a larger workspace of its own, never one the graph uses."""

    def __init__(self, module: nn.Module, example: torch.Tensor, warmup: int = 3):
        if module.training:
            raise _lib.FmoeError("capture the layer in eval mode (train mode updates host-side counters)")
        self.layer = module
        self.static_input = example.clone()
        side = torch.cuda.Stream(device=example.device)
        side.wait_stream(torch.cuda.current_stream(example.device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(warmup, 1)):  # at least one eager forward: the workspaces exist before the capture
                module(self.static_input)
        torch.cuda.current_stream(example.device).wait_stream(side)
        torch.cuda.synchronize(example.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.static_output, self.static_router_logits = module(self.static_input)
        self._workspaces = [ws for m in module.modules() if isinstance(m, FlashMoE) for ws in m._workspaces.values()]

    def replay(self) -> None:
        self.graph.replay()

    def __call__(self, hidden_states: torch.Tensor):
        self.static_input.copy_(hidden_states)
        self.graph.replay()
        return self.static_output, self.static_router_logits
