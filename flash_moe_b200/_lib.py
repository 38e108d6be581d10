"""ctypes binding of libfmoe_sm100a.so (the C ABI declared in include/fmoe.h).

There is no CPU path and no other backend: importing this module without the built
library, or calling an op with CPU tensors, raises.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libfmoe_sm100a.so")

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
NUM_STAGES = 6
STAGE_NAMES = ("router_front", "router_topk", "expert_scores", "expert_accum", "mlp_up", "mlp_down")

ERR_UNSUPPORTED = 2  # fmoe_error: a shape/dtype combination no kernel covers
STATUS_BAD_EXPERT_ID = 1
STATUS_WAIT_TIMEOUT = 2
STATUS_BAD_ROW_INDEX = 4


class FmoeError(RuntimeError):
    pass


class LayerArgs(ctypes.Structure):
    _fields_ = [
        ("x", ctypes.c_void_p),
        ("gate_proj", ctypes.c_void_p),
        ("up_proj", ctypes.c_void_p),
        ("down_proj", ctypes.c_void_p),
        ("router_gate", ctypes.c_void_p),
        ("down_embed", ctypes.c_void_p),
        ("up_embed", ctypes.c_void_p),
        ("running_mean", ctypes.c_void_p),
        ("running_var", ctypes.c_void_p),
        ("y", ctypes.c_void_p),
        ("router_logits", ctypes.c_void_p),
        ("indices_out", ctypes.c_void_p),
        ("gates_out", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("status", ctypes.c_void_p),
        ("stream", ctypes.c_void_p),
        ("aux_stream", ctypes.c_void_p),
        ("stage_events", ctypes.POINTER(ctypes.c_void_p)),
        ("num_tokens", ctypes.c_int64),
        ("num_experts", ctypes.c_int64),
        ("hidden", ctypes.c_int32),
        ("intermediate", ctypes.c_int32),
        ("num_keys", ctypes.c_int32),
        ("top_k", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
        ("training", ctypes.c_int32),
        ("norm_topk_prob", ctypes.c_int32),
        ("bn_momentum", ctypes.c_float),
        ("bn_eps", ctypes.c_float),
        ("bn_global_sums", ctypes.c_void_p),
        ("bn_global_count", ctypes.c_int64),
        ("residual", ctypes.c_void_p),
    ]


_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_int64
_Z = ctypes.c_size_t
_F = ctypes.c_float

# name -> (restype, argtypes); every symbol include/fmoe.h declares
SIGNATURES = {
    "fmoe_version": (_I, []),
    "fmoe_error_string": (ctypes.c_char_p, [_I]),
    "fmoe_router_topk": (_I, [_P, _I, _L, _I, _I, _P, _P, _P, _I, _P]),
    "fmoe_router_front_workspace_bytes": (_Z, [_L, _I, _I, _I]),
    "fmoe_router_front": (_I, [_P, _P, _P, _P, _I, _F, _F, _P, _P, _I, _L, _I, _I, _P, _Z, _P, _P]),
    "fmoe_bn_batch_sums_workspace_bytes": (_Z, [_I]),
    "fmoe_bn_batch_sums": (_I, [_P, _I, _L, _I, _P, _P, _Z, _P]),
    "fmoe_expert_forward_sharded": (_I, [_P, _P, _P, _I, _P, _P, _P, _I, _I, _L, _I, _L, _I, _P, _Z, _P, _P, _P, _P, _L]),
    "fmoe_peer_forward": (_I, [_P, _P, _P, _P, _P, _P, _I, _L, _I, _L, _I, _P, _Z, _P, _P]),
    "fmoe_pkm_workspace_bytes": (_Z, [_L, _I]),
    "fmoe_pkm_forward": (_I, [_P, _P, _P, _P, _I, _L, _I, _L, _I, _P, _Z, _P, _P]),
    "fmoe_mlp_forward_saving_preacts": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _L, _I, _I, _P, _Z, _P, _P]),
    "fmoe_router_topk_backward": (_I, [_P, _P, _I, _L, _I, _I, _P, _P]),
    "fmoe_expert_backward_workspace_bytes": (_Z, [_L, _I, _L, _I]),
    "fmoe_expert_forward_saving_scores": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _L, _I, _L, _I, _P, _Z, _P, _P]),
    "fmoe_expert_backward": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _L, _I, _L, _I, _P, _Z, _P, _P]),
    "fmoe_swiglu_backward": (_I, [_P, _P, _P, _P, _P, _P, _I, _L, _P]),
    "fmoe_gather_probe": (_I, [_P, _L, _P, _L, _I, _I, _I, _P, _P, _P]),
    "fmoe_rms_norm": (_I, [_P, _P, _P, _I, _L, _I, _F, _P]),
    "fmoe_selftest_wait_timeout": (_I, [ctypes.c_uint64, _P, _P, _P]),
    "fmoe_combine_partial_rows": (_I, [_P, _L, _P, _I, _L, _I, _P, _P, _P]),
    "fmoe_expert_workspace_bytes": (_Z, [_L, _I, _L, _I]),
    "fmoe_expert_forward": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _L, _I, _L, _I, _P, _Z, _P, _P]),
    "fmoe_expert_static_scratch_bytes": (_Z, []),
    "fmoe_expert_forward_static": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _L, _I, _L, _I, _P, _P]),
    "fmoe_mlp_workspace_bytes": (_Z, [_L, _I, _I, _I]),
    "fmoe_mlp_forward": (_I, [_P, _P, _P, _P, _P, _P, _I, _L, _I, _I, _P, _Z, _P, _P]),
    "fmoe_layer_workspace_bytes": (_Z, [_L, _I, _I, _L, _I, _I, _I]),
    "fmoe_layer_forward": (_I, [ctypes.POINTER(LayerArgs)]),
}

_lib: Optional[ctypes.CDLL] = None


def lib() -> ctypes.CDLL:
    """Load the shared library once; raise loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FmoeError(
                f"{LIB_PATH} is missing: build it with `python -m flash_moe_b200.build` "
                "(flash_moe_b200 has no fallback path)"
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().fmoe_error_string(rc).decode()
        raise FmoeError(f"{what} failed: {msg} (code {rc})")


def dtype_code(t: torch.Tensor) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise FmoeError(f"unsupported dtype {t.dtype}; supported: float32, bfloat16, float16") from None


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise FmoeError("flash_moe_b200 runs on CUDA tensors only (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise FmoeError(f"tensors on different devices: {dev} and {t.device}")
    return dev


def current_stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# one int32 status word per device; kernels OR error bits into it
_status = {}


def status_word(device: torch.device) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def read_status(device=None, clear: bool = True) -> int:
    """Synchronising read of the device status word (FMOE_STATUS_* bits)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = status_word(device)
    v = int(w.item())
    if clear and v:
        w.zero_()
    return v


def check_status(device=None) -> None:
    v = read_status(device)
    if v & STATUS_WAIT_TIMEOUT:
        raise FmoeError("a device-side wait timed out inside a flash_moe_b200 kernel")
    if v & STATUS_BAD_EXPERT_ID:
        raise FmoeError("expert index outside [0, num_experts) was skipped")
    if v & STATUS_BAD_ROW_INDEX:
        raise FmoeError("combine_partial_rows skipped a slot that points past the received rows")
