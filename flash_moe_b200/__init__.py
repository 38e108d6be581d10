"""flash_moe_b200: the hot path of the FlashMoE layer (fused forward, backward of its three ops) on NVIDIA B200 (sm_100a).

Python host code over a C-ABI shared library of hand-written CUDA kernels
(`libfmoe_sm100a.so`, declared in `include/fmoe.h`).  Mirrors the reference's
public interface: `FlashMoE` / `FlashMoEConfig` and the three op entry points.
"""

from ._lib import FmoeError, check_status, read_status  # noqa: F401
from .modules.flash_moe import FlashMoE, FlashMoEConfig, GraphedFlashMoE, StageTimer  # noqa: F401
from .ops.flash_expert import flash_expert_func, triton_flash_expert_func  # noqa: F401
from .ops.flash_mlp import flash_mlp_func, triton_flash_mlp_func  # noqa: F401
from .ops.flash_router import flash_router_func, triton_flash_router_func  # noqa: F401
from .ops.peer import peer_func, triton_peer_func  # noqa: F401
from .ops.pkm import pkm_func, triton_pkm_func  # noqa: F401

__version__ = "0.1.0"
