"""CPU-only checks of the drop-in boundary: the library loads, exports every symbol the header
declares, and the ctypes mirror of `fmoe_layer_args` has the C layout.  No kernels are launched."""

import ctypes
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fmoe.h")


@pytest.fixture(scope="module")
def built_lib():
    from flash_moe_b200 import build

    return build.build()


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(fmoe_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol(built_lib):
    from flash_moe_b200 import _lib

    names = declared_functions()
    assert "fmoe_layer_forward" in names and "fmoe_router_topk" in names
    handle = ctypes.CDLL(built_lib)
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in include/fmoe.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature in flash_moe_b200/_lib.py"
    assert _lib.lib().fmoe_version() >= 100
    assert _lib.lib().fmoe_error_string(3) == b"workspace missing or too small"


def test_layer_args_layout_matches_c(tmp_path):
    from flash_moe_b200 import _lib

    fields = [f[0] for f in _lib.LayerArgs._fields_]
    prog = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void){",
            'printf("%zu\\n", sizeof(fmoe_layer_args));']
    prog += [f'printf("%zu\\n", offsetof(fmoe_layer_args, {f}));' for f in fields]
    prog += ["return 0;}"]
    c = tmp_path / "layout.c"
    c.write_text("\n".join(prog))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", str(c), "-o", str(exe)], check=True)
    out = [int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    assert out[0] == ctypes.sizeof(_lib.LayerArgs)
    for f, off in zip(fields, out[1:]):
        assert getattr(_lib.LayerArgs, f).offset == off, f


def test_host_side_argument_errors_need_no_gpu(built_lib):
    """Argument validation happens before any CUDA call."""
    from flash_moe_b200 import _lib

    L = _lib.lib()
    assert L.fmoe_router_topk(None, 1, 4, 16, 17, None, None, None, 0, None) == 1  # k > num_keys
    assert L.fmoe_router_topk(None, 1, 0, 16, 4, None, None, None, 0, None) == 0  # no tokens: nothing to do
    assert L.fmoe_router_topk(None, 7, 4, 16, 4, ctypes.c_void_p(16), ctypes.c_void_p(16), None, 0, None) == 1
    assert L.fmoe_expert_workspace_bytes(4096, 1024, 16384, 64) > 4 * 4096 * 64 * 4
    assert L.fmoe_layer_workspace_bytes(4096, 1024, 4096, 16384, 128, 64, 1) > 4096 * 4096 * 2
    assert L.fmoe_layer_forward(None) == 1


def test_no_cpu_path():
    import torch

    from flash_moe_b200 import FmoeError
    from flash_moe_b200.ops.flash_router import flash_router_func

    with pytest.raises(FmoeError):
        flash_router_func(torch.zeros(2, 4, 8), 8, 2)


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "flash_moe_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, f"{f} mentions the oracle"
