"""Build libfmoe_sm100a.so in-tree with nvcc (no torch headers, no JIT cache).

    python -m flash_moe_b200.build [--force] [--verbose]
"""

from __future__ import annotations

import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libfmoe_sm100a.so")
SOURCES = ["api.cu", "router_topk.cu", "expert.cu", "expert_fused.cu", "gemm_sm100.cu", "gemm_sm100_pair.cu", "gemm_router_bn.cu", "simt_gemm.cu", "elementwise.cu", "gather_probe.cu", "backward.cu", "noalloc.cu", "selftest.cu"]
HEADERS = ["common.cuh", "ptx_sm100.cuh", "gemm_epilogue.cuh", os.path.join("..", "..", "include", "fmoe.h")]


def _sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = _sources() + [os.path.join(CSRC, h) for h in HEADERS]
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB_PATH
    cmd = [
        nvcc_path(),
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-O3", "-std=c++17", "-lineinfo",
        "--shared", "-Xcompiler", "-fPIC",
        "--threads", "0",
        "-o", LIB_PATH + ".tmp",
    ] + _sources()
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd))
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    os.replace(LIB_PATH + ".tmp", LIB_PATH)  # readers see the old library or the new one, never a partial file
    if verbose:
        print(res.stdout + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
