#!/usr/bin/env python
"""Benchmark of the FlashMoE layer forward (benchmark configuration 2: the reference's quick-start shape) on 1..N B200s.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the reference's eager CPU path on the box's host cores
    python bench.py --impl reference-gpu ...  # the unmodified reference module (Triton + cuBLAS) on cuda:0

One step = one forward of the layer over one batch of synthetic tokens.  At N > 1 every rank runs the same per-GPU
batch with replicated weights (tokens sharded, no data-path collective: weak scaling).  Rank 0 prints ONE JSON line.

After the timed region (and outside it) the same run measures what explains the headline: per-stage durations and
rooflines, the gather ceiling of the expert passes, library GEMMs of the same shapes, the end-to-end path from pinned
host memory, a sustained figure over >= 2 s of replays, the other benchmark configurations (router only, experts
only, 8-layer stack) as sub-records, the reference's own GPU module, and - at N > 1, before the timed region - the
multi-GPU correctness checks.  `--quick` skips the sub-records.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import re
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "FlashMoE layer fwd tokens/s (H=1024,N=16384,k=64,bf16) + % of HBM roofline"
WORKLOAD = dict(name="config2: 1x4096 tokens, H=1024, I=4096, N=16384 (128x128 keys), k=64, bf16, eval",
                T=4096, H=1024, I=4096, N=16384, k=64, norm=False)
C3 = dict(T=16384, H=2048, nk=512, k=128)                                   # router only
C4 = dict(T=32768, H=2048, N=1 << 20, k=16)                                 # experts only, Zipf(1.1) ids
C5 = dict(layers=8, T=64 * 2048, H=2048, I=5632, N=65536, k=32, norm=True)  # residual stack
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
L2_FLUSH_BYTES = 256 << 20
REF_DIR = os.path.join(ROOT, "baseline", "_ref")

# which committed ncu summary holds the DRAM traffic of each stage's kernel(s) at this workload
PROFILE_OF_STAGE = {
    "router_front": ["router_gemm_bn_config2.md"],
    "router_topk": ["router_topk_config2.md"],
    "expert_scores": ["expert_scores_config2.md"],
    "expert_accum": ["expert_accum_config2.md"],
    "mlp_up": ["gemm_swiglu_config2.md"],
    "mlp_down": ["gemm_down_add_config2.md"],
}
KERNEL_OF_STAGE = {
    "router_front": "router_gemm_bn_kernel<128> (batch-norm applied to the x tiles in shared memory + sub-key logits, tcgen05)",
    "router_topk": "router_topk_reg_kernel<bf16, 4> (log-softmax, product-key top-k, gates)",
    "expert_scores": "expert_scores_mma_kernel<bf16, 4 x 2 buffers> (gathered down rows x token row, silu * gate)",
    "expert_accum": "expert_accum_kernel<bf16, float, 2> (gate-weighted sum of gathered up rows)",
    "mlp_up": "gemm_tcgen05_pair_kernel<SWIGLU> (shared MLP gate/up GEMM + SiLU*up epilogue, CTA pairs)",
    "mlp_down": "gemm_tcgen05_pair_kernel<ADD> (shared MLP down GEMM + fp32 expert addend, CTA pairs)",
}


# ------------------------------------------------------------------------------------------------ small helpers
def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


_UNIT = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}


def ncu_dram_bytes(stage):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the stage's kernel(s), read from the committed
    ncu summaries under profiles/ (None when a summary is missing, so a stale literal can never be reported)."""
    total = 0.0
    for name in PROFILE_OF_STAGE[stage]:
        path = os.path.join(ROOT, "profiles", name)
        if not os.path.exists(path):
            return None
        text = open(path).read()
        for key in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
            m = re.search(r"`" + re.escape(key) + r"`\)\s*\|\s*([0-9.,]+)\s*(\w+)", text)
            if not m or m.group(2) not in _UNIT:
                return None
            total += float(m.group(1).replace(",", "")) * _UNIT[m.group(2)]
    return int(total)


def bench_config(world):
    """The `config` object, identical for every arm of this benchmark."""
    return {"workload": WORKLOAD["name"], "tokens_per_gpu": WORKLOAD["T"],
            "parallelism": f"tokens sharded x{world}, weights replicated"}


class ClockSampler:
    """SM clock and throttle-reason samples (NVML, read-only queries) taken by a thread while the
    measurement runs; falls back to one nvidia-smi query when NVML is unavailable."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(physical_gpu_index(self.gpu))
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None
            return self
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                bits = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def stop(self):
        if self._nvml is None:
            return self._smi_once()
        self._stop.set()
        self._thread.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}

    def _smi_once(self):
        try:
            out = subprocess.run(
                ["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
                 "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                 "clocks_event_reasons.sw_power_cap", "--format=csv,noheader,nounits", "-i", str(self.gpu)],
                capture_output=True, text=True, timeout=10).stdout.strip().split(",")
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            reasons = [n for n, v in zip(names, out[2:6]) if v.strip().lower().startswith("active")]
            return {"sm_mhz": float(out[0]), "sm_max_mhz": float(out[1]), "reasons": reasons, "samples": 1}
        except Exception:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock query unavailable"], "samples": 0}


def physical_gpu_index(local):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v.strip() for v in vis.split(",") if v.strip()]
        if local < len(ids) and ids[local].isdigit():
            return int(ids[local])
    return local


def parse_cpulist(text):
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_to_gpu_numa_node(local):
    """Pin this process (and therefore the pinned host buffers it allocates afterwards: first touch) to the CPUs of
    the NUMA node the GPU hangs off.  Read-only sysfs / NVML queries; returns a description for the JSON line."""
    info = {"bound": False}
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(physical_gpu_index(local))
        bus = pynvml.nvmlDeviceGetPciInfo(h).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        bus = bus.lower()
        if len(bus.split(":")[0]) == 8:  # NVML prints an 8-digit domain, sysfs a 4-digit one
            bus = bus[4:]
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read().strip())
        info["gpu_pci"] = bus
        info["numa_node"] = node
        if node < 0:
            info["note"] = "the platform reports no NUMA node for this GPU"
            return info
        cpus = parse_cpulist(open(f"/sys/devices/system/node/node{node}/cpulist").read())
        allowed = os.sched_getaffinity(0)
        info["_original_affinity"] = allowed
        use = cpus & allowed
        if not use:
            info["note"] = "none of the node's CPUs is available to this process"
            return info
        os.sched_setaffinity(0, use)
        info.update(bound=True, cpus=len(use))
    except Exception as e:  # noqa: BLE001 - binding is best effort
        info["note"] = f"{type(e).__name__}: {str(e)[:120]}"
    return info


def build_inputs(dtype):
    """Seeded default init (torch.manual_seed(0)) and x ~ N(0,1) generated on the CPU."""
    from flash_moe_b200 import FlashMoE, FlashMoEConfig

    w = WORKLOAD
    torch.manual_seed(0)
    layer = FlashMoE(FlashMoEConfig(w["H"], w["I"], "silu", w["N"], w["k"], w["norm"])).to(dtype).eval()
    x = torch.randn(1, w["T"], w["H"], generator=torch.Generator().manual_seed(1)).to(dtype)
    return layer, x


def cuda_time(fn, iters, flush=None, warmup=2):
    """Mean CUDA-event duration in ms of fn() on the current stream, L2 flushed before each timed call if asked."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for i in range(iters):
        if flush is not None:
            flush.fill_(i & 0xFF)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return sum(times) / len(times)


# ------------------------------------------------------------------------------------------------ CPU reference arm
def build_cpu_reference():
    """The reference's eager CPU path at the benchmark workload, float32 (on CPU its bf16 path is slower), all host
    threads.  The reference's own `FlashMoE_Pytorch` when an install of the package sits in baseline/_ref (kind
    "reference"; its config object lacks the `mlp_bias` attribute the class reads, so that one attribute is set
    here), else the oracle's restatement of it (kind "port")."""
    w = WORKLOAD
    x = torch.randn(1, w["T"], w["H"], generator=torch.Generator().manual_seed(1))
    try:
        if not os.path.isdir(os.path.join(REF_DIR, "flash_moe")):
            raise ImportError("no reference install under baseline/_ref")
        if REF_DIR not in sys.path:
            sys.path.insert(0, REF_DIR)
        from flash_moe.modules.flash_moe import FlashMoE_Pytorch, FlashMoEConfig as RefConfig

        cfg = RefConfig(w["H"], w["I"], "silu", w["N"], w["k"], w["norm"])
        cfg.mlp_bias = False
        torch.manual_seed(0)
        return FlashMoE_Pytorch(cfg).eval(), x, "reference", "flash_moe.modules.flash_moe.FlashMoE_Pytorch from baseline/_ref"
    except Exception as e:  # noqa: BLE001 - any failure of the foreign package falls back to the port
        from oracle.flashmoe_oracle import OracleFlashMoE

        torch.manual_seed(0)
        ref = OracleFlashMoE(w["H"], w["I"], w["N"], w["k"], w["norm"]).eval()
        return ref, x, "port", f"oracle port of the reference's eager module ({type(e).__name__}: {str(e)[:80]})"


def time_cpu_reference(steps, warmup):
    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except Exception:
        pass
    torch.set_num_threads(cores)
    ref, x, kind, what = build_cpu_reference()
    with torch.no_grad():
        for _ in range(warmup):
            ref(x)
        times = []
        for _ in range(steps):
            t0 = time.perf_counter()
            ref(x)
            times.append(time.perf_counter() - t0)
    return 1e3 * sum(times) / len(times), cores, kind, what


def run_reference_arm(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    ms, cores, kind, what = time_cpu_reference(args.steps, args.warmup)
    T = WORKLOAD["T"]
    val = T / (ms / 1e3)
    sample = f"{args.steps} full forwards of {T} tokens, float32 eager on CPU, {cores} threads ({what})"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": bench_config(args.gpus),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------ reference on the GPU
def reference_gpu_record(steps, warmup):
    """The UNMODIFIED reference package (its Triton `FlashMoE` module + cuBLAS) from baseline/_ref on cuda:0 at the
    benchmark workload, timed the reference's way (synchronise, perf_counter, synchronise: tests/testing.py:189-203
    of the reference) and with CUDA events + L2 flush like this library's arm."""
    try:
        if not os.path.isdir(os.path.join(REF_DIR, "flash_moe")):
            raise RuntimeError("no reference install under baseline/_ref")
        if REF_DIR not in sys.path:
            sys.path.insert(0, REF_DIR)
        from flash_moe.modules.flash_moe import FlashMoE as RefFlashMoE, FlashMoEConfig as RefConfig

        w = WORKLOAD
        T = w["T"]
        dev = torch.device("cuda", 0)
        torch.manual_seed(0)
        ref = RefFlashMoE(RefConfig(w["H"], w["I"], "silu", w["N"], w["k"], w["norm"])).to(torch.bfloat16).to(dev).eval()
        x_host = torch.randn(1, T, w["H"], generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).pin_memory()
        y_host = torch.empty_like(x_host).pin_memory()
        x_dev = x_host.to(dev)
        flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
        with torch.no_grad():
            for _ in range(warmup):  # includes Triton's JIT and autotuning
                ref(x_dev)
            torch.cuda.synchronize()
            ms = cuda_time(lambda: ref(x_dev), steps, flush, warmup=0)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                ref(x_dev)
            torch.cuda.synchronize()
            wall_ms = 1e3 * (time.perf_counter() - t0) / steps
            t0 = time.perf_counter()
            for _ in range(steps):
                x_dev.copy_(x_host, non_blocking=True)
                y, _ = ref(x_dev)
                y_host.copy_(y, non_blocking=True)
            torch.cuda.synchronize()
            e2e_ms = 1e3 * (time.perf_counter() - t0) / steps
        return {"impl": "reference-gpu", "metric": METRIC, "value": T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
                "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": bench_config(1),
                "arm": "unmodified reference FlashMoE (Triton kernels + cuBLAS) from baseline/_ref",
                "ms_per_step_reference_convention": wall_ms,
                "timing": "ms_per_step: CUDA events, L2 flushed between steps; ms_per_step_reference_convention: "
                          "synchronise / perf_counter / synchronise around back-to-back forwards, no flush",
                "e2e": {"value": T / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": x_host.numel() * 2,
                        "d2h_bytes_per_step": y_host.numel() * 2}}
    except Exception as e:  # noqa: BLE001 - any failure of the foreign package is reported, not raised
        return {"impl": "reference-gpu", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}


def reference_gpu_subprocess(timeout_s):
    """Runs the reference-GPU arm in a child process (its JIT and autotuner stay out of this process; a limit
    guards the default run) and returns its JSON record."""
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference-gpu", "--steps", "10", "--warmup", "3"]
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s, env=env)
        for line in reversed(res.stdout.strip().splitlines()):
            if line.startswith("{"):
                return json.loads(line)
        return {"unavailable": f"no record (rc {res.returncode}): {res.stderr[-200:]}"}
    except subprocess.TimeoutExpired:
        return {"unavailable": f"did not finish within {timeout_s} s"}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}


# ------------------------------------------------------------------------------------------------ sub-records
def zipf_indices(T, k, N, seed, dev):
    """Expert ids by inverse-CDF sampling of p_r ~ r^-1.1 over r = 1..N, id = rank - 1 (hot experts have low ids)."""
    g = torch.Generator(device=dev).manual_seed(seed)
    p = torch.arange(1, N + 1, dtype=torch.float64, device=dev).pow(-1.1)
    cdf = torch.cumsum(p / p.sum(), 0)
    u = torch.rand(T, k, generator=g, dtype=torch.float64, device=dev)
    return torch.searchsorted(cdf, u).clamp_(max=N - 1)


def record_c3(dev, peaks, flush):
    """Router only (configuration 3): 16384 tokens, hidden 2048 read as two 1024-wide query halves, 512 + 512
    sub-keys (N(0, 1/32^2): each logit ~ N(0,1)), per-half log-softmax, Cartesian top-128.  In the reference's
    interface a split query is a block-diagonal router weight [2*nk, H]."""
    from flash_moe_b200.ops.flash_router import flash_router_with_gates
    from flash_moe_b200.ops.router_front import router_front

    T, H, nk, k = C3["T"], C3["H"], C3["nk"], C3["k"]
    dt = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(31)
    q = torch.randn(T, H, generator=g, device=dev).to(dt)
    keys = (torch.randn(2, nk, H // 2, generator=g, device=dev) / math.sqrt(H // 2)).to(dt)
    w = torch.zeros(2 * nk, H, dtype=dt, device=dev)
    w[:nk, : H // 2] = keys[0]
    w[nk:, H // 2:] = keys[1]
    rm, rv = torch.zeros(H, dtype=dt, device=dev), torch.ones(H, dtype=dt, device=dev)
    logits, logp = router_front(q, w, rm, rv)
    front_ms = cuda_time(lambda: router_front(q, w, rm, rv), 5, flush)
    topk_ms = cuda_time(lambda: flash_router_with_gates(logp, nk, k), 5, flush)
    ms = front_ms + topk_ms
    flops_full, flops_split = 4.0 * T * H * nk, 2.0 * T * H * nk
    hbm = 2.0 * T * H + 2.0 * 2 * nk * H + (2 + 8 + 2) * T * k  # q, weight, scores + indices + gates out
    tensor_ms = 1e3 * flops_full / (peaks["bf16_tflops"] * 1e12)
    hbm_ms = 1e3 * hbm / (peaks["hbm_gbs"] * 1e9)
    bound = max(tensor_ms, hbm_ms)
    return {"workload": "config3: router only, 16384 tokens, H=2048 (2 x 1024 query halves), 512+512 sub-keys, top-128, bf16",
            "ms": round(ms, 4), "front_ms": round(front_ms, 4), "topk_ms": round(topk_ms, 4),
            "tokens_per_s": T / (ms * 1e-3),
            "roofline": {"bound": "tensor" if tensor_ms >= hbm_ms else "hbm", "bound_ms": round(bound, 4),
                         "frac": round(bound / ms, 4), "tensor_ms_full_H": round(tensor_ms, 4),
                         "tensor_ms_split_query": round(1e3 * flops_split / (peaks["bf16_tflops"] * 1e12), 4),
                         "hbm_ms": round(hbm_ms, 4),
                         "note": "the reference's router_gate feeds the full H to both halves, so the GEMM executes the "
                                 "full-H flop count (68.7 GF); a split-query router would need half (34.4 GF)"},
            "sub_keys": "N(0, (1/32)^2)", "timing": "op-level calls (router_front, router top-k with gates), CUDA events, L2 flushed"}


def record_c4(dev, peaks, flush, world, rank):
    """Experts only (configuration 4): 32768 tokens in total, hidden 2048, 2^20 experts (2 x 4 GiB bf16 tables),
    k = 16, Zipf(1.1) ids, gates = softmax of N(0,1).  One GPU: the unsharded op.  N > 1: tables sharded by id % N,
    tokens split over the ranks, with rows read in place over NVLink (peer) and with the all-to-all exchange."""
    import torch.distributed as dist

    from flash_moe_b200.ops.flash_expert import flash_expert_func
    from flash_moe_b200.parallel import ExpertShardedExperts, PeerShardedExperts, choose_hot_experts, token_shard

    T, H, N, k = C4["T"], C4["H"], C4["N"], C4["k"]
    dt = torch.bfloat16
    s, e = token_shard(T, rank, world)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    rows = (N - rank + world - 1) // world
    down = torch.empty(rows, H, dtype=dt, device=dev).normal_(0, 0.1, generator=g)
    up = torch.empty(rows, H, dtype=dt, device=dev).normal_(0, 0.1, generator=g)
    x = (torch.randn(e - s, H, generator=g, device=dev) * 0.5).to(dt)
    idx = zipf_indices(e - s, k, N, 7 + rank, dev)
    gates = torch.softmax(torch.randn(e - s, k, generator=g, device=dev), -1).to(dt)
    distinct = int(torch.unique(idx).numel())
    rec = {"workload": "config4: experts only, 32768 tokens, H=2048, N=2^20, k=16, Zipf(1.1) ids, bf16",
           "timing": "CUDA events, L2 flushed, max over ranks"}

    def finish(ms, extra):
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
        # algorithmic HBM bytes: touched rows of both tables once, x in, y out, ids and gates
        hbm = 2.0 * 2 * distinct * H + 2.0 * 2 * (e - s) * H + (8 + 2) * (e - s) * k
        out = {"ms": round(ms, 4), "tokens_per_s": T / (ms * 1e-3)}
        out.update(extra)
        if world == 1:
            out["roofline"] = {"bound": "hbm", "bytes": hbm, "achieved_gbs": round(hbm / (ms * 1e-3) / 1e9, 1),
                               "peak_gbs": peaks["hbm_gbs"], "frac": round(hbm / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                               "distinct_experts": distinct,
                               "gathered_row_bytes": 2.0 * 2 * (e - s) * k * H,
                               "note": "the gathered rows (2 per pair) are 4.3 GB, of which the hot experts hit L2"}
        return out

    if world == 1:
        ms = cuda_time(lambda: flash_expert_func(x, down, up, idx, gates), 5, flush)
        rec["one_gpu"] = finish(ms, {})
        return rec
    # ---- peer-memory form: no exchange, remote rows read in place by the gather kernels
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    hot = choose_hot_experts(idx, N, 256)
    try:
        peer = PeerShardedExperts(N, H, dt, dev)
    except Exception as exc:  # noqa: BLE001 - no symmetric memory on this machine
        peer = None
        rec["peer_sharded"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:160]}"}
    if peer is not None:
        peer.down_shard.copy_(down)
        peer.up_shard.copy_(up)
        peer.publish()
        ms = cuda_time(lambda: peer.forward(x, idx, gates), 5, flush)

        def remote_bytes(hot_ids):
            far = (idx % world) != rank
            if hot_ids is not None:
                far = far & ~torch.isin(idx, hot_ids)
            return 2.0 * 2 * float(far.sum()) * H

        remote = remote_bytes(None)
        limiter = "NVLink: every remote row crosses it once (measured peer copy 770 GB/s per direction)"
        rec["peer_sharded"] = finish(ms, {"nvlink_bytes_per_rank": remote, "limiter": limiter,
                                          "nvlink_gbs_per_rank": round(remote / (ms * 1e-3) / 1e9, 1)})
        # the 256 most popular experts of this batch copied to every GPU: their rows no longer cross NVLink
        peer.replicate_hot_experts(hot)
        ms = cuda_time(lambda: peer.forward(x, idx, gates), 5, flush)
        remote = remote_bytes(hot)
        pairs_hot = float(torch.isin(idx, hot).float().mean())
        rec["peer_sharded_hot256"] = finish(ms, {"nvlink_bytes_per_rank": remote, "limiter": limiter,
                                                 "nvlink_gbs_per_rank": round(remote / (ms * 1e-3) / 1e9, 1),
                                                 "share_of_pairs_on_replicated_experts": round(pairs_hot, 3)})
        del peer
    # ---- all-to-all form: token rows to the owners, partial rows back
    a2a = ExpertShardedExperts(down, up, N)
    ms = cuda_time(lambda: a2a.forward(x, idx, gates), 5, flush)

    def a2a_stats():
        st = a2a.last_stats
        moved = (st.get("dispatch_bytes") or 0) + (st.get("combine_bytes") or 0)
        return {"dispatch_bytes_per_rank": st.get("dispatch_bytes"), "combine_bytes_per_rank": st.get("combine_bytes"),
                "rows_sent": st.get("sent_rows"), "rows_received": st.get("received_rows"),
                "replicated_hot_experts": st.get("hot_experts", 0), "collectives": st.get("collectives"),
                "limiter": "NVLink payload (dispatch + float32 partial rows back) plus one host read of the count matrix",
                "nvlink_bytes_per_rank": moved}

    rec["all_to_all"] = finish(ms, a2a_stats())
    a2a.replicate_hot_experts(hot)
    ms = cuda_time(lambda: a2a.forward(x, idx, gates), 5, flush)
    rec["all_to_all_hot256"] = finish(ms, a2a_stats())
    return rec


def record_c5(dev, peaks, world, rank):
    """Residual stack of 8 layers (configuration 5): 64 x 2048 tokens in total, H=2048, I=5632, N=65536, k=32,
    norm_topk_prob, eval; tokens sharded over the ranks (strong scaling), weights replicated, no collective."""
    import torch.distributed as dist

    from flash_moe_b200 import FlashMoEConfig
    from flash_moe_b200.modules.stack import FlashMoEStack
    from flash_moe_b200.parallel import token_shard

    c = C5
    cfg = FlashMoEConfig(c["H"], c["I"], "silu", c["N"], c["k"], c["norm"])
    with torch.device(dev):
        stack = FlashMoEStack(cfg, c["layers"], seeds=list(range(c["layers"]))).to(torch.bfloat16).eval()
    s, e = token_shard(c["T"], rank, world)
    x = torch.randn(1, e - s, c["H"], device=dev, generator=torch.Generator(device=dev).manual_seed(100 + rank)).to(torch.bfloat16)
    with torch.no_grad():
        ms = cuda_time(lambda: stack(x), 3, None, warmup=2)
        y, _ = stack(x)
        finite = bool(torch.isfinite(y.float()).all())
        # the same stack as a pre-norm decoder block (RMS norm in front of every layer, skip connection un-normalised):
        # one more kernel per layer, and the activations stay in range
        stack.norms = torch.nn.ParameterList([torch.nn.Parameter(torch.ones(c["H"], device=dev, dtype=torch.bfloat16))
                                              for _ in range(c["layers"])])
        ms_norm = cuda_time(lambda: stack(x), 3, None, warmup=1)
        y, _ = stack(x)
        finite_norm = bool(torch.isfinite(y.float()).all())
    t = torch.tensor([ms, ms_norm], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_norm = float(t[0]), float(t[1])
    nk = int(math.isqrt(c["N"]))
    Tl = e - s
    flops = c["layers"] * (4.0 * Tl * c["H"] * nk + 6.0 * Tl * c["H"] * c["I"])
    hbm = c["layers"] * (2.0 * 2 * Tl * c["H"] + 4.0 * Tl * nk + 4.0 * nk * c["H"] + 6.0 * c["H"] * c["I"] + 4.0 * c["N"] * c["H"])
    bound = 1e3 * (flops / (peaks["bf16_tflops_sustained"] * 1e12) + hbm / (peaks["hbm_gbs"] * 1e9))
    return {"workload": "config5: 8-layer residual stack, 64x2048 tokens in total, H=2048, I=5632, N=65536, k=32, norm_topk_prob, bf16, eval",
            "ms": round(ms, 3), "ms_per_layer": round(ms / c["layers"], 3), "tokens_per_s": c["T"] / (ms * 1e-3),
            "tokens_per_gpu": Tl, "scaling": "strong",
            "roofline": {"bound": "tensor + hbm, summed per stage", "bound_ms": round(bound, 3), "frac": round(bound / ms, 4),
                         "peaks": "sustained bf16 (the pass runs for tens of ms) and copy bandwidth"},
            "finite_output": finite,
            "pre_norm": {"ms": round(ms_norm, 3), "tokens_per_s": c["T"] / (ms_norm * 1e-3), "finite_output": finite_norm},
            "note": "with default init and no normalisation between layers this synthetic stack leaves the bf16 range after "
                    "a few layers; the work done does not depend on it",
            "timing": "CUDA events over whole passes of the stack, max over ranks"}


def sustained_record(graphed, dev, local, T, world):
    """>= 2 s of back-to-back CUDA-graph replays (no L2 flush): tokens/s with the SM clock seen meanwhile."""
    sampler = ClockSampler(local).start()
    chunk, total, n = 500, 0.0, 0
    torch.cuda.synchronize()
    t_begin = time.perf_counter()
    while time.perf_counter() - t_begin < 2.2:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(chunk):
            graphed.replay()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
        n += chunk
    clocks = sampler.stop()
    ms = total / n
    return {"seconds": round(total / 1e3, 2), "replays": n, "ms_per_step": round(ms, 4),
            "tokens_per_s_per_gpu": T / (ms * 1e-3), "clocks": clocks,
            "note": "back-to-back replays, inputs and tables stay in L2 between steps (no flush)"}


def cublas_same_shapes(dev, flush):
    """torch.matmul (cuBLAS) at the three contraction shapes of the layer, for reference beside the stage times."""
    w = WORKLOAD
    T, H, I, nk = w["T"], w["H"], w["I"], int(math.isqrt(w["N"]))
    dt = torch.bfloat16
    x = torch.randn(T, H, device=dev).to(dt)
    wg, wu = torch.randn(I, H, device=dev).to(dt), torch.randn(I, H, device=dev).to(dt)
    wd = torch.randn(H, I, device=dev).to(dt)
    wr = torch.randn(2 * nk, H, device=dev).to(dt)
    h = torch.randn(T, I, device=dev).to(dt)
    return {"mlp_up_two_gemms_no_activation": round(cuda_time(lambda: (x @ wg.t(), x @ wu.t()), 10, flush), 4),
            "mlp_down": round(cuda_time(lambda: h @ wd.t(), 10, flush), 4),
            "router": round(cuda_time(lambda: x @ wr.t(), 10, flush), 4),
            "note": "library GEMMs only: no batch-norm, activation, addend or rounding fused; L2 flushed between calls"}


def training_step_record(dev, steps=20, graph=True):
    """Backward of the expert op alone, expert forward + backward, and one full training step of the layer (forward
    + backward through autograd, eager and replayed from one CUDA graph) at the benchmark workload; CUDA-event
    means over back-to-back iterations, inputs resident on the GPU."""
    from flash_moe_b200 import FlashMoE, FlashMoEConfig, check_status
    from flash_moe_b200.ops.flash_expert import _expert_backward, flash_expert_func

    w = WORKLOAD
    T, H, I, N, k = w["T"], w["H"], w["I"], w["N"], w["k"]

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    with torch.enable_grad():
        torch.manual_seed(0)
        layer = FlashMoE(FlashMoEConfig(H, I, "silu", N, k, False)).to(torch.bfloat16).to(dev).eval()
        g = torch.Generator(device=dev).manual_seed(1)
        x = torch.randn(1, T, H, device=dev, generator=g).to(torch.bfloat16).requires_grad_()
        dy = torch.randn(1, T, H, device=dev, generator=g).to(torch.bfloat16)
        idx = torch.randint(0, N, (T, k), device=dev, generator=g)
        gates = torch.softmax(torch.randn(T, k, device=dev, generator=g), -1).to(torch.bfloat16)
        xf, do = x.detach().view(T, H), dy.view(T, H)
        down, up = layer.down_embed.weight.detach(), layer.up_embed.weight.detach()
        out = {"workload": w["name"] + ", gradients of x and every parameter", "steps": steps}
        out["expert_backward_ms"] = round(timed(lambda: _expert_backward(do, xf, down, up, idx, gates)), 4)

        def expert_step():
            leaves = [t.detach().requires_grad_() for t in (xf, down, up, gates)]
            flash_expert_func(leaves[0], leaves[1], leaves[2], idx, leaves[3]).backward(do)

        out["expert_forward_backward_ms"] = round(timed(expert_step), 4)

        def layer_step():
            for p in layer.parameters():
                p.grad = None
            x.grad = None
            y, _ = layer(x)
            y.backward(dy)

        out["layer_forward_backward_ms"] = round(timed(layer_step), 4)
        best = out["layer_forward_backward_ms"]
        if graph:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                layer_step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            for p in layer.parameters():
                p.grad = None
            x.grad = None
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cg):
                y, _ = layer(x)
                y.backward(dy)
            out["layer_forward_backward_graph_ms"] = round(timed(cg.replay), 4)
            best = min(best, out["layer_forward_backward_graph_ms"])
    check_status()
    out["tokens_per_s_training_step"] = T / (best * 1e-3)
    return out


class ParityMismatch(RuntimeError):
    """A multi-GPU path produced a result that differs from the single-GPU one."""


def multi_gpu_check(dev, rank, world):
    """Small-shape correctness checks of every multi-GPU path, run by all ranks before the timed region; raises
    ParityMismatch (or torch's AssertionError) on a mismatch.  A path that cannot be set up on this machine at all
    (e.g. no peer mappings) is reported as unavailable instead.  (NVLS is off for this process and the peer path
    uses plain peer loads.)"""
    import torch.distributed as dist

    from flash_moe_b200 import FlashMoE, FlashMoEConfig, check_status
    from flash_moe_b200.ops.flash_expert import flash_expert_fp32, flash_expert_func
    from flash_moe_b200.parallel import (ExpertShardedExperts, PeerShardedExperts, choose_hot_experts,
                                         shard_expert_table, token_shard)

    out = {}
    dt = torch.bfloat16
    # tokens sharded, weights replicated: each rank's rows equal the unsharded rows
    torch.manual_seed(0)
    layer = FlashMoE(FlashMoEConfig(256, 512, "silu", 1024, 8)).to(dt).eval().to(dev)
    Tn = 300  # every shard and the whole batch stay on the same (small-shape) kernels, so rows must match bit for bit
    x = torch.randn(1, Tn, 256, generator=torch.Generator().manual_seed(1)).to(dt).to(dev)
    s, e = token_shard(Tn, rank, world)
    with torch.no_grad():
        full, _ = layer(x)
        part, _ = layer(x[:, s:e].contiguous())
    if not torch.equal(part, full[:, s:e]):
        raise ParityMismatch("multi_gpu_check: token shard differs from the unsharded forward")
    out["token_shard_rows_equal_unsharded"] = "ok"
    # training mode: batch-norm statistics of the WHOLE batch under token sharding
    torch.manual_seed(0)
    tl_full = FlashMoE(FlashMoEConfig(256, 512, "silu", 1024, 8)).to(dev).train()
    torch.manual_seed(0)
    tl_shard = FlashMoE(FlashMoEConfig(256, 512, "silu", 1024, 8)).to(dev).train()
    xf = (torch.randn(1, Tn, 256, generator=torch.Generator().manual_seed(2)) * 1.7 + 0.4).to(dev)
    with torch.no_grad():
        _, lf = tl_full(xf)
        _, lp = tl_shard(xf[:, s:e].contiguous(), bn_sync_group=dist.group.WORLD)
    torch.testing.assert_close(lp, lf[:, s:e], rtol=2e-4, atol=2e-5)
    torch.testing.assert_close(tl_shard.router_norm.running_mean, tl_full.router_norm.running_mean, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(tl_shard.router_norm.running_var, tl_full.router_norm.running_var, rtol=1e-5, atol=1e-6)
    out["train_bn_statistics_all_reduced"] = "ok"
    # experts sharded by id % world: all-to-all form and peer-memory form against the unsharded op
    g = torch.Generator().manual_seed(3)
    T, H, N, k = 64 * world, 256, 4099, 8
    xs = (torch.randn(T, H, generator=g) * 0.5).to(dt).to(dev)
    down = (torch.randn(N, H, generator=g) * 0.1).to(dt).to(dev)
    up = (torch.randn(N, H, generator=g) * 0.1).to(dt).to(dev)
    p = torch.arange(1, N + 1, dtype=torch.float64).pow(-1.1)
    idx = torch.multinomial((p / p.sum()).float(), T * k, replacement=True, generator=g).view(T, k).to(dev)
    idx[0, 0] = N - 1
    idx[1, 1] = -1
    gates = torch.softmax(torch.randn(T, k, generator=g), -1).to(dt).to(dev)
    want32 = flash_expert_fp32(xs, down, up, idx, gates)
    want16 = flash_expert_func(xs, down, up, idx, gates)
    s, e = token_shard(T, rank, world)
    a2a = ExpertShardedExperts(shard_expert_table(down, rank, world), shard_expert_table(up, rank, world), N)
    got = a2a.forward(xs[s:e], idx[s:e], gates[s:e])
    err = (got - want32[s:e]).abs().max().item() / want32.abs().max().item()
    if not err < 1e-5:
        raise ParityMismatch(f"multi_gpu_check: all-to-all experts differ from the unsharded op ({err:.2e})")
    out["all_to_all_experts_equal_unsharded"] = "ok"
    hot = choose_hot_experts(idx[s:e], N, 32)
    a2a.replicate_hot_experts(hot)
    got = a2a.forward(xs[s:e], idx[s:e], gates[s:e])
    err = (got - want32[s:e]).abs().max().item() / want32.abs().max().item()
    if not err < 1e-5:
        raise ParityMismatch(f"multi_gpu_check: all-to-all experts with replicated hot experts differ ({err:.2e})")
    try:
        peer = PeerShardedExperts(N, H, dt, dev)
    except Exception as exc:  # noqa: BLE001 - symmetric memory not available here: nothing to check, say so
        out["peer_sharded_experts_bit_equal_unsharded"] = f"unavailable: {type(exc).__name__}: {str(exc)[:120]}"
        check_status()
        dist.barrier()
        return out
    peer.down_shard.copy_(shard_expert_table(down, rank, world))
    peer.up_shard.copy_(shard_expert_table(up, rank, world))
    peer.publish()
    got16 = peer.forward(xs[s:e], idx[s:e], gates[s:e])
    torch.cuda.synchronize(dev)
    if not torch.equal(got16, want16[s:e]):
        raise ParityMismatch("multi_gpu_check: peer-sharded experts differ from the unsharded op")
    out["peer_sharded_experts_bit_equal_unsharded"] = "ok"
    peer.replicate_hot_experts(hot)
    got16 = peer.forward(xs[s:e], idx[s:e], gates[s:e])
    torch.cuda.synchronize(dev)
    if not torch.equal(got16, want16[s:e]):
        raise ParityMismatch("multi_gpu_check: peer-sharded experts with replicated hot experts differ")
    out["hot_expert_replication_keeps_results"] = "ok"
    check_status()
    dist.barrier()
    return out


# ------------------------------------------------------------------------------------------------ main arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true", help="skip the sub-records measured after the timed region")
    ap.add_argument("--no-overlap", action="store_true", help="(default) run the shared MLP on the main stream")
    ap.add_argument("--overlap", action="store_true", help="fork the shared-MLP up GEMM to a side stream")
    ap.add_argument("--eager", action="store_true", help="time plain module calls instead of CUDA-graph replays")
    ap.add_argument("--only", default=None, choices=["training_step", "training_step_eager", "layer_forward"],
                    help="run just this piece (what the ncu summaries under profiles/ were captured on): the training "
                         "step sub-record, or three eager forwards of the benchmark layer")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.impl == "reference-gpu":
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(reference_gpu_record(args.steps, args.warmup)))
        return

    if args.only == "layer_forward":
        from flash_moe_b200 import check_status

        layer, x = build_inputs(torch.bfloat16)
        layer, x = layer.cuda(), x.cuda()
        with torch.no_grad():
            for _ in range(3):
                layer(x)
        torch.cuda.synchronize()
        check_status()
        print(json.dumps({"only": "layer_forward", "forwards": 3, "workload": WORKLOAD["name"]}))
        return
    if args.only is not None:
        torch.cuda.set_device(0)
        print(json.dumps(training_step_record(torch.device("cuda", 0), args.steps, graph=args.only == "training_step")))
        return

    import torch.distributed as dist

    from flash_moe_b200 import GraphedFlashMoE, StageTimer, check_status

    t_start = time.perf_counter()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    numa = bind_to_gpu_numa_node(local)  # before any pinned allocation
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    mgc = None
    if world > 1:
        # every rank checks every multi-GPU path on small shapes first; a mismatch ends the run with a non-zero exit
        # code, and so does a check that does not come back (the paths it guards would not either)
        stuck = threading.Timer(240.0, lambda: (sys.stderr.write("multi_gpu_check did not finish within 240 s\n"), os._exit(3)))
        stuck.daemon = True
        stuck.start()
        mgc = multi_gpu_check(dev, rank, world)
        stuck.cancel()

    dtype = torch.bfloat16
    layer, x_cpu = build_inputs(dtype)
    layer = layer.to(dev)
    layer.overlap_shared_mlp = bool(args.overlap) and not args.no_overlap
    w = WORKLOAD
    T, H, I, N, k = w["T"], w["H"], w["I"], w["N"], w["k"]
    x_host = x_cpu.pin_memory()
    x_dev = x_host.to(dev, non_blocking=True)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev)

    # ---------------- device-resident timing ----------------
    def timed_pass(steps, with_stage_events, graphed=None):
        timers = [StageTimer() for _ in range(steps)] if with_stage_events else [None] * steps
        for t in timers:
            if t is not None:
                t.c_array()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        barrier()
        t_wall = time.perf_counter()
        for i in range(steps):
            flush.fill_(i & 0xFF)  # evict L2 between timed iterations
            starts[i].record(stream)
            if graphed is not None:
                graphed.replay()
            else:
                layer(x_dev, stage_timer=timers[i])
            ends[i].record(stream)
        barrier()
        wall = 1e3 * (time.perf_counter() - t_wall)
        step = [s.elapsed_time(e) for s, e in zip(starts, ends)]
        stages = None
        if with_stage_events:
            stages = {n: sum(t.elapsed_ms()[n] for t in timers) / len(timers) for n in timers[0].elapsed_ms()}
        return sum(step) / len(step), wall, stages

    sampler = ClockSampler(local).start()
    with torch.no_grad():
        for _ in range(args.warmup):
            layer(x_dev)
        torch.cuda.synchronize()
        check_status()
        # headline: K timed steps of the layer forward, replayed from a CUDA graph captured through the
        # module's public GraphedFlashMoE wrapper (input already resident in static_input)
        graphed = None if args.eager else GraphedFlashMoE(layer, x_dev)
        if graphed is not None:
            for _ in range(args.warmup):
                graphed.replay()
        ms, wall_ms, _ = timed_pass(args.steps, False, graphed)
        clocks = sampler.stop()
        # per-stage durations (and the dominant kernel's) from a second pass with every stage on the
        # main stream, so that they are not stretched by the concurrent shared-MLP GEMM
        was = layer.overlap_shared_mlp
        layer.overlap_shared_mlp = False
        for _ in range(2):
            layer(x_dev)
        serial_ms, _, stage_ms = timed_pass(args.steps, True)
        layer.overlap_shared_mlp = was
        layer(x_dev, return_routing=True)
        distinct_experts = int(torch.unique(layer.last_indices).numel())
    # ceiling for the two expert passes while the tables sit in L2: a load-only kernel gathering the same number of
    # random rows of the same size (measured here, outside every timed region)
    from flash_moe_b200.bench_gather_roof import measure_gather_roof
    gather_roof_gbs, gather_variants = measure_gather_roof(dev, row_bytes=2 * H, rows=N, count=T * k)
    check_status()

    # ---------------- end to end: pinned host in, pinned host out, copies inside the timed region ----
    y_host = [torch.empty(1, T, H, dtype=dtype).pin_memory() for _ in range(2)]
    e2e_graphs = None if args.eager else [GraphedFlashMoE(layer, x_dev) for _ in range(2)]
    xs = [g.static_input for g in e2e_graphs] if e2e_graphs else [torch.empty_like(x_dev) for _ in range(2)]
    s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    free_x = [torch.cuda.Event() for _ in range(2)]
    got_x = [torch.cuda.Event() for _ in range(2)]
    done_y = [torch.cuda.Event() for _ in range(2)]
    read_y = [torch.cuda.Event() for _ in range(2)]

    def e2e_steps(n):
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(free_x[b])
                xs[b].copy_(x_host, non_blocking=True)
                got_x[b].record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(got_x[b])
                if e2e_graphs:
                    s_cmp.wait_event(read_y[b])  # the previous result of this graph has left the device
                    e2e_graphs[b].replay()
                    y = e2e_graphs[b].static_output
                else:
                    y, _ = layer(xs[b])
                free_x[b].record(s_cmp)
                done_y[b].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done_y[b])
                y_host[b].copy_(y, non_blocking=True)
                y.record_stream(s_out)
                read_y[b].record(s_out)

    def copies_only(n):
        """The host<->device copies of the end-to-end path with the compute removed: the host-side ceiling."""
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(s_in):
                xs[b].copy_(x_host, non_blocking=True)
            with torch.cuda.stream(s_out):
                y_host[b].copy_(xs[b].view_as(y_host[b]), non_blocking=True)

    with torch.no_grad():
        e2e_steps(args.warmup)
        barrier()
        t0 = time.perf_counter()
        e2e_steps(args.steps)
        barrier()
        e2e_ms = 1e3 * (time.perf_counter() - t0) / args.steps
        copies_only(args.warmup)
        barrier()
        t0 = time.perf_counter()
        copies_only(4 * args.steps)
        barrier()
        copy_ms = 1e3 * (time.perf_counter() - t0) / (4 * args.steps)
    check_status()

    if world > 1:
        t = torch.tensor([ms, e2e_ms, copy_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, copy_ms = float(t[0]), float(t[1]), float(t[2])

    peaks, peak_kind = load_peaks()
    h2d_bytes = x_host.numel() * x_host.element_size()
    d2h_bytes = y_host[0].numel() * y_host[0].element_size()

    original_affinity = numa.pop("_original_affinity", None)
    line = None
    extras = {}
    if rank == 0:
        # per-kernel rooflines: algorithmic flops (tensor-bound GEMMs) or algorithmic HBM bytes (the rest;
        # intermediates such as h, gs and the fp32 accumulator are not algorithmic) over the stage's
        # CUDA-event duration.  U = distinct experts the router selected in this batch.
        P, U, nk = T * k, distinct_experts, int(math.isqrt(N))
        work = {
            "router_front": ("tensor", 4.0 * T * H * nk),
            "router_topk": ("hbm", 2.0 * T * 2 * nk + 8.0 * P + 2.0 * P + 2.0 * P),
            "expert_scores": ("hbm", 2.0 * U * H + 2.0 * T * H + 8.0 * P + 2.0 * P),
            "expert_accum": ("hbm", 2.0 * U * H + 8.0 * P),
            "mlp_up": ("tensor", 2.0 * T * (2 * I) * H),
            "mlp_down": ("tensor", 2.0 * T * H * I),
        }
        kernel_rooflines = {}
        for name, (bound, amount) in work.items():
            rate = amount / (stage_ms[name] * 1e-3) / (1e12 if bound == "tensor" else 1e9)
            peak = peaks["bf16_tflops"] if bound == "tensor" else peaks["hbm_gbs"]
            kernel_rooflines[name] = {
                "kernel": KERNEL_OF_STAGE[name], "bound": bound, "achieved": round(rate, 2), "peak": peak,
                "unit": "TFLOP/s" if bound == "tensor" else "GB/s", "frac": round(rate / peak, 4),
                "traffic": ncu_dram_bytes(name), "ms": round(stage_ms[name], 4),
                "peak_source": peak_kind + (" (burst)" if bound == "tensor" else "")}
        dominant = max(stage_ms, key=lambda n: stage_ms[n])
        # the two expert passes move P*H*2 bytes of gathered table rows from L2 to the SMs, which is what
        # bounds them once the tables sit in L2; report that rate beside the HBM figure
        for name in ("expert_scores", "expert_accum"):
            rate = 2.0 * P * H / (stage_ms[name] * 1e-3) / 1e9
            kernel_rooflines[name]["l2_gather_gbs"] = round(rate, 1)
            kernel_rooflines[name]["l2_gather_roof_gbs"] = gather_roof_gbs
            kernel_rooflines[name]["l2_gather_frac"] = round(rate / gather_roof_gbs, 4)
            kernel_rooflines[name]["l2_gather_note"] = ("tables are L2-resident: P*H*2 B of gathered rows cross L2->SM per launch; "
                                                        "the roof is the best load-only variant with the same gather pattern "
                                                        "measured in this run (python -m flash_moe_b200.bench_gather_roof)")
        # whole-layer roofline: sum of the stage bounds (tensor pipe for the GEMMs, HBM for the rest)
        tensor_flops = 4.0 * T * H * nk + 6.0 * T * H * I
        hbm_bytes = 2 * T * H * 2 + 4 * T * nk + 4 * nk * H + 6 * H * I + 4 * N * H
        bound_ms = 1e3 * (tensor_flops / (peaks["bf16_tflops"] * 1e12) + hbm_bytes / (peaks["hbm_gbs"] * 1e9))
        line = {
            "metric": METRIC, "value": world * T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": bench_config(world),
            "timing": {"l2": "flushed between timed steps (256 MiB write)",
                       "overlap_shared_mlp": bool(layer.overlap_shared_mlp),
                       "launch": "eager module calls" if args.eager else "CUDA graph replay (GraphedFlashMoE)"},
            "stage_ms": dict({n: round(v, 4) for n, v in stage_ms.items()},
                             experts=round(stage_ms["expert_scores"] + stage_ms["expert_accum"], 4)),
            "stage_ms_note": "second timed pass with the shared MLP on the main stream (no overlap): "
                             f"{round(serial_ms, 4)} ms/step",
            "layer_roofline": {"bound_ms": round(bound_ms, 4), "frac": round(bound_ms / ms, 4), "peaks": peak_kind},
            "roofline": dict(kernel_rooflines[dominant], choice="the kernel with the longest measured duration"),
            "kernel_rooflines": kernel_rooflines,
            "gather_roof_variants_gbs": gather_variants,
            "distinct_experts_selected": distinct_experts,
            "e2e": {"value": world * T / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                    "h2d_gbs_per_rank": round(h2d_bytes / (e2e_ms * 1e-3) / 1e9, 2),
                    "d2h_gbs_per_rank": round(d2h_bytes / (e2e_ms * 1e-3) / 1e9, 2),
                    "copies_only_ms_per_step": round(copy_ms, 4),
                    "copies_only_note": "the same pinned-host copies with the compute removed (max over ranks): the "
                                        "host-side ceiling of the end-to-end path",
                    "host_numa_binding": numa},
            "gpu_launches": layer.kernels_per_forward() * args.steps,
            "clocks": clocks, "timed_region_wall_ms": round(wall_ms, 3),
        }
        if mgc is not None:
            line["multi_gpu_check"] = mgc

    emitted = threading.Event()

    def emit():
        """Rank 0 prints the one JSON line (once), with whatever sub-records exist by then."""
        if rank != 0 or emitted.is_set():
            return
        emitted.set()
        if extras:
            for key in ("sustained", "cublas_same_shape_ms", "reference_gpu", "training_step"):
                if key in extras:
                    line[key] = extras.pop(key)
            if extras:
                line["configs"] = dict(extras)
        line["run_seconds"] = round(time.perf_counter() - t_start, 1)
        print(json.dumps(line), flush=True)

    def give_up():
        # a sub-record that involves every rank got stuck: keep the measured line, leave without the rest
        extras.setdefault("watchdog", "a multi-GPU sub-record did not finish within its limit and was abandoned")
        emit()
        os._exit(0)

    watchdog = None
    if world > 1 and not args.quick:
        watchdog = threading.Timer(360.0, give_up)
        watchdog.daemon = True
        watchdog.start()
    # ---------------- sub-records, after (and outside) the timed regions ----------------

    def guarded(name, fn, collective=False):
        """One sub-record; a failure is recorded, not raised.  Records that involve collectives are attempted by
        every rank, the others by rank 0 alone; skipped when the run has already taken long."""
        if args.quick:
            return
        if not collective and rank != 0:
            return
        if time.perf_counter() - t_start > 420 and not collective:
            extras[name] = {"skipped": "the run had already taken more than 7 minutes"}
            return
        try:
            t0 = time.perf_counter()
            with torch.no_grad():
                rec = fn()
            if isinstance(rec, dict):
                rec["measured_in_s"] = round(time.perf_counter() - t0, 1)
            extras[name] = rec
        except Exception as e:  # noqa: BLE001
            extras[name] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
        torch.cuda.empty_cache()

    if graphed is not None:
        guarded("sustained", lambda: sustained_record(graphed, dev, local, T, world))
    guarded("cublas_same_shape_ms", lambda: cublas_same_shapes(dev, flush))
    del e2e_graphs, graphed
    guarded("training_step", lambda: training_step_record(dev))
    guarded("c3", lambda: record_c3(dev, peaks, flush))
    guarded("c4", lambda: record_c4(dev, peaks, flush, world, rank), collective=world > 1)
    guarded("c5", lambda: record_c5(dev, peaks, world, rank), collective=world > 1)
    if world == 1:
        guarded("reference_gpu", lambda: reference_gpu_subprocess(300))

    if watchdog is not None:
        watchdog.cancel()
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        if original_affinity:
            os.sched_setaffinity(0, original_affinity)  # the CPU baseline may use every host core
        cpu_steps = 3
        cpu_ms, cores, kind, what = time_cpu_reference(cpu_steps, 1)
        line["cpu_baseline"] = {
            "value": T / (cpu_ms * 1e-3), "unit": "tokens/s", "cores": cores, "kind": kind,
            "sample": f"{cpu_steps} full forwards of {T} tokens, float32 eager on CPU ({what}; CPU bf16 is slower)"}
    emit()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
