#!/usr/bin/env python
"""Benchmark of the FlashMoE layer forward (benchmark configuration 2: the reference's quick-start shape) on 1..N B200s.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the eager CPU arm on the box's host cores

One step = one forward of the layer over one batch of synthetic tokens.  At N > 1 every rank
runs the same per-GPU batch with replicated weights (tokens sharded, no data-path collective:
weak scaling).  Rank 0 prints ONE JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
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
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
L2_FLUSH_BYTES = 256 << 20
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of each kernel of the layer at this
# workload, from the ncu captures summarised in profiles/*_config2.md
NCU_DRAM_BYTES = {
    "router_front": 8404992 + 8931072,  # bn_apply + router GEMM
    "router_topk": 2168576,
    "expert_scores": 44579328 + 82944,
    "expert_accum": 36716544 + 321024,
    "mlp_up": 25196032 + 64256,
    "mlp_down": 58740224 + 1576960,
}
KERNEL_OF_STAGE = {
    "router_front": "bn_apply_kernel + gemm_tcgen05_kernel<128, ROUTER> (batch-norm, sub-key logits)",
    "router_topk": "router_topk_reg_kernel<bf16, 4> (log-softmax, product-key top-k, gates)",
    "expert_scores": "expert_scores_mma_kernel<bf16, 4 x 2 buffers> (gathered down rows x token row, silu * gate)",
    "expert_accum": "expert_accum_kernel<bf16, float, 2> (gate-weighted sum of gathered up rows)",
    "mlp_up": "gemm_tcgen05_pair_kernel<SWIGLU> (shared MLP gate/up GEMM + SiLU*up epilogue, CTA pairs)",
    "mlp_down": "gemm_tcgen05_pair_kernel<ADD> (shared MLP down GEMM + fp32 expert addend, CTA pairs)",
}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"])}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


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
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.gpu < len(ids) and ids[self.gpu].isdigit():
                return int(ids[self.gpu])
        return self.gpu

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


def build_inputs(dtype):
    """Seeded default init (torch.manual_seed(0)) and x ~ N(0,1) generated on the CPU."""
    from flash_moe_b200 import FlashMoE, FlashMoEConfig

    w = WORKLOAD
    torch.manual_seed(0)
    layer = FlashMoE(FlashMoEConfig(w["H"], w["I"], "silu", w["N"], w["k"], w["norm"])).to(dtype).eval()
    x = torch.randn(1, w["T"], w["H"], generator=torch.Generator().manual_seed(1)).to(dtype)
    return layer, x


def cpu_reference_step(ref, x32):
    with torch.no_grad():
        y, _ = ref(x32)
    return y


def build_cpu_reference():
    """The eager CPU arm: the oracle's restatement of the reference's pure-PyTorch module, float32
    (on CPU the reference's bf16 eager path is slower than its fp32 one), all host threads."""
    from oracle.flashmoe_oracle import OracleFlashMoE

    w = WORKLOAD
    torch.manual_seed(0)
    ref = OracleFlashMoE(w["H"], w["I"], w["N"], w["k"], w["norm"]).eval()
    x = torch.randn(1, w["T"], w["H"], generator=torch.Generator().manual_seed(1))
    return ref, x


def time_cpu_reference(steps, warmup):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ref, x = build_cpu_reference()
    for _ in range(warmup):
        cpu_reference_step(ref, x)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_reference_step(ref, x)
        times.append(time.perf_counter() - t0)
    ms = 1e3 * sum(times) / len(times)
    return ms, cores


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ms, cores = time_cpu_reference(args.steps, args.warmup)
    T = WORKLOAD["T"]
    val = T / (ms / 1e3)
    sample = f"{args.steps} full forwards of {T} tokens, float32 eager on CPU, {cores} threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD["name"], "arm": "oracle port of the reference's eager module on host cores"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_reference_gpu_arm(args):
    """Informational third arm: the UNMODIFIED reference package (its Triton `FlashMoE` module), when an
    install of it sits in baseline/_ref, timed on cuda:0 at the same workload with the same timing rules.
    It is not the reference arm of the bench contract (that one is the CPU path above)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    try:
        if not os.path.isdir(os.path.join(ref_dir, "flash_moe")):
            raise RuntimeError("no reference install under baseline/_ref")
        sys.path.insert(0, ref_dir)
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
            for _ in range(args.warmup):  # includes Triton's JIT and autotuning
                ref(x_dev)
            torch.cuda.synchronize()
            times = []
            for _ in range(args.steps):
                flush.fill_(1)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                ref(x_dev)
                b.record()
                torch.cuda.synchronize()
                times.append(a.elapsed_time(b))
            ms = sum(times) / len(times)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                x_dev.copy_(x_host, non_blocking=True)
                y, _ = ref(x_dev)
                y_host.copy_(y, non_blocking=True)
            torch.cuda.synchronize()
            e2e_ms = 1e3 * (time.perf_counter() - t0) / args.steps
        print(json.dumps({
            "impl": "reference-gpu", "metric": METRIC, "value": T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["name"], "arm": "unmodified reference FlashMoE (Triton kernels + cuBLAS) from baseline/_ref",
                       "l2": "flushed between timed steps (256 MiB write)"},
            "e2e": {"value": T / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": y_host.numel() * 2}}))
    except Exception as e:  # noqa: BLE001 - any failure of the foreign package is reported, not raised
        print(json.dumps({"impl": "reference-gpu", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-overlap", action="store_true", help="(default) run the shared MLP on the main stream")
    ap.add_argument("--overlap", action="store_true", help="fork the shared-MLP up GEMM to a side stream")
    ap.add_argument("--eager", action="store_true", help="time plain module calls instead of CUDA-graph replays")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.impl == "reference-gpu":
        run_reference_gpu_arm(args)
        return

    import torch.distributed as dist

    from flash_moe_b200 import GraphedFlashMoE, StageTimer, check_status

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

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

    sampler = ClockSampler(local)
    with torch.no_grad():
        sampler.start()
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
    gather_roof_gbs, _ = measure_gather_roof(dev, row_bytes=2 * H, rows=N, count=T * k)
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

    with torch.no_grad():
        e2e_steps(args.warmup)
        barrier()
        t0 = time.perf_counter()
        e2e_steps(args.steps)
        barrier()
        e2e_ms = 1e3 * (time.perf_counter() - t0) / args.steps
    check_status()
    clocks = sampler.stop()

    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])

    if rank == 0:
        peaks, peak_kind = load_peaks()
        # per-kernel rooflines: algorithmic flops (tensor-bound GEMMs) or algorithmic HBM bytes (the rest;
        # intermediates such as h, gs and the fp32 accumulator are not algorithmic) over the stage's
        # CUDA-event duration.  U = distinct experts the router selected in this batch.
        P, U, nk = T * k, distinct_experts, w_nk()
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
                "traffic": NCU_DRAM_BYTES[name], "ms": round(stage_ms[name], 4),
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
                                                        "the roof is a load-only kernel with the same gather pattern measured "
                                                        "in this run (python -m flash_moe_b200.bench_gather_roof)")
        # whole-layer roofline: sum of the stage bounds (tensor pipe for the GEMMs, HBM for the rest)
        tensor_flops = 4.0 * T * H * w_nk() + 6.0 * T * H * I
        hbm_bytes = 2 * T * H * 2 + 4 * T * w_nk() + 4 * w_nk() * H + 6 * H * I + 4 * N * H
        bound_ms = 1e3 * (tensor_flops / (peaks["bf16_tflops"] * 1e12) + hbm_bytes / (peaks["hbm_gbs"] * 1e9))
        line = {
            "metric": METRIC, "value": world * T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["name"], "tokens_per_gpu": T, "parallelism": f"tokens sharded x{world}, weights replicated",
                       "l2": "flushed between timed steps (256 MiB write)",
                       "overlap_shared_mlp": bool(layer.overlap_shared_mlp),
                       "launch": "eager module calls" if args.eager else "CUDA graph replay (GraphedFlashMoE)"},
            "stage_ms": dict({n: round(v, 4) for n, v in stage_ms.items()},
                             experts=round(stage_ms["expert_scores"] + stage_ms["expert_accum"], 4)),
            "stage_ms_note": "second timed pass with the shared MLP on the main stream (no overlap): "
                             f"{round(serial_ms, 4)} ms/step",
            "layer_roofline": {"bound_ms": round(bound_ms, 4), "frac": round(bound_ms / ms, 4), "peaks": peak_kind},
            "roofline": dict(kernel_rooflines[dominant], choice="the kernel with the longest measured duration"),
            "kernel_rooflines": kernel_rooflines,
            "distinct_experts_selected": distinct_experts,
            "e2e": {"value": world * T / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": x_host.numel() * x_host.element_size(),
                    "d2h_bytes_per_step": y_host[0].numel() * y_host[0].element_size()},
            "gpu_launches": layer.kernels_per_forward() * args.steps,
            "clocks": clocks, "timed_region_wall_ms": round(wall_ms, 3),
        }
        if world == 1 and not args.no_cpu_baseline:
            cpu_steps = 3
            cpu_ms, cores = time_cpu_reference(cpu_steps, 1)
            line["cpu_baseline"] = {
                "value": T / (cpu_ms * 1e-3), "unit": "tokens/s", "cores": cores, "kind": "port",
                "sample": f"{cpu_steps} full forwards of {T} tokens (float32 eager oracle port; CPU bf16 is slower)"}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def w_nk():
    import math
    return math.floor(math.sqrt(WORKLOAD["N"]))


if __name__ == "__main__":
    main()
