"""The rate at which one GPU can gather random table rows into its SMs (load-only probe, fmoe_gather_probe):

    python -m flash_moe_b200.bench_gather_roof [--row-bytes 2048] [--rows 16384] [--count 262144]

Defaults are the benchmark shape of the expert passes: 262144 (token, expert) pairs, one 2 KB row each from a
16384-row (32 MB, L2-resident) table.  Prints one JSON line with the rate per grid size and the best one.
"""

from __future__ import annotations

import argparse
import json

import torch

from . import _lib


def measure_gather_roof(device, row_bytes: int = 2048, rows: int = 16384, count: int = 262144, reps: int = 5):
    """Best gathered-row rate in GB/s over the probe's variants, and the per-variant results: register loads at a
    few grid sizes, bulk copies and 16-byte cp.async copies into a shared-memory ring (the latter is how the fused expert
    kernel fetches its rows)."""
    dev = torch.device(device)
    table = torch.ones(rows * row_bytes, dtype=torch.uint8, device=dev)
    ids = torch.randint(0, rows, (count,), device=dev, dtype=torch.int32, generator=torch.Generator(device=dev).manual_seed(1))
    sink = torch.zeros(1, dtype=torch.float32, device=dev)
    L = _lib.lib()
    results = {}
    with torch.cuda.device(dev):
        stream = _lib.current_stream_ptr(dev)
        status = _lib.status_word(dev).data_ptr()
        for name, ctas, mode in (("4_ctas_per_sm", 4, 0), ("8_ctas_per_sm", 8, 0), ("12_ctas_per_sm", 12, 0),
                                 ("16_ctas_per_sm", 16, 0), ("bulk_ring", 1, 1), ("cp_async_ring", 1, 2)):
            best = None
            for _ in range(reps):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                rc = L.fmoe_gather_probe(table.data_ptr(), rows, ids.data_ptr(), count, row_bytes, ctas, mode,
                                         sink.data_ptr(), status, stream)
                if rc == _lib.ERR_UNSUPPORTED:  # this row size does not fit this variant's ring
                    break
                _lib.check(rc, "fmoe_gather_probe")
                b.record()
                torch.cuda.synchronize(dev)
                ms = a.elapsed_time(b)
                best = ms if best is None else min(best, ms)
            if best is not None:
                results[name] = round(count * row_bytes / (best * 1e-3) / 1e9, 1)
    return max(results.values()), results


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--row-bytes", type=int, default=2048)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--count", type=int, default=262144)
    args = ap.parse_args()
    best, per_grid = measure_gather_roof("cuda:0", args.row_bytes, args.rows, args.count)
    print(json.dumps({"metric": "gathered rows into the SMs", "unit": "GB/s", "best": best, "per_grid": per_grid,
                      "config": {"row_bytes": args.row_bytes, "table_rows": args.rows, "rows_gathered": args.count}}))


if __name__ == "__main__":
    main()
