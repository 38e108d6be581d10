"""The bench's reference arm runs on host cores only, so its JSON contract can be checked without a GPU."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "tokens/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["n_gpus"] == 1 and d["warmup"] >= 3 and d["gpu_launches"] == 0
    assert d["config"]["workload"].startswith("config2")
    assert set(d["cpu_baseline"]) >= {"value", "unit", "cores", "kind", "sample"}
    # the reference's own eager module when an install of it sits in baseline/_ref, else the oracle's restatement
    have_ref = os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "flash_moe"))
    assert d["cpu_baseline"]["kind"] == ("reference" if have_ref else "port"), d["cpu_baseline"]
    sys.path.insert(0, ROOT)
    import bench

    assert d["config"] == bench.bench_config(1)  # both arms print the same config object
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_other_ranks_of_the_reference_arm_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                         capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""


def test_bench_helpers():
    sys.path.insert(0, ROOT)
    import bench

    assert bench.parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert bench.bench_config(4)["parallelism"].startswith("tokens sharded x4")
    # DRAM traffic figures come from the committed ncu summaries, never from literals
    for stage in bench.PROFILE_OF_STAGE:
        v = bench.ncu_dram_bytes(stage)
        assert v is None or v > 1000
    assert bench.ncu_dram_bytes("expert_scores") > 40e6
