"""bench.py's reference arm runs on the host cores only, so its JSON contract is checked here
without a GPU (the GPU arm's line is produced by the same code path and checked on the box)."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_one_contract_line():
    env = dict(os.environ, OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--scale", "0.004",
                        "--steps", "2", "--warmup", "1"], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, r.stdout
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    assert line["metric"] == "spmm_gflops_warm" and line["unit"].startswith("GFLOP/s")
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["steps"] == 2
    assert line["value"] > 0 and line["ms_per_step"] > 0
    assert line["config"]["workload"].startswith("C4")
    cb = line["cpu_baseline"]
    assert cb["kind"] == "reference" and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0
    assert line["vs_baseline"] is None


import pytest  # noqa: E402


@pytest.mark.gpu
def test_gpu_arm_prints_one_contract_line_at_test_size():
    """The GPU arm end to end at 2^-7 of configuration 4: one JSON line with the roofline, CPU
    baseline, end-to-end, clock, launch-count and parity keys, and a parity check that holds."""
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--scale", str(2 ** -7), "--steps", "5", "--warmup", "3",
                        "--also", "off", "--inner-warmup", "3", "--inner-iters", "5"],
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, r.stdout
    line = json.loads(lines[0])
    assert "impl" not in line or line["impl"] != "reference"
    assert line["metric"] == "spmm_gflops_warm" and line["n_gpus"] == 1 and line["steps"] == 5 and line["warmup"] >= 3
    assert line["config"]["workload"].startswith("C4") and line["config"]["kernel"] == "SEGMENT_HYBRID_TF32"
    assert line["config"]["routed_kernel"] and line["config"]["plan_build_ms"] > 0
    roof = line["roofline"]
    assert roof["bound"] == "hbm" and roof["peak"] > 0 and 0 < roof["frac"] < 1.5
    assert abs(roof["achieved"] - roof["bytes_algo_per_step"] / (line["ms_per_step"] * 1e-3) / 1e9) < 1e-6 * roof["achieved"]
    e2e = line["e2e"]
    assert e2e["h2d_bytes_per_step"] == 4 * line["config"]["K"] * line["config"]["N"]
    assert e2e["d2h_bytes_per_step"] == 4 * line["config"]["M"] * line["config"]["N"]
    assert 0 < e2e["value"] < line["value"]
    assert line["gpu_launches"] >= 5 and "reasons" in line["clocks"]
    assert line["cpu_baseline"]["kind"] == "reference" and line["cpu_baseline"]["value"] > 0
    assert line["parity"]["ok"] and line["parity"]["rel_fro_vs_cpu_sparse_mm"] < line["parity"]["tolerance"]
