"""bench.py's contract: what it prints and how it exits without a GPU, and (on one) that every workload
still runs and prints its one JSON line with the keys the record is read by."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "bench.py")


def run(*args, timeout=900):
    return subprocess.run([sys.executable, BENCH, *args], capture_output=True, text=True, timeout=timeout, cwd=ROOT)


def test_more_than_one_gpu_is_refused_with_one_line():
    out = run("--gpus", "2")
    assert out.returncode == 2
    assert len(out.stdout.strip().splitlines()) == 1 and "--gpus 2" in out.stdout


def test_reference_arm_says_why_it_is_unavailable():
    out = run("--impl", "reference", "--gpus", "1", "--steps", "5", "--warmup", "3")
    assert out.returncode == 0
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and "\n" not in rec["unavailable"]


@pytest.mark.gpu
def test_headline_line_on_two_layers():
    out = run("--layers", "2", "--steps", "3", "--warmup", "3", "--skip-points")
    assert out.returncode == 0, out.stderr[-2000:]
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "prefill", "roofline", "points", "wait_errors"):
        assert key in rec, key
    assert rec["steps"] == 3 and rec["warmup"] == 3 and rec["n_gpus"] == 1 and rec["wait_errors"] == 0
    assert rec["config"]["layers"] == 36 and rec["config"]["layers_run"] == 2 and len(rec["config"]) <= 20
    assert all(not isinstance(v, (dict, list)) for v in rec["config"].values())
    assert rec["gpu_launches"] > 0 and rec["value"] > 0 and rec["e2e"]["value"] > 0
    assert rec["e2e"]["h2d_bytes_per_step"] > 0 and rec["e2e"]["d2h_bytes_per_step"] > 0
    assert set(rec["prefill"]) >= {"value", "tokens", "ms", "frac"} and rec["prefill"]["tokens"] == 2048
    assert rec["roofline"]["bound"] == "hbm" and rec["roofline"]["unit"] == "GB/s"


@pytest.mark.gpu
@pytest.mark.parametrize("workload,metric", [("serving", "serving_generated_tokens_per_s"), ("mixed_step", "mixed_step_ms")])
def test_other_workloads_print_their_line(workload, metric):
    out = run("--workload", workload)
    assert out.returncode == 0, out.stderr[-2000:]
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["metric"] == metric and rec["value"] > 0 and rec["wait_errors"] == 0
