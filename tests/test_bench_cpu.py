"""The benchmark's contract, as far as it can be checked without a GPU: the reference arm
(the CPU oracle timed on a bounded sample) prints one JSON line with the agreed keys, and the
product arm refuses to run without a CUDA device instead of falling back to the CPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*args, env=None):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT,
                          capture_output=True, text=True, timeout=600,
                          env=dict(os.environ, **(env or {})))


def test_reference_arm_prints_the_contract_line():
    r = run_bench("--impl", "reference", "--config", "C1", "--steps", "2", "--warmup", "1",
                  "--reference-tokens", "64")
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "MoE-layer tokens/s" and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["steps"] == 2 and line["warmup"] == 1
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["vs_baseline"] is None
    assert line["gpu_launches"] == 0
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert line["config"]["workload"].startswith("C1")


def test_reference_arm_uses_all_cores_under_a_launcher_that_sets_one_thread():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the reference arm asks
    for every core it may run on instead of inheriting that."""
    r = run_bench("--impl", "reference", "--config", "C1", "--steps", "1", "--warmup", "0",
                  "--reference-tokens", "64", env={"OMP_NUM_THREADS": "1"})
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))


def test_traffic_figure_comes_from_the_committed_summary():
    sys.path.insert(0, ROOT)
    import importlib
    bench = importlib.import_module("bench")
    total, commit = bench.ncu_traffic("C3")
    assert total and total > 2e9 and commit
    assert bench.ncu_traffic("no such workload") == (None, None)


def test_product_arm_needs_a_gpu():
    import torch
    if torch.cuda.is_available():
        return  # the GPU suite and the benchmark itself cover this side
    r = run_bench("--config", "C1", "--steps", "1", "--warmup", "1", "--no-cpu-baseline")
    assert r.returncode != 0
    assert "cuda" in (r.stderr + r.stdout).lower()
