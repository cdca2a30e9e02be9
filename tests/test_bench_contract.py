"""bench.py's output contract, as far as it can be checked without a GPU: the reference arm
(the CPU oracle timed on host cores) prints one JSON line with the agreed keys, rank != 0 stays
silent, and the workload definitions are what the benchmark says they are."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np

import workloads
from conftest import REPO, load_golden


def _run_bench(*args: str, env_extra: dict[str, str] | None = None) -> subprocess.CompletedProcess:
    env = dict(os.environ)
    for key in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        env.pop(key, None)
    env.update(env_extra or {})
    return subprocess.run([sys.executable, str(REPO / "bench.py"), *args], capture_output=True, text=True,
                          timeout=300, env=env, cwd=str(REPO))


def test_reference_arm_prints_one_contract_line() -> None:
    result = _run_bench("--impl", "reference", "--workload", "sim_64", "--steps", "2", "--warmup", "1")
    assert result.returncode == 0, result.stderr
    lines = [line for line in result.stdout.splitlines() if line.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "gemm_tflops" and line["unit"] == "TFLOP/s"
    assert line["higher_is_better"] is True and line["vs_baseline"] is None and line["data"] == "synthetic"
    assert line["steps"] == 2 and line["warmup"] == 1 and line["n_gpus"] == 1 and line["gpu_launches"] == 0
    assert line["config"]["workload"] == "sim_64" and "model" not in line["config"]
    assert line["value"] > 0 and line["ms_per_step"] > 0
    baseline = line["cpu_baseline"]
    assert baseline["kind"] == "port" and baseline["cores"] >= 1 and baseline["value"] == line["value"]
    assert "rows [0," in baseline["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}


def test_reference_arm_runs_on_rank_zero_only() -> None:
    quiet = _run_bench("--impl", "reference", "--workload", "sim_64", "--steps", "1", "--warmup", "0", "--gpus", "2",
                       env_extra={"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert quiet.returncode == 0 and quiet.stdout.strip() == ""
    loud = _run_bench("--impl", "reference", "--workload", "sim_64", "--steps", "1", "--warmup", "0", "--gpus", "2",
                      env_extra={"RANK": "0", "LOCAL_RANK": "0", "WORLD_SIZE": "2"})
    assert loud.returncode == 0 and json.loads(loud.stdout)["n_gpus"] == 2


def test_workload_definitions() -> None:
    shapes = {name: (w.m, w.n, w.k, w.dtype) for name, w in workloads.CONFIGS.items()}
    assert shapes == {
        "sim_64": (64, 64, 64, "float16"),
        "gemm_8192": (8192, 8192, 8192, "float16"),
        "ragged": (4095, 3073, 1031, "bfloat16"),
        "skinny": (8, 16384, 8192, "float16"),
        "sharded": (16384, 32768, 16384, "float16"),
        "long_k": (512, 512, 16384, "float16"),  # (an extra shape class, not one of the five configurations)
    }
    assert workloads.flops(8192, 8192, 8192) == 2.0 * 8192**3
    assert workloads.algorithmic_bytes(8, 16384, 8192) == 2 * 8 * 8192 + 2 * 8192 * 16384 + 4 * 8 * 16384
    a, b = workloads.make_inputs("sim_64")
    golden_a, golden_b, _ = load_golden("sim_f16_m64_n64_k64_normal_seed0")
    assert np.array_equal(a.view(np.uint16), golden_a.view(np.uint16))
    assert np.array_equal(b.view(np.uint16), golden_b.view(np.uint16))
    a, b = workloads.make_inputs("ragged")
    assert a.shape == (4095, 1031) and b.shape == (1031, 3073) and a.dtype.name == "bfloat16"
    assert float(np.abs(a.astype(np.float32)).max()) <= 1.0


def test_sharded_generator_is_slab_consistent() -> None:
    _, whole = workloads.make_sharded_inputs(0, 6144, m=8, k=64, with_a=False)
    for lo, hi in ((0, 2048), (2048, 6144), (4096, 6144)):
        _, slab = workloads.make_sharded_inputs(lo, hi, m=8, k=64, with_a=False)
        assert np.array_equal(slab, whole[:, lo:hi])
    a1, _ = workloads.make_sharded_inputs(0, 2048, m=8, k=64)
    a2, _ = workloads.make_sharded_inputs(2048, 4096, m=8, k=64)
    assert np.array_equal(a1, a2)  # A is the same on every rank


def test_tolerance_rule() -> None:
    rng = np.random.default_rng(0)
    a = rng.standard_normal((32, 48)).astype(np.float16)
    b = rng.standard_normal((48, 40)).astype(np.float16)
    exact = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    assert workloads.check_against_float64(exact, a, b)["ok"]
    wrong = exact.copy()
    wrong[3, 5] += 10.0
    report = workloads.check_against_float64(wrong, a, b)
    assert not report["ok"] and report["max_element_ratio"] > 1e-2
    nan = exact.copy()
    nan[0, 0] = np.nan
    assert not workloads.check_against_float64(nan, a, b)["ok"]
    assert workloads.check_against_float64(wrong, a, b, rows=np.array([0, 1]))["ok"]
