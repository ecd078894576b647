"""bench.py on a machine without a GPU: the reference arm prints the contract's JSON line (on a small
workload, so that the test stays short), and the GPU arm refuses to run instead of falling back."""
import json
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parents[1]


def run_bench(*arguments, timeout=600):
    return subprocess.run([sys.executable, str(REPO / "bench.py"), *arguments], capture_output=True, text=True, timeout=timeout)


def test_reference_arm_prints_the_contract_line():
    result = run_bench("--impl", "reference", "--workload", "gemm_fp32_17x4096x4096_fewrows", "--steps", "2", "--warmup", "1")
    assert result.returncode == 0, result.stderr[-500:]
    line = json.loads(result.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "fp32_gemm_tflops" and line["unit"] == "TFLOP/s"
    assert line["higher_is_better"] is True and line["vs_baseline"] is None and line["dtype"] == "f32"
    assert line["config"]["workload"] == "gemm_fp32_17x4096x4096_fewrows" and line["config"]["m"] == 17
    assert line["value"] > 0 and line["ms_per_step"] > 0
    baseline = line["cpu_baseline"]
    assert baseline["kind"] == "reference" and baseline["cores"] >= 1 and baseline["value"] == line["value"]
    assert "rows of A per step" in baseline["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["gpu_launches"] == 0


def test_reference_arm_on_other_ranks_and_on_the_sweep():
    import os

    environment = dict(os.environ, RANK="1", WORLD_SIZE="2")
    result = subprocess.run([sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--gpus", "2"], capture_output=True,
                            text=True, timeout=120, env=environment)
    assert result.returncode == 0 and result.stdout.strip() == ""  # only rank 0 works and prints
    result = run_bench("--impl", "reference", "--workload", "finder_sweep")
    assert result.returncode == 0
    assert "unavailable" in json.loads(result.stdout.strip().splitlines()[-1])


def test_gpu_arm_has_no_cpu_fallback():
    import torch

    if torch.cuda.is_available():
        return  # covered by the GPU runs
    result = run_bench("--steps", "1", "--warmup", "1", timeout=300)
    assert result.returncode != 0
    assert "no CUDA device" in result.stdout
