"""The benchmark script's contract as far as it can be checked without a GPU: the reference arm (the CPU
restatement of the reference's fp32 dequantise-then-matmul path) prints one JSON line with the agreed keys, and
the GPU arm refuses to run, loudly, where there is no CUDA device (no CPU fallback)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=600):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=timeout, cwd=ROOT)


def test_reference_arm_prints_the_agreed_line():
    res = _run("--impl", "reference", "--steps", "1", "--warmup", "0")
    assert res.returncode == 0, res.stderr[-500:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["metric"] == "nvfp4_dual_gemm_tflops" and line["unit"] == "TFLOP/s" and line["higher_is_better"] is True
    assert line["steps"] == 1 and line["warmup"] == 0 and line["n_gpus"] == 1
    assert line["config"]["workload"] == "dual_gemm_swiglu_m8192_n14336_k4096"
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] > 0
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # 4 * M * N * K floating-point operations per step
    assert abs(line["value"] - 4 * 8192 * 14336 * 4096 / (line["ms_per_step"] * 1e-3) / 1e12) < 1e-6 * line["value"]


def test_gpu_arm_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a CUDA device is present")
    res = _run("--steps", "1", "--warmup", "0", "--no-extra", timeout=300)
    assert res.returncode != 0
    assert not any(ln.startswith("{") and '"value"' in ln for ln in res.stdout.splitlines())
