"""The GPU arm of the benchmark script prints the agreed line: the metric, the end-to-end figure with its copy
sizes, the roofline block, the CPU baseline, the clocks and the number of kernel launches in the timed region."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_gpu_arm_prints_the_agreed_line():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "5", "--warmup", "3", "--no-extra"],
                         capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-800:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["metric"] == "nvfp4_dual_gemm_tflops" and line["unit"] == "TFLOP/s" and line["n_gpus"] == 1
    assert line["steps"] == 5 and line["warmup"] == 3 and line["gpu_launches"] == 5
    assert line["config"]["workload"] == "dual_gemm_swiglu_m8192_n14336_k4096"
    flops = 4 * 8192 * 14336 * 4096
    assert abs(line["value"] - flops / (line["ms_per_step"] * 1e-3) / 1e12) < 1e-6 * line["value"]
    assert 1000.0 < line["value"] < 9000.0                      # a B200 does neither 1 nor 9 PFLOP/s of NVFP4 here
    e2e = line["e2e"]
    assert e2e["h2d_bytes_per_step"] > 80e6 and e2e["d2h_bytes_per_step"] == 8192 * 14336 * 2
    assert 0 < e2e["value"] < line["value"]
    roof = line["roofline"]
    assert roof["bound"] == "tensor" and roof["unit"] == "TFLOP/s" and "nvfp4_gemm_pair" in roof["kernel"]
    assert abs(roof["frac"] - roof["achieved"] / roof["peak"]) < 1e-9 and 0.3 < roof["frac"] < 1.3
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and 0 < base["value"] < 100
    assert line["clocks"]["sm_max_mhz"] >= line["clocks"]["sm_mhz"] > 0
