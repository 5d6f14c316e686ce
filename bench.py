#!/usr/bin/env python
"""Benchmark of the NVFP4 dual GEMM / grouped GEMM path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A "step" is one launch of the dual GEMM C = silu(A.B1^T) * (A.B2^T) on the
SwiGLU-FFN shape M=8192, N=14336, K=4096 (NVFP4 operands, e4m3 scale factors per
16 k, fp32 accumulation, fp16 output).  With N GPUs the problem is sharded along
its output columns (rows of B1/B2), A replicated, no collective on the data path:
total work is fixed, so this is strong scaling.  Rank 0 prints ONE JSON line.

value      algorithmic TFLOP/s (4*M*N*K per step), inputs resident in HBM
e2e        same metric through custom_kernel() with host buffers: pinned-host ->
           device copies of every input and a device -> host read of C inside
           the timed region
roofline   tensor-core roofline of the dual-GEMM kernel: algorithmic FLOP per launch /
           CUDA-event time, against 4 x the measured cuBLAS bf16 rate
cpu_baseline / --impl reference
           the reference's fp32 dequantise-then-matmul CPU path (torch CPU ops,
           all host threads) on the same workload, a few passes
extra      the other benchmark configurations (skinny-M dual GEMM, G=8 grouped
           GEMM, 64-expert MoE grouped GEMM) in microseconds per launch; a block of
           launches at least a second long ("sustained"); and, in a child process,
           the reference's own sm_100a kernel and the cuBLASLt NVFP4 GEMM on the same GPU

Timing protocol.  The reference times 15 or more data sets launched back to back between
two CUDA events after one L2 flush, and stops when the error of the mean falls under 0.1 %
(group_gemm/group_gemm_cute4.py:1586-1664, utils/dual_gemm/utils.py:165-172).  Here the
step count is given on the command line, so the region is exactly K launches, and the L2
is defeated by rotating input sets that together exceed it instead of one flush.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M, N, K = 8192, 14336, 4096
WORKLOAD = "dual_gemm_swiglu_m8192_n14336_k4096"
METRIC = "nvfp4_dual_gemm_tflops"
UNIT = "TFLOP/s"
L2_BYTES = 126 * 1024 * 1024
NOMINAL_FP4_TFLOPS = 9000.0
# CPU sample of the same problem
CPU_SAMPLE = (M, N, K)          # the whole workload: about 1.5-5 s per pass on 8-16 host cores


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = []
        for ts, line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7 and parts[0].isdigit():
                rows.append((ts, parts))
        inside = [p for ts, p in rows if t0 - 0.05 <= ts <= t1 + 0.15] or [p for _, p in rows]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = sorted(int(p[0]) for p in inside)
        reasons = []
        for idx, name in ((3, "hw_slowdown"), (4, "hw_thermal_slowdown"), (5, "sw_thermal_slowdown"),
                          (6, "sw_power_cap")):
            if any(p[idx].lower().startswith("active") for p in inside):
                reasons.append(name)
        return {"sm_mhz": int(statistics.median(busy)), "sm_max_mhz": int(inside[0][1]), "samples": len(inside),
                "power_w_max": max((float(p[2]) for p in inside if p[2].replace(".", "", 1).isdigit()), default=None),
                "reasons": reasons}


# --------------------------------------------------------------------------- reference arm (CPU)
def cpu_reference_sample(steps: int, warmup: int):
    """The reference's CPU check (fp32 dequantise, matmul, silu*mul, fp16 cast)
    on the benchmark problem.  Returns (TFLOP/s, seconds per step, threads)."""
    import torch
    pkg = importlib.import_module("llm-assisted-kernel-dev_b200")
    from oracle import nvfp4_oracle as orc
    m, n, k = CPU_SAMPLE
    # the launcher of multi-rank runs exports OMP_NUM_THREADS=1; this arm runs on one
    # rank only and may use every host core
    torch.set_num_threads(max(torch.get_num_threads(), os.cpu_count() or 1))
    data = pkg.inputs.generate_input(m, n, k, 1, 0, dist="uniform16", device="cpu")
    for _ in range(warmup):
        orc.dual_gemm(data)
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.dual_gemm(data)
    dt = (time.perf_counter() - t0) / steps
    flops = 4.0 * m * n * k
    return flops / dt / 1e12, dt, torch.get_num_threads()


def base_config():
    """The `config` object, identical in both arms."""
    return {"workload": WORKLOAD, "m": M, "n": N, "k": K, "l": 1,
            "operands": "e2m1 codes uniform over 16 values, e4m3 scales U[0.25,2], seeds 0,42,.."}


def run_reference(args):
    """`--impl reference`: the reference's CPU path on the box's host cores, rank 0 only.  Every step is one
    pass over the workload; when the requested steps would take more than a few minutes the passes run on
    the first columns of the problem only (TFLOP/s does not depend on the width) and `sample` says so."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    global CPU_SAMPLE
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    budget_passes = 150                       # about 0.9-1.5 s per full pass on 8-16 host cores
    n_cols = N
    if steps + warmup > budget_passes:
        n_cols = max(128, (N * budget_passes // (steps + warmup)) // 128 * 128)
    CPU_SAMPLE = (M, n_cols, K)
    tflops, dt, threads = cpu_reference_sample(steps, warmup)
    sample = (f"{'the whole workload' if n_cols == N else f'a problem {n_cols} instead of {N} columns wide'} per step: "
              f"{M}x{n_cols}x{K} (4*{M}*{n_cols}*{K} flop), {steps} timed passes after {warmup} warm-up passes")
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": dt * 1e3 * (N / n_cols), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32 (dequantised e2m1 x e4m3)", "data": "synthetic",
        "config": base_config(),
        "details": {"path": "reference CPU check: fp32 dequantise-then-matmul, silu*mul, fp16 cast (torch CPU ops)"},
        "cpu_baseline": {"value": tflops, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- same-box comparison (child process)
def run_same_box(args):
    """`--same-box`: in a process of its own, time on this GPU (a) the reference's own sm_100a dual-GEMM
    kernel, `custom_kernel` of dual_gemm/submission.py:894-957 (one CTA per 128 x 128 tile, CuTe DSL JIT),
    and (b) the cuBLASLt NVFP4 GEMM behind `torch._scaled_mm` -- the library kernel the reference's
    `ref_kernel` calls twice -- with the same event protocol as this library's figures.  Prints one JSON
    object; a part that cannot run is reported as {"unavailable": reason}."""
    import torch
    pkg = importlib.import_module("llm-assisted-kernel-dev_b200")
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import ref_loader
    torch.cuda.set_device(0)
    out = {}
    shapes = {"dual_skinny_m256_n4096_k7168": (256, 4096, 7168), "dual_one_eighth_shard_m8192_n1792_k4096": (8192, 1792, 4096)}
    steps, warmup = max(5, args.steps), max(3, args.warmup)

    def timed(fn_for_set, n_sets):
        sec, _, _ = time_launches(torch, lambda i: fn_for_set(i % n_sets), steps, warmup, lambda: None)
        return sec / steps * 1e6

    try:
        if not ref_loader.available():
            raise RuntimeError("baseline/_ref is not installed")
        os.environ.setdefault("CUTE_DSL_ARCH", "sm_100a")
        _ref, _specs, sub = ref_loader.load_dual(with_kernel=True)
        k1 = {}
        for name, (m, n, k) in shapes.items():
            per_set = m * k // 2 + n * k
            n_sets = max(2, min(8, -(-2 * L2_BYTES // per_set)))
            sets = [pkg.inputs.generate_input(m, n, k, 1, 42 * i, dist="uniform16", device="cuda:0") for i in range(n_sets)]
            sub.custom_kernel(sets[0])
            torch.cuda.synchronize()
            ours = pkg.dual_gemm.custom_kernel(tuple(t.clone() if t is not None else None for t in sets[0]))
            torch.cuda.synchronize()
            same = bool(torch.equal(torch.nan_to_num(ours.float(), 0.0, 1.0, -1.0).cpu(),
                                    torch.nan_to_num(sets[0][9].float(), 0.0, 1.0, -1.0).cpu())) or None
            us_ref = timed(lambda j: sub.custom_kernel(sets[j]), n_sets)
            us_ours = timed(lambda j: pkg.dual_gemm.custom_kernel(sets[j]), n_sets)
            k1[name] = {"reference_kernel_us": us_ref, "this_library_us": us_ours, "speedup": us_ref / us_ours,
                        "bit_identical_outputs": same, "input_sets": n_sets}
            del sets
        out["reference_submission_kernel"] = k1
    except Exception as exc:  # noqa: BLE001 - any import, JIT or launch failure is reported, not retried
        out["reference_submission_kernel"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
    try:
        # (c) the reference's grouped kernel with compile-time group dispatch, custom_kernel of
        # group_gemm/group_gemm_cute4.py:1252-1399, on the task's first benchmark list
        if not ref_loader.available():
            raise RuntimeError("baseline/_ref is not installed")
        k4 = ref_loader.load_grouped_kernel()
        gm, gn, gk = [80, 176, 128, 72, 64, 248, 96, 160], 4096, 7168
        g = len(gm)
        n_in = 3
        gsets = [pkg.inputs.generate_grouped_input(gm, [gn] * g, [gk] * g, g, 1111 + 42 * i, dist="reference",
                                                   device="cuda:0") for i in range(n_in)]
        ref_out = [c.clone() for c in k4.custom_kernel(gsets[0])]
        torch.cuda.synchronize()
        ours_out = pkg.group_gemm.custom_kernel(gsets[0])
        torch.cuda.synchronize()
        same = all(bool(torch.equal(a_, b_)) for a_, b_ in zip(ref_out, ours_out))
        for j in range(1, n_in):
            k4.custom_kernel(gsets[j])          # the reference compiles once per list and caches per pointer set
        torch.cuda.synchronize()
        us_ref = timed(lambda j: k4.custom_kernel(gsets[j]), n_in)
        us_ours = timed(lambda j: pkg.group_gemm.custom_kernel(gsets[j]), n_in)
        out["reference_grouped_kernel_cute4"] = {"list": "G=8, M 64..248, N=4096, K=7168 (utils/group_gemm/task.yml:59)",
                                                 "reference_kernel_us": us_ref, "this_library_us": us_ours,
                                                 "speedup": us_ref / us_ours, "bit_identical_outputs": same,
                                                 "input_sets": n_in}
    except Exception as exc:  # noqa: BLE001
        out["reference_grouped_kernel_cute4"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
    try:
        from oracle import nvfp4_oracle as orc
        m, n, k = M, N, K
        data = pkg.inputs.generate_input(m, n, k, 1, 0, dist="uniform16", device="cuda:0")
        sa = orc.to_blocked(data[3][:, :, 0]).view(torch.float8_e4m3fn).cuda()
        sb = orc.to_blocked(data[4][:, :, 0]).view(torch.float8_e4m3fn).cuda()
        a2, b2 = data[0][:, :, 0], data[1][:, :, 0].transpose(0, 1)
        us = timed(lambda j: torch._scaled_mm(a2, b2, sa, sb, bias=None, out_dtype=torch.float16), 1)
        out["cublaslt_nvfp4_gemm"] = {"shape": [m, n, k], "us_per_gemm": us, "tflops": 2.0 * m * n * k / us / 1e6,
                                      "note": "one plain block-scaled GEMM with fp16 output, no activation; the dual "
                                              "GEMM is two of these plus silu*mul"}
    except Exception as exc:  # noqa: BLE001
        out["cublaslt_nvfp4_gemm"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
    try:
        # a second library kernel for the same plain GEMM: the CUTLASS block-scaled GEMM that vLLM ships
        from vllm import _custom_ops as vops
        a8, b8 = a2.view(torch.uint8), data[1][:, :, 0].view(torch.uint8)
        sa2 = sa.view(-1, k // 16) if sa.dim() == 1 else sa
        sb2 = sb.view(-1, k // 16) if sb.dim() == 1 else sb
        alpha = torch.ones(1, dtype=torch.float32, device="cuda:0")
        got = vops.cutlass_scaled_fp4_mm(a8, b8, sa2, sb2, alpha, torch.float16)
        want = torch._scaled_mm(a2, b2, sa, sb, bias=None, out_dtype=torch.float16)
        same = bool(torch.equal(torch.nan_to_num(got.float(), posinf=7e4, neginf=-7e4),
                                torch.nan_to_num(want.float(), posinf=7e4, neginf=-7e4)))
        us = timed(lambda j: vops.cutlass_scaled_fp4_mm(a8, b8, sa2, sb2, alpha, torch.float16), 1)
        out["vllm_cutlass_nvfp4_gemm"] = {"shape": [m, n, k], "us_per_gemm": us, "tflops": 2.0 * m * n * k / us / 1e6,
                                          "equals_cublaslt": same,
                                          "note": "vllm._custom_ops.cutlass_scaled_fp4_mm, one plain GEMM, fp16 output"}
    except Exception as exc:  # noqa: BLE001
        out["vllm_cutlass_nvfp4_gemm"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
    try:
        # the activation quantiser beside vLLM's (same buffers for the same consumer, global scale 1)
        from vllm import _custom_ops as vops
        rows, kq = 32768, 8192
        x = (torch.randn(rows, kq, device="cuda:0") * 4).to(torch.bfloat16)
        one = torch.ones(1, dtype=torch.float32, device="cuda:0")
        qbytes = rows * kq * 2 + rows * kq // 2 + rows * kq // 16
        us_theirs = timed(lambda j: vops.scaled_fp4_quant(x, one), 1)
        us_ours = timed(lambda j: pkg.quantize.quantize_nvfp4(x), 1)
        out["vllm_nvfp4_quantiser"] = {"shape": [rows, kq], "vllm_us": us_theirs, "this_library_us": us_ours,
                                       "vllm_gbs": qbytes / us_theirs / 1e3, "this_library_gbs": qbytes / us_ours / 1e3,
                                       "note": "bf16 in, packed e2m1 + swizzled e4m3 scale factors out; both calls "
                                               "allocate their outputs"}
    except Exception as exc:  # noqa: BLE001
        out["vllm_nvfp4_quantiser"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
    try:
        # the 64-expert list beside the CUTLASS grouped block-scaled GEMM that vLLM's fused MoE calls
        from vllm import _custom_ops as vops
        experts, n_g, k_g = 64, 2048, 7168
        counts = pkg.inputs.moe_expert_counts(8192, experts, 8, seed=0)
        gdata = pkg.inputs.generate_grouped_input(counts, [n_g] * experts, [k_g] * experts, experts, 0, dist="uniform16",
                                                  device="cuda:0")

        def flat_sf(perm, rows):      # the buffer behind a permuted view: [row tile][k tile][32][4][4]
            return perm.view(torch.uint8).permute(5, 2, 4, 0, 1, 3).contiguous().view(-1, k_g // 16)

        a_cat = torch.cat([abc[0][:, :, 0].view(torch.uint8) for abc in gdata[0]], dim=0)
        b_all = torch.stack([abc[1][:, :, 0].view(torch.uint8) for abc in gdata[0]], dim=0)
        sfa_cat = torch.cat([flat_sf(sf[0], m) for sf, m in zip(gdata[2], counts)], dim=0).view(torch.float8_e4m3fn)
        sfb_all = torch.stack([flat_sf(sf[1], n_g) for sf in gdata[2]], dim=0).view(torch.float8_e4m3fn)
        offs = [0]
        sf_offs = [0]
        for m_g in counts:
            offs.append(offs[-1] + m_g)
            sf_offs.append(sf_offs[-1] + -(-m_g // 128) * 128)
        expert_offsets = torch.tensor(offs[:-1], dtype=torch.int32, device="cuda:0")     # first row of every expert
        sf_offsets = torch.tensor(sf_offs[:-1], dtype=torch.int32, device="cuda:0")     # ... in the padded scale factors
        sizes = torch.tensor([[m_g, n_g, k_g] for m_g in counts], dtype=torch.int32, device="cuda:0")
        alphas = torch.ones(experts, dtype=torch.float32, device="cuda:0")
        y = torch.empty((offs[-1], n_g), dtype=torch.float16, device="cuda:0")
        vops.cutlass_fp4_moe_mm(y, a_cat, b_all, sfa_cat, sfb_all, alphas, sizes, expert_offsets, sf_offsets)
        ours = pkg.group_gemm.custom_kernel(gdata)
        torch.cuda.synchronize()
        ours_cat = torch.cat([c[:, :, 0] for c in ours], dim=0).float()
        finite = torch.isfinite(ours_cat) & torch.isfinite(y.float())
        rel = ((ours_cat - y.float()).abs() / (ours_cat.abs() + 1.0))[finite].max().item()
        us_theirs = timed(lambda j: vops.cutlass_fp4_moe_mm(y, a_cat, b_all, sfa_cat, sfb_all, alphas, sizes,
                                                            expert_offsets, sf_offsets), 1)
        us_ours = timed(lambda j: pkg.group_gemm.custom_kernel(gdata), 1)
        out["vllm_cutlass_nvfp4_grouped_gemm"] = {
            "list": "64 experts, 8192 tokens top-8 (sum M = 65536), N=2048, K=7168", "vllm_us": us_theirs,
            "this_library_us": us_ours, "speedup": us_theirs / us_ours, "max_relative_difference": rel,
            "note": "vllm._custom_ops.cutlass_fp4_moe_mm on the same operands, concatenated the way it wants them"}
    except Exception as exc:  # noqa: BLE001
        out["vllm_cutlass_nvfp4_grouped_gemm"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
    try:
        # the routing kernel beside vLLM's fused grouped_topk (8192 tokens, 256 experts in 8 groups, top-8)
        from vllm import _custom_ops as vops
        logits = torch.randn((8192, 256), device="cuda:0")
        bias = torch.randn((256,), device="cuda:0") * 0.1
        us_theirs = timed(lambda j: vops.grouped_topk(logits, 8, 4, 8, True, 2.5, bias, 1), 1)
        bufs = pkg.moe.route(logits, bias, 8, 4, 8, 2.5)
        us_ours = timed(lambda j: pkg.moe.route(logits, bias, 8, 4, 8, 2.5, out=bufs), 1)
        out["vllm_grouped_topk"] = {"tokens": 8192, "experts": 256, "vllm_us": us_theirs, "this_library_us": us_ours}
    except Exception as exc:  # noqa: BLE001
        out["vllm_grouped_topk"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
    print(json.dumps(out), flush=True)


# --------------------------------------------------------------------------- our arm (GPU)
def input_sets(pkg, torch, shard_fn, device, count, m, n, k):
    sets = []
    for i in range(count):
        data = pkg.inputs.generate_input(m, n, k, 1, 42 * i, dist="uniform16", device="cpu")
        data = shard_fn(data)
        sets.append(data)
    return sets


def to_device(torch, pkg, data, device):
    """Move the tensors custom_kernel reads (and c) to the device, keeping strides."""
    a, b1, b2, sfa, sfb1, sfb2, sfa_p, sfb1_p, sfb2_p, c = data

    def sf(t):
        dense = t.view(torch.uint8).permute(5, 2, 4, 0, 1, 3).contiguous().to(device)
        return dense.permute(3, 4, 1, 5, 2, 0).view(torch.float8_e4m3fn)

    def fp4(t):
        raw = t.view(torch.uint8).permute(2, 0, 1).contiguous().to(device)
        return raw.permute(1, 2, 0).view(pkg.formats.FP4X2)
    cc = torch.empty((1, c.shape[0], c.shape[1]), dtype=torch.float16, device=device).permute(1, 2, 0)
    return (fp4(a), fp4(b1), fp4(b2), None, None, None, sf(sfa_p), sf(sfb1_p), sf(sfb2_p), cc)


def time_launches(torch, fn, steps, warmup, barrier):
    for i in range(warmup):
        fn(i)
    barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    start.record()
    for i in range(steps):
        fn(warmup + i)
    stop.record()
    torch.cuda.synchronize()
    t1 = time.time()
    barrier()
    return start.elapsed_time(stop) / 1e3, t0, t1


def run_grouped_only(args):
    """`--grouped g8|moe`: warm-up + timed launches of one grouped list and nothing else."""
    import torch
    pkg = importlib.import_module("llm-assisted-kernel-dev_b200")
    device = "cuda:0"
    torch.cuda.set_device(0)
    if args.grouped == "g8":
        ms = pkg.inputs.uniform_group_rows(8, seed=0)
        data = pkg.inputs.generate_grouped_input(ms, [4096] * 8, [7168] * 8, 8, 0, dist="uniform16", device=device)
    else:
        ms = pkg.inputs.moe_expert_counts(8192, 64, 8, seed=0)
        data = pkg.inputs.generate_grouped_input(ms, [2048] * 64, [7168] * 64, 64, 0, dist="uniform16", device=device)
    launches0 = pkg._lib.launch_count()
    sec, _, _ = time_launches(torch, lambda i: pkg.group_gemm.custom_kernel(data), args.steps, args.warmup, lambda: None)
    status = pkg._lib.read_status(0)
    if status:
        raise SystemExit(f"device status word {status:#x}: an on-device wait timed out")
    flops = pkg.formats.grouped_gemm_flops(data[3])
    print(json.dumps({"workload": "grouped_" + args.grouped, "us_per_launch": sec / args.steps * 1e6,
                      "tflops": flops * args.steps / sec / 1e12, "steps": args.steps, "warmup": args.warmup,
                      "gpu_launches": int(pkg._lib.launch_count() - launches0 - args.warmup),
                      "note": "grouped-only run for profiler captures"}), flush=True)


def run_quantize_only(args):
    """`--quantize ROWS,K`: warm-up + timed launches of the fp16 -> NVFP4 quantiser and nothing else."""
    import torch
    pkg = importlib.import_module("llm-assisted-kernel-dev_b200")
    torch.cuda.set_device(0)
    rows, k = (int(v) for v in args.quantize.split(","))
    x = torch.randn(rows, k, device="cuda:0", dtype=torch.float16)
    sec, _, _ = time_launches(torch, lambda i: pkg.quantize.quantize_nvfp4(x), args.steps, args.warmup, lambda: None)
    nbytes = rows * k * 2 + rows * k // 2 + rows * k // 16
    print(json.dumps({"workload": f"quantize_f16_m{rows}_k{k}", "us_per_launch": sec / args.steps * 1e6,
                      "hbm_gbs": nbytes * args.steps / sec / 1e9, "steps": args.steps, "warmup": args.warmup,
                      "note": "quantiser-only run for profiler captures"}), flush=True)


def run_moe(torch, pkg, device, peaks, steps, warmup):
    tokens, experts, top_k, n, k = 8192, 64, 8, 2048, 7168
    gen = torch.Generator().manual_seed(0)
    x = torch.randn((tokens, k), generator=gen).to(torch.bfloat16).to(device)
    logits = torch.randn((tokens, experts), generator=gen).to(device)
    wdata = pkg.inputs.generate_grouped_input([0] * experts, [n] * experts, [k] * experts, experts, 0, dist="uniform16",
                                              device=device)
    weights = pkg.moe.MoEWeights([abc[1] for abc in wdata[0]], [sf[1] for sf in wdata[2]])
    lib = pkg._lib.load()
    run = (lambda i: pkg.moe.moe_forward(x, logits, None, weights, n_group=8, topk_group=4, top_k=top_k,
                                         routed_scaling=2.5, return_plan=True))
    out, buf = run(0)
    stream = torch.cuda.current_stream().cuda_stream
    dev = torch.cuda.current_device()
    rows = tokens * top_k
    two_pass_scratch = torch.empty(int(lib.b200_moe_gather_scratch_bytes(tokens, k)), dtype=torch.uint8, device=device)
    steps_of = {
        "route": lambda i: pkg.moe.route(logits, None, 8, 4, top_k, 2.5, out=(buf.topk_idx, buf.topk_w)),
        "plan": lambda i: lib.b200_moe_plan(buf.topk_idx.data_ptr(), tokens, experts, top_k, buf.counts.data_ptr(),
                                            buf.row_offsets.data_ptr(), buf.sfa_atom_offsets.data_ptr(),
                                            buf.row_of.data_ptr(), buf.src_token.data_ptr(), buf.scratch.data_ptr(),
                                            buf.scratch.numel(), stream, dev),
        "quantize_scatter": lambda i: lib.b200_moe_quantize_scatter(x.data_ptr(), pkg._lib.DTYPE_BF16, tokens, k, x.stride(0),
                                                                    buf.row_of.data_ptr(), buf.row_offsets.data_ptr(),
                                                                    buf.sfa_atom_offsets.data_ptr(), experts, top_k,
                                                                    buf.a_q.data_ptr(), buf.sfa.data_ptr(), stream, dev),
        "gather_quantize_two_pass": lambda i: lib.b200_moe_gather_quantize(
            x.data_ptr(), pkg._lib.DTYPE_BF16, tokens, k, x.stride(0), buf.src_token.data_ptr(), buf.row_offsets.data_ptr(),
            buf.sfa_atom_offsets.data_ptr(), experts, top_k, buf.a_q.data_ptr(), buf.sfa.data_ptr(),
            two_pass_scratch.data_ptr(), two_pass_scratch.numel(), stream, dev),
        "grouped_gemm": lambda i: lib.b200_moe_grouped_gemm_nvfp4(experts, buf.a_q.data_ptr(), buf.sfa.data_ptr(), rows,
                                                                  weights.b_ptrs, weights.sfb_ptrs, n, k,
                                                                  buf.counts.data_ptr(), buf.row_offsets.data_ptr(),
                                                                  buf.sfa_atom_offsets.data_ptr(), buf.y.data_ptr(),
                                                                  buf.ws_ptr, buf.ws_bytes, stream, dev, None),
        "combine": lambda i: lib.b200_moe_combine(buf.y.data_ptr(), n, buf.row_of.data_ptr(), buf.topk_w.data_ptr(), tokens,
                                                  top_k, pkg._lib.DTYPE_BF16, out.data_ptr(), out.stride(0), stream, dev),
    }
    # algorithmic bytes of the HBM-bound steps
    algo = {"route": tokens * experts * 4 + rows * 8,
            # quantise every token once (2 B in, 9/16 B out per element), then read and write 9/16 B per element of
            # every permuted row
            "gather_quantize_two_pass": tokens * k * 2 + tokens * (k // 2 + k // 16) + 2 * rows * (k // 2 + k // 16),
            # read every token once (2 B per element), write 9/16 B per element of every permuted row
            "quantize_scatter": tokens * k * 2 + rows * (k // 2 + k // 16),
            "combine": rows * n * 2 + tokens * n * 2 + rows * 8}
    res = {}
    for name, fn in steps_of.items():
        sec, _, _ = time_launches(torch, fn, steps, warmup, lambda: None)
        us = sec / steps * 1e6
        res[name] = {"us": us}
        if name in algo:
            res[name]["hbm_gbs"] = algo[name] / us / 1e3
            res[name]["frac_hbm_peak"] = algo[name] / us / 1e3 / peaks["hbm_gbs"]
    sec, _, _ = time_launches(torch, run, steps, warmup, lambda: None)
    res["whole_layer_us"] = sec / steps * 1e6
    res["grouped_gemm"]["tflops"] = 2.0 * rows * n * k / res["grouped_gemm"]["us"] / 1e6
    res["note"] = ("quantize_scatter (what the layer runs) = every token row read and quantised once and written straight "
                   "to its top_k rows; gather_quantize_two_pass = the older entry point (quantise into scratch, then copy "
                   "every quantised row to its top_k places); no step reads anything back to the host")
    return res


def run_extra(torch, pkg, device, peaks, steps, warmup):
    """Other benchmark configurations, one GPU: microseconds per launch."""
    extra = {}
    fmts = pkg.formats
    # skinny-M dual GEMM (HBM-leaning): rotate 8 input sets (290 MB > L2)
    m, n, k = 256, 4096, 7168
    sets = [pkg.inputs.generate_input(m, n, k, 1, 42 * i, dist="uniform16", device=device) for i in range(8)]
    sec, _, _ = time_launches(torch, lambda i: pkg.dual_gemm.custom_kernel(sets[i % 8]), steps * 4, warmup, lambda: None)
    us = sec / (steps * 4) * 1e6
    byts, flops = fmts.dual_gemm_bytes(m, n, k), fmts.dual_gemm_flops(m, n, k)
    extra["dual_skinny_m256_n4096_k7168"] = {
        "us_per_launch": us, "kernel": pkg._lib.last_kernel(), "tflops": flops / us / 1e6, "hbm_gbs": byts / us / 1e3,
        "frac_hbm_peak": byts / us / 1e3 / peaks["hbm_gbs"], "input_sets": 8}
    del sets
    # grouped GEMM, G=8, M_i ~ U{64..1024}, N=4096, K=7168: 2 input sets (2 x 140 MB > L2)
    ms = pkg.inputs.uniform_group_rows(8, seed=0)
    gsets = [pkg.inputs.generate_grouped_input(ms, [4096] * 8, [7168] * 8, 8, 42 * i, dist="uniform16", device=device)
             for i in range(2)]
    sec, _, _ = time_launches(torch, lambda i: pkg.group_gemm.custom_kernel(gsets[i % 2]), steps * 2, warmup, lambda: None)
    us = sec / (steps * 2) * 1e6
    sizes = gsets[0][3]
    byts, flops = fmts.grouped_gemm_bytes(sizes), fmts.grouped_gemm_flops(sizes)
    extra["grouped_g8_n4096_k7168"] = {"us_per_launch": us, "m": ms, "kernel": pkg._lib.last_kernel(),
                                       "tflops": flops / us / 1e6,
                                       "hbm_gbs": byts / us / 1e3, "frac_hbm_peak": byts / us / 1e3 / peaks["hbm_gbs"]}
    del gsets
    # the benchmark dual GEMM with its result re-quantised to NVFP4 in the epilogue (input of a down projection)
    dq = pkg.inputs.generate_input(M, N, K, 1, 0, dist="uniform16", device=device)
    sec, _, _ = time_launches(torch, lambda i: pkg.dual_gemm.dual_gemm_quantized(dq[0], dq[1], dq[2], dq[6], dq[7], dq[8]),
                              steps, warmup, lambda: None)
    us = sec / steps * 1e6
    extra["dual_quantised_output_m8192_n14336_k4096"] = {"us_per_launch": us, "tflops": 4.0 * M * N * K / us / 1e6,
                                                         "output_bytes": M * N // 2 + M * N // 16}
    del dq
    # activation quantiser fp16 -> NVFP4 (HBM-bound): the benchmark's A shape (4 inputs, 268 MB > L2; at 67 MB
    # per launch a kernel runs ~20 us and launch + ramp-up keep any streaming kernel near 3.8 TB/s) and a
    # 512 MB input that shows the steady rate
    for name, qm, qk, n_in in (("quantize_f16_m8192_k4096", 8192, 4096, 4), ("quantize_f16_m32768_k8192", 32768, 8192, 1)):
        xs = [torch.randn(qm, qk, device=device, dtype=torch.float16) for _ in range(n_in)]
        sec, _, _ = time_launches(torch, lambda i: pkg.quantize.quantize_nvfp4(xs[i % n_in]), steps * 2, warmup,
                                  lambda: None)
        us = sec / (steps * 2) * 1e6
        qbytes = qm * qk * 2 + qm * qk // 2 + qm * qk // 16
        extra[name] = {"us_per_launch": us, "hbm_gbs": qbytes / us / 1e3,
                       "frac_hbm_peak": qbytes / us / 1e3 / peaks["hbm_gbs"]}
        del xs
    # the reference task's own benchmark shapes with its speed-of-light targets in microseconds
    # (utils/dual_gemm/task.yml:33-38 and 59-62, utils/group_gemm/task.yml:35-39 and 59-62), reference distribution
    task = {}
    for (tm, tn, tk, sol) in ((256, 4096, 7168, 4.708), (512, 4096, 7168, 8.714), (256, 3072, 4096, 2.125),
                              (512, 3072, 7168, 6.535)):
        per_set = tm * tk // 2 + tn * tk
        n_in = max(2, min(16, -(-2 * L2_BYTES // per_set)))
        tsets = [pkg.inputs.generate_input(tm, tn, tk, 1, 1111 + 42 * i, dist="reference", device=device)
                 for i in range(n_in)]
        sec, _, _ = time_launches(torch, lambda i: pkg.dual_gemm.custom_kernel(tsets[i % n_in]), steps * 4, warmup,
                                  lambda: None)
        us = sec / (steps * 4) * 1e6
        task[f"dual_m{tm}_n{tn}_k{tk}"] = {"us_per_launch": us, "speed_of_light_us": sol, "kernel": pkg._lib.last_kernel(),
                                            "hbm_gbs": fmts.dual_gemm_bytes(tm, tn, tk) / us / 1e3, "input_sets": n_in}
        del tsets
    for (gm, gn, gk, sol) in (([80, 176, 128, 72, 64, 248, 96, 160], 4096, 7168, 18.833),
                              ([40, 76, 168, 72, 164, 148, 196, 160], 7168, 2048, 10.667),
                              ([192, 320], 3072, 4096, 2.406), ([128, 384], 4096, 1536, 1.525)):
        g = len(gm)
        per_set = g * gn * gk // 2
        n_in = max(2, min(16, -(-2 * L2_BYTES // per_set)))
        gsets = [pkg.inputs.generate_grouped_input(gm, [gn] * g, [gk] * g, g, 1111 + 42 * i, dist="reference",
                                                   device=device) for i in range(n_in)]
        sec, _, _ = time_launches(torch, lambda i: pkg.group_gemm.custom_kernel(gsets[i % n_in]), steps * 4, warmup,
                                  lambda: None)
        us = sec / (steps * 4) * 1e6
        task[f"grouped_g{g}_n{gn}_k{gk}"] = {"us_per_launch": us, "speed_of_light_us": sol,
                                             "kernel": pkg._lib.last_kernel(),
                                             "hbm_gbs": fmts.grouped_gemm_bytes(gsets[0][3]) / us / 1e3, "input_sets": n_in}
        del gsets
    extra["reference_task_benchmarks"] = task
    # the whole MoE layer around that grouped GEMM: routing, plan, gather + quantise, GEMM, combine, each step
    # timed on its own (8192 tokens, 64 experts in 8 groups of which 4 stay, top-8, N=2048, K=7168, bf16 in and out)
    extra["moe_layer_t8192_e64_n2048_k7168"] = run_moe(torch, pkg, device, peaks, max(5, steps // 4), warmup)
    # MoE grouped GEMM, 64 experts, 8192 tokens top-8 (sum M = 65536), N=2048, K=7168
    counts = pkg.inputs.moe_expert_counts(8192, 64, 8, seed=0)
    data = pkg.inputs.generate_grouped_input(counts, [2048] * 64, [7168] * 64, 64, 0, dist="uniform16", device=device)
    sec, _, _ = time_launches(torch, lambda i: pkg.group_gemm.custom_kernel(data), steps, warmup, lambda: None)
    us = sec / steps * 1e6
    byts, flops = fmts.grouped_gemm_bytes(data[3]), fmts.grouped_gemm_flops(data[3])
    extra["grouped_moe_g64_n2048_k7168"] = {
        "us_per_launch": us, "kernel": pkg._lib.last_kernel(), "m_min": min(counts), "m_max": max(counts), "zero_groups": counts.count(0),
        "tflops": flops / us / 1e6, "frac_fp4_nominal": flops / us / 1e6 / NOMINAL_FP4_TFLOPS,
        "hbm_gbs": byts / us / 1e3}
    extra["l2_to_shared_memory_feed"] = run_feed_probe(torch, pkg, device)
    return extra


def run_feed_probe(torch, pkg, device):
    """What the memory system sustains when a kernel does nothing but the GEMMs' kind of loads (TMA from an
    L2-resident window into shared memory), next to what the dual GEMM draws: 38 KB per k-tile and CTA."""
    dev = torch.device(device).index or 0
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    rows = []
    for ctas, share, tiled in ((1, 1, True), (sms, 1, True), (sms, 1, False), (sms, 2, True), (sms, 32, True)):
        rows.append(pkg._lib.probe_l2_feed(dev, ctas, share, tiled))
    drawn = (M // 128) * (N // 128) * (K // 256) * 38 * 1024
    return {"runs": rows, "dual_gemm_bytes_from_l2_per_launch": drawn,
            "note": "16 KiB copies, 12 in flight per CTA, 4 issuing warps; share = CTAs reading the same tiles at the same time"}


def run_ours(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the NVFP4 kernels have no CPU path")
    torch.cuda.set_device(local)
    device = f"cuda:{local}"
    pkg = importlib.import_module("llm-assisted-kernel-dev_b200")
    pkg._lib.load()
    if world > 1:
        # the launcher exports OMP_NUM_THREADS=1; generating the synthetic inputs on the host may use this rank's
        # share of the cores
        torch.set_num_threads(max(1, (os.cpu_count() or world) // world))
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(device))

    def barrier():
        if dist is not None:
            dist.barrier()

    peaks = load_peaks()
    lo, hi = pkg.shard.column_range(N, rank, world)
    n_local = hi - lo
    shard = (lambda d: pkg.shard.shard_dual_input(d, rank, world))
    # rotate enough input sets that their bytes exceed 2 x L2
    per_set = M * K // 2 + 2 * (n_local * K // 2)
    n_sets = max(2, min(8, -(-2 * L2_BYTES // per_set)))
    host_sets = input_sets(pkg, torch, shard, device, n_sets, M, N, K)
    dev_sets = [to_device(torch, pkg, d, device) for d in host_sets]

    launches0 = pkg._lib.launch_count()
    sampler = ClockSampler(local)
    sampler.start()
    run_step = (lambda i: pkg.dual_gemm.custom_kernel(dev_sets[i % n_sets]))
    # One region of exactly K launches on one GPU.  With several GPUs a K-launch region of a
    # column shard lasts a millisecond or two and its max over ranks is dominated by jitter:
    # the region is then timed five times and the median region is reported.
    repeats = 1 if world == 1 else 5
    regions = []
    for rep in range(repeats):
        sec, t0, t1 = time_launches(torch, run_step, args.steps, args.warmup if rep == 0 else 0, barrier)
        t = torch.tensor([sec], dtype=torch.float64, device=device)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        regions.append((float(t.item()), sec, t0, t1))
    regions.sort()
    sec_max, sec, t0, t1 = regions[len(regions) // 2]
    clocks = sampler.stop(min(r[2] for r in regions), max(r[3] for r in regions))
    launches = (pkg._lib.launch_count() - launches0 - args.warmup) // repeats
    kernel_name = pkg._lib.last_kernel()
    status = pkg._lib.read_status(local)
    if status:
        raise SystemExit(f"device status word {status:#x}: an on-device wait timed out")
    flops_total = 4.0 * M * N * K
    value = flops_total * args.steps / sec_max / 1e12

    # SM clock this kernel really runs at: clock64 span of its first CTA / CUDA-event time of the same
    # launch (nvidia-smi samples every 100 ms and cannot see a region of a few milliseconds)
    eff = []
    for i in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run_step(i)
        e1.record()
        torch.cuda.synchronize()
        eff.append(pkg._lib.last_launch_cycles(local) / (e0.elapsed_time(e1) * 1e3))
    clocks["effective_sm_mhz"] = round(statistics.median(eff), 1)
    clocks["effective_sm_mhz_how"] = "clock64 span of CTA 0 / CUDA-event time of the same launch, median of 5"

    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                              "warmup": args.warmup, "ms_per_step": sec_max / args.steps * 1e3,
                              "config": {"workload": WORKLOAD}, "gpu_launches": int(launches), "clocks": clocks,
                              "kernel": kernel_name, "note": "kernel-only run for profiler captures"}), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- end to end: pinned host buffers -> device, kernel, C back to the host
    hs = host_sets[0]

    def pin_bytes(t_):
        return t_.view(torch.uint8).permute(2, 0, 1).contiguous().pin_memory()

    def pin_sf(t_):
        return t_.view(torch.uint8).permute(5, 2, 4, 0, 1, 3).contiguous().pin_memory()
    h_ops = [pin_bytes(x) for x in hs[:3]]
    h_sfs = [pin_sf(x) for x in hs[6:9]]
    h_c = torch.empty((1, M, n_local), dtype=torch.float16).pin_memory()
    # With several GPUs, A and its scale factors (the same on every rank) cross PCIe once, on rank 0,
    # and reach the other ranks by an NCCL broadcast over NVLink; every rank uploads only its own rows
    # of B1 / B2 and their scale factors.
    shared_in = [h_ops[0], h_sfs[0]]
    own_in = [h_ops[1], h_ops[2], h_sfs[1], h_sfs[2]]
    shared_bytes = sum(x.numel() for x in shared_in)
    own_bytes = sum(x.numel() for x in own_in)
    h2d = shared_bytes + own_bytes if (dist is None or rank == 0) else own_bytes
    d2h = h_c.numel() * 2
    # Two device buffer sets and three streams: while step i computes, step i+1's inputs
    # arrive and step i-1's C leaves (PCIe is full duplex).  Every step still copies all
    # of its inputs in and all of its result out; the events keep each buffer's copy-in,
    # kernel and copy-out in order.
    bufs = []
    for _ in range(2):
        flat = torch.empty(shared_bytes, dtype=torch.uint8, device=device)      # A bytes, then SFA bytes
        d_a = flat[:h_ops[0].numel()].view(h_ops[0].shape)
        d_sfa = flat[h_ops[0].numel():].view(h_sfs[0].shape)
        d_ops = [d_a] + [torch.empty_like(x, device=device) for x in h_ops[1:]]
        d_sfs = [d_sfa] + [torch.empty_like(x, device=device) for x in h_sfs[1:]]
        d_c = torch.empty((1, M, n_local), dtype=torch.float16, device=device)
        d_data = tuple(x.permute(1, 2, 0).view(pkg.formats.FP4X2) for x in d_ops) + (None, None, None) + \
            tuple(x.permute(3, 4, 1, 5, 2, 0).view(torch.float8_e4m3fn) for x in d_sfs) + (d_c.permute(1, 2, 0),)
        bufs.append({"flat": flat, "ops": d_ops, "sfs": d_sfs, "c": d_c, "data": d_data, "in_done": torch.cuda.Event(),
                     "kernel_done": torch.cuda.Event(), "out_done": torch.cuda.Event()})
    s_in, s_run, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device), torch.cuda.Stream(device)
    e2e_steps = max(4, min(args.steps, 20))

    def e2e_step(i):
        b = bufs[i % 2]
        with torch.cuda.stream(s_in):
            s_in.wait_event(b["kernel_done"])          # the kernel that last read these inputs
            if dist is None or rank == 0:
                b["ops"][0].copy_(h_ops[0], non_blocking=True)
                b["sfs"][0].copy_(h_sfs[0], non_blocking=True)
            for src, dst in zip(own_in, [b["ops"][1], b["ops"][2], b["sfs"][1], b["sfs"][2]]):
                dst.copy_(src, non_blocking=True)
            if dist is not None:
                dist.broadcast(b["flat"], src=0)       # ordered behind the copies above on this stream
            b["in_done"].record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(b["in_done"])
            s_run.wait_event(b["out_done"])            # C of two steps ago has left this buffer
            pkg.dual_gemm.custom_kernel(b["data"])
            b["kernel_done"].record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(b["kernel_done"])
            h_c.copy_(b["c"], non_blocking=True)
            b["out_done"].record(s_out)

    for b in bufs:                                      # events start out "recorded"
        for name in ("in_done", "kernel_done", "out_done"):
            b[name].record(torch.cuda.current_stream(device))
    for i in range(2):
        e2e_step(i)
    torch.cuda.synchronize()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(s_in)
    for i in range(e2e_steps):
        e2e_step(2 + i)
    s_out.wait_stream(s_in)
    s_out.wait_stream(s_run)
    stop.record(s_out)                                  # after the last C has reached the host
    torch.cuda.synchronize()
    barrier()
    sec_e2e = start.elapsed_time(stop) / 1e3
    t = torch.tensor([sec_e2e], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = flops_total * e2e_steps / float(t.item()) / 1e12

    io = torch.tensor([float(h2d), float(d2h)], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(io, op=dist.ReduceOp.SUM)      # bytes per step over all ranks
    h2d_total, d2h_total = int(io[0].item()), int(io[1].item())

    # MoE grouped GEMM sharded by group (N > 1): the one-GPU list (seed 0) is generated once on the host
    # and every rank keeps the experts shard.shard_grouped_input gives it; no collective on the data
    # path; time = max over ranks
    moe_sharded = None
    if dist is not None and not args.no_extra:
        counts = pkg.inputs.moe_expert_counts(8192, 64, 8, seed=0)
        whole = pkg.inputs.generate_grouped_input(counts, [2048] * 64, [7168] * 64, 64, 0, dist="uniform16", device="cpu")
        mine = pkg.shard.assign_groups(whole[3], world)[rank]
        gdata = pkg.inputs.grouped_to_device(pkg.shard.shard_grouped_input(whole, rank, world), device)
        del whole
        gsteps = max(5, min(args.steps, 50))
        gsec, _, _ = time_launches(torch, lambda i: pkg.group_gemm.custom_kernel(gdata), gsteps, 3, barrier)
        tg = torch.tensor([gsec], dtype=torch.float64, device=device)
        dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        us = float(tg.item()) / gsteps * 1e6
        total_flops = sum(2.0 * c_ * 2048 * 7168 for c_ in counts)
        moe_sharded = {"us_per_launch": us, "tflops": total_flops / us / 1e6, "groups_per_gpu": len(mine),
                       "kernel": pkg._lib.last_kernel(),
                       "parallelism": f"64 experts (one seed-0 list) sharded by group x{world}, no collective"}
        del gdata

    gather_ms = gather_ok = fused_gather = None
    if dist is not None:
        # after the metric: full C on every rank (one NCCL all-gather of the column shards); the gathered
        # matrix is checked against this rank's own shard
        pkg.dual_gemm.custom_kernel(dev_sets[0])
        shard_c = dev_sets[0][9]
        for _ in range(2):
            pkg.shard.gather_dual_output(shard_c, N)
        torch.cuda.synchronize()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(5):
            full_c = pkg.shard.gather_dual_output(shard_c, N)
        g1.record()
        torch.cuda.synchronize()
        tg = torch.tensor([g0.elapsed_time(g1) / 5], dtype=torch.float64, device=device)
        dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        gather_ms = float(tg.item())
        same = torch.equal(full_c[:, lo:hi].view(torch.int16), shard_c.view(torch.int16)) and \
            tuple(full_c.shape) == (M, N, 1)
        ok = torch.tensor([1.0 if same else 0.0], dtype=torch.float64, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        gather_ok = bool(ok.item() == 1.0)
        # the same result from ONE kernel per rank: the GEMM's epilogue stores every tile into the full C of
        # every rank through peer-mapped symmetric memory (plain TMA stores over NVLink, no multicast, no NCCL)
        try:
            import torch.distributed._symmetric_memory as symm_mem
            c_sym = symm_mem.empty((M, N), dtype=torch.float16, device=torch.device(device))
            hdl = symm_mem.rendezvous(c_sym, dist.group.WORLD)
            ptrs = [int(x) for x in hdl.buffer_ptrs]
            c_sym.fill_(float("nan"))
            torch.cuda.synchronize()
            barrier()
            pkg.shard.dual_gemm_gathered(dev_sets[0], ptrs, rank, world, N)
            torch.cuda.synchronize()
            barrier()
            same = bool(torch.equal(c_sym.view(torch.int16), full_c[:, :, 0].view(torch.int16)))
            fsec, _, _ = time_launches(torch, lambda i: pkg.shard.dual_gemm_gathered(dev_sets[i % n_sets], ptrs, rank, world, N),
                                       args.steps, 3, barrier)
            tf = torch.tensor([fsec, 1.0 if same else 0.0], dtype=torch.float64, device=device)
            tmax = tf.clone()
            dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
            dist.all_reduce(tf, op=dist.ReduceOp.MIN)
            fused_gather = {"ms_per_step": float(tmax[0].item()) / args.steps * 1e3, "matches_all_gather": bool(tf[1].item() == 1.0),
                            "kernel": pkg._lib.last_kernel(), "bytes_over_nvlink_per_rank": int(2 * M * n_local * (world - 1)),
                            "note": "GEMM + all-gather in one kernel per rank; compare with ms_per_step + c_all_gather_ms"}
            del c_sym
        except Exception as exc:  # noqa: BLE001 - symmetric memory may be unavailable; the NCCL path above stands
            fused_gather = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
        del full_c

    # a block of launches at least a second long: the power-capped regime a serving loop sees
    sustained_block = None
    if not args.no_extra:
        n_long = max(args.steps, int(1.2 / (sec_max / args.steps)) + 1)
        sampler = ClockSampler(local)
        sampler.start()
        lsec, lt0, lt1 = time_launches(torch, run_step, n_long, 0, barrier)
        lclocks = sampler.stop(lt0, lt1)
        t = torch.tensor([lsec], dtype=torch.float64, device=device)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        lval = flops_total * n_long / float(t.item()) / 1e12
        sustained_block = {"value": lval, "unit": UNIT, "steps": n_long, "ms_per_step": float(t.item()) / n_long * 1e3,
                           "clocks": lclocks,
                           "frac_of_4x_bf16_sustained": lval / world / (4.0 * peaks["bf16_tflops_sustained"]),
                           "frac_nominal": lval / world / NOMINAL_FP4_TFLOPS}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # Denominator: 4 x the measured cuBLAS bf16 rate (no FP4 figure is measured).  A long run of
    # back-to-back launches is in the power-capped regime, like the "sustained" bf16 figure;
    # a short one is compared with the burst figure.  Both fractions are reported.
    sustained = sec > 0.2 and "sw_power_cap" in (clocks.get("reasons") or [])
    peak_key = "bf16_tflops_sustained" if sustained else "bf16_tflops"
    fp4_peak = 4.0 * peaks[peak_key]
    per_launch_flops = 4.0 * M * n_local * K
    achieved = per_launch_flops * args.steps / sec / 1e12     # this rank's kernel
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": fp4_peak, "unit": "TFLOP/s", "frac": achieved / fp4_peak,
        "peak_basis": f"4 x {peaks['source']} cuBLAS bf16 {'sustained' if sustained else 'burst'} "
                      f"({peaks[peak_key]} TFLOP/s; timed region {sec:.2f} s, "
                      f"{'power-capped' if sustained else 'not power-capped or short'}): no measured FP4 figure "
                      f"exists; nominal dense NVFP4 is {NOMINAL_FP4_TFLOPS:.0f}",
        "frac_of_burst_peak": achieved / (4.0 * peaks["bf16_tflops"]),
        "frac_nominal": achieved / NOMINAL_FP4_TFLOPS,
        # An MMA-only loop of this library's instrumented build (every SM issuing 128x256x64 block-scaled
        # MMAs back to back on random operand bytes, no loads, no epilogue) reached 8140-8190 TFLOP/s on this
        # pool at 1.68 GHz (8850 with constant operands at 1.83 GHz): the ceiling for this data, below nominal.
        "peak_mma_only": MMA_ONLY_TFLOPS, "frac_of_mma_only": achieved / MMA_ONLY_TFLOPS,
        "kernel": kernel_name, "avg_launch_us": sec / args.steps * 1e6,
        "traffic": TRAFFIC_BYTES_PER_LAUNCH if (world == 1 and (M, N, K) == (8192, 14336, 4096)) else None,
        "traffic_source": "one-pass ncu capture of a full-size launch, profiles/dual_gemm_pair_m8192_n14336_k4096_launches.md",
        "algorithmic_bytes": pkg.formats.dual_gemm_bytes(M, n_local, K),
    }
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec_max / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3 block scale), f32 accumulate, f16 out",
        "data": "synthetic", "gpu_launches": int(launches),
        "config": base_config(),
        "details": {"n_per_gpu": n_local, "parallelism": f"column-sharded x{world}, A replicated, no collective",
                    "l2": f"rotating {n_sets} input sets ({n_sets * per_set / 1e6:.0f} MB > L2 126 MB) plus "
                          f"{2 * M * n_local / 1e6:.0f} MB of C written per step",
                    "timing": "one region of K launches" if repeats == 1 else
                              f"median of {repeats} regions of K launches each (max over ranks per region); regions "
                              f"in ms per step: {[round(r[0] / args.steps * 1e3, 4) for r in regions]}"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_total, "d2h_bytes_per_step": d2h_total,
                "steps": e2e_steps, "overlap": "copy-in, kernel and copy-out of consecutive steps on three streams",
                "inputs": "every rank uploads its rows of B1/B2 and their scale factors" +
                          ("" if world == 1 else "; A and its scale factors are uploaded on rank 0 and broadcast over NVLink (NCCL)")},
        "clocks": clocks, "roofline": roofline,
    }
    extra = {}
    if gather_ms is not None:
        line["c_all_gather_ms"] = gather_ms
        line["c_all_gather_matches_shards"] = gather_ok
        line["c_gather_fused_in_epilogue"] = fused_gather
    if moe_sharded is not None:
        extra["grouped_moe_g64_n2048_k7168_sharded"] = moe_sharded
    if sustained_block is not None:
        extra["sustained"] = sustained_block
    if world == 1:
        cpu_tflops, cpu_dt, threads = cpu_reference_sample(4, 1)
        m_, n_, k_ = CPU_SAMPLE
        line["cpu_baseline"] = {"value": cpu_tflops, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": f"the whole workload ({m_}x{n_}x{k_}), 4 timed passes "
                                          f"({cpu_dt:.2f} s each)"}
        if not args.no_extra:
            del dev_sets, host_sets, bufs
            torch.cuda.empty_cache()
            extra.update(run_extra(torch, pkg, device, peaks, max(5, min(args.steps, 200)), max(3, args.warmup)))
            extra["same_gpu"] = same_box_child()
    if extra:
        line["extra"] = extra
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def same_box_child():
    """Run `bench.py --same-box` in a child process (the reference's JIT-compiled kernel and the cuBLASLt
    GEMM stay out of this process) and return its JSON object."""
    try:
        res = subprocess.run([sys.executable, os.path.abspath(__file__), "--same-box", "--steps", "30", "--warmup", "5"],
                             capture_output=True, text=True, timeout=600, cwd=ROOT)
        for ln in reversed(res.stdout.strip().splitlines()):
            if ln.startswith("{"):
                return json.loads(ln)
        return {"unavailable": f"no JSON from the child (exit {res.returncode}): {res.stderr[-300:]}"}
    except Exception as exc:  # noqa: BLE001
        return {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}


# TFLOP/s of an MMA-only loop on all SMs with random operand bytes (instrumented build, this pool)
MMA_ONLY_TFLOPS = 8140.0

# DRAM bytes (read + write) of one full-size dual-GEMM launch: dram__bytes_read.sum 85.4 MB +
# dram__bytes_write.sum 191.9 MB from a one-pass ncu capture of `bench.py --kernel-only`
# (summary under profiles/).  Reads are the operands once;
# part of C is still in the L2 when the launch ends.
TRAFFIC_BYTES_PER_LAUNCH = 277.3e6


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="default: 1000 (GPU arm), 10 (reference arm)")
    ap.add_argument("--warmup", type=int, default=None, help="default: 20 (GPU arm), 2 (reference arm)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary configurations")
    ap.add_argument("--kernel-only", action="store_true",
                    help="only the device-timed launches (no e2e, CPU baseline or extras): for profiler captures")
    ap.add_argument("--shape", default=None, help="M,N,K override of the dual-GEMM shape (profiler captures)")
    ap.add_argument("--same-box", action="store_true",
                    help="one GPU: time the reference's own sm_100a kernel and the cuBLASLt NVFP4 GEMM (child process of the default run)")
    ap.add_argument("--quantize", default=None, help="ROWS,K: launch only the activation quantiser (profiler captures)")
    ap.add_argument("--moe-layer", action="store_true",
                    help="run only the MoE layer steps (routing, plan, gather, grouped GEMM, combine; profiler captures, one GPU)")
    ap.add_argument("--feed-probe", action="store_true",
                    help="only measure how fast TMA loads fill shared memory from L2 (one JSON line)")
    ap.add_argument("--grouped", default=None, choices=["g8", "moe"],
                    help="launch only the G=8 or the 64-expert grouped GEMM (profiler captures, one GPU)")
    args = ap.parse_args()
    if args.shape:
        global M, N, K, WORKLOAD
        M, N, K = (int(x) for x in args.shape.split(","))
        WORKLOAD = f"dual_gemm_m{M}_n{N}_k{K}"
    if args.steps is None:
        args.steps = 10 if args.impl == "reference" else 1000
    if args.warmup is None:
        args.warmup = 2 if args.impl == "reference" else 20
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.same_box:
        run_same_box(args)
    elif args.moe_layer:
        import torch
        torch.cuda.set_device(0)
        pkg = importlib.import_module("llm-assisted-kernel-dev_b200")
        print(json.dumps({"workload": "moe_layer_t8192_e64_n2048_k7168",
                          **run_moe(torch, pkg, "cuda:0", load_peaks(), args.steps, args.warmup)}), flush=True)
    elif args.feed_probe:
        import torch
        torch.cuda.set_device(0)
        pkg = importlib.import_module("llm-assisted-kernel-dev_b200")
        print(json.dumps({"workload": "l2_to_shared_memory_feed", **run_feed_probe(torch, pkg, "cuda:0")}), flush=True)
    elif args.grouped:
        run_grouped_only(args)
    elif args.quantize:
        run_quantize_only(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
