"""NVFP4 block-scaled grouped GEMM ``C_g = A_g @ B_g.T`` (all groups in one launch).

``custom_kernel(data)`` is a drop-in for the reference's grouped entry point
(group_gemm/group_gemm_cute5_v2.py:4245-4424, group_gemm/group_gemm_cute4.py:1252-1399):
``data = (abc_tensors, sfasfb_tensors, sfasfb_reordered_tensors, problem_sizes)``;
every ``c`` tensor is written in place on the current CUDA stream and the list
of those same tensors is returned without synchronising.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .formats import is_kernel_sf_layout

# signature of a call -> (ctypes argument arrays, device workspace).  The
# reference's harness passes the same tensors again and again while timing, so
# the per-call host work is one dictionary lookup (cf. the reference's pointer
# caches, group_gemm/group_gemm_cute5_v2.py:4319-4345).
_plans: dict = {}
_MAX_PLANS = 64
# Workspaces of evicted plans, per (device, bytes).  They are never handed back to the
# torch allocator while the library may still believe its descriptor table is in them:
# eviction first tells the library to forget the address, then parks the tensor here for
# the next plan of that size.
_free_workspaces: dict = {}


class _Plan:
    __slots__ = ("g", "a", "b", "sfa", "sfb", "c", "mnk", "workspace", "ws_bytes", "device")


def _build_plan(abc, sf_perm, sizes, validate: bool) -> _Plan:
    g = len(sizes)
    if g == 0:
        raise ValueError("grouped gemm needs at least one group")
    if len(abc) != g or len(sf_perm) != g:
        raise ValueError("abc_tensors, reordered scale factors and problem_sizes must have equal length")
    dev = abc[0][2].device
    if dev.type != "cuda":
        raise ValueError("grouped gemm needs CUDA tensors (there is no CPU path)")
    plan = _Plan()
    plan.g, plan.device = g, dev.index
    arr = ctypes.c_void_p * g
    plan.a, plan.b, plan.c, plan.sfa, plan.sfb = arr(), arr(), arr(), arr(), arr()
    plan.mnk = (ctypes.c_int * (3 * g))()
    for i, ((a, b, c), (sfa, sfb), (m, n, k, l)) in enumerate(zip(abc, sf_perm, sizes)):
        if l != 1:
            raise ValueError(f"group {i}: l={l}; the grouped path supports l == 1 only")
        if validate:
            if c.dtype != torch.float16 or tuple(c.shape) != (m, n, 1):
                raise ValueError(f"group {i}: c must be float16 [{m}, {n}, 1]")
            if m > 0 and (c.stride(0) != n or c.stride(1) != 1):
                raise ValueError(f"group {i}: c must be row-major with pitch n")
            if tuple(a.shape) != (m, k // 2, 1) or tuple(b.shape) != (n, k // 2, 1):
                raise ValueError(f"group {i}: operand shapes do not match problem size {(m, n, k)}")
            if m > 0 and (a.stride(1) != 1 or a.stride(0) != k // 2 or b.stride(1) != 1 or b.stride(0) != k // 2):
                raise ValueError(f"group {i}: a and b must be K-major packed bytes")
            if m > 0 and not (is_kernel_sf_layout(sfa, m, k, 1) and is_kernel_sf_layout(sfb, n, k, 1)):
                raise ValueError(f"group {i}: scale factors are not in the reordered (32,4,rest,4,K/64,1) layout")
            for t in (a, b, c, sfa, sfb):
                if t.device != dev:
                    raise ValueError("all tensors must live on the same CUDA device")
        plan.a[i], plan.b[i], plan.c[i] = a.data_ptr(), b.data_ptr(), c.data_ptr()
        plan.sfa[i], plan.sfb[i] = sfa.data_ptr(), sfb.data_ptr()
        plan.mnk[3 * i], plan.mnk[3 * i + 1], plan.mnk[3 * i + 2] = m, n, k
    plan.ws_bytes = int(_lib.load().b200_grouped_workspace_bytes(g))
    pool = _free_workspaces.get((dev.index, plan.ws_bytes))
    plan.workspace = pool.pop() if pool else torch.empty(plan.ws_bytes + 256, dtype=torch.uint8, device=dev)
    return plan


def _workspace_ptr(plan: _Plan) -> int:
    return (plan.workspace.data_ptr() + 255) & ~255


def _evict(plan: _Plan) -> None:
    _lib.check(_lib.load().b200_grouped_workspace_forget(plan.device, _workspace_ptr(plan)))
    _free_workspaces.setdefault((plan.device, plan.ws_bytes), []).append(plan.workspace)


def _signature(abc, sf_perm, sizes):
    return (tuple((a.data_ptr(), b.data_ptr(), c.data_ptr()) for a, b, c in abc),
            tuple((x.data_ptr(), y.data_ptr()) for x, y in sf_perm),
            tuple(tuple(s) for s in sizes))


def grouped_gemm(abc_tensors, sfasfb_reordered_tensors, problem_sizes, *, variant: int = _lib.VARIANT_AUTO,
                 tile_n: int = 0, status: torch.Tensor | None = None, validate: bool = True):
    """Launch every group's GEMM in one kernel; returns the list of ``c`` tensors."""
    sig = _signature(abc_tensors, sfasfb_reordered_tensors, problem_sizes)
    plan = _plans.get(sig)
    if plan is None:
        plan = _build_plan(abc_tensors, sfasfb_reordered_tensors, problem_sizes, validate)
        if len(_plans) >= _MAX_PLANS:
            _evict(_plans.pop(next(iter(_plans))))
        _plans[sig] = plan
    ws_ptr = _workspace_ptr(plan)
    stream = torch.cuda.current_stream(plan.device).cuda_stream
    code = _lib.load().b200_grouped_gemm_nvfp4_ex(
        plan.g, plan.a, plan.b, plan.sfa, plan.sfb, plan.c, plan.mnk, ws_ptr, plan.ws_bytes, variant, tile_n,
        stream, plan.device, status.data_ptr() if status is not None else None)
    _lib.check(code)
    return [c for (_a, _b, c) in abc_tensors]


def custom_kernel(data, *, variant: int = _lib.VARIANT_AUTO, tile_n: int = 0, events=None, stats=None):
    """``custom_kernel(data) -> list[c]``.  ``events`` / ``stats`` are accepted
    for signature compatibility with the reference's profiling hooks
    (group_gemm/group_gemm_cute5_v2.py:4245-4251) and ignored."""
    abc_tensors, _, sfasfb_reordered_tensors, problem_sizes = data
    return grouped_gemm(abc_tensors, sfasfb_reordered_tensors, problem_sizes, variant=variant, tile_n=tile_n)


def custom_kernel_no_alloc(data):
    """Same contract as ``custom_kernel`` for callers that must not allocate
    device memory: the per-group descriptor table lives in a fixed array inside
    the library instead of a workspace tensor, so this wrapper creates no
    tensors at all.  At most ``_lib.STATIC_MAX_GROUPS`` groups; calls whose GPU
    work may overlap must not use this entry point concurrently (they share the
    one table).  The first call on a device should precede any stream capture."""
    abc_tensors, _, sf_perm, problem_sizes = data
    g = len(problem_sizes)
    if g == 0:
        raise ValueError("grouped gemm needs at least one group")
    dev = abc_tensors[0][2].device
    if dev.type != "cuda":
        raise ValueError("grouped gemm needs CUDA tensors (there is no CPU path)")
    arr = ctypes.c_void_p * g
    a, b, c, sfa, sfb = arr(), arr(), arr(), arr(), arr()
    mnk = (ctypes.c_int * (3 * g))()
    for i, ((ta, tb, tc), (tsfa, tsfb), (m, n, k, l)) in enumerate(zip(abc_tensors, sf_perm, problem_sizes)):
        if l != 1:
            raise ValueError(f"group {i}: l={l}; the grouped path supports l == 1 only")
        a[i], b[i], c[i], sfa[i], sfb[i] = ta.data_ptr(), tb.data_ptr(), tc.data_ptr(), tsfa.data_ptr(), tsfb.data_ptr()
        mnk[3 * i], mnk[3 * i + 1], mnk[3 * i + 2] = m, n, k
    stream = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(_lib.load().b200_grouped_gemm_nvfp4_static(g, a, b, sfa, sfb, c, mnk, stream, dev.index, None))
    return [tc for (_ta, _tb, tc) in abc_tensors]
