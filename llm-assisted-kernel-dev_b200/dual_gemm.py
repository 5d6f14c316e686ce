"""NVFP4 block-scaled dual GEMM ``C = silu(A @ B1.T) * (A @ B2.T)`` on B200.

``custom_kernel(data)`` is a drop-in for the reference's entry point
(dual_gemm/submission.py:894-957, dual_gemm/dual_gemm_opt_cute.py:2706-2832):
same 10-tuple, the caller-allocated ``c`` (``data[9]``) is written in place on
the current CUDA stream and returned without synchronising.  The arithmetic runs
in libb200nvfp4.so; nothing here computes on the CPU.
"""
from __future__ import annotations

import torch

from . import _lib
from .formats import is_kernel_sf_layout


def _ptr(t: torch.Tensor) -> int:
    return t.data_ptr()


# Split-k workspaces (zero-filled once; the kernel leaves the arrival counters at
# zero), one per device and size.  Shapes that are not split need none.
_workspaces: dict = {}


def _splitk_workspace(lib, device: torch.device, m: int, n: int, k: int, l: int):
    nbytes = int(lib.b200_dual_splitk_workspace_bytes(m, n, k, l))
    if nbytes == 0:
        return None, 0
    key = (device.index, nbytes)
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.zeros(nbytes + 256, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return (ws.data_ptr() + 255) & ~255, nbytes


# Scratch of the CTA-pair kernel's stream-k tail (fp32 partial sums of the tiles that two pairs
# share + flag words; zero-filled once): one per device and stream, because launches that overlap
# on the GPU must not share it.
_streamk_workspaces: dict = {}


def _streamk_workspace(lib, device: torch.device, stream: int, m: int, n: int, k: int, l: int):
    nbytes = int(lib.b200_dual_streamk_workspace_bytes(m, n, k, l))
    if nbytes == 0:
        return None, 0
    key = (device.index, stream)
    ws = _streamk_workspaces.get(key)
    if ws is None or ws.numel() < nbytes + 256:
        ws = torch.zeros(nbytes + 256, dtype=torch.uint8, device=device)
        _streamk_workspaces[key] = ws
    return (ws.data_ptr() + 255) & ~255, nbytes


def _validate(a, b1, b2, sfa_perm, sfb1_perm, sfb2_perm, c, m, n, k, l) -> None:
    if c.dtype != torch.float16:
        raise ValueError(f"c must be float16, got {c.dtype}")
    if tuple(a.shape) != (m, k // 2, l) or tuple(b1.shape) != (n, k // 2, l) or tuple(b2.shape) != (n, k // 2, l):
        raise ValueError(f"operand shapes {tuple(a.shape)} {tuple(b1.shape)} {tuple(b2.shape)} do not match "
                         f"c {tuple(c.shape)}")
    for name, t, rows in (("a", a, m), ("b1", b1, n), ("b2", b2, n)):
        if t.element_size() != 1 or t.stride(1) != 1 or t.stride(0) != k // 2 or \
                (l > 1 and t.stride(2) != rows * (k // 2)):
            raise ValueError(f"{name} must be K-major packed bytes with strides (K/2, 1, rows*K/2)")
    if c.stride(1) != 1:
        raise ValueError("c must have unit stride along N")
    for name, t, rows in (("sfa", sfa_perm, m), ("sfb1", sfb1_perm, n), ("sfb2", sfb2_perm, n)):
        if not is_kernel_sf_layout(t, rows, k, l):
            raise ValueError(f"{name} is not in the (32,4,rest,4,K/64,L) reordered scale-factor layout")
    dev = c.device
    for t in (a, b1, b2, sfa_perm, sfb1_perm, sfb2_perm):
        if t.device != dev:
            raise ValueError("all tensors must live on the same CUDA device")


# (tensor addresses, shape, strides, variant) -> ready-made argument tuple.  The
# reference's harness calls custom_kernel on the same tensors over and over while
# timing (cholesky/eval.py:179-183), so a repeated call costs one dictionary
# lookup and one foreign call; the layout checks run once per distinct call.
_plans: dict = {}
_MAX_PLANS = 256


def dual_gemm(a, b1, b2, sfa_perm, sfb1_perm, sfb2_perm, c, *, variant: int = _lib.VARIANT_AUTO,
              status: torch.Tensor | None = None, validate: bool = True) -> torch.Tensor:
    """Launch the dual GEMM.

    a            [M, K/2, L] packed e2m1 (``float4_e2m1fn_x2`` or uint8), K-major
    b1, b2       [N, K/2, L] packed e2m1
    sf*_perm     (32, 4, rest, 4, K/64, L) e4m3 views of the reference's
                 reordered scale-factor buffers
    c            [M, N, L] fp16 with strides (ldc, 1, batch); written in place
    status       optional 1-element uint32/int32 CUDA tensor receiving a non-zero
                 code if an on-device wait times out
    """
    stream = torch.cuda.current_stream(c.device).cuda_stream if c.is_cuda else 0
    key = (a.data_ptr(), b1.data_ptr(), b2.data_ptr(), sfa_perm.data_ptr(), sfb1_perm.data_ptr(),
           sfb2_perm.data_ptr(), c.data_ptr(), c.shape, c.stride(), a.shape[1], variant,
           0 if status is None else status.data_ptr(), stream)
    plan = _plans.get(key)
    if plan is None:
        if not c.is_cuda:
            raise ValueError("dual_gemm needs CUDA tensors (there is no CPU path)")
        m, n, l = c.shape
        k = a.shape[1] * 2
        if validate:
            _validate(a, b1, b2, sfa_perm, sfb1_perm, sfb2_perm, c, m, n, k, l)
        lib = _lib.load()
        ws_ptr, ws_bytes = (None, 0)
        if variant == _lib.VARIANT_SPLITK:
            ws_ptr, ws_bytes = _splitk_workspace(lib, c.device, m, n, k, l)
        elif variant == _lib.VARIANT_PAIR_STREAMK and m % 256 == 0:
            ws_ptr, ws_bytes = _streamk_workspace(lib, c.device, stream, m, n, k, l)
        args = (key[0], key[1], key[2], key[3], key[4], key[5], key[6], m, n, k, l, c.stride(0),
                c.stride(2) if l > 1 else 0, 0, 0, variant, ws_ptr, ws_bytes)
        plan = (lib.b200_dual_gemm_nvfp4_ex, args, c.device, c.device.index,
                status.data_ptr() if status is not None else None)
        if len(_plans) >= _MAX_PLANS:
            _plans.pop(next(iter(_plans)))
        _plans[key] = plan
    fn, args, device, index, status_ptr = plan
    code = fn(*args, stream, index, status_ptr)
    if code:
        _lib.check(code)
    return c


def dual_gemm_quantized(a, b1, b2, sfa_perm, sfb1_perm, sfb2_perm):
    """``silu(A @ B1.T) * (A @ B2.T)`` re-quantised to NVFP4 in the epilogue:
    returns ``(q, sf_perm)`` -- ``q`` [M, N/2, 1] packed e2m1 and the
    (32, 4, M/128, 4, N/64, 1) e4m3 view of a fresh reordered scale-factor buffer --
    equal byte for byte to ``quantize.quantize_nvfp4`` applied to the fp16 result of
    ``dual_gemm``.  M % 256 == 0, L == 1.  The input of the next block-scaled GEMM
    (the reference stores fp16: dual_gemm/submission.py:596-611)."""
    from .formats import E4M3, FP4X2
    if not a.is_cuda:
        raise ValueError("dual_gemm_quantized needs CUDA tensors (there is no CPU path)")
    m, n, k = a.shape[0], b1.shape[0], a.shape[1] * 2
    if a.shape[2] != 1:
        raise ValueError("dual_gemm_quantized supports l == 1 only")
    for name, t, rows in (("sfa", sfa_perm, m), ("sfb1", sfb1_perm, n), ("sfb2", sfb2_perm, n)):
        if not is_kernel_sf_layout(t, rows, k, 1):
            raise ValueError(f"{name} is not in the (32,4,rest,4,K/64,L) reordered scale-factor layout")
    lib = _lib.load()
    q = torch.empty((m, n // 2), dtype=torch.uint8, device=a.device)
    sf = torch.empty((1, max(m // 128, 1), max(n // 64, 1), 32, 4, 4), dtype=torch.uint8, device=a.device)
    code = lib.b200_dual_gemm_nvfp4_quant(a.data_ptr(), b1.data_ptr(), b2.data_ptr(), sfa_perm.data_ptr(),
                                          sfb1_perm.data_ptr(), sfb2_perm.data_ptr(), q.data_ptr(), sf.data_ptr(),
                                          m, n, k, torch.cuda.current_stream(a.device).cuda_stream, a.device.index,
                                          None)
    _lib.check(code)
    return q.view(m, n // 2, 1).view(FP4X2), sf.permute(3, 4, 1, 5, 2, 0).view(E4M3)


def custom_kernel(data, *, variant: int = _lib.VARIANT_AUTO):
    """``custom_kernel(data) -> output``; ``data`` is the reference's
    ``(a, b1, b2, sfa, sfb1, sfb2, sfa_perm, sfb1_perm, sfb2_perm, c)``.
    Only ``data[0:3]``, ``data[6:9]`` and ``data[9]`` are used, like the
    reference (dual_gemm/dual_gemm_opt_cute.py:2731)."""
    a, b1, b2, _, _, _, sfa_perm, sfb1_perm, sfb2_perm, c = data
    return dual_gemm(a, b1, b2, sfa_perm, sfb1_perm, sfb2_perm, c, variant=variant)
