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
    if not c.is_cuda:
        raise ValueError("dual_gemm needs CUDA tensors (there is no CPU path)")
    m, n, l = c.shape
    k = a.shape[1] * 2
    if validate:
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
    lib = _lib.load()
    stream = torch.cuda.current_stream(c.device).cuda_stream
    c_batch = c.stride(2) if l > 1 else 0
    code = lib.b200_dual_gemm_nvfp4_ex(
        _ptr(a), _ptr(b1), _ptr(b2), _ptr(sfa_perm), _ptr(sfb1_perm), _ptr(sfb2_perm), _ptr(c),
        m, n, k, l, c.stride(0), c_batch, 0, 0, variant, None, 0, stream, c.device.index,
        status.data_ptr() if status is not None else None)
    _lib.check(code)
    return c


def custom_kernel(data, *, variant: int = _lib.VARIANT_AUTO):
    """``custom_kernel(data) -> output``; ``data`` is the reference's
    ``(a, b1, b2, sfa, sfb1, sfb2, sfa_perm, sfb1_perm, sfb2_perm, c)``.
    Only ``data[0:3]``, ``data[6:9]`` and ``data[9]`` are used, like the
    reference (dual_gemm/dual_gemm_opt_cute.py:2731)."""
    a, b1, b2, _, _, _, sfa_perm, sfb1_perm, sfb2_perm, c = data
    return dual_gemm(a, b1, b2, sfa_perm, sfb1_perm, sfb2_perm, c, variant=variant)
