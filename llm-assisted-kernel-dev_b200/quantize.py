"""fp16 / bf16 activations -> NVFP4 operand (packed e2m1 + reordered e4m3 scale
factors) on the GPU, in exactly the form ``dual_gemm.custom_kernel`` and
``group_gemm.custom_kernel`` take as ``a`` / ``sfa_perm``.

The reference has no quantiser: its ``generate_input`` draws pre-quantised
operands (dual_gemm/reference.py:114-190).  This is the step that precedes the
GEMMs in a real FFN.  The arithmetic runs in libb200nvfp4.so; there is no CPU path.
"""
from __future__ import annotations

import torch

from . import _lib
from .formats import E4M3, FP4X2, sf_atoms


def quantize_nvfp4(x: torch.Tensor):
    """x [rows, k] (fp16 or bf16, CUDA, unit stride along k, k % 64 == 0) ->
    ``(q, sf_perm)``: ``q`` [rows, k/2, 1] packed e2m1 and ``sf_perm`` the
    (32, 4, ceil(rows/128), 4, k/64, 1) e4m3 view of a freshly allocated
    reordered scale-factor buffer.  Runs on the current stream, no synchronisation."""
    if not x.is_cuda:
        raise ValueError("quantize_nvfp4 needs a CUDA tensor (there is no CPU path)")
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be [rows, k] with unit stride along k")
    if x.dtype == torch.float16:
        dtype = _lib.DTYPE_F16
    elif x.dtype == torch.bfloat16:
        dtype = _lib.DTYPE_BF16
    else:
        raise ValueError(f"x must be float16 or bfloat16, got {x.dtype}")
    rows, k = x.shape
    lib = _lib.load()
    rm, rk = sf_atoms(rows, k) if k % 64 == 0 and rows > 0 else (1, 1)
    q = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
    sf = torch.empty((1, rm, rk, 32, 4, 4), dtype=torch.uint8, device=x.device)
    code = lib.b200_quantize_nvfp4(x.data_ptr(), dtype, rows, k, x.stride(0), q.data_ptr(), sf.data_ptr(),
                                   torch.cuda.current_stream(x.device).cuda_stream, x.device.index)
    _lib.check(code)
    return q.view(rows, k // 2, 1).view(FP4X2), sf.permute(3, 4, 1, 5, 2, 0).view(E4M3)
