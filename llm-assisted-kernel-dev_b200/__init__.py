"""B200-native NVFP4 block-scaled dual GEMM and grouped GEMM.

Drop-in ``custom_kernel(data)`` entry points for the dual-GEMM and grouped-GEMM
problems of whatdhack/llm-assisted-kernel-dev, backed by hand-written sm_100a
kernels in ``libb200nvfp4.so`` (C ABI: include/b200_nvfp4.h).

    from <this package>.dual_gemm import custom_kernel      # dual GEMM
    from <this package>.group_gemm import custom_kernel     # grouped GEMM
"""
from . import _lib, formats, inputs  # noqa: F401
from . import dual_gemm, group_gemm, moe, quantize, shard  # noqa: F401

__all__ = ["dual_gemm", "group_gemm", "moe", "inputs", "formats", "shard"]
