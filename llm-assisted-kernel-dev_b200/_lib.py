"""ctypes binding of libb200nvfp4.so (the C ABI in include/b200_nvfp4.h).

There is no fallback: if the library is missing or a call fails, an exception is
raised.  The library is looked for next to this file (built in-tree by
``build.py``).
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200nvfp4.so")

VARIANT_AUTO, VARIANT_PERSISTENT, VARIANT_SERIAL, VARIANT_SERIAL_2MMA, VARIANT_SPLITK, VARIANT_PAIR = 0, 1, 2, 3, 4, 5

VARIANT_PAIR_NARROW, VARIANT_PAIR_STREAMK, VARIANT_SELFTEST_LOST_LOAD = 6, 7, 8

E_NULL, E_SHAPE, E_ALIGN, E_WORKSPACE, E_VARIANT, E_DRIVER, E_LIMIT, E_CAPTURE = -1, -2, -3, -4, -5, -6, -7, -8

STATIC_MAX_GROUPS = 64
DTYPE_F16, DTYPE_BF16 = 0, 1

_vp = ctypes.c_void_p
_i = ctypes.c_int
_i64 = ctypes.c_int64
_sz = ctypes.c_size_t
_u32p = ctypes.POINTER(ctypes.c_uint32)

SIGNATURES = {
    "b200_version": (ctypes.c_char_p, []),
    "b200_last_error": (ctypes.c_char_p, []),
    "b200_launch_count": (ctypes.c_uint64, []),
    "b200_last_kernel": (ctypes.c_char_p, []),
    "b200_dual_gemm_nvfp4": (_i, [_vp] * 7 + [_i] * 4 + [_i64, _vp, _i, _vp]),
    "b200_dual_gemm_nvfp4_ex": (_i, [_vp] * 7 + [_i] * 4 + [_i64] * 4 + [_i, _vp, _sz, _vp, _i, _vp]),
    "b200_dual_gemm_nvfp4_gather": (_i, [_vp] * 7 + [_i] * 7 + [_vp, _i, _vp]),
    "b200_dual_splitk_workspace_bytes": (_sz, [_i] * 4),
    "b200_dual_streamk_workspace_bytes": (_sz, [_i] * 4),
    "b200_grouped_gemm_nvfp4": (_i, [_i] + [_vp] * 6 + [_vp, _sz, _vp, _i, _vp]),
    "b200_grouped_gemm_nvfp4_ex": (_i, [_i] + [_vp] * 6 + [_vp, _sz, _i, _i, _vp, _i, _vp]),
    "b200_grouped_workspace_bytes": (_sz, [_i]),
    "b200_grouped_gemm_nvfp4_static": (_i, [_i] + [_vp] * 6 + [_vp, _i, _vp]),
    "b200_dual_gemm_nvfp4_quant": (_i, [_vp] * 8 + [_i] * 3 + [_vp, _i, _vp]),
    "b200_quantize_sf_bytes": (_sz, [_i, _i]),
    "b200_quantize_nvfp4": (_i, [_vp, _i, _i, _i, _i64, _vp, _vp, _vp, _i]),
    "b200_moe_route": (_i, [_vp, _vp, _i, _i, _i, _i, _i, ctypes.c_float, _vp, _vp, _vp, _i]),
    "b200_moe_plan_scratch_bytes": (_sz, [_i, _i, _i]),
    "b200_moe_plan": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _i]),
    "b200_moe_sfa_bytes": (_sz, [_i, _i, _i, _i]),
    "b200_moe_gather_scratch_bytes": (_sz, [_i, _i]),
    "b200_moe_gather_quantize": (_i, [_vp, _i, _i, _i, _i64, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _sz, _vp, _i]),
    "b200_moe_quantize_scatter": (_i, [_vp, _i, _i, _i, _i64, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _i]),
    "b200_moe_gemm_workspace_bytes": (_sz, [_i]),
    "b200_moe_grouped_gemm_nvfp4": (_i, [_i, _vp, _vp, _i, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _i, _vp]),
    "b200_moe_combine": (_i, [_vp, _i, _vp, _vp, _i, _i, _i, _vp, _i64, _vp, _i]),
    "b200_read_status": (_i, [_i, _vp, _u32p]),
    "b200_read_last_cycles": (_i, [_i, _vp, ctypes.POINTER(ctypes.c_uint64)]),
    "b200_probe_l2_feed": (_i, [_i, _i, _i, _i, _i, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double),
                                ctypes.POINTER(ctypes.c_double)]),
    "b200_grouped_workspace_forget": (_i, [_i, _vp]),
}

_lib = None


class B200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libb200nvfp4 error {code}: {message}")
        self.code = code


def load() -> ctypes.CDLL:
    """Load the shared library (once) and declare every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python __graft_entry__.py` or "
            f"`python llm-assisted-kernel-dev_b200/build.py` (needs nvcc). There is no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)        # AttributeError if a declared symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(code: int) -> None:
    """Raise for a non-zero return: ValueError for rejected arguments (< 0),
    B200Error for CUDA errors (> 0)."""
    if code == 0:
        return
    msg = load().b200_last_error().decode()
    if code < 0:
        err = ValueError(f"libb200nvfp4 rejected the call ({code}): {msg}")
        err.code = code
        raise err
    raise B200Error(code, msg)


def read_status(device: int, stream: int = 0) -> int:
    out = ctypes.c_uint32(0)
    check(load().b200_read_status(device, stream, ctypes.byref(out)))
    return out.value


def raise_on_status(device: int, stream: int = 0) -> None:
    """Synchronise and raise B200Error if a bounded on-device wait gave up since the last check."""
    word = read_status(device, stream)
    if word:
        raise B200Error(word, f"device status word {word:#x}: an on-device wait ran out (bits: 1 producer, 2/4 MMA, "
                              f"8 epilogue, 0x10 serial, 0x20 split-k, 0x40 scale factors, 0x80 CTA pair)")


def last_launch_cycles(device: int, stream: int = 0) -> int:
    """SM-clock cycles the first CTA of the last GEMM launch on ``device`` ran for."""
    out = ctypes.c_uint64(0)
    check(load().b200_read_last_cycles(device, stream, ctypes.byref(out)))
    return int(out.value)


def probe_l2_feed(device: int, ctas: int, share: int = 1, tiled: bool = True, copies_per_cta: int = 8000) -> dict:
    """Rate at which TMA loads alone fill shared memory from L2 (``b200_probe_l2_feed``): aggregate TB/s,
    bytes per SM clock of the slowest CTA, SM clock during the run."""
    tbs, bpc, mhz = ctypes.c_double(0), ctypes.c_double(0), ctypes.c_double(0)
    check(load().b200_probe_l2_feed(device, ctas, share, 1 if tiled else 0, copies_per_cta, ctypes.byref(tbs),
                                    ctypes.byref(bpc), ctypes.byref(mhz)))
    return {"ctas": ctas, "share": share, "tiled": bool(tiled), "tb_per_s": tbs.value,
            "bytes_per_clk_per_sm": bpc.value, "sm_mhz": mhz.value}


def last_kernel() -> str:
    return load().b200_last_kernel().decode()


def launch_count() -> int:
    return int(load().b200_launch_count())
