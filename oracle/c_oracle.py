"""ctypes binding of the plain-C oracle (oracle/nvfp4_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/ and by the benchmark's CPU-baseline
leg, never by the shipped package.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle_nvfp4.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "nvfp4_oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-B", "liboracle_nvfp4.so"], check=True, capture_output=True)
    return LIB


def load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(build())
        vp, i, lg = ctypes.c_void_p, ctypes.c_int, ctypes.c_long
        lib.oracle_dual_gemm.restype = i
        lib.oracle_dual_gemm.argtypes = [vp] * 7 + [i, i, i, lg]
        lib.oracle_gemm.restype = i
        lib.oracle_gemm.argtypes = [vp] * 5 + [i, i, i, lg]
        lib.oracle_e4m3_to_f32.restype = ctypes.c_float
        lib.oracle_e4m3_to_f32.argtypes = [ctypes.c_uint8]
        lib.oracle_f32_to_f16.restype = ctypes.c_uint16
        lib.oracle_f32_to_f16.argtypes = [ctypes.c_float]
        _lib = lib
    return _lib


def _dense_bytes(t: torch.Tensor) -> np.ndarray:
    """Bytes of a [rows, cols, 1] operand, row-major."""
    return np.ascontiguousarray(t.detach().cpu().view(torch.uint8)[:, :, 0].numpy())


def _sf_buffer(perm: torch.Tensor) -> np.ndarray:
    """The dense (rest_mn, rest_k, 32, 4, 4) byte buffer behind a permuted view (L == 1)."""
    u8 = perm.detach().cpu().view(torch.uint8)
    return np.ascontiguousarray(u8.permute(5, 2, 4, 0, 1, 3)[0].numpy())


def dual_gemm(data) -> torch.Tensor:
    """fp16 [M, N, 1] from the C oracle, reading the permuted scale factors."""
    a, b1, b2 = (_dense_bytes(t) for t in data[:3])
    sfa, sfb1, sfb2 = (_sf_buffer(t) for t in data[6:9])
    m, n, k = a.shape[0], b1.shape[0], a.shape[1] * 2
    out = np.zeros((m, n), dtype=np.uint16)
    rc = load().oracle_dual_gemm(a.ctypes.data, b1.ctypes.data, b2.ctypes.data, sfa.ctypes.data,
                                 sfb1.ctypes.data, sfb2.ctypes.data, out.ctypes.data, m, n, k, n)
    if rc:
        raise MemoryError("oracle_dual_gemm failed")
    return torch.from_numpy(out.view(np.float16).copy()).unsqueeze(-1)


def gemm(a, b, sfa_perm, sfb_perm) -> torch.Tensor:
    """fp16 [M, N, 1] = A.B^T from the C oracle (grouped path, one group)."""
    an, bn = _dense_bytes(a), _dense_bytes(b)
    m, n, k = an.shape[0], bn.shape[0], bn.shape[1] * 2
    out = np.zeros((m, n), dtype=np.uint16)
    if m:
        rc = load().oracle_gemm(an.ctypes.data, bn.ctypes.data, _sf_buffer(sfa_perm).ctypes.data,
                                _sf_buffer(sfb_perm).ctypes.data, out.ctypes.data, m, n, k, n)
        if rc:
            raise MemoryError("oracle_gemm failed")
    return torch.from_numpy(out.view(np.float16).copy()).unsqueeze(-1)
