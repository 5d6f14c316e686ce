"""NVFP4 operand and scale-factor formats used on the dual / grouped GEMM path.

Host-side layout arithmetic only (index maps, shapes, byte counts); no matrix
arithmetic lives here.

* operands: e2m1, two per byte, element 2j in the low nibble of byte j
  (reference: group_gemm/group_gemm_cute5_v2.py:4444-4449)
* scale factors: one ``float8_e4m3fn`` byte per 16 consecutive k
  (reference: dual_gemm/reference.py:6,146-147)
* kernel-facing scale-factor layout: a contiguous (L, rest_mn, rest_k, 32, 4, 4)
  byte buffer viewed as (32, 4, rest_mn, 4, rest_k, L)
  (reference: dual_gemm/reference.py:151-188)
"""
from __future__ import annotations

import torch

SF_VEC = 16          # k elements per scale factor
SF_ROW_ATOM = 128    # rows covered by one 512-byte scale-factor atom
SF_K_ATOM = 4        # scale factors (= 64 k) covered by one atom
TILE_M = 128
TILE_N = 128
TILE_K = 256

FP4X2 = getattr(torch, "float4_e2m1fn_x2", torch.uint8)
E4M3 = torch.float8_e4m3fn


def ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def sf_atoms(mn: int, k: int) -> tuple[int, int]:
    """(rest_mn, rest_k): number of 512-byte atoms along rows and along k."""
    return ceil_div(mn, SF_ROW_ATOM), ceil_div(ceil_div(k, SF_VEC), SF_K_ATOM)


def sf_perm_bytes(mn: int, k: int, l: int = 1) -> int:
    rm, rk = sf_atoms(mn, k)
    return l * rm * rk * 512


def sf_offset(i: int, j: int, b: int, rest_mn: int, rest_k: int) -> int:
    """Byte offset of scale factor (row i, 16-k block j, batch b) in the
    kernel-facing buffer."""
    return (((b * rest_mn + i // 128) * rest_k + j // 4) * 512
            + (i % 32) * 16 + ((i % 128) // 32) * 4 + (j % 4))


def permute_scale_factors(sf: torch.Tensor, pad_bytes: torch.Tensor | None = None) -> torch.Tensor:
    """[mn, sf_k, L] e4m3 -> kernel-facing (32, 4, rest_mn, 4, rest_k, L) view
    with strides (16, 4, 512*rest_k, 1, 512, 512*rest_k*rest_mn).

    Rows beyond ``mn`` keep whatever ``pad_bytes`` holds (the reference leaves
    them uninitialised / random: dual_gemm/reference.py:166-167,
    group_gemm/group_gemm_cute5_v2.py:4506); zero when not given."""
    u8 = sf.view(torch.uint8)
    mn, sf_k, l = u8.shape
    rest_mn, rest_k = ceil_div(mn, 128), ceil_div(sf_k, 4)
    shape = (l, rest_mn, rest_k, 32, 4, 4)
    if pad_bytes is None:
        buf = torch.zeros(shape, dtype=torch.uint8, device=u8.device)
    else:
        buf = pad_bytes.to(u8.device).view(torch.uint8).reshape(shape).clone()
    view = buf.permute(3, 4, 1, 5, 2, 0)
    i = torch.arange(mn, device=u8.device).view(-1, 1, 1)
    j = torch.arange(sf_k, device=u8.device).view(1, -1, 1)
    b = torch.arange(l, device=u8.device).view(1, 1, -1)
    view[i % 32, (i % 128) // 32, i // 128, j % 4, j // 4, b] = u8
    return view.view(E4M3)


def is_kernel_sf_layout(t: torch.Tensor, mn: int, k: int, l: int) -> bool:
    """True when ``t`` is the (32,4,rest_mn,4,rest_k,L) view of a dense
    (L,rest_mn,rest_k,32,4,4) buffer, i.e. what the kernels index."""
    rm, rk = sf_atoms(mn, k)
    if tuple(t.shape) != (32, 4, rm, 4, rk, l) or t.element_size() != 1:
        return False
    want = (16, 4, 512 * rk, 1, 512, 512 * rk * rm)
    return all(sz == 1 or st == w for sz, st, w in zip(t.shape, t.stride(), want))


def dual_gemm_flops(m: int, n: int, k: int, l: int = 1) -> int:
    """Two GEMMs of 2*M*N*K each; epilogue not counted."""
    return 4 * m * n * k * l


def dual_gemm_bytes(m: int, n: int, k: int, l: int = 1) -> int:
    """Algorithmic bytes: packed operands + scale factors + fp16 output, once."""
    return l * (m * k // 2 + 2 * (n * k // 2) + m * k // 16 + 2 * (n * k // 16) + 2 * m * n)


def grouped_gemm_flops(problem_sizes) -> int:
    return sum(2 * m * n * k * l for (m, n, k, l) in problem_sizes)


def grouped_gemm_bytes(problem_sizes) -> int:
    """Reference accounting (group_gemm/group_gemm_cute4.py:1910-1913) with the
    A-side scale factors padded to 128-row atoms."""
    total = 0
    for (m, n, k, l) in problem_sizes:
        total += l * (m * k // 2 + n * k // 2 + ceil_div(m, 128) * 128 * k // 16 + n * k // 16 + 2 * m * n)
    return total
