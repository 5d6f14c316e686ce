"""Seeded synthetic inputs in the reference's tuple layouts.

Mirrors ``generate_input`` of the reference (dual: dual_gemm/reference.py:81-197;
grouped: group_gemm/group_gemm_cute5_v2.py:4538-4702) -- same tensor shapes,
strides, dtypes and placement -- with two operand distributions:

``"reference"``  codes ``randint(255) & 0xBB`` (values 0, +-0.5, +-1, +-1.5) and
                 scale factors ``rand[0,1) -> e4m3`` (dual_gemm/reference.py:117-121,146-147)
``"uniform16"``  codes uniform over all 16 e2m1 values, scale factors uniform in
                 [0.25, 2] rounded to e4m3 (the benchmark configurations)

Random draws come from a CPU ``torch.Generator`` so the bytes are identical on
every machine; tensors are then moved to ``device``.
"""
from __future__ import annotations

import torch

from .formats import E4M3, FP4X2, SF_VEC, ceil_div, permute_scale_factors

E2M1_CODE = {0.0: 0x0, 0.5: 0x1, 1.0: 0x2, 1.5: 0x3, 2.0: 0x4, 3.0: 0x5, 4.0: 0x6, 6.0: 0x7,
             -0.5: 0x9, -1.0: 0xA, -1.5: 0xB, -2.0: 0xC, -3.0: 0xD, -4.0: 0xE, -6.0: 0xF}


def _fp4_bytes(gen, l, mn, k, dist):
    if dist == "reference":
        raw = torch.randint(255, (l, mn, k // 2), dtype=torch.uint8, generator=gen)
        raw = raw & 0b1011_1011
    elif dist == "uniform16":
        raw = torch.randint(256, (l, mn, k // 2), dtype=torch.uint8, generator=gen)
    else:
        raise ValueError(f"unknown distribution {dist!r}")
    return raw


def _sf_e4m3(gen, l, mn, sf_k, dist):
    r = torch.rand((l, mn, sf_k), dtype=torch.float32, generator=gen)
    if dist == "uniform16":
        r = 0.25 + 1.75 * r
    return r.to(E4M3)


def _as_fp4(raw_lmk: torch.Tensor, device) -> torch.Tensor:
    """(L, rows, K/2) bytes -> [rows, K/2, L] fp4x2 view, strides (K/2, 1, rows*K/2)."""
    return raw_lmk.to(device).permute(1, 2, 0).view(FP4X2)


def _sf_pair(gen, l, mn, sf_k, dist, device, random_padding):
    sf = _sf_e4m3(gen, l, mn, sf_k, dist).permute(1, 2, 0)          # [mn, sf_k, L]
    pad = None
    if random_padding:
        nbytes = l * ceil_div(mn, 128) * ceil_div(sf_k, 4) * 512
        pad = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, generator=gen)
    return sf, _to_device_keep_strides(permute_scale_factors(sf, pad), device)


def _to_device_keep_strides(view: torch.Tensor, device) -> torch.Tensor:
    """Move a permuted view to ``device`` preserving its strides (``.to`` may
    re-pack a non-contiguous tensor)."""
    if str(device) == "cpu":
        return view
    l = view.shape[5]
    rm, rk = view.shape[2], view.shape[4]
    dense = view.view(torch.uint8).permute(5, 2, 4, 0, 1, 3).contiguous()
    assert dense.shape == (l, rm, rk, 32, 4, 4)
    return dense.to(device).permute(3, 4, 1, 5, 2, 0).view(E4M3)


def generate_input(m: int, n: int, k: int, l: int, seed: int, dist: str = "reference",
                   device: str = "cuda"):
    """Dual-GEMM 10-tuple ``(a, b1, b2, sfa, sfb1, sfb2, sfa_perm, sfb1_perm,
    sfb2_perm, c)``; argument meaning as dual_gemm/reference.py:81-112."""
    gen = torch.Generator().manual_seed(seed)
    a = _as_fp4(_fp4_bytes(gen, l, m, k, dist), device)
    b1 = _as_fp4(_fp4_bytes(gen, l, n, k, dist), device)
    b2 = _as_fp4(_fp4_bytes(gen, l, n, k, dist), device)
    sf_k = ceil_div(k, SF_VEC)
    sfa, sfa_p = _sf_pair(gen, l, m, sf_k, dist, device, False)
    sfb1, sfb1_p = _sf_pair(gen, l, n, sf_k, dist, device, False)
    sfb2, sfb2_p = _sf_pair(gen, l, n, sf_k, dist, device, False)
    c = torch.randn((l, m, n), dtype=torch.float32, generator=gen).to(torch.float16)
    c = c.to(device).permute(1, 2, 0)
    return (a, b1, b2, sfa.to(device), sfb1.to(device), sfb2.to(device), sfa_p, sfb1_p, sfb2_p, c)


def _kat_fp4(rows, k, l, kind, single=None):
    t = torch.zeros((l, rows, k // 2), dtype=torch.uint8)
    if kind == "identity":
        idx = torch.arange(min(rows, k))
        t[:, idx, idx // 2] |= torch.where(idx % 2 == 0, 0x02, 0x20).to(torch.uint8)
    elif kind == "constant":
        t.fill_(0x22)
    elif kind == "single":
        r, c, val = single
        code = E2M1_CODE[float(val)]
        t[:, r, c // 2] = code << 4 if c % 2 else code
    return t


def generate_grouped_input(m, n, k, g: int, seed: int, dist: str = "reference", device: str = "cuda",
                           identity_a=False, identity_b=False, constant_a=False, constant_b=False,
                           single_a=None, unit_sfa=False, unit_sfb=False, fill_c=None,
                           random_sf_padding=True):
    """Grouped 4-tuple ``(abc_tensors, sfasfb_tensors, sfasfb_reordered_tensors,
    problem_sizes)``; options follow the reference's known-answer input modes
    (group_gemm/group_gemm_cute5_v2.py:4538-4702).  Scale factors use the chosen
    distribution (never NaN); padding rows of the reordered scale factors hold
    random bytes like the reference's."""
    gen = torch.Generator().manual_seed(seed)
    abc, sfs, sfs_perm, sizes = [], [], [], []
    l = 1
    for gi in range(g):
        mi, ni, ki = int(m[gi]), int(n[gi]), int(k[gi])
        sf_k = ceil_div(ki, SF_VEC)
        if identity_a:
            a_raw = _kat_fp4(mi, ki, l, "identity")
        elif constant_a:
            a_raw = _kat_fp4(mi, ki, l, "constant")
        elif single_a is not None:
            a_raw = _kat_fp4(mi, ki, l, "single", single_a)
        else:
            a_raw = _fp4_bytes(gen, l, mi, ki, dist)
        if identity_b:
            b_raw = _kat_fp4(ni, ki, l, "identity")
        elif constant_b:
            b_raw = _kat_fp4(ni, ki, l, "constant")
        else:
            b_raw = _fp4_bytes(gen, l, ni, ki, dist)
        if fill_c is not None:
            c = torch.full((l, mi, ni), float(fill_c), dtype=torch.float16)
        else:
            c = torch.randn((l, mi, ni), dtype=torch.float32, generator=gen).to(torch.float16)
        if unit_sfa:
            sfa = torch.full((l, mi, sf_k), 0x38, dtype=torch.uint8).view(E4M3).permute(1, 2, 0)
            sfa_p = _to_device_keep_strides(permute_scale_factors(sfa), device)
        else:
            sfa, sfa_p = _sf_pair(gen, l, mi, sf_k, dist, device, random_sf_padding)
        if unit_sfb:
            sfb = torch.full((l, ni, sf_k), 0x38, dtype=torch.uint8).view(E4M3).permute(1, 2, 0)
            sfb_p = _to_device_keep_strides(permute_scale_factors(sfb), device)
        else:
            sfb, sfb_p = _sf_pair(gen, l, ni, sf_k, dist, device, False)
        abc.append((_as_fp4(a_raw, device), _as_fp4(b_raw, device), c.to(device).permute(1, 2, 0)))
        sfs.append((sfa, sfb))              # CPU, like the reference (:4657-4670)
        sfs_perm.append((sfa_p, sfb_p))
        sizes.append((mi, ni, ki, l))
    return (abc, sfs, sfs_perm, sizes)


def grouped_to_device(data, device):
    """Move a grouped 4-tuple generated on the CPU to ``device``, keeping every stride
    (the un-reordered scale factors stay on the CPU, like the reference's)."""
    abc, sfs, sfs_perm, sizes = data

    def op(t):
        return t.view(torch.uint8).permute(2, 0, 1).contiguous().to(device).permute(1, 2, 0).view(FP4X2)

    def out(t):
        return t.permute(2, 0, 1).contiguous().to(device).permute(1, 2, 0)
    return ([(op(a), op(b), out(c)) for (a, b, c) in abc], list(sfs),
            [(_to_device_keep_strides(x, device), _to_device_keep_strides(y, device)) for (x, y) in sfs_perm],
            list(sizes))


def moe_expert_counts(tokens: int, experts: int, top_k: int, seed: int) -> list[int]:
    """Tokens routed to each expert by top-k of softmax(N(0,1) logits); counts
    sum to tokens*top_k and may contain zeros."""
    gen = torch.Generator().manual_seed(seed)
    logits = torch.randn((tokens, experts), dtype=torch.float32, generator=gen)
    choice = torch.softmax(logits, dim=-1).topk(top_k, dim=-1).indices
    return torch.bincount(choice.flatten(), minlength=experts).tolist()


def uniform_group_rows(g: int, seed: int, choices=tuple(range(64, 1025, 64))) -> list[int]:
    """M_i drawn uniformly from ``choices`` (the G=8 grouped benchmark)."""
    gen = torch.Generator().manual_seed(seed)
    idx = torch.randint(len(choices), (g,), generator=gen)
    return [choices[i] for i in idx.tolist()]
