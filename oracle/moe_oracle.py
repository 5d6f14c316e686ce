"""CPU oracle for the mixture-of-experts steps around the NVFP4 grouped GEMM.

TEST INFRASTRUCTURE ONLY: imported by tests/ and nothing else.  Restates with torch CPU ops

* the reference's DeepSeek-V3 "no-aux" routing: sigmoid, bias, group scores = sum of the
  two largest biased scores of a group, topk_group groups kept, top_k experts among them,
  weights = unbiased score / (their sum + 1e-20) * scale  (moe/moe_fibench_ref.py:106-134);
* its per-expert token selection in token order (``nonzero`` of the selection mask,
  moe/moe_fibench_ref.py:144-149), its gather (:152) and its weighted fp32 accumulation
  with ``index_add_`` in expert order (:172-176).

Pins: ``route`` is checked against vectors produced by *executing the reference's own routing
lines* (tests/golden/make_moe_golden.py -> tests/golden/moe_routing_vectors.npz).  The expert
arithmetic of the reference is FP8 with 128-block scales (moe/moe_fibench_ref.py:74-101) and
cannot pin an NVFP4 path: the per-expert product here is the NVFP4 oracle (quantise_nvfp4 ->
dequantise -> fp32 matmul -> fp16) and that part of the parity is UNPINNED.
"""
from __future__ import annotations

import torch

from . import nvfp4_oracle as orc


def route(logits: torch.Tensor, bias, n_group: int, topk_group: int, top_k: int, scale: float,
          exact_sigmoid: bool = False):
    """Returns (topk_idx [T, top_k] int64, unordered like the reference's, and the dense weight
    matrix [T, E] fp32)."""
    logits = logits.detach().cpu().float()
    t, e = logits.shape
    b = torch.zeros(e) if bias is None else bias.detach().cpu().float().reshape(-1)
    if exact_sigmoid:
        # in double precision, rounded to fp32: the correctly rounded value of the reference's fp32 expression
        # (moe/moe_fibench_ref.py:103), independent of which vectorised fp32 exp the host's torch build dispatches
        # to (on one machine a large tensor's fp32 exp came back 1e-5 off in about one process out of a dozen)
        s = (1.0 / (1.0 + torch.exp(-logits.double()))).float()
    else:
        s = 1.0 / (1.0 + torch.exp(-logits))      # the reference's expression, bit for bit
    swb = s + b
    group_size = e // n_group
    grouped = swb.view(t, n_group, group_size)
    top2, _ = torch.topk(grouped, k=min(2, group_size), dim=2, largest=True, sorted=False)
    group_scores = top2.sum(dim=2)
    _, group_idx = torch.topk(group_scores, k=topk_group, dim=1, largest=True, sorted=False)
    group_mask = torch.zeros_like(group_scores)
    group_mask.scatter_(1, group_idx, 1.0)
    score_mask = group_mask.unsqueeze(2).expand(t, n_group, group_size).reshape(t, e)
    pruned = swb.masked_fill(score_mask == 0, torch.finfo(torch.float32).min)
    _, topk_idx = torch.topk(pruned, k=top_k, dim=1, largest=True, sorted=False)
    m = torch.zeros_like(s)
    m.scatter_(1, topk_idx, 1.0)
    weights = s * m
    weights = weights / (weights.sum(dim=1, keepdim=True) + 1e-20) * scale
    return topk_idx, weights


def plan(topk_idx: torch.Tensor, experts: int):
    """counts [E], row_offsets [E + 1] and, per expert, its tokens in ascending order."""
    tokens_of = []
    for e in range(experts):
        sel = (topk_idx == e).any(dim=1)
        tokens_of.append(torch.nonzero(sel, as_tuple=False).squeeze(1))
    counts = torch.tensor([len(x) for x in tokens_of], dtype=torch.int64)
    offsets = torch.zeros(experts + 1, dtype=torch.int64)
    offsets[1:] = torch.cumsum(counts, 0)
    return counts, offsets, tokens_of


def moe_forward(x: torch.Tensor, logits, bias, b_list, sfb_list, n_group, topk_group, top_k, scale,
                out_dtype=torch.bfloat16):
    """out [T, n]; b_list[e] [n, k/2, 1] packed e2m1 bytes, sfb_list[e] [n, k/16, 1] e4m3 (un-reordered)."""
    x = x.detach().cpu()
    t, k = x.shape
    experts = len(b_list)
    topk_idx, weights = route(logits, bias, n_group, topk_group, top_k, scale, exact_sigmoid=True)
    _counts, _offsets, tokens_of = plan(topk_idx, experts)
    n = orc.as_u8(b_list[0]).shape[0]
    out = torch.zeros((t, n), dtype=torch.float32)
    for e in range(experts):
        tok = tokens_of[e]
        if tok.numel() == 0:
            continue
        a_e = x.index_select(0, tok)
        packed, sf = orc.quantize_nvfp4(a_e)
        y = orc.gemm_fp32(packed.unsqueeze(-1), sf.unsqueeze(-1), b_list[e], sfb_list[e])[:, :, 0].to(torch.float16)
        w = weights.index_select(0, tok)[:, e]
        out.index_add_(0, tok, y.float() * w.unsqueeze(1))
    return out.to(out_dtype), topk_idx, weights
