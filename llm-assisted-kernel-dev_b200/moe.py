"""Mixture-of-experts layer around the NVFP4 grouped GEMM on B200: routing, permutation of
token rows into per-expert ranges (with quantisation to NVFP4), one grouped GEMM over all
experts, weighted combination.

Mirrors the structure of the reference's MoE (moe/moe_fibench_ref.py:20-33: DeepSeek-V3
no-aux routing :106-134, per-expert token gather :144-153, expert GEMM :155-170, weighted
accumulation :172-176) with one NVFP4 GEMM per expert instead of its FP8 GEMM1 -> SwiGLU ->
GEMM2.  All arithmetic runs in libb200nvfp4.so (csrc/moe_kernels.cuh and the grouped GEMM
kernels); nothing here computes on the CPU and nothing is read back to the host between
the steps."""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .formats import is_kernel_sf_layout


class MoEWeights:
    """The experts' weights, quantised: ``b[e]`` [n, k/2, 1] packed e2m1 and ``sfb_perm[e]`` the
    reordered (32, 4, n/128, 4, k/64, 1) scale factors -- the layout ``group_gemm`` takes."""

    def __init__(self, b, sfb_perm):
        if len(b) == 0 or len(b) != len(sfb_perm):
            raise ValueError("need one weight tensor and one scale-factor tensor per expert")
        self.experts = len(b)
        self.n, half_k = b[0].shape[0], b[0].shape[1]
        self.k = half_k * 2
        dev = b[0].device
        if dev.type != "cuda":
            raise ValueError("MoE weights must be CUDA tensors (there is no CPU path)")
        for i, (w, sf) in enumerate(zip(b, sfb_perm)):
            if tuple(w.shape) != (self.n, half_k, 1) or w.stride(1) != 1 or w.stride(0) != half_k:
                raise ValueError(f"expert {i}: weights must be [n, k/2, 1] K-major packed bytes")
            if not is_kernel_sf_layout(sf, self.n, self.k, 1):
                raise ValueError(f"expert {i}: scale factors are not in the reordered (32,4,rest,4,K/64,1) layout")
            if w.device != dev or sf.device != dev:
                raise ValueError("all weights must live on the same CUDA device")
        self.device = dev
        self._keep = (list(b), list(sfb_perm))
        arr = ctypes.c_void_p * self.experts
        self.b_ptrs = arr(*[w.data_ptr() for w in b])
        self.sfb_ptrs = arr(*[sf.data_ptr() for sf in sfb_perm])


class _Buffers:
    """Device buffers of one (tokens, experts, top_k, k, n) configuration, allocated once."""

    def __init__(self, lib, dev, tokens, experts, top_k, k, n):
        rows = tokens * top_k
        i32 = dict(dtype=torch.int32, device=dev)
        self.topk_idx = torch.empty((tokens, top_k), **i32)
        self.topk_w = torch.empty((tokens, top_k), dtype=torch.float32, device=dev)
        self.counts = torch.empty(experts, **i32)
        self.row_offsets = torch.empty(experts + 1, **i32)
        self.sfa_atom_offsets = torch.empty(experts + 1, **i32)
        self.row_of = torch.empty(rows, **i32)
        self.src_token = torch.empty(rows, **i32)
        self.scratch = torch.empty(max(1, int(lib.b200_moe_plan_scratch_bytes(tokens, experts, top_k))),
                                   dtype=torch.uint8, device=dev)
        self.a_q = torch.empty((rows, k // 2), dtype=torch.uint8, device=dev)
        self.sfa = torch.zeros(int(lib.b200_moe_sfa_bytes(tokens, experts, top_k, k)), dtype=torch.uint8, device=dev)
        self.y = torch.empty((rows, n), dtype=torch.float16, device=dev)
        ws_bytes = int(lib.b200_moe_gemm_workspace_bytes(experts))
        self.ws = torch.empty(ws_bytes + 256, dtype=torch.uint8, device=dev)
        self.ws_ptr = (self.ws.data_ptr() + 255) & ~255
        self.ws_bytes = ws_bytes


_buffers: dict = {}


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return _lib.DTYPE_F16
    if t.dtype == torch.bfloat16:
        return _lib.DTYPE_BF16
    raise ValueError(f"expected float16 or bfloat16, got {t.dtype}")


def route(logits: torch.Tensor, bias, n_group: int, topk_group: int, top_k: int, routed_scaling: float = 1.0,
          out=None):
    """``(topk_idx [T, top_k] int32, topk_w [T, top_k] float32)`` of the no-aux routing
    (moe/moe_fibench_ref.py:106-134); slots in descending order of the biased score."""
    if not logits.is_cuda:
        raise ValueError("route needs CUDA tensors (there is no CPU path)")
    if logits.dtype != torch.float32 or logits.dim() != 2 or not logits.is_contiguous():
        raise ValueError("logits must be a contiguous float32 [tokens, experts] tensor")
    tokens, experts = logits.shape
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != experts or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous float32 [experts] tensor")
    dev = logits.device
    idx, w = out if out is not None else (torch.empty((tokens, top_k), dtype=torch.int32, device=dev),
                                          torch.empty((tokens, top_k), dtype=torch.float32, device=dev))
    code = _lib.load().b200_moe_route(logits.data_ptr(), bias.data_ptr() if bias is not None else None, tokens, experts,
                                      n_group, topk_group, top_k, float(routed_scaling), idx.data_ptr(), w.data_ptr(),
                                      torch.cuda.current_stream(dev).cuda_stream, dev.index)
    _lib.check(code)
    return idx, w


def moe_forward(x: torch.Tensor, logits: torch.Tensor, bias, weights: MoEWeights, *, n_group: int = 1,
                topk_group: int = 1, top_k: int = 8, routed_scaling: float = 1.0, out_dtype=torch.bfloat16,
                return_plan: bool = False):
    """``out[t] = sum_e weight[t, e] * (quantise(x[t]) @ W_e.T)`` over the token's ``top_k`` experts.

    x        [tokens, k] fp16 / bf16 activations (unit stride along k)
    logits   [tokens, experts] fp32 router logits, ``bias`` [experts] fp32 or None
    weights  ``MoEWeights`` (NVFP4 expert weights)
    Five launches (+ a one-block table kernel) on the current stream, no host synchronisation.
    """
    if not x.is_cuda:
        raise ValueError("moe_forward needs CUDA tensors (there is no CPU path)")
    if x.dim() != 2 or x.stride(1) != 1 or x.shape[1] != weights.k:
        raise ValueError(f"x must be [tokens, {weights.k}] with unit stride along k")
    tokens, k = x.shape
    experts, n = weights.experts, weights.n
    if tuple(logits.shape) != (tokens, experts):
        raise ValueError(f"logits must be [{tokens}, {experts}]")
    lib = _lib.load()
    dev = x.device
    key = (dev.index, tokens, experts, top_k, k, n)
    buf = _buffers.get(key)
    if buf is None:
        buf = _buffers[key] = _Buffers(lib, dev, tokens, experts, top_k, k, n)
    stream = torch.cuda.current_stream(dev).cuda_stream
    route(logits, bias, n_group, topk_group, top_k, routed_scaling, out=(buf.topk_idx, buf.topk_w))
    _lib.check(lib.b200_moe_plan(buf.topk_idx.data_ptr(), tokens, experts, top_k, buf.counts.data_ptr(),
                                 buf.row_offsets.data_ptr(), buf.sfa_atom_offsets.data_ptr(), buf.row_of.data_ptr(),
                                 buf.src_token.data_ptr(), buf.scratch.data_ptr(), buf.scratch.numel(), stream, dev.index))
    _lib.check(lib.b200_moe_quantize_scatter(x.data_ptr(), _dtype_code(x), tokens, k, x.stride(0), buf.row_of.data_ptr(),
                                             buf.row_offsets.data_ptr(), buf.sfa_atom_offsets.data_ptr(), experts, top_k,
                                             buf.a_q.data_ptr(), buf.sfa.data_ptr(), stream, dev.index))
    _lib.check(lib.b200_moe_grouped_gemm_nvfp4(experts, buf.a_q.data_ptr(), buf.sfa.data_ptr(), tokens * top_k,
                                               weights.b_ptrs, weights.sfb_ptrs, n, k, buf.counts.data_ptr(),
                                               buf.row_offsets.data_ptr(), buf.sfa_atom_offsets.data_ptr(),
                                               buf.y.data_ptr(), buf.ws_ptr, buf.ws_bytes, stream, dev.index, None))
    out = torch.empty((tokens, n), dtype=out_dtype, device=dev)
    _lib.check(lib.b200_moe_combine(buf.y.data_ptr(), n, buf.row_of.data_ptr(), buf.topk_w.data_ptr(), tokens, top_k,
                                    _dtype_code(out), out.data_ptr(), out.stride(0), stream, dev.index))
    return (out, buf) if return_plan else out
