"""Generate tests/golden/reference_vectors.npz by running the reference's own
helper functions (unmodified, imported from a checkout of
whatdhack/llm-assisted-kernel-dev) on the CPU.

Usage (only where the reference checkout is available):
    python tests/golden/make_golden.py /path/to/llm-assisted-kernel-dev

The reference allocates on "cuda" and its oracle calls ``torch._scaled_mm`` with
fp4 operands, neither of which exists on a CPU-only machine.  This script runs
the reference's *input generators and layout helpers* (not its GEMM) with a
small device shim that turns ``device="cuda"`` / ``.cuda()`` into CPU
placement; the arithmetic of those helpers is pure index manipulation, so the
bytes are what a GPU run would produce for the same random draws.  The vectors
pin: the e2m1 decode table and nibble order (``nvfp4_to_fp16``), ``to_blocked``
(both copies), and the permuted scale-factor layout written by the reference's
index scatter (dual ``generate_input`` and grouped
``create_reordered_scale_factor_tensor``).
"""
from __future__ import annotations

import contextlib
import importlib.util
import os
import sys
import types

import numpy as np
import torch

_FACTORIES = ["randint", "rand", "randn", "empty", "arange", "full", "zeros", "ones", "tensor"]


@contextlib.contextmanager
def cpu_device_shim():
    saved = {name: getattr(torch, name) for name in _FACTORIES}
    saved_cuda = torch.Tensor.cuda
    saved_to = torch.Tensor.to

    def wrap(fn):
        def inner(*args, **kwargs):
            if str(kwargs.get("device", "")).startswith("cuda"):
                kwargs["device"] = "cpu"
            return fn(*args, **kwargs)
        return inner

    def to(self, *args, **kwargs):
        args = tuple("cpu" if isinstance(a, str) and a.startswith("cuda") else a for a in args)
        if str(kwargs.get("device", "")).startswith("cuda"):
            kwargs["device"] = "cpu"
        return saved_to(self, *args, **kwargs)

    try:
        for name, fn in saved.items():
            setattr(torch, name, wrap(fn))
        torch.Tensor.cuda = lambda self, *a, **k: self
        torch.Tensor.to = to
        yield
    finally:
        for name, fn in saved.items():
            setattr(torch, name, fn)
        torch.Tensor.cuda = saved_cuda
        torch.Tensor.to = saved_to


def load_module(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def u8(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).numpy() if t.dtype != torch.uint8 else t.contiguous().numpy()


def main(ref_root: str) -> None:
    out = {}
    # --- dual GEMM reference.py (needs its task.py / utils.py on sys.path)
    sys.path.insert(0, os.path.join(ref_root, "utils", "dual_gemm"))
    dual_ref = load_module(os.path.join(ref_root, "dual_gemm", "reference.py"), "ref_dual_reference")
    sys.path.pop(0)

    sf = torch.arange(256 * 8, dtype=torch.int64).remainder(251).to(torch.uint8).view(256, 8)
    out["to_blocked_in"] = sf.numpy()
    out["to_blocked_out"] = dual_ref.to_blocked(sf).numpy()

    with cpu_device_shim():
        data = dual_ref.generate_input(m=128, n=256, k=512, l=2, seed=1111)
    names = ["a", "b1", "b2", "sfa", "sfb1", "sfb2", "sfa_perm", "sfb1_perm", "sfb2_perm"]
    for name, t in zip(names, data[:9]):
        out["dual_" + name] = u8(t) if "perm" not in name else u8(t.permute(5, 2, 4, 0, 1, 3))
        out["dual_" + name + "_shape"] = np.array(t.shape)
        out["dual_" + name + "_stride"] = np.array(t.stride())

    # --- grouped helpers live in group_gemm_cute5_v2.py, which imports modal at
    # top level; a stub module is enough for the import to succeed.
    for missing in ("modal",):
        if missing not in sys.modules:
            stub = types.ModuleType(missing)

            class _Any:
                def __init__(self, *a, **k): pass
                def __call__(self, *a, **k): return _Any()
                def __getattr__(self, _): return _Any()
            stub.__getattr__ = lambda _name: _Any()
            sys.modules[missing] = stub
    os.environ.setdefault("CUTE_DSL_ARCH", "sm_100a")
    try:
        grp = load_module(os.path.join(ref_root, "group_gemm", "group_gemm_cute5_v2.py"), "ref_group_v2")
    except Exception as exc:  # pragma: no cover - depends on the installed DSL
        print("grouped reference module did not import:", repr(exc))
        grp = None
    if grp is not None:
        all_bytes = torch.arange(256, dtype=torch.uint8).view(16, 16, 1)
        out["decode_in"] = all_bytes.numpy()
        out["decode_out"] = grp.nvfp4_to_fp16(all_bytes).float().numpy()
        sf72 = torch.arange(72 * 16, dtype=torch.int64).remainder(119).to(torch.uint8).view(72, 16)
        out["to_blocked_pad_in"] = sf72.numpy()
        out["to_blocked_pad_out"] = grp.to_blocked(sf72).numpy()
        ref_sf = torch.arange(72 * 16, dtype=torch.int64).remainder(126).to(torch.uint8).view(1, 72, 16)
        ref_sf = ref_sf.view(torch.float8_e4m3fn).permute(1, 2, 0)
        with cpu_device_shim():
            torch.manual_seed(7)
            perm = grp.create_reordered_scale_factor_tensor(1, 72, 256, ref_sf)
        out["grp_sf_in"] = u8(ref_sf)
        out["grp_sf_perm"] = u8(perm.permute(5, 2, 4, 0, 1, 3))
        out["grp_sf_perm_shape"] = np.array(perm.shape)
        out["grp_sf_perm_stride"] = np.array(perm.stride())
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
