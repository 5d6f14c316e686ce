"""Import the reference's own task modules from ``baseline/_ref/`` (see install_ref.py).

The reference keeps one ``task.py`` / ``utils.py`` pair per problem under the same module
names and its files do ``from task import ...`` / ``from utils import ...``; they are
loaded here under those names and the names are taken out of ``sys.modules`` again, so
nothing leaks into the importing process.  Used by the GPU harness test and by the
same-box comparison of ``bench.py``; never by the product package."""
from __future__ import annotations

import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def available() -> bool:
    return os.path.exists(os.path.join(REF, "dual_gemm", "reference.py"))


def _load(name: str, path: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def load_dual(with_kernel: bool = False):
    """Returns (reference module, specs dict[, submission module]) of the dual-GEMM task:
    ``reference.generate_input / ref_kernel / check_implementation`` as the reference
    defines them, ``specs["tests"]`` and ``specs["benchmarks"]`` from its task.yml."""
    import yaml
    saved = {k: sys.modules.get(k) for k in ("task", "utils", "reference", "submission")}
    try:
        _load("task", os.path.join(REF, "utils", "dual_gemm", "task.py"))
        _load("utils", os.path.join(REF, "utils", "dual_gemm", "utils.py"))
        reference = _load("reference", os.path.join(REF, "dual_gemm", "reference.py"))
        submission = _load("submission", os.path.join(REF, "dual_gemm", "submission.py")) if with_kernel else None
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    with open(os.path.join(REF, "utils", "dual_gemm", "task.yml")) as f:
        specs = yaml.safe_load(f)
    return (reference, specs, submission) if with_kernel else (reference, specs)


def load_grouped_kernel():
    """The reference's grouped kernel file group_gemm/group_gemm_cute4.py (``custom_kernel`` at :1252-1399),
    imported unmodified.  The file runs ``pip install`` at import time when no ``tvm`` module can be found
    (:12-25) and builds Modal objects at module level (:1408-1426, :1722, :1964); inert stand-ins for both
    module names are registered first so that neither happens, and removed again afterwards."""
    import importlib.machinery
    import types

    class _Chain:
        """Absorbs any attribute access or call; used as a decorator it returns the function unchanged."""
        def __getattr__(self, name):
            if name.startswith("__"):
                raise AttributeError(name)
            return self

        def __call__(self, *args, **kwargs):
            if len(args) == 1 and callable(args[0]) and not kwargs and not isinstance(args[0], _Chain):
                return args[0]
            return self

    names = ("task", "utils", "modal", "tvm", "group_gemm_cute4")
    saved = {k: sys.modules.get(k) for k in names}
    try:
        modal = types.ModuleType("modal")
        def _modal_attr(name):
            if name.startswith("__"):
                raise AttributeError(name)
            return _Chain()
        modal.__getattr__ = _modal_attr
        sys.modules["modal"] = modal
        if importlib.util.find_spec("tvm") is None:
            tvm = types.ModuleType("tvm")
            tvm.__spec__ = importlib.machinery.ModuleSpec("tvm", None)
            sys.modules["tvm"] = tvm
        _load("task", os.path.join(REF, "utils", "group_gemm", "task.py"))
        _load("utils", os.path.join(REF, "utils", "group_gemm", "utils.py"))
        return _load("group_gemm_cute4", os.path.join(REF, "group_gemm", "group_gemm_cute4.py"))
    finally:
        for k, v in saved.items():
            if k == "group_gemm_cute4":
                continue
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def grouped_specs():
    import yaml
    with open(os.path.join(REF, "utils", "group_gemm", "task.yml")) as f:
        return yaml.safe_load(f)
