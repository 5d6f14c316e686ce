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


def grouped_specs():
    import yaml
    with open(os.path.join(REF, "utils", "group_gemm", "task.yml")) as f:
        return yaml.safe_load(f)
