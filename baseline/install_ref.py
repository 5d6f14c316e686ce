"""Copy the few reference files that the GPU-side harness test and the same-box
comparison need into ``baseline/_ref/`` (git-ignored; it travels to the GPU box with
the working tree, where the reference checkout itself does not exist).

    python baseline/install_ref.py [/path/to/reference]

Files taken, unmodified:
  dual_gemm/reference.py              generate_input, ref_kernel, check_implementation
  dual_gemm/submission.py             the reference's own sm_100a kernel (one CTA per tile)
  group_gemm/group_gemm_cute4.py      the reference's grouped kernel with compile-time group dispatch
  utils/dual_gemm/{task.py,utils.py,task.yml}      task types, comparison rule, test / benchmark specs
  utils/group_gemm/{task.py,utils.py,task.yml}     the same for the grouped problem
The reference's other kernels (dual_gemm/dual_gemm_opt_cute.py, group_gemm/group_gemm_cute5*.py)
are left out on purpose: their sources name cluster-multicast TMA loads, which must not be
present in a tree that runs on more than one GPU of this pool.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
FILES = [
    "dual_gemm/reference.py",
    "dual_gemm/submission.py",
    "group_gemm/group_gemm_cute4.py",
    "utils/dual_gemm/task.py",
    "utils/dual_gemm/utils.py",
    "utils/dual_gemm/task.yml",
    "utils/group_gemm/task.py",
    "utils/group_gemm/utils.py",
    "utils/group_gemm/task.yml",
]


# the reference checkout sits beside this repository
DEFAULT_ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


def install(reference_root: str = DEFAULT_ROOT) -> bool:
    """Returns True when every file is in place afterwards."""
    if not os.path.isdir(reference_root):
        return all(os.path.exists(os.path.join(DEST, f)) for f in FILES)
    for rel in FILES:
        src = os.path.join(reference_root, rel)
        dst = os.path.join(DEST, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        with open(src, "rb") as f:
            text = f.read()
        if b"multicast" in text:
            raise RuntimeError(f"{rel} names a multicast load; it must not travel")
        shutil.copyfile(src, dst)
    return True


if __name__ == "__main__":
    ok = install(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_ROOT)
    print("baseline/_ref", "ready" if ok else "incomplete")
