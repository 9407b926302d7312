"""Stages the reference's Python package for runs on a GPU box.  TEST INFRASTRUCTURE ONLY.

    python oracle/make_ref.py [<reference source tree>]
    (default: $TRITONIX_REFERENCE_ROOT, else the directory `reference` beside this repository)

The reference (ayghri/tritonix) is pure Python + Triton, so "building" it is copying the
`tritonix` package's .py files, unmodified, into oracle/_ref/ — a directory that version
control ignores (nothing of the reference enters this repository's history) but that travels
with the working tree to the machine that has the GPU, where the reference tree itself is not
mounted.  oracle/reference_gpu.py loads it from there to run the reference's own Triton kernels
(tritonix/ops/matmul.py:42-108, :147-202, tritonix/ops/swiglu.py:24-110) on the same GPU as
the CUDA kernels under test.  Nothing in the product imports oracle/_ref.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def default_root() -> str:
    """Where the reference's source tree is expected: the environment's answer, else a checkout
    named `reference` in the directory that holds this repository."""
    return os.environ.get("TRITONIX_REFERENCE_ROOT") or os.path.join(
        os.path.dirname(os.path.dirname(HERE)), "reference")


def stage(root: str | None = None) -> str | None:
    """Copies <root>/tritonix/**/*.py to oracle/_ref/tritonix.  Returns the destination, or None
    when there is no reference tree at ``root`` (then whatever was staged before stays)."""
    root = root or default_root()
    src = os.path.join(root, "tritonix")
    if not os.path.isdir(src):
        return None
    dst = os.path.join(DEST, "tritonix")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(src, dst, ignore=lambda d, names: [
        n for n in names if not (n.endswith(".py") or os.path.isdir(os.path.join(d, n)))
        or n == "__pycache__"])
    with open(os.path.join(DEST, "STAGED_FROM"), "w") as f:
        f.write(root + "\n")
    return DEST


if __name__ == "__main__":
    out = stage(sys.argv[1] if len(sys.argv) > 1 else None)
    print(out if out else "no reference tree found; nothing staged")
