"""Loads the reference implementation (ayghri/tritonix) from a source tree for comparison runs.
TEST INFRASTRUCTURE ONLY — used by tests/golden/make_golden.py (CPU, Triton's interpreter) where
the reference tree is mounted, and by oracle/reference_gpu.py (a process of its own that runs the
reference's kernels on a GPU from the copy staged by oracle/make_ref.py); nothing in the product
imports it.

`import tritonix` fails on the reference as shipped: tritonix/autotune.py:8-11 imports
`CoordinateMonotonicFunction`, which tritonix/utils/pruners.py:172 defines under the name
`CoordinateUnimodalFunction`.  The loader therefore registers stub packages (so the package
__init__ files, which import everything, are skipped), aliases the missing name, and imports the
two op modules.  With TRITON_INTERPRET=1 set before Triton is imported, the @triton.jit kernels
run on CPU tensors through Triton's NumPy interpreter.
"""
from __future__ import annotations

import importlib
import os
import sys
import types


def load_reference(root: str, interpret: bool = True):
    """Returns (matmul_module, swiglu_module) of the reference source tree at ``root`` (the
    directory that contains its ``tritonix`` package)."""
    if interpret:
        os.environ.setdefault("TRITON_INTERPRET", "1")
    if not os.path.isdir(os.path.join(root, "tritonix")):
        raise FileNotFoundError(f"no reference tree at {root}")
    for name, sub in (("tritonix", "tritonix"), ("tritonix.ops", "tritonix/ops")):
        mod = types.ModuleType(name)
        mod.__path__ = [os.path.join(root, sub)]
        sys.modules[name] = mod
    pruners = importlib.import_module("tritonix.utils.pruners")
    pruners.CoordinateMonotonicFunction = pruners.CoordinateUnimodalFunction
    return (importlib.import_module("tritonix.ops.matmul"),
            importlib.import_module("tritonix.ops.swiglu"))
