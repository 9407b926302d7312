"""Shared access to the convolution golden cases (inputs regenerated from the seeds of
tests/golden/make_conv2d_golden.py)."""
import importlib.util
import os

import numpy as np
import torch

_here = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location(
    "make_conv2d_golden", os.path.join(_here, "golden", "make_conv2d_golden.py"))


def _load():
    before = os.environ.get("TRITON_INTERPRET")  # the generator sets it on import
    mod = importlib.util.module_from_spec(_spec)
    _spec.loader.exec_module(mod)
    if before is None:
        os.environ.pop("TRITON_INTERPRET", None)
    else:
        os.environ["TRITON_INTERPRET"] = before
    return mod


_mod = _load()
CASES = _mod.CASES
make_inputs = _mod.make_inputs
GOLDEN_PATH = os.path.join(_here, "golden", "conv2d_reference.npz")


def case_ids():
    return [c[0] for c in CASES]


def load_case(golden, name):
    """(x, w, bias, stride, padding, dilation, reference_output, dtype name)."""
    case = next(c for c in CASES if c[0] == name)
    _, xshape, wshape, stride, padding, dilation, has_bias, dtype = case
    x, w, b = make_inputs(name, xshape, wshape, has_bias, dtype)
    chk = golden[name + "/checksum"]
    assert abs(x.double().sum().item() - chk[0]) < 1e-6 * max(1.0, abs(chk[0])), "input drift (x)"
    assert abs(w.double().sum().item() - chk[1]) < 1e-6 * max(1.0, abs(chk[1])), "input drift (w)"
    return x, w, b, stride, padding, dilation, torch.from_numpy(golden[name + "/out"]), dtype


def golden():
    return np.load(GOLDEN_PATH)
