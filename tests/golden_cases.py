"""Shared access to the golden cases (inputs regenerated from the seeds of make_golden.py)."""
import importlib.util
import os

import numpy as np
import torch

_here = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(_here, "golden", "make_golden.py"))


def _load_cases():
    # make_golden.py sets TRITON_INTERPRET on import; keep the environment as it was
    before = os.environ.get("TRITON_INTERPRET")
    mod = importlib.util.module_from_spec(_spec)
    _spec.loader.exec_module(mod)
    if before is None:
        os.environ.pop("TRITON_INTERPRET", None)
    else:
        os.environ["TRITON_INTERPRET"] = before
    return mod


_mod = _load_cases()
CASES = _mod.CASES
make_inputs = _mod.make_inputs


def case_ids(kind=None):
    return [c[0] for c in CASES if kind is None or c[1] == kind]


def get_case(name):
    for c in CASES:
        if c[0] == name:
            return c
    raise KeyError(name)


def inputs_and_reference(golden, name):
    """(a, b, reference_output, case) with the generator-drift check applied."""
    case = get_case(name)
    _, kind, m, n, k, dtype, cfg, extra = case
    a, b = make_inputs(name, kind, m, n, k, dtype)
    chk = golden[name + "/checksum"]
    assert abs(a.double().sum().item() - chk[0]) < 1e-6 * max(1.0, abs(chk[0])), "input drift (a)"
    assert abs(b.double().sum().item() - chk[1]) < 1e-6 * max(1.0, abs(chk[1])), "input drift (b)"
    if name + "/a" in golden.files:
        assert np.array_equal(golden[name + "/a"], a.numpy())
    ref = torch.from_numpy(golden[name + "/out"])
    return a, b, ref, case
