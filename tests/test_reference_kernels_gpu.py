"""The CUDA kernels against the reference's OWN Triton kernels run on a B200, on identical
seeded inputs — bf16 included, which the CPU interpreter behind reference_outputs.npz cannot do.

Two forms of the same comparison:
 * against tests/golden/reference_b200.npz, outputs of the reference's matmul_kernel
   (tritonix/ops/matmul.py:42-108), gemm_splitk_kernel (:147-202) and glu_kernel
   (tritonix/ops/swiglu.py:24-110) recorded on a B200 by tests/golden/make_b200_golden.py;
 * live, when the unmodified reference package is staged under oracle/_ref (oracle/make_ref.py):
   oracle/reference_gpu.py runs it in a process of its own on this GPU, then this process runs
   the CUDA kernels on the same inputs.

Tolerance: max|err|/max|ref| <= 2e-3 (fp16), 8e-3 (bf16).  The reference's split-K rounds every
slice's partial to the output type and adds the roundings with atomics (tritonix/ops/matmul.py:
195-202), so its own distance from the exact product is added to the allowance there.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import contraction as O
from oracle.reference_gpu import from_numpy, make_inputs
from tests.gpu_util import DEV, TOL
from tests.reference_cases import CASES, case_ids, get_case
from tritonix_b200 import _cabi

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FIXTURE = os.path.join(REPO, "tests", "golden", "reference_b200.npz")
STAGED = os.path.join(REPO, "oracle", "_ref", "tritonix")

OURS = {
    "matmul": lambda c: {"kernel": "tcgen05", "tile_n": 128},
    "splitk": lambda c: {"kernel": "tcgen05", "tile_n": 128, "tile_k": 128,
                         "split_k": c["cfg"]["split_k"], "stages": 4},
    "glu": lambda c: {"kernel": "tcgen05", "tile_n": 128},
}
EPILOGUE = {"silu": _cabi.EPI_GLU_SILU, "none": _cabi.EPI_GLU_LINEAR}


def run_ours(case):
    a_cpu, b_cpu = make_inputs(case)
    a, b = a_cpu.to(DEV), b_cpu.to(DEV)
    glu = case["kind"] == "glu"
    epi = EPILOGUE[case["activation"]] if glu else _cabi.EPI_NONE
    c = torch.full((case["m"], case["n"] // 2 if glu else case["n"]), float("nan"), device=DEV,
                   dtype=a.dtype)
    _cabi.launch(a, b, c, OURS[case["kind"]](case), epi)
    _cabi.check_status(c.device)
    rows = case["rows"]
    if glu:
        exact = O.glu_oracle(a_cpu[rows], b_cpu, case["activation"], out_dtype=torch.float32)
    else:
        exact = O.matmul_oracle(a_cpu[rows], b_cpu, out_dtype=torch.float32)
    return c[rows].cpu(), exact, (a_cpu, b_cpu)


def compare(case, ours, reference, exact):
    dtype = ours.dtype
    assert reference.shape == ours.shape and reference.dtype == dtype
    assert not torch.isnan(ours.float()).any()
    tol = TOL[dtype]
    err_ours = O.rel_err(ours, exact)
    err_ref = O.rel_err(reference, exact)
    assert err_ours <= tol, f"CUDA kernel vs fp32 product: {err_ours:.2e}"
    allowance = tol + (err_ref if case["kind"] == "splitk" else 0.0)
    err = O.rel_err(ours, reference.float())
    assert err <= allowance, (f"CUDA kernel vs reference Triton kernel: {err:.2e} > {allowance:.2e} "
                              f"(reference vs fp32 product: {err_ref:.2e})")


@pytest.fixture(scope="module")
def recorded():
    if not os.path.exists(FIXTURE):
        pytest.skip("tests/golden/reference_b200.npz has not been generated")
    return np.load(FIXTURE)


@pytest.mark.parametrize("name", case_ids())
def test_against_recorded_reference_kernel_outputs(recorded, name):
    case = get_case(name)
    ours, exact, (a_cpu, b_cpu) = run_ours(case)
    chk = recorded[name + "/checksum"]
    assert abs(a_cpu.double().sum().item() - chk[0]) <= 1e-6 * max(1.0, abs(chk[0])), "input drift (a)"
    assert abs(b_cpu.double().sum().item() - chk[1]) <= 1e-6 * max(1.0, abs(chk[1])), "input drift (b)"
    assert list(recorded[name + "/rows"]) == case["rows"]
    compare(case, ours, from_numpy(recorded[name + "/out"], case["dtype"]), exact)


@pytest.fixture(scope="module")
def live(tmp_path_factory):
    if not os.path.isdir(STAGED):
        pytest.skip("the reference package is not staged under oracle/_ref "
                    "(python oracle/make_ref.py <reference tree>)")
    tmp = tmp_path_factory.mktemp("reference_gpu")
    spec, out = tmp / "spec.json", tmp / "out.npz"
    spec.write_text(json.dumps(CASES))
    env = {k: v for k, v in os.environ.items() if k != "TRITON_INTERPRET"}
    env["TRITON_CACHE_DIR"] = str(tmp / "triton_cache")
    done = subprocess.run([sys.executable, os.path.join(REPO, "oracle", "reference_gpu.py"),
                           "--spec", str(spec), "--out", str(out)], env=env, capture_output=True,
                          text=True, timeout=900)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    return np.load(out)


@pytest.mark.parametrize("name", case_ids())
def test_against_reference_kernels_run_now(live, name):
    case = get_case(name)
    ours, exact, _ = run_ours(case)
    compare(case, ours, from_numpy(live[name + "/out"], case["dtype"]), exact)
