"""Generates tests/golden/reference_b200.npz: outputs of the REFERENCE's own Triton kernels
(matmul_kernel, gemm_splitk_kernel, glu_kernel of ayghri/tritonix) compiled by Triton's JIT and
run on an NVIDIA B200, for the seeded cases of tests/reference_cases.py (bf16 and fp16).

    python oracle/make_ref.py <reference source tree>       # where the reference is mounted
    python tests/golden/make_b200_golden.py [--out FILE]    # on a machine with a B200

The first step stages the unmodified reference package under oracle/_ref/ (ignored by version
control); the second runs oracle/reference_gpu.py on it in a process of its own and keeps, per
case, the output rows the case lists plus fp64 checksums of the seeded inputs (to detect
generator drift).  The file complements reference_outputs.npz, which holds CPU-interpreter runs
of the same kernels and therefore no bf16.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, REPO)

import numpy as np  # noqa: E402

from oracle.reference_gpu import make_inputs  # noqa: E402
from tests.reference_cases import CASES  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(REPO, "tests", "golden", "reference_b200.npz"))
    args = ap.parse_args()
    with tempfile.TemporaryDirectory() as tmp:
        spec, raw = os.path.join(tmp, "spec.json"), os.path.join(tmp, "raw.npz")
        with open(spec, "w") as f:
            json.dump(CASES, f)
        subprocess.run([sys.executable, os.path.join(REPO, "oracle", "reference_gpu.py"),
                        "--spec", spec, "--out", raw], check=True)
        got = np.load(raw)
        out = {}
        for case in CASES:
            a, b = make_inputs(case)
            out[case["name"] + "/out"] = got[case["name"] + "/out"]
            out[case["name"] + "/rows"] = np.array(case["rows"])
            out[case["name"] + "/checksum"] = np.array([a.double().sum().item(), b.double().sum().item()])
    import torch
    out["meta/gpu"] = np.array(torch.cuda.get_device_name(0))
    import triton
    out["meta/triton"] = np.array(triton.__version__)
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
