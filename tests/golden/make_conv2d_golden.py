"""Generates tests/golden/conv2d_reference.npz by running the REFERENCE's own conv2d_forward
(ayghri/tritonix, tritonix/ops/conv2d/forward.py) on CPU under Triton's interpreter, on seeded
inputs.  Run once where the reference tree is mounted:

    TRITON_INTERPRET=1 python tests/golden/make_conv2d_golden.py <path to the reference tree>

Tests regenerate the inputs from the case name (make_inputs below) and compare checksums, so a
drift of the generator is noticed.  fp16 and fp32 only: Triton 3.6's interpreter returns garbage
for bf16 dot products.
"""
from __future__ import annotations

import importlib
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, REPO)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from oracle.ref_loader import load_reference  # noqa: E402

CASES = [
    # name, (N, C, H, W), (C_OUT, R, S), stride, padding, dilation, bias, dtype
    ("cv_3x3_pad1_f16", (2, 16, 12, 12), (32, 3, 3), (1, 1), (1, 1), (1, 1), True, "float16"),
    ("cv_1x1_f16", (1, 64, 9, 7), (24, 1, 1), (1, 1), (0, 0), (1, 1), False, "float16"),
    ("cv_3x3_stride2_f16", (2, 8, 15, 13), (16, 3, 3), (2, 2), (1, 1), (1, 1), True, "float16"),
    ("cv_5x3_dil2_f16", (1, 8, 14, 16), (8, 5, 3), (1, 1), (2, 3), (2, 1), False, "float16"),
    ("cv_odd_channels_f16", (2, 3, 10, 11), (5, 3, 3), (1, 2), (0, 1), (1, 1), True, "float16"),
    ("cv_3x3_pad1_f32", (1, 6, 9, 10), (7, 3, 3), (1, 1), (1, 1), (1, 1), True, "float32"),
    ("cv_stride2_dil2_f32", (2, 4, 13, 12), (6, 3, 2), (2, 1), (2, 0), (2, 2), False, "float32"),
]
BLOCKS = dict(BLOCK_SIZE_M=32, BLOCK_SIZE_N=32, BLOCK_SIZE_K=16, GROUP_SIZE_M=4)


def make_inputs(name, xshape, wshape, has_bias, dtype):
    """Seeded inputs; tests call this same function."""
    seed = sum(ord(ch) for ch in name)
    g = torch.Generator().manual_seed(seed)
    dt = getattr(torch, dtype)
    n, c, h, w = xshape
    c_out, r, s = wshape
    x = torch.randn(n, c, h, w, generator=g, dtype=torch.float32)
    wt = torch.randn(c_out, c, r, s, generator=g, dtype=torch.float32) * (c * r * s) ** -0.5
    b = torch.randn(c_out, generator=g, dtype=torch.float32) if has_bias else None
    return x.to(dt), wt.to(dt), (b.to(dt) if b is not None else None)


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python " + sys.argv[0] + " <path to the reference source tree>")
    load_reference(sys.argv[1])  # registers the stub packages and the pruner alias
    fwd = importlib.import_module("tritonix.ops.conv2d.forward")
    out = {}
    for name, xshape, wshape, stride, padding, dilation, has_bias, dtype in CASES:
        x, w, b = make_inputs(name, xshape, wshape, has_bias, dtype)
        y = fwd.conv2d_forward(x, w, b, stride, padding, dilation, use_tf32=False, config=dict(BLOCKS))
        out[name + "/out"] = y.numpy()
        out[name + "/checksum"] = np.array([x.double().sum().item(), w.double().sum().item()])
        print(name, tuple(y.shape), float(y.float().abs().max()))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "conv2d_reference.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
