"""Generates tests/golden/reference_outputs.npz by running the REFERENCE's own Triton kernels
(matmul_kernel, gemm_splitk_kernel, glu_kernel of ayghri/tritonix) on CPU under Triton's
interpreter, on seeded inputs.  Run once where the reference tree is mounted:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py <path to the reference source tree>

Inputs are regenerated from the recorded seeds by tests (torch CPU generator); for every case
the file stores the reference output, the inputs' fp64 checksums (to detect generator drift)
and, for the small cases, the inputs themselves.  bf16 is not generated: Triton 3.6's
interpreter returns garbage for bf16 dot products.
"""
from __future__ import annotations

import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, REPO)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from oracle.ref_loader import load_reference  # noqa: E402

CASES = [
    # name, kind, m, n, k, dtype, cfg (reference's block sizes), extra
    ("mm_small_f16", "matmul", 128, 96, 160, "float16", dict(block_m=32, block_n=32, block_k=32, group_m=4), {}),
    ("mm_ragged_f16", "matmul", 100, 70, 90, "float16", dict(block_m=32, block_n=32, block_k=32, group_m=4), {}),
    ("mm_c1_f16", "matmul", 1024, 768, 512, "float16", dict(block_m=128, block_n=128, block_k=64, group_m=8), {}),
    ("mm_small_f32", "matmul", 96, 80, 72, "float32", dict(block_m=32, block_n=32, block_k=16, group_m=4), {}),
    ("sk2_f16", "splitk", 64, 128, 256, "float16", dict(block_m=32, block_n=64, block_k=32, group_m=4, split_k=2), {}),
    ("sk4_f16", "splitk", 64, 128, 256, "float16", dict(block_m=32, block_n=64, block_k=32, group_m=4, split_k=4), {}),
    ("sk8_f16", "splitk", 64, 128, 256, "float16", dict(block_m=32, block_n=64, block_k=32, group_m=4, split_k=8), {}),
    ("sk4_c3scaled_f16", "splitk", 64, 512, 1792, "float16", dict(block_m=64, block_n=128, block_k=64, group_m=8, split_k=4), {}),
    ("glu_silu_small_f16", "glu", 64, 80, 48, "float16", dict(block_m=32, block_n=32, block_k=16, group_m=4), {"activation": "silu"}),
    ("glu_none_small_f16", "glu", 64, 80, 48, "float16", dict(block_m=32, block_n=32, block_k=16, group_m=4), {"activation": "none"}),
    ("glu_silu_f16", "glu", 256, 768, 512, "float16", dict(block_m=64, block_n=128, block_k=64, group_m=8), {"activation": "silu"}),
    ("glu_silu_f32", "glu", 64, 96, 40, "float32", dict(block_m=32, block_n=32, block_k=16, group_m=4), {"activation": "silu", "use_tf32": False}),
]


def make_inputs(name, kind, m, n, k, dtype):
    """Seeded inputs; tests call this same function."""
    seed = sum(ord(c) for c in name)
    g = torch.Generator().manual_seed(seed)
    dt = getattr(torch, dtype)
    a = torch.randn(m, k, generator=g, dtype=torch.float32)
    b = torch.randn(k, n, generator=g, dtype=torch.float32)
    if kind == "glu":
        b = b * 0.05 * (64.0 / k) ** 0.5
    elif kind == "splitk":
        a, b = a * k ** -0.25, b * k ** -0.25
    return a.to(dt), b.to(dt)


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python " + sys.argv[0] + " <path to the reference source tree>")
    root = sys.argv[1]
    ref_mm, ref_sw = load_reference(root)
    import triton

    out = {}
    for name, kind, m, n, k, dtype, cfg, extra in CASES:
        a, b = make_inputs(name, kind, m, n, k, dtype)
        if kind == "matmul":
            c = ref_mm._launch_matmul(a, b, dict(cfg))
        elif kind == "splitk":
            c = ref_mm._launch_splitk(a, b, dict(cfg))
        else:
            c = torch.empty(m, n // 2, dtype=a.dtype)
            grid = (triton.cdiv(m, cfg["block_m"]), triton.cdiv(n, cfg["block_n"]))
            ref_sw.glu_kernel[grid](a, b, c, m, n, k, a.stride(0), a.stride(1), b.stride(0),
                                    b.stride(1), c.stride(0), c.stride(1), **cfg, **extra)
        out[name + "/out"] = c.numpy()
        out[name + "/checksum"] = np.array([a.double().sum().item(), b.double().sum().item()])
        if m * k + k * n <= 40000:
            out[name + "/a"] = a.numpy()
            out[name + "/b"] = b.numpy()
        fp32 = a.float() @ b.float()
        print(f"{name}: out {tuple(c.shape)} {c.dtype}  |ref|max={fp32.abs().max():.3f}", flush=True)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_outputs.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
