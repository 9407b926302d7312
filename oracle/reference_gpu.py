"""Runs the reference's own Triton kernels on a GPU.  TEST INFRASTRUCTURE ONLY.

    python oracle/reference_gpu.py --spec cases.json --out outputs.npz

It is always run as a process of its own: the reference package is also called `tritonix`, so
it cannot share an interpreter with code that aliased this package under that name, and the
Triton JIT should not share a CUDA context with the kernels under test.  The reference tree is
the unmodified copy that oracle/make_ref.py staged under oracle/_ref/ (loaded through
oracle/ref_loader.py, which only works around the reference's broken `import tritonix`).

Each case of the JSON list names a kernel of the reference and a seeded problem:
  {"name", "kind": "matmul" | "splitk" | "glu", "m", "n", "k", "dtype": "bfloat16" | "float16",
   "seed", "a_scale", "b_scale", "cfg": {block_m, block_n, block_k, group_m, [split_k],
   num_stages, num_warps}, ["activation"], ["rows": [...]], ["time": true]}
and is launched exactly as the reference launches it: `_launch_matmul` (tritonix/ops/matmul.py:
217-237), `_launch_splitk` (:240-264), and for the GLU the direct `glu_kernel[grid](...)` call
of the reference's only example (playground/opt_glu.py:33-56).  Only tile-aligned shapes are
accepted: `matmul_kernel` masks the K tail but not the M/N tails on load
(tritonix/ops/matmul.py:92-96), so a ragged M or N would read out of bounds on a GPU.
`swiglu_kernel` (tritonix/ops/swiglu.py:113-230) is never launched: its W3 indexing runs out of
bounds beyond one tile.

The .npz holds, per case, "<name>/out" (all rows, or the rows listed in "rows"; bf16 is stored
as its uint16 bit pattern) and, with "time", "<name>/ms" = [mean, min] milliseconds per launch
(CUDA events, L2 flushed between launches).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")


def make_inputs(case):
    """Seeded operands of a case on the CPU (the tests build theirs with this same function)."""
    import torch
    g = torch.Generator().manual_seed(int(case["seed"]))
    dt = getattr(torch, case["dtype"])
    a = torch.randn(case["m"], case["k"], generator=g, dtype=torch.float32) * case.get("a_scale", 1.0)
    b = torch.randn(case["k"], case["n"], generator=g, dtype=torch.float32) * case.get("b_scale", 1.0)
    return a.to(dt), b.to(dt)


def to_numpy(t):
    import torch
    t = t.detach().cpu().contiguous()
    return t.view(torch.int16).numpy().view("uint16") if t.dtype == torch.bfloat16 else t.numpy()


def from_numpy(arr, dtype_name):
    import numpy as np
    import torch
    if dtype_name == "bfloat16":
        return torch.from_numpy(np.ascontiguousarray(arr).view("int16")).view(torch.bfloat16)
    return torch.from_numpy(np.ascontiguousarray(arr))


def check_aligned(case):
    cfg = case["cfg"]
    if case["m"] % cfg["block_m"] or case["n"] % cfg["block_n"]:
        raise ValueError(f"{case['name']}: M and N must be multiples of the reference's tile "
                         "(its loads are not masked along M and N)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--spec", required=True)
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(REF_ROOT, "tritonix")):
        sys.exit("oracle/_ref is empty: run `python oracle/make_ref.py` where the reference tree is mounted")
    os.environ.pop("TRITON_INTERPRET", None)
    sys.path.insert(0, os.path.dirname(HERE))
    import numpy as np
    import torch
    from oracle.ref_loader import load_reference
    ref_mm, ref_sw = load_reference(REF_ROOT, interpret=False)
    import triton

    dev = torch.device("cuda", 0)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    out = {}
    with open(args.spec) as f:
        cases = json.load(f)
    for case in cases:
        check_aligned(case)
        a_cpu, b_cpu = make_inputs(case)
        a, b = a_cpu.to(dev), b_cpu.to(dev)
        cfg = dict(case["cfg"])
        m, n, k = case["m"], case["n"], case["k"]
        if case["kind"] == "matmul":
            run = lambda: ref_mm._launch_matmul(a, b, cfg)  # noqa: E731
        elif case["kind"] == "splitk":
            run = lambda: ref_mm._launch_splitk(a, b, cfg)  # noqa: E731
        elif case["kind"] == "glu":
            z = torch.empty(m, n // 2, dtype=a.dtype, device=dev)
            grid = (triton.cdiv(m, cfg["block_m"]), triton.cdiv(n, cfg["block_n"]))
            extra = {"activation": case.get("activation", "silu")}

            def run():
                ref_sw.glu_kernel[grid](a, b, z, m, n, k, a.stride(0), a.stride(1), b.stride(0),
                                        b.stride(1), z.stride(0), z.stride(1), **cfg, **extra)
                return z
        else:
            raise ValueError(case["kind"])
        c = run()
        torch.cuda.synchronize(dev)
        rows = case.get("rows")
        out[case["name"] + "/out"] = to_numpy(c[rows] if rows else c)
        if case.get("time"):
            for _ in range(3):
                run()
            times = []
            for _ in range(int(case.get("reps", 10))):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                run()
                e1.record()
                e1.synchronize()
                times.append(e0.elapsed_time(e1))
            out[case["name"] + "/ms"] = np.array([sum(times) / len(times), min(times)])
        print(f"{case['name']}: {case['kind']} {m}x{n}x{k} {case['dtype']} done", flush=True)
    np.savez_compressed(args.out, **out)


if __name__ == "__main__":
    main()
