"""Cases on which the CUDA kernels are compared with the reference's own Triton kernels RUN ON A
B200 (oracle/reference_gpu.py): bf16 — the type of every headline workload, which Triton's CPU
interpreter cannot compute — and fp16, at shapes that are multiples of the reference's tiles
(its loads are not masked along M and N, tritonix/ops/matmul.py:92-96).  The configurations lie
inside the reference's own search spaces (tritonix/ops/matmul.py:33-38, :136-141,
tritonix/ops/swiglu.py:15-20).

Used by tests/golden/make_b200_golden.py (which stores the reference kernels' outputs for the
listed rows in tests/golden/reference_b200.npz) and by tests/test_reference_kernels_gpu.py.
"""
import random


def _rows(m, count, seed):
    r = random.Random(seed)
    return sorted(set([0, m - 1] + [r.randrange(m) for _ in range(count)]))


_MM = dict(block_m=128, block_n=128, block_k=64, group_m=8, num_stages=3, num_warps=8)
_SK = dict(block_m=64, block_n=128, block_k=64, group_m=8, num_stages=3, num_warps=4)
_GLU = dict(block_m=128, block_n=128, block_k=64, group_m=8, num_stages=3, num_warps=8)

CASES = [
    dict(name="mm_bf16_2048", kind="matmul", m=2048, n=2048, k=2048, dtype="bfloat16", seed=101,
         a_scale=1.0, b_scale=2048 ** -0.5, cfg=_MM, rows=_rows(2048, 30, 1)),
    dict(name="mm_f16_c1", kind="matmul", m=1024, n=768, k=512, dtype="float16", seed=102,
         a_scale=1.0, b_scale=512 ** -0.5, cfg=_MM, rows=_rows(1024, 30, 2)),
    dict(name="mm_bf16_c5down_slice", kind="matmul", m=1024, n=4096, k=14336, dtype="bfloat16",
         seed=103, a_scale=0.05, b_scale=0.02, cfg=_MM, rows=_rows(1024, 14, 3)),
    dict(name="sk4_f16_c3", kind="splitk", m=64, n=4096, k=14336, dtype="float16", seed=104,
         a_scale=14336 ** -0.25, b_scale=14336 ** -0.25, cfg=dict(_SK, split_k=4), rows=_rows(64, 14, 4)),
    dict(name="sk8_bf16_c3", kind="splitk", m=64, n=4096, k=14336, dtype="bfloat16", seed=105,
         a_scale=14336 ** -0.25, b_scale=14336 ** -0.25, cfg=dict(_SK, split_k=8), rows=_rows(64, 14, 5)),
    dict(name="glu_silu_bf16_c4_slice", kind="glu", m=1024, n=2048, k=4096, dtype="bfloat16",
         seed=106, a_scale=1.0, b_scale=0.02, cfg=_GLU, activation="silu", rows=_rows(1024, 30, 6)),
    dict(name="glu_none_bf16_c4_slice", kind="glu", m=1024, n=2048, k=4096, dtype="bfloat16",
         seed=107, a_scale=1.0, b_scale=0.02, cfg=_GLU, activation="none", rows=_rows(1024, 30, 7)),
    dict(name="glu_silu_f16", kind="glu", m=512, n=1024, k=1024, dtype="float16", seed=108,
         a_scale=1.0, b_scale=0.03, cfg=_GLU, activation="silu", rows=_rows(512, 30, 8)),
]


def case_ids():
    return [c["name"] for c in CASES]


def get_case(name):
    for c in CASES:
        if c["name"] == name:
            return c
    raise KeyError(name)
