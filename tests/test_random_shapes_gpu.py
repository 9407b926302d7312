"""Seeded sweep over random problem sizes, dtypes, kernel configurations and epilogues: every
case goes through the C ABI and is compared with the CPU oracle.  Sizes are drawn so that all
kernel families and their ragged-edge paths are hit (TMA-legal and not, one tile and many,
M below and above a tile, K not a multiple of the K block)."""
import random

import pytest
import torch

from oracle import contraction as O
from tests.gpu_util import assert_close, run_gemm, seeded
from tritonix_b200 import OutOfResources, _cabi

pytestmark = pytest.mark.gpu
EPI = {0: None, _cabi.EPI_GLU_LINEAR: "none", _cabi.EPI_GLU_SILU: "silu", _cabi.EPI_GLU_SIGMOID: "sigmoid"}


def draw_case(rng: random.Random):
    legal = rng.random() < 0.75
    step = 8 if legal else 1
    m = rng.choice([1, 7, 64, 100, 128, 129, 255, 256, 300, 512, 777, 1024])
    n = rng.randrange(step, 1400, step)
    k = rng.randrange(step, 2100, step)
    epi = rng.choice([0, 0, 0, _cabi.EPI_GLU_SILU, _cabi.EPI_GLU_SIGMOID, _cabi.EPI_GLU_LINEAR])
    if epi:
        n = max(16, n // 16 * 16) if legal else max(2, n // 2 * 2)
    dtype = rng.choice([torch.float16, torch.bfloat16] + ([torch.float32] if not legal else []))
    cfg = {}
    if legal:
        cfg["tile_n"] = rng.choice([128, 256] if epi else [64, 128, 256])
        cfg["tile_k"] = rng.choice([64, 128])
        cfg["cta_group"] = rng.choice([1, 2]) if cfg["tile_n"] >= 128 else 1
        cfg["stages"] = rng.choice([2, 3, 4])
        cfg["acc_stages"] = rng.choice([1, 2])
        cfg["group_m"] = rng.choice([1, 3, 8])
        cfg["tile_order"] = rng.choice(["grouped", "serpentine", "hilbert"])
        cfg["split_k"] = rng.choice([1, 1, 2, 3, 4, 8])
        cfg["max_ctas"] = rng.choice([0, 0, 2, 8])
    return m, n, k, dtype, epi, cfg


@pytest.mark.parametrize("seed", range(120))
def test_random_problem(seed):
    rng = random.Random(1000 + seed)
    m, n, k, dtype, epi, cfg = draw_case(rng)
    a, b = seeded(m, k, n, dtype, seed=seed, b_scale=(0.5 * k ** -0.5) if epi else None)
    try:
        out, res = run_gemm(a, b, cfg, epi)
    except OutOfResources:
        cfg["stages"] = 2   # the draw exceeded shared memory: the two-stage ring always fits
        out, res = run_gemm(a, b, cfg, epi)
    ref = O.glu_oracle(a, b, EPI[epi]) if epi else O.matmul_oracle(a, b)
    scale = 10 if dtype == torch.float32 else 1
    assert_close(out, ref, dtype, scale=scale)


def draw_double_tile_case(rng: random.Random):
    m = rng.choice([1, 100, 129, 256, 300, 512, 777, 1024, 1500])
    n = rng.randrange(8, 2600, 8)
    k = rng.randrange(8, 2100, 8)
    epi = rng.choice([0, 0, _cabi.EPI_GLU_SILU, _cabi.EPI_GLU_LINEAR])
    if epi:
        n = max(16, n // 16 * 16)
    tile_k = rng.choice([64, 64, 128])
    cfg = {"tile_n": 512, "cta_group": 2, "tile_k": tile_k,
           "stages": 2 if tile_k == 128 else rng.choice([2, 3, 4]),
           "group_m": rng.choice([1, 3, 8]), "tile_order": rng.choice(["grouped", "serpentine"]),
           "max_ctas": rng.choice([0, 0, 2, 6])}
    return m, n, k, rng.choice([torch.float16, torch.bfloat16]), epi, cfg


@pytest.mark.parametrize("seed", range(40))
def test_random_problem_on_double_tiles(seed):
    """tile_n = 512 (two 256-column tiles per CTA pair): against the oracle, and bit for bit
    against the same problem on single tiles."""
    rng = random.Random(5000 + seed)
    m, n, k, dtype, epi, cfg = draw_double_tile_case(rng)
    a, b = seeded(m, k, n, dtype, seed=seed, b_scale=(0.5 * k ** -0.5) if epi else None)
    out, res = run_gemm(a, b, cfg, epi)
    assert res.kernel == _cabi.KERNEL_TCGEN05
    ref = O.glu_oracle(a, b, EPI[epi]) if epi else O.matmul_oracle(a, b)
    assert_close(out, ref, dtype)
    single, _ = run_gemm(a, b, {"tile_n": 256, "cta_group": 2, "tile_k": cfg["tile_k"]}, epi)
    assert torch.equal(out, single)
