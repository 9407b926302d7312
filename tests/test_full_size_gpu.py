"""Parity at the full sizes of the benchmark configurations that the other files only cover at
reduced scale: the skinny split-K GEMM for every factor of the sweep, the Llama-3-8B-shaped
SwiGLU MLP block (d = 4096, ff = 14336, 32768 tokens) and the 8192^3 GEMM split along M the way
2, 4 and 8 GPUs would split it.  Outputs are checked on sampled rows against the CPU oracle
(fp32 accumulation, one rounding; tolerance 2e-3 fp16 / 8e-3 bf16) and through size-independent
properties: bit-identical repeats, and shards that reproduce the rows of the unsharded result."""
import pytest
import torch

from oracle import contraction as O
from tests.gpu_util import DEV, assert_close
from tritonix_b200 import _cabi

pytestmark = pytest.mark.gpu
bf16, f16 = torch.bfloat16, torch.float16
T = {"kernel": "tcgen05"}


def device_randn(shape, dtype, seed, scale):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(shape, device=DEV, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("split_k", [1, 2, 4, 8, 16])
def test_skinny_split_k_sweep_at_full_size(split_k):
    """fp16 M = 64, K = 14336, N = 4096, entries N(0,1)/sqrt(K): every factor of the sweep,
    all 64 rows against the oracle, and two runs bit-identical."""
    m, k, n = 64, 14336, 4096
    a = device_randn((m, k), f16, 40, k ** -0.5)
    b = device_randn((k, n), f16, 41, 1.0)
    cfg = {**T, "tile_n": 128, "tile_k": 128, "stages": 4, "split_k": split_k}
    c1 = torch.full((m, n), float("nan"), device=DEV, dtype=f16)
    c2 = torch.full((m, n), float("nan"), device=DEV, dtype=f16)
    res = _cabi.launch(a, b, c1, cfg)
    _cabi.launch(a, b, c2, cfg)
    _cabi.check_status(c1.device)
    assert res.split_k == split_k
    assert torch.equal(c1, c2)
    assert_close(c1.cpu(), O.splitk_oracle(a.cpu(), b.cpu(), split_k, 128), f16)


def test_llama_mlp_block_at_full_size():
    """32768 tokens through d = 4096 -> ff = 14336 -> 4096 on one GPU: the two-launch
    `swiglu_mlp` and `TensorParallelSwiGLU` at world size 1 agree bit for bit, and 64 sampled
    tokens pushed through the full weights match the oracle."""
    import tritonix_b200 as tnx
    from tritonix_b200.distributed import TensorParallelSwiGLU
    m, d, ff = 32768, 4096, 14336
    x = device_randn((m, d), bf16, 50, 1.0)
    w12 = device_randn((d, 2 * ff), bf16, 51, 0.02)
    wd = device_randn((ff, d), bf16, 52, 0.02)
    glu_cfg = {**T, "tile_n": 256, "cta_group": 2, "tile_k": 128, "stages": 3, "group_m": 16}
    y = tnx.swiglu_mlp(x, w12, wd, cfg=glu_cfg, down_cfg=glu_cfg)
    y_tp = TensorParallelSwiGLU(w12, wd, chunks=1, gate_up_cfg=glu_cfg, down_cfg=glu_cfg)(x)
    _cabi.check_status(y.device)
    assert torch.equal(y, y_tp)
    rows = sorted(set(torch.randint(0, m, (62,), generator=torch.Generator().manual_seed(7)).tolist()
                      + [0, m - 1]))
    ref = O.swiglu_mlp_oracle(x[rows].cpu(), w12.cpu(), wd.cpu(), hidden_dtype=bf16)
    assert_close(y[rows].cpu(), ref, bf16)


@pytest.mark.parametrize("parts", [2, 4, 8])
def test_square_gemm_split_along_m(parts):
    """The 8192^3 bf16 problem with A and C cut into `parts` row blocks (B replicated), the
    blocks run one after another on this GPU as the ranks of a `parts`-GPU job would run them:
    every block equals the same rows of the unsharded product bit for bit (a row of C depends
    on its row of A and on B only), and sampled rows match the oracle."""
    m = n = k = 8192
    a = device_randn((m, k), bf16, 60, k ** -0.5)
    b = device_randn((k, n), bf16, 61, 1.0)
    cfg = {**T, "tile_n": 256, "cta_group": 2, "tile_k": 128, "stages": 3, "group_m": 16}
    whole = torch.empty(m, n, device=DEV, dtype=bf16)
    _cabi.launch(a, b, whole, cfg)
    rows_per = m // parts
    sharded = torch.full((m, n), float("nan"), device=DEV, dtype=bf16)
    for r in range(parts):
        lo, hi = r * rows_per, (r + 1) * rows_per
        _cabi.launch(a[lo:hi], b, sharded[lo:hi], cfg)
    _cabi.check_status(whole.device)
    assert torch.equal(whole, sharded)
    rows = sorted({0, m - 1, rows_per - 1, rows_per, 3 * rows_per // 2})
    assert_close(sharded[rows].cpu(), O.matmul_oracle(a[rows].cpu(), b.cpu()), bf16)
