"""Fused GLU / SwiGLU parity: gate and up columns interleaved in W12, activation on the fp32
accumulator, one rounding (tritonix/ops/swiglu.py:82-110)."""
import pytest
import torch

from oracle import contraction as O
from tests.golden_cases import case_ids, inputs_and_reference
from tests.gpu_util import DEV, assert_close, run_gemm, seeded
from tritonix_b200 import _cabi

pytestmark = pytest.mark.gpu
bf16, f16, f32 = torch.bfloat16, torch.float16, torch.float32
T = {"kernel": "tcgen05"}
EPI = {"none": _cabi.EPI_GLU_LINEAR, "silu": _cabi.EPI_GLU_SILU, "sigmoid": _cabi.EPI_GLU_SIGMOID}


@pytest.mark.parametrize("name", case_ids("glu"))
def test_matches_reference_kernel_outputs(golden, name):
    x, w12, ref, case = inputs_and_reference(golden, name)
    act = case[7]["activation"]
    out, _ = run_gemm(x, w12, None, EPI[act])
    assert_close(out, ref, x.dtype, scale=10 if x.dtype == f32 else 1)
    assert_close(out, O.glu_oracle(x, w12, act), x.dtype, scale=10 if x.dtype == f32 else 1)


@pytest.mark.parametrize("act", ["silu", "sigmoid", "none"])
@pytest.mark.parametrize("m,f,k,dtype,cfg", [
    (128, 64, 128, bf16, {"tile_n": 128}),
    (512, 512, 512, bf16, {"tile_n": 256}),
    (512, 512, 512, f16, {"tile_n": 256, "cta_group": 2}),
    (300, 200, 520, f16, {"tile_n": 128}),                       # ragged; F multiple of 8
    (1000, 1000, 264, bf16, {"tile_n": 256, "cta_group": 2, "tile_k": 128, "stages": 3}),
    (2048, 1792, 1024, bf16, {"tile_n": 256, "cta_group": 2}),   # per-rank hidden width at TP=8
])
def test_tcgen05_against_oracle(act, m, f, k, dtype, cfg):
    x, w12 = seeded(m, k, 2 * f, dtype, seed=f, b_scale=0.02 * (4096 / k) ** 0.5)
    out, res = run_gemm(x, w12, {**T, **cfg}, EPI[act])
    assert res.kernel == _cabi.KERNEL_TCGEN05 and out.shape == (m, f)
    assert_close(out, O.glu_oracle(x, w12, act), dtype)


@pytest.mark.parametrize("m,f,k,dtype", [(512, 512, 512, bf16), (1000, 328, 264, f16), (300, 136, 2048, bf16)])
def test_double_tiles_with_glu_epilogue(m, f, k, dtype):
    """tile_n = 512 (two 256-column tiles per CTA pair) under the GLU epilogue: bit-identical to
    single tiles, including a last double tile whose right half is empty or ragged."""
    x, w12 = seeded(m, k, 2 * f, dtype, seed=f + 1, b_scale=0.02 * (4096 / k) ** 0.5)
    wide, res = run_gemm(x, w12, {**T, "tile_n": 512, "cta_group": 2, "tile_k": 64, "stages": 4}, EPI["silu"])
    assert res.kernel == _cabi.KERNEL_TCGEN05 and wide.shape == (m, f)
    assert_close(wide, O.glu_oracle(x, w12, "silu"), dtype)
    single, _ = run_gemm(x, w12, {**T, "tile_n": 256, "cta_group": 2, "tile_k": 64}, EPI["silu"])
    assert torch.equal(wide, single)


@pytest.mark.parametrize("m,f,k,dtype", [(64, 36, 50, f16), (100, 35, 90, bf16), (64, 48, 40, f32)])
def test_strided_kernel_glu(m, f, k, dtype):
    x, w12 = seeded(m, k, 2 * f, dtype, seed=1, b_scale=0.1)
    for act in ("silu", "sigmoid", "none"):
        out, res = run_gemm(x, w12, None, EPI[act])
        assert res.kernel == _cabi.KERNEL_STRIDED
        assert_close(out, O.glu_oracle(x, w12, act), dtype, scale=10 if dtype == f32 else 1)


def test_full_size_swiglu_by_sampled_rows():
    """x 8192x4096 N(0,1), W1/W2 4096x14336 N(0, 0.02^2) interleaved to 4096x28672, bf16."""
    m, k, f = 8192, 4096, 14336
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn(m, k, device=DEV, generator=g).to(bf16)
    w12 = (torch.randn(k, 2 * f, device=DEV, generator=g) * 0.02).to(bf16)
    rows = torch.randint(0, m, (32,), generator=torch.Generator().manual_seed(2)).tolist() + [0, m - 1]
    for act in ("silu", "sigmoid"):
        z = torch.empty(m, f, device=DEV, dtype=bf16)
        _cabi.launch(x, w12, z, {**T, "tile_n": 256, "cta_group": 2, "tile_k": 128, "stages": 3, "group_m": 16}, EPI[act])
        _cabi.check_status(z.device)
        assert_close(z[rows].cpu(), O.glu_oracle(x[rows].cpu(), w12.cpu(), act), bf16)


def test_interleave_matches_separate_weights():
    import tritonix_b200 as t
    g = torch.Generator().manual_seed(5)
    x = torch.randn(256, 512, generator=g).to(f16)
    w1 = (torch.randn(512, 384, generator=g) * 0.04).to(f16)
    w2 = (torch.randn(512, 384, generator=g) * 0.04).to(f16)
    w12 = t.interleave_weights(w1, w2)
    assert torch.equal(w12[:, 0::2], w1) and torch.equal(w12[:, 1::2], w2)
    z = t.swiglu(x.to(DEV), w12.to(DEV), cfg={"tile_n": 128})
    t.check_status()
    ref = (torch.nn.functional.silu(x.float() @ w1.float()) * (x.float() @ w2.float())).to(f16)
    assert_close(z.cpu(), ref, f16)
