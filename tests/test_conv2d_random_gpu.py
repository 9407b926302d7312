"""Seeded random convolution geometries against the CPU oracle: every combination of filter
size, stride, padding, dilation, channel counts, batch, layout and dtype that the draw produces
must agree with the reference arithmetic, whichever internal route the library takes for it
(im2col-mode boxes, width folding for thin inputs, the batched GEMM for 1 x 1 over NCHW, the
fp32 kernel)."""
import random

import pytest
import torch

from oracle import conv2d as OC
from tritonix_b200 import _cabi
from tritonix_b200.ops.conv2d import conv2d_forward_kernel

pytestmark = pytest.mark.gpu
TOL = {torch.float16: 2e-3, torch.bfloat16: 8e-3, torch.float32: 1e-5}
DEV = "cuda"


def draw(seed):
    rng = random.Random(seed)
    r, s = rng.choice([1, 1, 2, 3, 3, 3, 5]), rng.choice([1, 1, 2, 3, 3, 3, 4, 7])
    stride = (rng.choice([1, 1, 1, 2, 3]), rng.choice([1, 1, 1, 2, 3]))
    dilation = (rng.choice([1, 1, 1, 2]), rng.choice([1, 1, 1, 2, 3]))
    padding = (rng.choice([0, 0, 1, 1, 2, 3]), rng.choice([0, 0, 1, 1, 2, 4]))
    c_in = rng.choice([1, 3, 4, 8, 16, 17, 24, 40, 64, 72, 130])
    c_out = rng.choice([1, 5, 8, 16, 40, 64, 72, 128, 136, 200])
    batch = rng.choice([1, 1, 2, 3])
    h = rng.randint((r - 1) * dilation[0] + 1, 26)
    w = rng.randint((s - 1) * dilation[1] + 1, 34)
    if rng.random() < 0.25:  # shapes the batched-GEMM route accepts: h * w and c_in multiples of 8
        r = s = 1
        stride, padding = (1, 1), (0, 0)
        h, w, c_in = rng.choice([2, 4, 8]), rng.choice([4, 8, 12]), rng.choice([8, 24, 64, 136])
    dtype = rng.choice([torch.float16, torch.float16, torch.bfloat16, torch.bfloat16, torch.float32])
    channels_last = rng.random() < 0.4
    bias = rng.random() < 0.6
    return (batch, c_in, h, w), (c_out, r, s), stride, padding, dilation, dtype, channels_last, bias


@pytest.mark.parametrize("seed", range(96))
def test_random_geometry(seed):
    xshape, wshape, stride, padding, dilation, dtype, channels_last, has_bias = draw(seed)
    g = torch.Generator().manual_seed(1000 + seed)
    n, c, h, w = xshape
    c_out, r, s = wshape
    x = torch.randn(n, c, h, w, generator=g).to(dtype)
    wt = (torch.randn(c_out, c, r, s, generator=g) * (c * r * s) ** -0.5).to(dtype)
    b = torch.randn(c_out, generator=g).to(dtype) if has_bias else None
    h_out, w_out = OC.conv_output_size(h, w, r, s, stride, padding, dilation)
    xd = x.to(DEV)
    out = torch.full((n, c_out, h_out, w_out), float("nan"), device=DEV, dtype=dtype)
    if channels_last:
        xd = xd.contiguous(memory_format=torch.channels_last)
        out = out.contiguous(memory_format=torch.channels_last)
    conv2d_forward_kernel[(1,)](out, xd, wt.to(DEV), b.to(DEV) if has_bias else None, n, c, h, w,
                                c_out, h_out, w_out, r, s, stride[0], stride[1], padding[0],
                                padding[1], dilation[0], dilation[1])
    _cabi.check_status(out.device)
    got = out.cpu().contiguous()
    ref = OC.conv2d_oracle(x, wt, b, stride, padding, dilation)
    assert got.shape == ref.shape and not torch.isnan(got.float()).any()
    err = OC.rel_err(got, ref)
    assert err <= TOL[dtype], (f"seed {seed}: {xshape} * {wshape} stride {stride} pad {padding} "
                               f"dil {dilation} {dtype} cl={channels_last}: err {err:.3e}")
