"""Pins the convolution oracle to outputs of the reference's own kernel (tests/golden) and to
torch's CPU convolution."""
import pytest
import torch

from oracle import conv2d as OC
from tests import conv_cases

TOL = {"float16": 2e-3, "float32": 1e-5}


@pytest.fixture(scope="module")
def conv_golden():
    return conv_cases.golden()


@pytest.mark.parametrize("name", conv_cases.case_ids())
def test_oracle_matches_reference_kernel(conv_golden, name):
    x, w, b, stride, padding, dilation, ref, dtype = conv_cases.load_case(conv_golden, name)
    out = OC.conv2d_oracle(x, w, b, stride, padding, dilation)
    assert out.shape == ref.shape and out.dtype == ref.dtype
    assert OC.rel_err(out, ref) <= TOL[dtype]


@pytest.mark.parametrize("geom", [
    ((2, 5, 9, 8), (7, 3, 3), (1, 1), (1, 1), (1, 1)),
    ((1, 4, 11, 6), (3, 2, 4), (2, 3), (1, 2), (1, 1)),
    ((3, 2, 7, 7), (4, 3, 3), (1, 1), (0, 0), (2, 2)),
    ((1, 1, 5, 5), (1, 5, 5), (1, 1), (0, 0), (1, 1)),   # one output pixel
    ((1, 3, 4, 4), (2, 3, 3), (1, 1), (3, 3), (1, 1)),   # more padding than image
])
def test_oracle_matches_torch_conv2d(geom):
    xshape, (c_out, r, s), stride, padding, dilation = geom
    g = torch.Generator().manual_seed(7)
    x = torch.randn(*xshape, generator=g, dtype=torch.float64)
    w = torch.randn(c_out, xshape[1], r, s, generator=g, dtype=torch.float64)
    b = torch.randn(c_out, generator=g, dtype=torch.float64)
    want = torch.nn.functional.conv2d(x, w, b, stride, padding, dilation)
    got = OC.conv2d_oracle(x.float(), w.float(), b.float(), stride, padding, dilation,
                           out_dtype=torch.float64)
    assert got.shape == want.shape
    assert OC.rel_err(got, want) <= 1e-6


def test_output_size_formula():
    assert OC.conv_output_size(12, 12, 3, 3, (1, 1), (1, 1), (1, 1)) == (12, 12)
    assert OC.conv_output_size(15, 13, 3, 3, (2, 2), (1, 1), (1, 1)) == (8, 7)
    assert OC.conv_output_size(14, 16, 5, 3, (1, 1), (2, 3), (2, 1)) == (10, 20)


@pytest.mark.parametrize("seed", range(24))
def test_oracle_matches_torch_conv2d_on_random_geometries(seed):
    import random
    rng = random.Random(seed)
    r, s = rng.randint(1, 5), rng.randint(1, 5)
    stride = (rng.randint(1, 3), rng.randint(1, 3))
    dilation = (rng.randint(1, 3), rng.randint(1, 2))
    padding = (rng.randint(0, 3), rng.randint(0, 4))
    n, c, c_out = rng.randint(1, 3), rng.randint(1, 9), rng.randint(1, 7)
    h = rng.randint((r - 1) * dilation[0] + 1, 14)
    w = rng.randint((s - 1) * dilation[1] + 1, 15)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, c, h, w, generator=g, dtype=torch.float64)
    wt = torch.randn(c_out, c, r, s, generator=g, dtype=torch.float64)
    b = torch.randn(c_out, generator=g, dtype=torch.float64) if seed % 2 else None
    want = torch.nn.functional.conv2d(x, wt, b, stride, padding, dilation)
    got = OC.conv2d_oracle(x.float(), wt.float(), None if b is None else b.float(), stride, padding,
                           dilation, out_dtype=torch.float64)
    assert got.shape == want.shape
    assert OC.rel_err(got, want) <= 1e-6
