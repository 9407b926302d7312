"""GPU parity of the convolution forward (tnx_conv2d_forward through the C ABI) against the
CPU oracle and against outputs of the reference's own kernel."""
import pytest
import torch

from oracle import conv2d as OC
from tests import conv_cases
from tritonix_b200 import _cabi
from tritonix_b200.ops.conv2d import conv2d_forward, conv2d_forward_kernel

pytestmark = pytest.mark.gpu
TOL = {torch.float16: 2e-3, torch.bfloat16: 8e-3, torch.float32: 1e-5}
DEV = "cuda"


@pytest.fixture(autouse=True)
def fresh_conv_caches():
    """Tests flip the TNX_CONV_* switches, which the Python layer reads when it first sees a call
    signature: start every test without remembered calls."""
    from tritonix_b200.ops import conv2d as conv_module
    conv_module.clear_caches()
    yield
    conv_module.clear_caches()


def run_conv(x, w, b, stride, padding, dilation, cfg=None, channels_last=False):
    """One launch through the C ABI into a NaN-filled output."""
    xd, wd = x.to(DEV), w.to(DEV)
    bd = b.to(DEV) if b is not None else None
    if channels_last:
        xd = xd.contiguous(memory_format=torch.channels_last)
    n, c, h, wi = x.shape
    c_out, _, r, s = w.shape
    h_out, w_out = OC.conv_output_size(h, wi, r, s, stride, padding, dilation)
    out = torch.full((n, c_out, h_out, w_out), float("nan"), device=DEV, dtype=x.dtype)
    if channels_last:
        out = out.contiguous(memory_format=torch.channels_last)
    res = conv2d_forward_kernel[(1,)](out, xd, wd, bd, n, c, h, wi, c_out, h_out, w_out, r, s,
                                      stride[0], stride[1], padding[0], padding[1], dilation[0],
                                      dilation[1], n * h_out * w_out, c_out, c * r * s,
                                      **(cfg or {}))
    _cabi.check_status(out.device)
    return out.cpu().contiguous(), res


def check(out, ref, dtype, scale=1.0):
    assert out.shape == ref.shape and out.dtype == ref.dtype
    assert not torch.isnan(out.float()).any(), "output has unwritten / NaN elements"
    err = OC.rel_err(out, ref)
    assert err <= TOL[dtype] * scale, f"max|err|/max|ref| = {err:.3e}"


def seeded(xshape, wshape, dtype, bias=True, seed=0):
    g = torch.Generator().manual_seed(seed)
    n, c, h, w = xshape
    c_out, r, s = wshape
    x = torch.randn(n, c, h, w, generator=g).to(dtype)
    wt = (torch.randn(c_out, c, r, s, generator=g) * (c * r * s) ** -0.5).to(dtype)
    b = torch.randn(c_out, generator=g).to(dtype) if bias else None
    return x, wt, b


@pytest.fixture(scope="module")
def conv_golden():
    return conv_cases.golden()


@pytest.mark.parametrize("name", conv_cases.case_ids())
def test_matches_reference_kernel_output(conv_golden, name):
    x, w, b, stride, padding, dilation, ref, dtype = conv_cases.load_case(conv_golden, name)
    out, res = run_conv(x, w, b, stride, padding, dilation)
    assert res.kernel == (_cabi.KERNEL_STRIDED if dtype == "float32" else _cabi.KERNEL_TCGEN05)
    check(out, ref, x.dtype)
    check(out, OC.conv2d_oracle(x, w, b, stride, padding, dilation), x.dtype)


GEOMS = [
    # xshape, (c_out, r, s), stride, padding, dilation
    ((1, 64, 56, 56), (64, 3, 3), (1, 1), (1, 1), (1, 1)),     # ResNet 3x3
    ((2, 64, 56, 56), (128, 3, 3), (2, 2), (1, 1), (1, 1)),    # strided 3x3
    ((2, 256, 14, 14), (512, 1, 1), (1, 1), (0, 0), (1, 1)),   # 1x1, 4 channel blocks
    ((1, 3, 64, 64), (32, 7, 7), (2, 2), (3, 3), (1, 1)),      # stem: 3 channels, 7x7 / 2
    ((1, 32, 20, 24), (48, 3, 3), (1, 1), (2, 2), (2, 2)),     # dilated
    ((3, 96, 7, 7), (160, 3, 3), (1, 1), (1, 1), (1, 1)),      # small image, 49 pixels
    ((1, 40, 17, 19), (72, 3, 5), (2, 1), (0, 2), (1, 1)),     # ragged everything
    ((1, 128, 28, 28), (200, 3, 3), (1, 1), (1, 1), (1, 1)),   # c_out not a tile multiple
    ((2, 16, 9, 9), (8, 3, 3), (3, 3), (0, 0), (1, 1)),        # stride 3, tiny c_out
    ((1, 8, 5, 300), (16, 1, 3), (1, 1), (0, 1), (1, 1)),      # wide rows
    ((1, 130, 33, 21), (24, 5, 2), (1, 1), (4, 0), (1, 3)),    # 3 channel blocks, 5x2 dilated filter
    ((2, 64, 12, 126), (32, 3, 3), (1, 1), (1, 1), (1, 1)),    # rows of 126 pixels
    ((5, 72, 9, 9), (136, 3, 3), (1, 1), (0, 0), (1, 1)),      # no padding, odd tile counts
]


@pytest.fixture(params=["default", "im2col", "tiled"])
def box_mode(request, monkeypatch):
    """The ways the kernel fetches input pixels: the library's own choice (a halo patch per
    channel block for layers of at most 64 output channels where it applies, else one im2col-mode
    box per tap), im2col-mode boxes everywhere, rectangular tiled boxes everywhere."""
    monkeypatch.delenv("TNX_CONV_TILED", raising=False)
    monkeypatch.delenv("TNX_CONV_NO_HALO", raising=False)
    if request.param != "default":
        monkeypatch.setenv("TNX_CONV_NO_HALO", "1")
    if request.param == "tiled":
        monkeypatch.setenv("TNX_CONV_TILED", "1")
    return request.param


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("geom", GEOMS)
def test_geometries_against_oracle(geom, dtype, box_mode):
    xshape, wshape, stride, padding, dilation = geom
    x, w, b = seeded(xshape, wshape, dtype, bias=True, seed=xshape[1])
    out, res = run_conv(x, w, b, stride, padding, dilation)
    assert res.kernel == _cabi.KERNEL_TCGEN05
    check(out, OC.conv2d_oracle(x, w, b, stride, padding, dilation), dtype)


THIN = [
    ((2, 3, 64, 64), (32, 7, 7), (2, 2), (3, 3), (1, 1)),      # the classic stem
    ((1, 3, 33, 47), (24, 3, 3), (1, 1), (1, 1), (1, 1)),
    ((2, 8, 20, 24), (16, 3, 5), (1, 2), (1, 2), (1, 1)),      # 40 folded channels
    ((1, 16, 18, 18), (40, 3, 4), (1, 1), (0, 2), (2, 1)),     # exactly 64 folded channels
    ((1, 4, 9, 120), (8, 1, 5), (1, 11), (0, 0), (1, 1)),      # horizontal stride 11
    ((3, 1, 28, 28), (8, 5, 5), (1, 1), (2, 2), (1, 2)),       # one channel, dilated columns
]


@pytest.mark.parametrize("fold", [True, False])
@pytest.mark.parametrize("layout", ["nchw", "channels_last"])
@pytest.mark.parametrize("geom", THIN)
def test_thin_inputs(geom, layout, fold, monkeypatch):
    """Inputs with few channels: the filter row is folded into the channels (default) or every
    tap gets its own zero-padded 64-channel block (TNX_CONV_NO_FOLD); same numbers either way."""
    xshape, wshape, stride, padding, dilation = geom
    if not fold:
        if stride[1] > 8:
            pytest.skip("strides above 8 need the folded path")
        monkeypatch.setenv("TNX_CONV_NO_FOLD", "1")
    x, w, b = seeded(xshape, wshape, torch.float16, bias=True, seed=wshape[0])
    out, res = run_conv(x, w, b, stride, padding, dilation, channels_last=(layout == "channels_last"))
    assert res.kernel == _cabi.KERNEL_TCGEN05
    check(out, OC.conv2d_oracle(x, w, b, stride, padding, dilation), torch.float16)


POINTWISE = [
    ((2, 64, 8, 8), (24, 1, 1)),        # fewer output channels than a tile has rows
    ((3, 128, 28, 28), (256, 1, 1)),    # CTA pairs by default
    ((1, 40, 4, 6), (72, 1, 1)),        # 24 pixels: one ragged column tile
    ((5, 72, 12, 10), (200, 1, 1)),     # ragged rows, columns and K
]


@pytest.mark.parametrize("as_gemm", [True, False])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("geom", POINTWISE)
def test_pointwise_on_nchw_is_a_batch_of_gemms(geom, dtype, as_gemm, monkeypatch):
    """1 x 1 / stride 1 / no padding on NCHW tensors: one launch, no workspace, bias per output
    row; TNX_CONV_NO_BATCHED_GEMM sends the same call through the repacking path."""
    xshape, wshape = geom
    if not as_gemm:
        monkeypatch.setenv("TNX_CONV_NO_BATCHED_GEMM", "1")
    x, w, b = seeded(xshape, wshape, dtype, bias=True, seed=wshape[0])
    out, res = run_conv(x, w, b, (1, 1), (0, 0), (1, 1))
    assert (res.workspace_bytes == 0) == as_gemm
    check(out, OC.conv2d_oracle(x, w, b, (1, 1), (0, 0), (1, 1)), dtype)
    xd, wd, bd = x.to(DEV), w.to(DEV), b.to(DEV)
    via_entry = conv2d_forward(xd, wd, bd)
    _cabi.check_status(via_entry.device)
    check(via_entry.cpu(), OC.conv2d_oracle(x, w, b, (1, 1), (0, 0), (1, 1)), dtype)


@pytest.mark.parametrize("cfg", [
    dict(BLOCK_SIZE_M=128, BLOCK_SIZE_N=64, BLOCK_SIZE_K=64),
    dict(BLOCK_SIZE_M=128, BLOCK_SIZE_N=128, BLOCK_SIZE_K=128),
    dict(BLOCK_SIZE_M=128, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64, num_stages=3),
    dict(BLOCK_SIZE_M=256, BLOCK_SIZE_N=128, BLOCK_SIZE_K=64),
    dict(BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=128, GROUP_SIZE_M=4),
    dict(tile_n=128, tile_k=64, cta_group=2, stages=2),
])
def test_configurations(cfg, box_mode):
    x, w, b = seeded((2, 192, 30, 30), (320, 3, 3), torch.bfloat16, seed=11)
    out, res = run_conv(x, w, b, (1, 1), (1, 1), (1, 1), cfg)
    assert (res.tile_w, res.tile_h) == ((30, 4) if box_mode == "tiled" else (128, 1))
    check(out, OC.conv2d_oracle(x, w, b, (1, 1), (1, 1), (1, 1)), torch.bfloat16)


@pytest.mark.parametrize("channels", [(64, 64), (24, 40), (30, 64), (64, 20)])
def test_channels_last_in_and_out(channels, box_mode):
    """torch.channels_last tensors: used in place when the channel counts are multiples of 8,
    through the padding passes otherwise; same numbers either way."""
    c_in, c_out = channels
    x, w, b = seeded((2, c_in, 18, 22), (c_out, 3, 3), torch.float16, seed=5)
    ref = OC.conv2d_oracle(x, w, b, (1, 1), (1, 1), (1, 1))
    out_cl, _ = run_conv(x, w, b, (1, 1), (1, 1), (1, 1), channels_last=True)
    out, _ = run_conv(x, w, b, (1, 1), (1, 1), (1, 1))
    check(out_cl, ref, torch.float16)
    assert torch.equal(out_cl, out)


@pytest.mark.parametrize("geom", GEOMS[:5])
def test_fp32_kernel(geom):
    xshape, wshape, stride, padding, dilation = geom
    x, w, b = seeded(xshape, wshape, torch.float32, seed=3)
    out, res = run_conv(x, w, b, stride, padding, dilation)
    assert res.kernel == _cabi.KERNEL_STRIDED and res.workspace_bytes == 0
    check(out, OC.conv2d_oracle(x, w, b, stride, padding, dilation), torch.float32)
    out_cl, _ = run_conv(x, w, b, stride, padding, dilation, channels_last=True)
    check(out_cl, OC.conv2d_oracle(x, w, b, stride, padding, dilation), torch.float32)


def test_public_entry_tunes_and_repeats():
    x, w, b = seeded((2, 64, 28, 28), (96, 3, 3), torch.bfloat16, seed=9)
    xd, wd, bd = x.to(DEV), w.to(DEV), b.to(DEV)
    first = conv2d_forward(xd, wd, bd, stride=1, padding=1)
    second = conv2d_forward(xd, wd, bd, stride=(1, 1), padding=(1, 1))
    _cabi.check_status(first.device)
    assert torch.equal(first, second)
    check(first.cpu(), OC.conv2d_oracle(x, w, b, (1, 1), (1, 1), (1, 1)), torch.bfloat16)
    fixed = conv2d_forward(xd, wd, bd, padding=(1, 1),
                           config=dict(BLOCK_SIZE_M=128, BLOCK_SIZE_N=128, BLOCK_SIZE_K=64))
    check(fixed.cpu(), OC.conv2d_oracle(x, w, b, (1, 1), (1, 1), (1, 1)), torch.bfloat16)
    cl = conv2d_forward(xd.contiguous(memory_format=torch.channels_last), wd, bd, padding=1)
    assert cl.is_contiguous(memory_format=torch.channels_last)
    check(cl.cpu().contiguous(), OC.conv2d_oracle(x, w, b, (1, 1), (1, 1), (1, 1)), torch.bfloat16)


def test_linearity_at_full_size():
    """conv(x1 + x2) = conv(x1) + conv(x2) for inputs whose sums are exact in bf16, at a size the
    CPU oracle would take too long on (ResNet-50 layer, batch 32)."""
    g = torch.Generator().manual_seed(1)
    x1 = torch.randint(-4, 5, (32, 128, 28, 28), generator=g).to(torch.bfloat16).to(DEV)
    x2 = torch.randint(-4, 5, (32, 128, 28, 28), generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randint(-2, 3, (128, 128, 3, 3), generator=g).to(torch.bfloat16).to(DEV)
    y1 = conv2d_forward(x1, w, None, padding=1, config=dict(BLOCK_SIZE_M=256, BLOCK_SIZE_N=128))
    y2 = conv2d_forward(x2, w, None, padding=1, config=dict(BLOCK_SIZE_M=256, BLOCK_SIZE_N=128))
    y12 = conv2d_forward(x1 + x2, w, None, padding=1,
                         config=dict(BLOCK_SIZE_M=128, BLOCK_SIZE_N=128))
    _cabi.check_status(y1.device)
    # small integers: every product and partial sum is exact in fp32, the results in bf16 are
    # exact whenever they stay below 256 in magnitude; compare in fp32 with the bf16 tolerance
    err = OC.rel_err(y12.float().cpu(), (y1.float() + y2.float()).cpu())
    assert err <= 8e-3


HALO = [
    # xshape, (c_out, r, s), padding, dilation  (stride 1, at most 64 input and 64 output channels)
    ((2, 64, 56, 56), (64, 3, 3), (1, 1), (1, 1)),     # 58-pixel patch rows, 2 output rows per tile
    ((3, 48, 28, 28), (48, 3, 3), (1, 1), (1, 1)),     # 30-pixel rows, 4 per tile, ragged channels
    ((1, 40, 33, 21), (24, 3, 2), (2, 0), (1, 3)),     # 3x2 filter, dilated columns, ragged rows
    ((2, 64, 12, 126), (32, 3, 3), (1, 1), (1, 1)),    # patch rows of exactly 128 pixels
    ((5, 24, 9, 9), (64, 2, 2), (0, 0), (1, 1)),       # even filter, no padding, many tiles per CTA
    ((1, 56, 7, 7), (8, 3, 3), (1, 1), (2, 2)),        # dilated 3x3 on a 7x7 image
    ((40, 32, 20, 20), (16, 3, 3), (1, 1), (1, 1)),    # 160 tiles: every CTA reuses its resident weights
]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("geom", HALO)
def test_halo_patch_variant(geom, dtype, monkeypatch):
    """Layers of at most 64 output channels: one patch load per channel block, every tap a
    shifted window of it.  Same numbers as one load per tap (TNX_CONV_NO_HALO)."""
    xshape, wshape, padding, dilation = geom
    x, w, b = seeded(xshape, wshape, dtype, bias=True, seed=wshape[0] + xshape[1])
    ref = OC.conv2d_oracle(x, w, b, (1, 1), padding, dilation)
    out, res = run_conv(x, w, b, (1, 1), padding, dilation)
    halo_w = ref.shape[3] + (wshape[2] - 1) * dilation[1]
    assert res.tile_w == halo_w and res.tile_h == min(128 // halo_w, ref.shape[2])
    check(out, ref, dtype)
    monkeypatch.setenv("TNX_CONV_NO_HALO", "1")
    per_tap, res2 = run_conv(x, w, b, (1, 1), padding, dilation)
    assert (res2.tile_w, res2.tile_h) == (128, 1)
    check(per_tap, ref, dtype)


def test_wide_padding_uses_rectangles():
    """Padding beyond what an im2col box can express (128) falls back to rectangles of pixels."""
    x, w, b = seeded((1, 16, 6, 6), (16, 3, 3), torch.float16, seed=2)
    out, res = run_conv(x, w, b, (1, 1), (130, 2), (1, 1))
    assert (res.tile_w, res.tile_h) != (128, 1)
    check(out, OC.conv2d_oracle(x, w, b, (1, 1), (130, 2), (1, 1)), torch.float16)


def test_packed_weights_match_and_follow_updates():
    """Weights packed once (tnx_conv2d_pack_weights) give the same bits as weights packed inside
    the call, and the public entry repacks after an in-place update of the weight tensor."""
    x, w, b = seeded((2, 48, 16, 16), (40, 3, 3), torch.float16, seed=4)
    ref, _ = run_conv(x, w, b, (1, 1), (1, 1), (1, 1))
    xd, wd, bd = x.to(DEV), w.to(DEV), b.to(DEV)
    problem = _cabi.make_conv_problem(2, 48, 16, 16, 40, 3, 3, (1, 1), (1, 1), (1, 1),
                                      torch.float16, True)
    packed = _cabi.conv_pack_weights(problem, wd)
    out = torch.full((2, 40, 16, 16), float("nan"), device=DEV, dtype=torch.float16)
    conv2d_forward_kernel[(1,)](out, xd, packed, bd, 2, 48, 16, 16, 40, 16, 16, 3, 3, 1, 1, 1, 1,
                                1, 1, weights_packed=True)
    _cabi.check_status(out.device)
    assert torch.equal(out.cpu(), ref)

    y1 = conv2d_forward(xd, wd, bd, padding=1)
    y1_again = conv2d_forward(xd, wd, bd, padding=1)       # served from the packed-weight cache
    assert torch.equal(y1, y1_again)
    wd.mul_(2.0)                                           # in place: same storage, new version
    y2 = conv2d_forward(xd, wd, bd, padding=1)
    _cabi.check_status(y2.device)
    check(y2.cpu(), OC.conv2d_oracle(x, w * 2.0, b, (1, 1), (1, 1), (1, 1)), torch.float16)
    assert not torch.equal(y1, y2)


def test_tuner_drives_the_convolution_handle():
    """conv2d_forward_kernel.tune(launcher): the grid search walks the space under the
    reference's key names, prunes what does not fit an SM (OutOfResources from the library's
    resource check) and returns a configuration that computes the right numbers."""
    x, w, b = seeded((2, 64, 20, 20), (96, 3, 3), torch.bfloat16, seed=13)
    xd, wd, bd = x.to(DEV), w.to(DEV), b.to(DEV)
    out = torch.empty((2, 96, 20, 20), device=DEV, dtype=torch.bfloat16)
    seen = []

    def launcher(cfg):
        seen.append(dict(cfg))
        conv2d_forward_kernel[(1,)](out, xd, wd, bd, 2, 64, 20, 20, 96, 20, 20, 3, 3, 1, 1, 1, 1,
                                    1, 1, **cfg)

    best = conv2d_forward_kernel.tune(launcher, max_configs=24, warmup=1, rep=3)
    _cabi.check_status(out.device)
    assert best is not None and set(best) == set(conv2d_forward_kernel.space)
    assert 1 <= len(seen) and all(c["BLOCK_SIZE_M"] in (128, 256) for c in seen)
    out.fill_(float("nan"))
    launcher(best)
    _cabi.check_status(out.device)
    check(out.cpu(), OC.conv2d_oracle(x, w, b, (1, 1), (1, 1), (1, 1)), torch.bfloat16)
    # a ring that cannot fit is reported the way the tuner expects
    with pytest.raises(_cabi.OutOfResources):
        launcher(dict(BLOCK_SIZE_M=128, BLOCK_SIZE_N=256, BLOCK_SIZE_K=128, GROUP_SIZE_M=8, num_stages=8))


def test_torch_custom_op_and_fake_kernel():
    import tritonix_b200  # noqa: F401  (registers torch.ops.tritonix.*)
    from torch._subclasses.fake_tensor import FakeTensorMode
    x, w, b = seeded((2, 32, 12, 10), (24, 3, 3), torch.float16, seed=6)
    y = torch.ops.tritonix.conv2d_forward(x.to(DEV), w.to(DEV), b.to(DEV), [2, 1], [1, 1], [1, 1], [])
    _cabi.check_status(y.device)
    check(y.cpu(), OC.conv2d_oracle(x, w, b, (2, 1), (1, 1), (1, 1)), torch.float16)
    with FakeTensorMode():
        fx = torch.empty(2, 32, 12, 10, device=DEV, dtype=torch.float16)
        fw = torch.empty(24, 32, 3, 3, device=DEV, dtype=torch.float16)
        assert torch.ops.tritonix.conv2d_forward(fx, fw, None, [2, 1], [1, 1], [1, 1], []).shape \
            == (2, 24, 6, 10)


def test_errors():
    x = torch.zeros(1, 8, 4, 4, device=DEV, dtype=torch.float16)
    w = torch.zeros(8, 8, 7, 7, device=DEV, dtype=torch.float16)
    with pytest.raises(ValueError):
        conv2d_forward(x, w)  # filter larger than the input
    with pytest.raises(ValueError):
        conv2d_forward(x, torch.zeros(8, 4, 3, 3, device=DEV, dtype=torch.float16))
    with pytest.raises(RuntimeError):
        conv2d_forward(x.cpu(), w.cpu())
    with pytest.raises(ValueError):
        conv2d_forward(x, torch.zeros(8, 8, 3, 3, device=DEV, dtype=torch.float16),
                       config=dict(BLOCK_SIZE_M=64))


def test_strided_view_does_not_reuse_a_prepared_channels_last_call():
    """A prepared call is keyed by the input's strides: after a channels_last call, an arbitrary
    strided view of the same shape must be rejected (as the general path does), not read as
    dense N x H x W x C memory."""
    x, w, b = seeded((2, 32, 12, 12), (24, 3, 3), torch.float16, seed=21)
    xd, wd, bd = x.to(DEV), w.to(DEV), b.to(DEV)
    cl = xd.contiguous(memory_format=torch.channels_last)
    y1 = conv2d_forward(cl, wd, bd, padding=1)
    y2 = conv2d_forward(cl, wd, bd, padding=1)      # prepared call
    assert torch.equal(y1, y2)
    wide = torch.zeros(2, 32, 12, 16, device=DEV, dtype=torch.float16)
    view = wide[..., :12]
    view.copy_(xd)
    assert view.shape == cl.shape and not view.is_contiguous()
    with pytest.raises(ValueError, match="contiguous"):
        conv2d_forward(view, wd, bd, padding=1)
    y3 = conv2d_forward(view.contiguous(), wd, bd, padding=1)
    _cabi.check_status(y3.device)
    check(y3.cpu(), OC.conv2d_oracle(x, w, b, (1, 1), (1, 1), (1, 1)), torch.float16)


def test_weights_written_through_data_need_the_static_switch():
    x, w, b = seeded((2, 48, 16, 16), (40, 3, 3), torch.float16, seed=8)
    xd, wd, bd = x.to(DEV), w.to(DEV), b.to(DEV)
    conv2d_forward(xd, wd, bd, padding=1)
    wd.data.copy_((w * 3.0).to(DEV))               # does not move the version counter
    y = conv2d_forward(xd, wd, bd, padding=1, weights_static=False)
    _cabi.check_status(y.device)
    check(y.cpu(), OC.conv2d_oracle(x, w * 3.0, b, (1, 1), (1, 1), (1, 1)), torch.float16)
