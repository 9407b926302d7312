"""Host-side logic of the convolution entry points: geometry, kernel family, workspace layout
and validation through tnx_conv2d_query (no device work)."""
import ctypes

import pytest
import torch

from oracle import conv2d as OC
from tritonix_b200 import _cabi


def query(xshape, wshape, stride=(1, 1), padding=(0, 0), dilation=(1, 1), dtype=torch.bfloat16,
          cfg=None, **kw):
    n, c, h, w = xshape
    c_out, r, s = wshape
    p = _cabi.make_conv_problem(n, c, h, w, c_out, r, s, stride, padding, dilation, dtype, False, **kw)
    return _cabi.conv_query(p, _cabi.make_config(cfg) if cfg else None), p


@pytest.mark.parametrize("geom", [
    ((2, 16, 12, 12), (32, 3, 3), (1, 1), (1, 1), (1, 1)),
    ((2, 8, 15, 13), (16, 3, 3), (2, 2), (1, 1), (1, 1)),
    ((1, 8, 14, 16), (8, 5, 3), (1, 1), (2, 3), (2, 1)),
    ((1, 3, 224, 224), (64, 7, 7), (2, 2), (3, 3), (1, 1)),
])
def test_output_geometry_matches_reference_formula(geom):
    xshape, wshape, stride, padding, dilation = geom
    res, _ = query(xshape, wshape, stride, padding, dilation)
    assert (res.h_out, res.w_out) == OC.conv_output_size(xshape[2], xshape[3], wshape[1], wshape[2],
                                                         stride, padding, dilation)


def test_kernel_family_and_workspace():
    res, _ = query((2, 64, 56, 56), (128, 3, 3), padding=(1, 1))
    assert res.kernel == _cabi.KERNEL_TCGEN05 and (res.tile_w, res.tile_h) == (128, 1)
    x_bytes = 2 * 56 * 56 * 64 * 2
    w_bytes = 128 * 9 * 64 * 2
    y_bytes = 2 * 56 * 56 * 128 * 2
    assert res.workspace_bytes >= x_bytes + w_bytes + y_bytes
    assert res.workspace_bytes <= x_bytes + w_bytes + y_bytes + 3 * 256
    # channels_last in and out with channel counts that are multiples of 8: only the weights
    res_cl, _ = query((2, 64, 56, 56), (128, 3, 3), padding=(1, 1),
                      input_layout=_cabi.LAYOUT_NHWC, output_layout=_cabi.LAYOUT_NHWC)
    assert w_bytes <= res_cl.workspace_bytes <= w_bytes + 256
    # 24 input channels are padded to 64 in the packed weights (one 64-channel block per tap)
    res24, p24 = query((1, 24, 32, 32), (16, 3, 3), input_layout=_cabi.LAYOUT_NHWC)
    assert res24.workspace_bytes >= 16 * 9 * 64 * 2
    assert _cabi.lib.tnx_conv2d_packed_weight_bytes(ctypes.byref(p24)) == 16 * 9 * 64 * 2
    # fp32: CUDA-core kernel, nothing to repack
    res32, p32 = query((2, 64, 56, 56), (128, 3, 3), padding=(1, 1), dtype=torch.float32)
    assert res32.kernel == _cabi.KERNEL_STRIDED and res32.workspace_bytes == 0
    assert _cabi.lib.tnx_conv2d_packed_weight_bytes(ctypes.byref(p32)) == 0


def test_thin_inputs_fold_the_filter_row_into_channels(monkeypatch):
    """C <= 16 and S*C <= 64: the S taps of a filter row become channels of a repacked input
    (N x H x W_OUT x S*C, padded to 8), the kernel then sees an R x 1 filter and the horizontal
    stride disappears (so strides above 8 are fine there)."""
    res, p = query((2, 3, 64, 64), (32, 7, 7), stride=(2, 2), padding=(3, 3))
    assert (res.h_out, res.w_out) == (32, 32)
    folded_in = 2 * 64 * 32 * 24 * 2                 # 7 * 3 = 21 channels -> 24
    packed = 32 * 7 * 64 * 2                         # one 64-wide K block per filter row
    y_nhwc = 2 * 32 * 32 * 32 * 2
    assert folded_in + packed + y_nhwc <= res.workspace_bytes <= folded_in + packed + y_nhwc + 3 * 256
    assert _cabi.lib.tnx_conv2d_packed_weight_bytes(ctypes.byref(p)) == packed
    res, _ = query((1, 4, 16, 200), (8, 1, 5), stride=(1, 11))     # stride_w folded away
    assert res.w_out == (200 - 5) // 11 + 1
    monkeypatch.setenv("TNX_CONV_NO_FOLD", "1")
    res, p = query((2, 3, 64, 64), (32, 7, 7), stride=(2, 2), padding=(3, 3))
    assert _cabi.lib.tnx_conv2d_packed_weight_bytes(ctypes.byref(p)) == 32 * 49 * 64 * 2
    with pytest.raises(ValueError):
        query((1, 4, 16, 200), (8, 1, 5), stride=(1, 11))
    monkeypatch.delenv("TNX_CONV_NO_FOLD")
    # not for 17+ channels, 1-wide filters or fp32
    for kw in (dict(xshape=(1, 17, 16, 16), wshape=(8, 3, 3)), dict(xshape=(1, 8, 16, 16), wshape=(8, 3, 1))):
        _, p = query(**kw)
        taps = kw["wshape"][1] * kw["wshape"][2]
        assert _cabi.lib.tnx_conv2d_packed_weight_bytes(ctypes.byref(p)) == 8 * taps * 64 * 2


def test_pointwise_nchw_needs_no_workspace(monkeypatch):
    """1 x 1, stride 1, no padding, NCHW: a batch of GEMMs on the tensors as they are."""
    res, p = query((4, 64, 28, 28), (256, 1, 1))
    assert res.kernel == _cabi.KERNEL_TCGEN05 and res.workspace_bytes == 0
    assert (res.h_out, res.w_out) == (28, 28) and res.grid % 2 == 0      # CTA pairs for 256 channels
    # anything that breaks the plain-GEMM shape goes through the repacking path
    for kw in (dict(stride=(2, 2)), dict(padding=(1, 1)), dict(input_layout=_cabi.LAYOUT_NHWC),
               dict(output_layout=_cabi.LAYOUT_NHWC), dict(weight_layout=_cabi.WEIGHT_PACKED)):
        res, _ = query((4, 64, 28, 28), (256, 1, 1), **kw)
        assert res.workspace_bytes > 0
    res, _ = query((4, 64, 7, 7), (256, 1, 1))        # 49 pixels per image: not a multiple of 8
    assert res.workspace_bytes > 0
    res, _ = query((4, 20, 8, 8), (256, 1, 1))        # 20 channels: not a multiple of 8
    assert res.workspace_bytes > 0
    monkeypatch.setenv("TNX_CONV_NO_BATCHED_GEMM", "1")
    res, _ = query((4, 64, 28, 28), (256, 1, 1))
    assert res.workspace_bytes > 0


def test_halo_tiles_for_layers_with_few_output_channels(monkeypatch):
    res, _ = query((1, 64, 56, 56), (64, 3, 3), padding=(1, 1))
    assert (res.tile_w, res.tile_h) == (58, 2)            # full rows plus the halo columns
    res, _ = query((1, 64, 28, 28), (32, 3, 3), padding=(1, 1), dilation=(1, 2))
    assert (res.tile_w, res.tile_h) == (26 + 4, 4)
    # not for strided or wide layers, more than 64 input or output channels, K steps of 128 or
    # CTA pairs
    for kw in (dict(stride=(2, 2)), dict(xshape=(1, 64, 8, 200)), dict(wshape=(128, 3, 3)),
               dict(xshape=(1, 128, 56, 56)), dict(cfg=dict(tile_n=64, tile_k=128)),
               dict(cfg=dict(tile_m=256, tile_n=128))):
        kw = dict(kw)
        res, _ = query(kw.pop("xshape", (1, 64, 56, 56)), kw.pop("wshape", (64, 3, 3)),
                       padding=(1, 1), **kw)
        assert (res.tile_w, res.tile_h) == (128, 1)
    # 5 x 5 filters: the weights of 25 taps do not fit in shared memory next to two patches
    res, _ = query((1, 64, 56, 56), (64, 5, 5), padding=(2, 2))
    assert (res.tile_w, res.tile_h) == (128, 1)
    monkeypatch.setenv("TNX_CONV_NO_HALO", "1")
    res, _ = query((1, 64, 56, 56), (64, 3, 3), padding=(1, 1))
    assert (res.tile_w, res.tile_h) == (128, 1)


def test_rectangular_tiles_when_im2col_boxes_cannot_be_used(monkeypatch):
    monkeypatch.setenv("TNX_CONV_NO_HALO", "1")
    res, _ = query((1, 64, 56, 56), (64, 3, 3), padding=(1, 1))
    assert (res.tile_w, res.tile_h) == (128, 1)
    monkeypatch.setenv("TNX_CONV_TILED", "1")
    res, _ = query((1, 64, 56, 56), (64, 3, 3), padding=(1, 1))
    assert (res.tile_w, res.tile_h) == (56, 2)          # 112 pixels, no tile crosses an image row
    res, _ = query((3, 96, 7, 7), (160, 3, 3), padding=(1, 1))
    assert res.tile_w * res.tile_h % 8 == 0 and res.tile_w >= 7 and res.tile_h >= 7
    monkeypatch.delenv("TNX_CONV_TILED")
    res, _ = query((1, 16, 6, 6), (16, 3, 3), padding=(130, 2))   # corner does not fit 8 bits
    assert (res.tile_w, res.tile_h) != (128, 1)


def test_configuration_is_honoured_and_checked():
    res, _ = query((4, 64, 28, 28), (256, 3, 3), padding=(1, 1),
                   cfg=dict(tile_m=256, tile_n=256, tile_k=64, stages=3))
    assert res.tmem_columns == 512 and res.grid % 2 == 0
    with pytest.raises(_cabi.OutOfResources):
        query((4, 64, 28, 28), (256, 3, 3), padding=(1, 1),
              cfg=dict(tile_m=128, tile_n=256, tile_k=128, stages=8))
    with pytest.raises(ValueError):
        query((4, 64, 28, 28), (256, 3, 3), cfg=dict(tile_m=64))
    with pytest.raises(ValueError):
        query((4, 64, 28, 28), (256, 3, 3), cfg=dict(tile_k=32))


@pytest.mark.parametrize("bad", [
    dict(xshape=(1, 8, 4, 4), wshape=(8, 7, 7)),                        # filter larger than input
    dict(xshape=(1, 8, 32, 32), wshape=(8, 3, 3), stride=(9, 1)),       # stride beyond a TMA box step
    dict(xshape=(1, 8, 32, 32), wshape=(8, 3, 3), stride=(0, 1)),
    dict(xshape=(1, 8, 32, 32), wshape=(8, 3, 3), dilation=(1, 0)),
    dict(xshape=(1, 8, 32, 32), wshape=(8, 3, 3), padding=(-1, 0)),
    dict(xshape=(0, 8, 32, 32), wshape=(8, 3, 3)),
    dict(xshape=(1, 8, 32, 32), wshape=(8, 3, 3), input_layout=7),
    dict(xshape=(1, 8, 32, 32), wshape=(8, 3, 3), dtype=torch.float32,
         weight_layout=_cabi.WEIGHT_PACKED),
])
def test_invalid_problems_are_rejected(bad):
    with pytest.raises(ValueError):
        query(**bad)


def test_null_pointers_are_rejected_before_any_launch():
    _, p = query((1, 8, 8, 8), (8, 3, 3))
    rc = _cabi.lib.tnx_conv2d_forward(ctypes.byref(p), None, None, None, None, None, None, 0,
                                      None, None)
    assert rc == _cabi.ERR_INVALID and "NULL" in _cabi.last_error()
    assert _cabi.lib.tnx_conv2d_query(None, None, None) == _cabi.ERR_INVALID


def test_public_entry_refuses_host_tensors():
    from tritonix_b200.ops.conv2d import conv2d_forward
    with pytest.raises(RuntimeError):
        conv2d_forward(torch.zeros(1, 8, 8, 8), torch.zeros(8, 8, 3, 3))
