"""Registers the contraction kernels as torch custom operators (namespace ``tritonix``) so
they are visible to ``torch.ops``, autograd-free tracing and ``torch.compile`` (fake kernels
give the output shapes).  ``cfg`` is the tnx_config of include/tritonix_b200.h as a list of
ints in field order (tile_m, tile_n, tile_k, stages, acc_stages, cta_group, split_k, group_m,
tile_order, kernel, max_ctas); missing trailing entries and zeros select the defaults.
"""
from __future__ import annotations

from typing import List

import torch

from tritonix_b200 import _cabi

_FIELDS = ("tile_m", "tile_n", "tile_k", "stages", "acc_stages", "cta_group", "split_k",
           "group_m", "tile_order", "kernel", "max_ctas")

_lib = torch.library.Library("tritonix", "DEF")
_lib.define("gemm(Tensor a, Tensor b, int[] cfg) -> Tensor")
_lib.define("gemm_splitk(Tensor a, Tensor b, int split_k, int[] cfg) -> Tensor")
_lib.define("glu(Tensor x, Tensor w12, int activation, int[] cfg) -> Tensor")
_lib.define("conv2d_forward(Tensor input, Tensor weight, Tensor? bias, int[] stride, int[] padding, "
            "int[] dilation, int[] cfg) -> Tensor")


def cfg_to_list(cfg: dict | None) -> List[int]:
    c = _cabi.make_config(cfg)
    return [int(getattr(c, f)) for f in _FIELDS]


def _cfg_dict(cfg: List[int]) -> dict:
    return {f: int(v) for f, v in zip(_FIELDS, cfg) if int(v) != 0}


def _gemm(a, b, cfg):
    c = torch.empty((a.shape[0], b.shape[1]), device=a.device, dtype=a.dtype)
    _cabi.launch(a, b, c, _cfg_dict(cfg))
    return c


def _gemm_splitk(a, b, split_k, cfg):
    c = torch.empty((a.shape[0], b.shape[1]), device=a.device, dtype=a.dtype)
    _cabi.launch(a, b, c, {**_cfg_dict(cfg), "split_k": int(split_k)})
    return c


def _glu(x, w12, activation, cfg):
    z = torch.empty((x.shape[0], w12.shape[1] // 2), device=x.device, dtype=x.dtype)
    _cabi.launch(x, w12, z, _cfg_dict(cfg), epilogue=int(activation))
    return z


def _conv_out_shape(input, weight, stride, padding, dilation):
    n, _, h, w = input.shape
    c_out, _, r, s = weight.shape
    h_out = (h + 2 * padding[0] - dilation[0] * (r - 1) - 1) // stride[0] + 1
    w_out = (w + 2 * padding[1] - dilation[1] * (s - 1) - 1) // stride[1] + 1
    return (n, c_out, h_out, w_out)


def _conv2d_forward(input, weight, bias, stride, padding, dilation, cfg):
    from tritonix_b200.ops.conv2d import conv2d_forward
    config = _cfg_dict(cfg)
    return conv2d_forward(input, weight, bias, tuple(stride), tuple(padding), tuple(dilation),
                          config=config or None)


_lib.impl("gemm", _gemm, "CUDA")
_lib.impl("conv2d_forward", _conv2d_forward, "CUDA")
_lib.impl("gemm_splitk", _gemm_splitk, "CUDA")
_lib.impl("glu", _glu, "CUDA")


@torch.library.register_fake("tritonix::gemm")
def _gemm_fake(a, b, cfg):
    return a.new_empty((a.shape[0], b.shape[1]))


@torch.library.register_fake("tritonix::gemm_splitk")
def _gemm_splitk_fake(a, b, split_k, cfg):
    return a.new_empty((a.shape[0], b.shape[1]))


@torch.library.register_fake("tritonix::glu")
def _glu_fake(x, w12, activation, cfg):
    return x.new_empty((x.shape[0], w12.shape[1] // 2))


@torch.library.register_fake("tritonix::conv2d_forward")
def _conv2d_forward_fake(input, weight, bias, stride, padding, dilation, cfg):
    channels_last = (not input.is_contiguous()
                     and input.is_contiguous(memory_format=torch.channels_last))
    return torch.empty(_conv_out_shape(input, weight, stride, padding, dilation),
                       device=input.device, dtype=input.dtype,
                       memory_format=torch.channels_last if channels_last
                       else torch.contiguous_format)
