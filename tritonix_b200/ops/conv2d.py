"""2-D convolution forward: ``conv2d_forward`` and the ``conv2d_forward_kernel`` handle — the
surface of tritonix/ops/conv2d/forward.py:8-319 (forward only; the reference's backward and
channel-sparse kernels are not part of this package).

The convolution is an implicit GEMM, GEMM_M = N*H_OUT*W_OUT, GEMM_N = C_OUT, GEMM_K = C_IN*R*S.
For fp16/bf16 it runs on the tcgen05 kernel: a tile's 128 rows are a rectangle of output pixels,
each filter tap is one TMA box load from the N x H x W x C input (zero fill outside the image is
the padding), the weights are a K-major operand.  NCHW tensors are repacked on the way in and
out; ``torch.channels_last`` tensors with channel counts that are multiples of 8 are used in
place; inputs with at most 16 channels are repacked so that a filter row's taps become channels
(a 3-channel 7x7 stem then multiplies 448 instead of 3136 K elements per output).  fp32 runs on
a CUDA-core kernel.

Search space, under the reference's key names (forward.py:8-18):
  BLOCK_SIZE_M  output pixels per tile: 128 = one SM per tile, 256 = a CTA pair
  BLOCK_SIZE_N  output channels per tile (64 / 128 / 256)
  BLOCK_SIZE_K  K elements per pipeline stage (64 / 128)
  GROUP_SIZE_M  band height of the grouped tile order
  num_stages    depth of the TMA -> shared-memory ring
"""
from __future__ import annotations

import ctypes
import os
import weakref

import torch

from tritonix_b200 import _cabi
from tritonix_b200.autotune import Choice, PowerOfTwo, Range, tunable

_CONV_ALIASES = {"BLOCK_SIZE_M": "tile_m", "BLOCK_SIZE_N": "tile_n", "BLOCK_SIZE_K": "tile_k",
                 "GROUP_SIZE_M": "group_m"}
_CONV_IGNORED = {"OUT_DTYPE", "USE_TF32"}


def _pair(v):
    if isinstance(v, int):
        return (v, v)
    v = tuple(int(x) for x in v)
    if len(v) != 2:
        raise ValueError(f"expected an int or a pair, got {v}")
    return v


def _conv_config(cfg: dict | None) -> _cabi.Config | None:
    """Reference config keys (forward.py:302-305) -> the C ABI's."""
    if not cfg:
        return None
    out = {}
    for key, value in cfg.items():
        if key in _CONV_IGNORED:
            continue
        out[_CONV_ALIASES.get(key, key)] = value
    return _cabi.make_config(out)


def _layout(t: torch.Tensor) -> int:
    if t.is_contiguous():
        return _cabi.LAYOUT_NCHW
    if t.is_contiguous(memory_format=torch.channels_last):
        return _cabi.LAYOUT_NHWC
    raise ValueError("tensor must be contiguous NCHW or torch.channels_last")


class _Conv2dKernel:
    """Handle with the reference's launch syntax (forward.py:277-290):

        conv2d_forward_kernel[grid](out, input, weight, bias, N, C_IN, H_IN, W_IN, C_OUT, H_OUT,
                                    W_OUT, R, S, str_h, str_w, pad_h, pad_w, dil_h, dil_w,
                                    GEMM_M, GEMM_N, GEMM_K, BLOCK_SIZE_M=..., ...)

    ``grid`` is accepted and ignored (the kernel is persistent and sizes its own grid)."""

    __name__ = "conv2d_forward_kernel"

    def __init__(self):
        self._plans: dict = {}

    def __getitem__(self, grid):
        def launch(*args, **kwargs):
            return self.run(*args, **kwargs)
        return launch

    def run(self, out, input, weight, bias, *geometry, **cfg):
        problem, config, res = self.plan(out, input, weight, bias, *geometry, **cfg)
        _cabi.conv_launch(problem, config, res, input, weight, bias, out)
        return res

    def plan(self, out, input, weight, bias, batch, c_in, h_in, w_in, c_out, h_out, w_out,
             filter_h, filter_w, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w, gemm_m=None,
             gemm_n=None, gemm_k=None, **cfg):
        """Validates a launch and returns its (problem, config, resources) C structs."""
        _cabi.require_cuda(out, input, weight)
        # weights_packed=True: ``weight`` is the buffer _cabi.conv_pack_weights() returned
        packed = bool(cfg.pop("weights_packed", False))
        if not (input.dtype == out.dtype and (packed or weight.dtype == input.dtype)):
            raise ValueError(f"dtype mismatch {input.dtype}/{weight.dtype}/{out.dtype}")
        if bias is not None and (bias.dtype != input.dtype or not bias.is_cuda):
            raise ValueError("bias must be a CUDA tensor of the input's dtype")
        # problem / config / resources are remembered per distinct call signature
        key = (batch, c_in, h_in, w_in, c_out, filter_h, filter_w, stride_h, stride_w, pad_h,
               pad_w, dil_h, dil_w, h_out, w_out, input.dtype, bias is not None, _layout(input),
               _layout(out), packed, tuple(sorted(cfg.items())),
               os.environ.get("TNX_CONV_TILED"), os.environ.get("TNX_CONV_NO_FOLD"),
               os.environ.get("TNX_CONV_NO_BATCHED_GEMM"), os.environ.get("TNX_CONV_NO_HALO"))
        plan = self._plans.get(key)
        if plan is None:
            problem = _cabi.make_conv_problem(
                batch, c_in, h_in, w_in, c_out, filter_h, filter_w, (stride_h, stride_w),
                (pad_h, pad_w), (dil_h, dil_w), input.dtype, bias is not None, _layout(input),
                _layout(out), _cabi.WEIGHT_PACKED if packed else _cabi.WEIGHT_KCRS)
            config = _conv_config(cfg)
            res = _cabi.conv_query(problem, config)
            if (res.h_out, res.w_out) != (h_out, w_out):
                raise ValueError(f"H_OUT x W_OUT = {h_out} x {w_out} does not match the geometry "
                                 f"({res.h_out} x {res.w_out})")
            if len(self._plans) >= 1024:
                self._plans.clear()
            plan = self._plans[key] = (problem, config, res)
        return plan

    def __repr__(self):
        return "<tritonix_b200 CUDA kernel conv2d_forward_kernel>"


conv2d_forward_kernel = tunable(
    keys=["GEMM_M", "GEMM_N", "GEMM_K"],
    space={
        "BLOCK_SIZE_M": PowerOfTwo(128, 256),
        "BLOCK_SIZE_N": PowerOfTwo(64, 256),
        "BLOCK_SIZE_K": PowerOfTwo(64, 128),
        "GROUP_SIZE_M": Choice([4, 8, 16]),
        "num_stages": Range(2, 8),
    },
    memory_params={"BLOCK_SIZE_M", "BLOCK_SIZE_N", "BLOCK_SIZE_K", "num_stages"},
    memory_rank={"BLOCK_SIZE_M": lambda rows: -rows},
)(_Conv2dKernel())

# Packed copies of weight tensors seen recently, so that a layer called again with unchanged
# weights (inference, or several micro-batches per optimiser step) does not repack them.  An
# entry is valid while the tensor is alive and its version counter (bumped by every in-place
# write) has not moved.  Two limits of that test: a write through ``weight.data`` (``p.data.copy_``,
# some optimisers and state-dict loaders) does not move the counter, so after one call
# ``clear_caches()`` or pass ``weights_static=False``; and weights that require grad while
# autograd is recording are assumed to be in training and are repacked on every call.
# The packed copy is written on the stream of its first use; the event recorded there is waited
# on by any other stream that reads the copy later.
_PACKED_WEIGHTS: "dict[tuple, tuple]" = {}
_PACKED_WEIGHTS_MAX = 64


def _packed_weights(weight: torch.Tensor, problem_of, static: bool = True) -> torch.Tensor:
    if not static or (weight.requires_grad and torch.is_grad_enabled()):
        return _cabi.conv_pack_weights(problem_of(), weight)
    key = (weight.data_ptr(), weight.shape, weight.dtype, weight.device)
    stream = torch.cuda.current_stream(weight.device)
    hit = _PACKED_WEIGHTS.get(key)
    if hit is not None:
        ref, version, packed, packed_on, done = hit
        if ref() is weight and version == weight._version:
            if packed_on != stream.cuda_stream:
                stream.wait_event(done)
            return packed
    packed = _cabi.conv_pack_weights(problem_of(), weight)
    done = torch.cuda.Event()
    done.record(stream)
    if len(_PACKED_WEIGHTS) >= _PACKED_WEIGHTS_MAX:
        _PACKED_WEIGHTS.pop(next(iter(_PACKED_WEIGHTS)))
    _PACKED_WEIGHTS[key] = (weakref.ref(weight), weight._version, packed, stream.cuda_stream, done)
    return packed


# Tuned configuration per problem, as the reference keeps one (forward.py:171, 244-300).
_CONV_FWD_CONFIG_CACHE: dict[tuple, dict] = {}
# (BLOCK_SIZE_M, BLOCK_SIZE_N, BLOCK_SIZE_K, GROUP_SIZE_M) tried on the first call for a problem.
_CANDIDATE_CONFIGS = [
    (256, 256, 64, 8),
    (256, 256, 128, 8),
    (256, 128, 64, 8),
    (256, 128, 128, 8),
    (128, 256, 64, 8),
    (128, 256, 128, 8),
    (128, 128, 64, 8),
    (128, 128, 128, 8),
    (128, 64, 64, 8),
    (128, 64, 128, 8),
]


def _time_kernel(fn, launches: int = 6) -> float:
    """Milliseconds per launch of ``fn``: one untimed call (compilation of nothing, but first-use
    set-up such as the shared-memory opt-in), then ``launches`` back-to-back calls between two
    events on the current stream."""
    fn()
    first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first.record()
    for _ in range(launches):
        fn()
    last.record()
    last.synchronize()
    return first.elapsed_time(last) / launches


# Call signatures seen before (shapes, dtypes, devices, layout, geometry) -> a closure that goes
# straight to the C entry point with the structs prepared the first time.  Eager calls of small
# layers are bound by the host; this path costs about half of the general one.
_FAST_CALLS: dict = {}


def clear_caches() -> None:
    """Forgets tuned configurations, packed weights, prepared calls and launch plans.  The
    ``TNX_CONV_*`` environment switches are read when a call signature is first seen, so call
    this after changing one of them."""
    _FAST_CALLS.clear()
    _CONV_FWD_CONFIG_CACHE.clear()
    _PACKED_WEIGHTS.clear()
    conv2d_forward_kernel.kernel._plans.clear()


def _signature(input, weight, bias, stride, padding, dilation):
    if isinstance(stride, list) or isinstance(padding, list) or isinstance(dilation, list):
        stride, padding, dilation = _pair(stride), _pair(padding), _pair(dilation)
    return (input.shape, weight.shape, input.dtype, weight.dtype, input.device, weight.device,
            None if bias is None else (bias.shape, bias.dtype, bias.device, bias.is_contiguous()),
            stride, padding, dilation, input.stride(), weight.stride())


def _prepare_fast_call(plan, out_shape, channels_last, packed, device, dtype):
    problem, config, res = plan
    forward = _cabi.lib.tnx_conv2d_forward
    problem_ref = ctypes.byref(problem)
    config_ref = ctypes.byref(config) if config is not None else None
    layout = torch.channels_last if channels_last else torch.contiguous_format
    status_ptr = _cabi.status_word(device).data_ptr()
    ws_bytes = int(res.workspace_bytes)
    index = device.index if device.index is not None else torch.cuda.current_device()

    def call(input, weight, bias):
        if torch.cuda.current_device() != index:
            return None  # the general path switches devices
        out = torch.empty(out_shape, device=device, dtype=dtype, memory_format=layout)
        if packed:
            weight = _packed_weights(weight, lambda: problem)
        stream = torch.cuda.current_stream().cuda_stream
        ws = _cabi.conv_workspace(device, ws_bytes, stream) if ws_bytes else None
        rc = forward(problem_ref, config_ref, input.data_ptr(), weight.data_ptr(),
                     None if bias is None else bias.data_ptr(), out.data_ptr(),
                     None if ws is None else ws.data_ptr(), ws_bytes, status_ptr, stream)
        if rc:
            _cabi.raise_for(rc)
        return out

    return call


def conv2d_forward(input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                   stride=(1, 1), padding=(0, 0), dilation=(1, 1), use_tf32: bool = True,
                   config: dict | None = None, weights_static: bool = True) -> torch.Tensor:
    """Forward of ``torch.nn.functional.conv2d`` (groups = 1), the reference's
    ``conv2d_forward`` (forward.py:202-319): input N x C x H x W, weight C_OUT x C x R x S,
    optional bias, fp32 accumulation, output N x C_OUT x H_OUT x W_OUT of the input's dtype.

    A ``torch.channels_last`` input gives a ``channels_last`` output and skips the repacking
    passes.  ``config`` fixes the kernel configuration (reference keys ``BLOCK_SIZE_M/N/K``,
    ``GROUP_SIZE_M``, or this package's ``tile_n``/``tile_k``/``stages``/``cta_group``);
    without it the first call for a problem times a handful of candidates and remembers the
    best.  ``use_tf32`` is accepted for compatibility: fp32 inputs are computed in full fp32.
    ``weights_static=False`` repacks the weights on every call instead of reusing the packed
    copy of an unchanged tensor (needed when the weights are written through ``.data``, which
    the version counter does not see).
    """
    signature = None
    if config is None and weights_static:
        signature = _signature(input, weight, bias, stride, padding, dilation)
        fast = _FAST_CALLS.get(signature)
        if fast is not None:
            out = fast(input, weight, bias)
            if out is not None:
                return out
    _cabi.require_cuda(input, weight)
    if input.dim() != 4 or weight.dim() != 4:
        raise ValueError("input must be N x C x H x W and weight C_OUT x C x R x S")
    if input.shape[1] != weight.shape[1]:
        raise ValueError(f"channel mismatch: input has {input.shape[1]}, weight {weight.shape[1]}")
    if weight.dtype != input.dtype or (bias is not None and bias.dtype != input.dtype):
        raise ValueError("input, weight and bias must share one dtype")
    stride, padding, dilation = _pair(stride), _pair(padding), _pair(dilation)
    channels_last = (not input.is_contiguous()
                     and input.is_contiguous(memory_format=torch.channels_last))
    if not channels_last and not input.is_contiguous():
        raise ValueError("input must be contiguous NCHW or torch.channels_last")
    weight = weight.contiguous()
    if bias is not None:
        bias = bias.contiguous()
    n, c_in, h_in, w_in = input.shape
    c_out, _, r, s = weight.shape
    h_out = (h_in + 2 * padding[0] - dilation[0] * (r - 1) - 1) // stride[0] + 1
    w_out = (w_in + 2 * padding[1] - dilation[1] * (s - 1) - 1) // stride[1] + 1
    if h_out < 1 or w_out < 1:
        raise ValueError("the dilated filter is larger than the padded input")
    out = torch.empty((n, c_out, h_out, w_out), device=input.device, dtype=input.dtype,
                      memory_format=torch.channels_last if channels_last
                      else torch.contiguous_format)
    extra = {}
    # A 1 x 1, stride-1, unpadded convolution over NCHW tensors runs as one GEMM per image on the
    # tensors as they are: nothing to repack, weights included (tnx_conv2d_forward decides by the
    # same rule).
    plain_gemm = (r == 1 and s == 1 and stride == (1, 1) and padding == (0, 0) and not channels_last
                  and (h_in * w_in) % 8 == 0 and c_in % 8 == 0
                  and os.environ.get("TNX_CONV_NO_BATCHED_GEMM") is None)
    if input.dtype != torch.float32 and not plain_gemm:
        weight = _packed_weights(weight, lambda: _cabi.make_conv_problem(
            n, c_in, h_in, w_in, c_out, r, s, stride, padding, dilation, input.dtype,
            bias is not None), weights_static)
        extra["weights_packed"] = True
    args = (out, input, weight, bias, n, c_in, h_in, w_in, c_out, h_out, w_out, r, s,
            stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1],
            n * h_out * w_out, c_out, c_in * r * s)

    def launch(*a, **cfg):
        return conv2d_forward_kernel.run(*a, **cfg, **extra)

    if config is None and input.dtype != torch.float32:
        key = (n, c_in, h_in, w_in, c_out, r, s, stride, padding, dilation, input.dtype,
               channels_last)
        config = _CONV_FWD_CONFIG_CACHE.get(key)
        if config is None:
            best_time, best = float("inf"), None
            for bm, bn, bk, g in _CANDIDATE_CONFIGS:
                cand = dict(BLOCK_SIZE_M=bm, BLOCK_SIZE_N=bn, BLOCK_SIZE_K=bk, GROUP_SIZE_M=g)
                if bn > 64 and bn // 2 >= c_out:
                    continue  # half of the tile's columns would be padding
                try:
                    t = _time_kernel(lambda: launch(*args, **cand))
                except (ValueError, _cabi.OutOfResources):
                    continue
                if t < best_time:
                    best_time, best = t, cand
            config = best or {}
            _cabi.check_status(input.device)
            _CONV_FWD_CONFIG_CACHE[key] = config
    plan = conv2d_forward_kernel.plan(*args, **(config or {}), **extra)
    _cabi.conv_launch(*plan, input, weight, bias, out)
    if signature is not None and weight.is_contiguous() and (bias is None or bias.is_contiguous()):
        if len(_FAST_CALLS) >= 4096:
            _FAST_CALLS.clear()
        _FAST_CALLS[signature] = _prepare_fast_call(
            plan, tuple(out.shape), channels_last, "weights_packed" in extra, input.device,
            input.dtype)
    return out


def torch_conv2d_forward(input, weight, bias=None, stride=(1, 1), padding=(0, 0),
                         dilation=(1, 1)):
    """PyTorch's own convolution, for comparisons only (forward.py:322-331); never used as a
    fallback by this package."""
    return torch.nn.functional.conv2d(input, weight, bias, stride, padding, dilation)
