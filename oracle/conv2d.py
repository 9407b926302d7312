"""CPU restatement of the reference's convolution forward.  TEST INFRASTRUCTURE ONLY.

It is the checker for tnx_conv2d_forward; only tests/, __graft_entry__.smoke() and bench.py's
CPU legs may import it, never the product path.

conv2d_oracle restates conv2d_forward_kernel (tritonix/ops/conv2d/forward.py:52-165) as the
implicit GEMM it is: row gemm_m = (n, h_out, w_out) (forward.py:84-87), column = output channel,
K index gemm_k = (c_in, filter row, filter column) (forward.py:104-107); the input element of a
(row, k) pair sits at h = h_out*stride_h - pad_h + r*dil_h, w = w_out*stride_w - pad_w + s*dil_w
and counts as zero outside the image (forward.py:109-126); products are accumulated in fp32
(forward.py:95, :145), the bias is added in fp32 (forward.py:148-153) and the sum is cast once to
the operand type (forward.py:163-165).  The dot product itself is Triton's tl.dot (third-party,
`triton >=3.4.0,<4.0.0` in the reference's pyproject.toml): fp32-accumulated products of the
operands as stored.

Pinning: tests/test_conv2d_oracle.py checks it against tests/golden/conv2d_reference.npz, which
tests/golden/make_conv2d_golden.py produced by running the reference's own kernel on CPU under
Triton's interpreter.
"""
from __future__ import annotations

import torch

ERR_TOLERANCE = {torch.float16: 2e-3, torch.bfloat16: 8e-3, torch.float32: 1e-5}


def conv_output_size(h_in, w_in, r, s, stride, padding, dilation):
    """H_OUT, W_OUT as conv2d_forward computes them (forward.py:226-227)."""
    h_out = (h_in + 2 * padding[0] - dilation[0] * (r - 1) - 1) // stride[0] + 1
    w_out = (w_in + 2 * padding[1] - dilation[1] * (s - 1) - 1) // stride[1] + 1
    return h_out, w_out


def im2col(x: torch.Tensor, r: int, s: int, stride, padding, dilation) -> torch.Tensor:
    """The GEMM's left operand: (N*H_OUT*W_OUT) x (C*R*S), zero where a tap leaves the image."""
    n, c, h_in, w_in = x.shape
    h_out, w_out = conv_output_size(h_in, w_in, r, s, stride, padding, dilation)
    ho = torch.arange(h_out).view(h_out, 1, 1, 1)
    wo = torch.arange(w_out).view(1, w_out, 1, 1)
    fr = torch.arange(r).view(1, 1, r, 1)
    fs = torch.arange(s).view(1, 1, 1, s)
    hi = (ho * stride[0] - padding[0] + fr * dilation[0]).expand(h_out, w_out, r, s)
    wi = (wo * stride[1] - padding[1] + fs * dilation[1]).expand(h_out, w_out, r, s)
    valid = (hi >= 0) & (hi < h_in) & (wi >= 0) & (wi < w_in)
    hi_c, wi_c = hi.clamp(0, h_in - 1), wi.clamp(0, w_in - 1)
    cols = x[:, :, hi_c, wi_c]  # N x C x H_OUT x W_OUT x R x S
    cols = cols * valid.to(x.dtype)
    return cols.permute(0, 2, 3, 1, 4, 5).reshape(n * h_out * w_out, c * r * s)


def conv2d_oracle(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
                  stride=(1, 1), padding=(0, 0), dilation=(1, 1),
                  out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """N x C_OUT x H_OUT x W_OUT; operands are taken as stored, sums run in fp32 (fp64 for fp32
    operands, so that the checker is more exact than what it checks)."""
    x, w = x.detach().cpu(), w.detach().cpu()
    out_dtype = out_dtype or x.dtype
    acc = torch.float64 if x.dtype == torch.float32 else torch.float32
    n, c, h_in, w_in = x.shape
    c_out, _, r, s = w.shape
    h_out, w_out = conv_output_size(h_in, w_in, r, s, stride, padding, dilation)
    a = im2col(x.to(acc), r, s, stride, padding, dilation)
    y = a @ w.to(acc).reshape(c_out, c * r * s).t()
    if bias is not None:
        y = y + bias.detach().cpu().to(acc).view(1, c_out)
    return y.view(n, h_out, w_out, c_out).permute(0, 3, 1, 2).contiguous().to(out_dtype)


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.detach().cpu().double(), want.detach().cpu().double()
    return ((got - want).abs().max() / want.abs().max().clamp_min(1e-30)).item()
