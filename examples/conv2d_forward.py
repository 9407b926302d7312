"""Convolution forward on the CUDA kernels, the way the reference's README uses conv2d_forward:
NCHW tensors in, NCHW out; then the same layer on channels_last tensors (no repacking passes),
a fixed configuration, and the C ABI underneath.

    python examples/conv2d_forward.py [N C H W C_OUT R]
"""
import sys
import time

import torch

import tritonix_b200 as tritonix
from tritonix_b200 import _cabi

args = [int(v) for v in sys.argv[1:7]]
N, C, H, W, C_OUT, R = args if len(args) == 6 else (32, 128, 28, 28, 128, 3)
DTYPE = torch.bfloat16


def timed(fn, reps=20):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) / reps * 1e6


def main():
    dev = torch.device("cuda")
    x = torch.randn(N, C, H, W, device=dev, dtype=DTYPE)
    w = torch.randn(C_OUT, C, R, R, device=dev, dtype=DTYPE) * (C * R * R) ** -0.5
    b = torch.randn(C_OUT, device=dev, dtype=DTYPE)
    pad = R // 2

    # 1. drop-in call: the first call for a problem times a few configurations and keeps the best
    y = tritonix.conv2d_forward(x, w, b, stride=1, padding=pad)
    ref = tritonix.torch_conv2d_forward(x, w, b, (1, 1), (pad, pad))
    err = ((y.float() - ref.float()).abs().max() / ref.float().abs().max()).item()
    print(f"NCHW {tuple(x.shape)} * {tuple(w.shape)} -> {tuple(y.shape)}  max|err|/max|ref| = {err:.2e}")
    print(f"  tritonix_b200 {timed(lambda: tritonix.conv2d_forward(x, w, b, 1, pad)):8.1f} us per call")
    print(f"  torch (cuDNN) {timed(lambda: tritonix.torch_conv2d_forward(x, w, b, (1, 1), (pad, pad))):8.1f} us per call")

    # 2. channels_last tensors are used in place: one kernel, output channels_last as well
    xcl = x.contiguous(memory_format=torch.channels_last)
    ycl = tritonix.conv2d_forward(xcl, w, b, stride=1, padding=pad)
    assert ycl.is_contiguous(memory_format=torch.channels_last)
    print(f"channels_last: {timed(lambda: tritonix.conv2d_forward(xcl, w, b, 1, pad)):8.1f} us per call")

    # 3. a fixed configuration (reference key names) instead of the tuned one
    cfg = dict(BLOCK_SIZE_M=128, BLOCK_SIZE_N=128, BLOCK_SIZE_K=64, GROUP_SIZE_M=8)
    yfix = tritonix.conv2d_forward(x, w, b, stride=1, padding=pad, config=cfg)
    print("fixed config agrees:", torch.allclose(yfix.float(), y.float(), atol=2e-2, rtol=2e-2))

    # 4. what the C ABI reports for this problem
    problem = _cabi.make_conv_problem(N, C, H, W, C_OUT, R, R, (1, 1), (pad, pad), (1, 1), DTYPE, True)
    res = _cabi.conv_query(problem)
    print(f"tnx_conv2d_query: {res.h_out} x {res.w_out} output, {res.grid} CTAs, "
          f"{res.smem_bytes} B shared memory, {res.workspace_bytes} B workspace")
    tritonix.check_status()


if __name__ == "__main__":
    main()
