"""Contraction ops (the reference's tritonix/ops/__init__.py:1-4, restricted to the dense path:
GEMM, split-K GEMM, GLU/SwiGLU and the convolution forward)."""
from tritonix_b200.ops.matmul import (cuda_matmul, gemm_splitk_kernel, matmul, matmul_kernel,
                                      matmul_splitk, triton_matmul)
from tritonix_b200.ops.swiglu import (glu, glu_kernel, interleave_weights, swiglu, swiglu_kernel,
                                      swiglu_mlp)
from tritonix_b200.ops.conv2d import (conv2d_forward, conv2d_forward_kernel,
                                      torch_conv2d_forward)
from tritonix_b200.ops import _torch_ops  # noqa: F401  (registers torch.ops.tritonix.*)

__all__ = ["matmul", "matmul_splitk", "cuda_matmul", "triton_matmul", "matmul_kernel",
           "gemm_splitk_kernel", "glu_kernel", "swiglu_kernel", "glu", "swiglu", "swiglu_mlp",
           "interleave_weights", "conv2d_forward", "conv2d_forward_kernel", "torch_conv2d_forward"]
