"""tritonix_b200 — the dense-contraction path of tritonix (tiled GEMM, split-K GEMM, fused
GLU/SwiGLU, convolution forward, autotuner, dispatcher) on hand-written CUDA kernels for NVIDIA
B200 (sm_100a).

The public names follow the reference package (tritonix/__init__.py:3-13) for this path:
``matmul``, ``matmul_splitk``, ``glu_kernel``, ``swiglu_kernel``, ``conv2d_forward``,
``torch_conv2d_forward``, ``tunable``, ``TunableKernel``, ``PowerOfTwo``, ``Range``, ``Choice``.  There is one backend, ``"cuda"``;
nothing falls back to Triton, PyTorch or the CPU.
"""
from tritonix_b200._cabi import DeviceStatusError, OutOfResources, check_status
from tritonix_b200.autotune import (Choice, ConfigSpace, PowerOfTwo, Range, SpaceConfig,
                                    TunableKernel, tunable)
from tritonix_b200.dispatcher import DynamicDispatcher, dynamic_dispatch
from tritonix_b200.ops import (conv2d_forward, conv2d_forward_kernel, cuda_matmul,
                               gemm_splitk_kernel, glu, glu_kernel, interleave_weights, matmul,
                               matmul_kernel, matmul_splitk, swiglu, swiglu_kernel, swiglu_mlp,
                               torch_conv2d_forward, triton_matmul)
from tritonix_b200.host_io import HostRowPipeline, matmul_from_host
from tritonix_b200.testing import do_bench
from tritonix_b200.utils.pruners import (CoordinateMonotonicFunction, CoordinateUnimodalFunction,
                                         MonotonicCascadeTrie)

__version__ = "0.1.0"

__all__ = ["matmul", "matmul_splitk", "cuda_matmul", "triton_matmul", "matmul_kernel",
           "gemm_splitk_kernel", "glu_kernel", "swiglu_kernel", "glu", "swiglu", "swiglu_mlp",
           "interleave_weights", "tunable", "TunableKernel", "PowerOfTwo", "Range", "Choice",
           "SpaceConfig", "ConfigSpace", "MonotonicCascadeTrie", "CoordinateUnimodalFunction",
           "CoordinateMonotonicFunction", "DynamicDispatcher", "dynamic_dispatch",
           "OutOfResources", "DeviceStatusError", "check_status", "do_bench", "install_as_tritonix",
           "HostRowPipeline", "matmul_from_host", "conv2d_forward", "conv2d_forward_kernel",
           "torch_conv2d_forward"]


def install_as_tritonix() -> None:
    """Makes ``import tritonix`` resolve to this package (and ``tritonix.ops``,
    ``tritonix.autotune``, ``tritonix.dispatcher``, ``tritonix.utils`` to its modules), so
    code written against the reference runs unchanged on the dense-contraction path."""
    import sys

    from tritonix_b200 import autotune, dispatcher, ops, utils
    from tritonix_b200.utils import hilbert, pruners, spaces

    me = sys.modules[__name__]
    # the submodules, not the same-named objects they export
    ops_matmul = sys.modules["tritonix_b200.ops.matmul"]
    ops_swiglu = sys.modules["tritonix_b200.ops.swiglu"]
    ops_conv2d = sys.modules["tritonix_b200.ops.conv2d"]
    alias = {"tritonix": me, "tritonix.ops": ops, "tritonix.ops.matmul": ops_matmul,
             "tritonix.ops.swiglu": ops_swiglu, "tritonix.ops.conv2d": ops_conv2d,
             "tritonix.ops.conv2d.forward": ops_conv2d, "tritonix.autotune": autotune,
             "tritonix.dispatcher": dispatcher, "tritonix.utils": utils,
             "tritonix.utils.hilbert": hilbert, "tritonix.utils.pruners": pruners,
             "tritonix.utils.spaces": spaces}
    sys.modules.update(alias)
