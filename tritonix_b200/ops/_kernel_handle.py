"""Kernel handles: Python objects that accept the reference's Triton launch syntax

    kernel[grid](a, b, c, m, n, k, stride_am, stride_ak, stride_bk, stride_bn, stride_cm,
                 stride_cn, **cfg)

(tritonix/ops/matmul.py:222-236, tritonix/ops/swiglu.py:24-43) and enqueue the CUDA kernels of
libtritonix_b200.so.  ``grid`` is accepted for compatibility and ignored: the kernels are
persistent and size their own grid.  The explicit sizes and strides are honoured exactly as
passed (they need not equal the tensors' own), as with a Triton launch.
"""
from __future__ import annotations

from typing import Callable, List

import torch

from tritonix_b200 import _cabi

class CudaKernel:
    """One entry of the kernel family.  ``epilogue`` is fixed per handle except for the GLU
    handle, whose ``activation=`` keyword selects it per launch."""

    def __init__(self, name: str, epilogue: int = _cabi.EPI_NONE, glu: bool = False,
                 doc: str | None = None):
        self.__name__ = name
        self.__doc__ = doc
        self._epilogue = epilogue
        self._glu = glu
        self._pre_hooks: List[Callable] = []
        self.specialize_keys: list = []

    def add_pre_run_hook(self, hook: Callable) -> None:
        """``hook(*args, **kwargs)`` runs before every launch with the launch's arguments
        (Triton's JITFunction.add_pre_run_hook, used at tritonix/ops/matmul.py:210)."""
        self._pre_hooks.append(hook)

    def __getitem__(self, grid):
        def launch(*args, **kwargs):
            return self.run(*args, grid=grid, **kwargs)
        return launch

    def run(self, a, b, c, m, n, k, stride_am, stride_ak, stride_bk, stride_bn, stride_cm,
            stride_cn, grid=None, **cfg):
        for hook in self._pre_hooks:
            hook(a, b, c, m, n, k, stride_am, stride_ak, stride_bk, stride_bn, stride_cm,
                 stride_cn, **cfg)
        for t in (a, b, c):
            if not isinstance(t, torch.Tensor) or not t.is_cuda:
                raise RuntimeError(f"{self.__name__}: operands must be CUDA tensors "
                                   "(tritonix_b200 has no CPU path)")
        if not (a.dtype == b.dtype == c.dtype):
            raise ValueError(f"{self.__name__}: dtype mismatch {a.dtype}/{b.dtype}/{c.dtype}")
        epilogue = self._epilogue
        if self._glu:
            # The reference applies SiLU iff activation == "silu" and no activation otherwise
            # (tritonix/ops/swiglu.py:100-102); "sigmoid" is this package's addition.
            activation = cfg.pop("activation", "silu")
            epilogue = _cabi.ACTIVATIONS.get(activation, _cabi.EPI_GLU_LINEAR)
        table = cfg.pop("tile_table", None)
        return _cabi.launch_raw(a.device, a.dtype, a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                m, n, k, (stride_am, stride_ak, stride_bk, stride_bn, stride_cm,
                                          stride_cn), cfg, epilogue, table)

    def __repr__(self):
        return f"<tritonix_b200 CUDA kernel {self.__name__}>"
