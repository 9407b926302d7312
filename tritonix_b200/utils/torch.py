"""Global PyTorch precision toggles (the reference's tritonix/utils/torch.py:44-105).  They only
affect PyTorch's own kernels — e.g. a cuBLAS or CPU comparison run — never this package's."""
from __future__ import annotations

import torch


def _ampere_or_newer() -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] >= 8


def enable_cudnn_optimizations() -> None:
    if torch.backends.cudnn.is_available():
        torch.backends.cudnn.benchmark = True


def enable_torch_optimizations(allow_tf32: bool = True, fp16_reduced_precision: bool = False) -> None:
    """cuDNN autotuning on; TF32 for fp32 matmuls and convolutions on or off; optionally
    reduced-precision accumulation for fp16/bf16 matmuls."""
    enable_cudnn_optimizations()
    if _ampere_or_newer():
        torch.backends.cuda.matmul.allow_tf32 = bool(allow_tf32)
        torch.backends.cudnn.allow_tf32 = bool(allow_tf32)
    if fp16_reduced_precision:
        torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = True
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = True


def disable_torch_optimizations() -> None:
    """Deterministic cuDNN, no TF32, fp32 matmuls at the highest precision."""
    if torch.backends.cudnn.is_available():
        torch.backends.cudnn.benchmark = False
        torch.backends.cudnn.deterministic = True
    if _ampere_or_newer():
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        torch.set_float32_matmul_precision("highest")
