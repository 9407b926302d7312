"""Fused gated-linear-unit entry points.

``glu_kernel`` computes Z = act(X.W1) * (X.W2) in one pass over a column-interleaved weight
matrix W12 (column 2j = W1[:, j], column 2j+1 = W2[:, j]), as the reference's Triton kernel of
the same name (tritonix/ops/swiglu.py:12-110): the gate and up accumulators of a tile live side
by side in TMEM, are activated and multiplied in registers, and only Z is written.
``activation``: "silu" (default, SwiGLU), "sigmoid" (the classic GLU; described by the
reference's README but not implemented there), anything else = no activation (bilinear), which
is the reference's behaviour for any non-"silu" value.

``swiglu_kernel`` has the call signature of the reference's three-matrix kernel
(tritonix/ops/swiglu.py:113-230), Z = (silu(X.W1) * (X.W2)).W3.  The reference's version
accumulates with atomics and indexes W3 incorrectly beyond one tile; here it is ONE
deterministic launch (``tnx_swiglu_mlp``: hidden-activation tiles and output tiles interleaved
in one persistent kernel, the hidden activation kept in the input precision in a small ring
that stays in L2) for fp16/bf16 operands with contiguous rows, and two launches (fused
gate/up, then the down projection) for anything else.

Host wrappers: ``glu``, ``swiglu``, ``swiglu_mlp``, ``interleave_weights``.
"""
from __future__ import annotations

import os

import torch

from tritonix_b200 import _cabi
from tritonix_b200.autotune import Choice, PowerOfTwo, Range, tunable
from tritonix_b200.ops._kernel_handle import CudaKernel
import tritonix_b200.ops.matmul  # noqa: F401
import sys as _sys

_mm = _sys.modules["tritonix_b200.ops.matmul"]  # the module (ops.matmul is also a dispatcher)

glu_kernel = tunable(
    keys=["m", "n", "k"],
    space={
        "block_m": PowerOfTwo(128, 256),
        "block_n": PowerOfTwo(128, 256),
        "block_k": PowerOfTwo(64, 128),
        "group_m": Choice([4, 8, 16]),
        "num_stages": Range(2, 8),
        "acc_stages": Choice([1, 2]),
    },
    memory_params={"block_m", "block_n", "block_k", "num_stages", "acc_stages"},
    memory_rank={"block_m": lambda rows: -rows},
)(CudaKernel("glu_kernel", glu=True,
             doc="Z = act(X.W1) * (X.W2) over interleaved W12; n counts W12's columns (2F)."))


class _SwigluMlpKernel(CudaKernel):
    """Handle with the reference's swiglu_kernel argument list."""

    def run(self, x, w12, w3, z, m, n, k, f, stride_xm, stride_xk, stride_wk, stride_wn,
            stride_w3n, stride_w3l, stride_zm, stride_zl, grid=None, **cfg):
        activation = cfg.pop("activation", "silu")
        cfg.pop("block_l", None)
        fused = cfg.pop("fused", True)
        if fused and self._run_fused(x, w12, w3, z, m, n, k, f, stride_xm, stride_xk, stride_wk,
                                     stride_wn, stride_w3n, stride_w3l, stride_zm, stride_zl,
                                     activation, cfg):
            return
        hidden = torch.empty((m, n // 2), device=x.device, dtype=x.dtype)
        glu_kernel[grid](x, w12, hidden, m, n, k, stride_xm, stride_xk, stride_wk, stride_wn,
                         hidden.stride(0), hidden.stride(1), activation=activation, **cfg)
        down_cfg = _mm.default_config(m, f, n // 2)
        _mm.matmul_kernel[grid](hidden, w3, z, m, f, n // 2, hidden.stride(0), hidden.stride(1),
                                stride_w3n, stride_w3l, stride_zm, stride_zl, **down_cfg)


    @staticmethod
    def _run_fused(x, w12, w3, z, m, n, k, f, stride_xm, stride_xk, stride_wk, stride_wn, stride_w3n,
                   stride_w3l, stride_zm, stride_zl, activation, cfg) -> bool:
        """One launch when the operands qualify and the arguments describe the tensors as they
        are; returns False to let the two-launch path take the call."""
        tensors = all(isinstance(t, torch.Tensor) for t in (x, w12, w3, z))
        if not tensors or not _cabi.mlp_eligible(x, w12, w3, z):
            return False
        if (tuple(x.shape) != (m, k) or tuple(w12.shape) != (k, n) or tuple(w3.shape) != (n // 2, f)
                or tuple(z.shape) != (m, f)
                or (stride_xm, stride_xk, stride_wk, stride_wn) != (*x.stride(), *w12.stride())
                or (stride_w3n, stride_w3l, stride_zm, stride_zl) != (*w3.stride(), *z.stride())):
            return False
        keep = {"block_k": "tile_k", "tile_k": "tile_k", "num_stages": "stages", "stages": "stages",
                "group_m": "group_m", "max_ctas": "max_ctas"}
        mlp_cfg = {keep[key]: v for key, v in cfg.items() if key in keep}
        if mlp_cfg.get("tile_k") not in (None, 64, 128):
            return False
        _cabi.launch_mlp(x, w12, w3, z, mlp_cfg, _cabi.ACTIVATIONS.get(activation, _cabi.EPI_GLU_LINEAR))
        return True


swiglu_kernel = tunable(
    keys=["m", "n", "k"],
    space=dict(glu_kernel.space),
    memory_params={"block_m", "block_n", "block_k", "num_stages", "acc_stages"},
    memory_rank={"block_m": lambda rows: -rows},
)(_SwigluMlpKernel("swiglu_kernel",
                   doc="Z[M, f] = (silu(X.W1) * (X.W2)) . W3, W12 interleaved, W3 is (n/2, f)."))


def interleave_weights(w1: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """(K, F), (K, F) -> (K, 2F) with columns alternating W1, W2 — the layout the kernels read."""
    if w1.shape != w2.shape:
        raise ValueError(f"w1 and w2 must have the same shape, got {w1.shape} and {w2.shape}")
    return torch.stack((w1, w2), dim=2).reshape(w1.shape[0], 2 * w1.shape[1])


def default_glu_config(m: int, n: int, k: int) -> dict:
    if m > 128:
        return {"block_m": 256, "block_n": 256, "block_k": 128, "group_m": 16, "num_stages": 3}
    return {"block_m": 128, "block_n": 256 if n >= 256 else 128, "block_k": 64, "group_m": 8,
            "num_stages": 4}


def _launch_glu(x: torch.Tensor, w12: torch.Tensor, cfg: dict, activation: str,
                out=None) -> torch.Tensor:
    m, k = x.shape
    _, n = w12.shape
    z = out if out is not None else torch.empty((m, n // 2), device=x.device, dtype=x.dtype)
    if tuple(z.shape) != (m, n // 2) or z.dtype != x.dtype:
        raise ValueError(f"out must be a {(m, n // 2)} {x.dtype} tensor")
    glu_kernel[(1,)](x, w12, z, m, n, k, x.stride(0), x.stride(1), w12.stride(0), w12.stride(1),
                     z.stride(0), z.stride(1), activation=activation, **cfg)
    return z


_glu_cfg: dict = {}


def glu(x: torch.Tensor, w12: torch.Tensor, activation: str = "sigmoid",
        cfg: dict | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """act(x @ W1) * (x @ W2) with W12 = interleave_weights(W1, W2); tuned once per shape."""
    _cabi.require_cuda(x, w12)
    if x.dim() != 2 or w12.dim() != 2 or x.shape[1] != w12.shape[0] or w12.shape[1] % 2:
        raise ValueError(f"glu expects x (M, K) and w12 (K, 2F); got {tuple(x.shape)}, "
                         f"{tuple(w12.shape)}")
    m, k = x.shape
    n = w12.shape[1]
    if cfg is None:
        key = (m, n, k)
        cfg = _glu_cfg.get(key)
        if cfg is None:
            tune = os.environ.get("TRITONIX_B200_TUNE", "1") not in ("0", "false", "off")
            if tune and _cabi.umma_eligible_tensors(x, w12) and (n // 2) % 8 == 0:
                seeds = [dict(block_m=256, block_n=256, block_k=bk, group_m=16, num_stages=st, acc_stages=2)
                         for bk, st in ((128, 3), (64, 6))]
                cfg = _mm._tuned(glu_kernel, lambda c: _launch_glu(x, w12, c, activation), key, x,
                                 _mm._plausible(m, n), seeds, 2.0 * m * n * k)
            cfg = cfg or default_glu_config(m, n, k)
            _glu_cfg[key] = cfg
    return _launch_glu(x, w12, cfg, activation, out)


def swiglu(x: torch.Tensor, w12: torch.Tensor, cfg: dict | None = None,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """silu(x @ W1) * (x @ W2)."""
    return glu(x, w12, activation="silu", cfg=cfg, out=out)


def swiglu_mlp(x: torch.Tensor, w12: torch.Tensor, w_down: torch.Tensor,
               cfg: dict | None = None, down_cfg: dict | None = None,
               out: torch.Tensor | None = None, fused: bool = False,
               fused_cfg: dict | None = None) -> torch.Tensor:
    """The SwiGLU MLP block (silu(x W1) * (x W2)) W_down: two launches (fused gate/up, then the
    down projection), or with ``fused=True`` the one-launch kernel (``fused_cfg``: tile_k,
    stages, group_m = 256-row tiles per band)."""
    if fused:
        _cabi.require_cuda(x, w12, w_down)
        y = out if out is not None else torch.empty((x.shape[0], w_down.shape[1]), device=x.device,
                                                    dtype=x.dtype)
        _cabi.launch_mlp(x, w12, w_down, y, fused_cfg, _cabi.EPI_GLU_SILU)
        return y
    hidden = swiglu(x, w12, cfg=cfg)
    if down_cfg is not None:
        return _mm._launch_matmul(hidden, w_down, down_cfg, out)
    return _mm.cuda_matmul(hidden, w_down, out=out)
