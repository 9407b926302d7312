"""CPU restatement of the reference's contraction algorithms.  TEST INFRASTRUCTURE ONLY.

This file is the checker for the CUDA kernels of tritonix_b200; it is never part of the
product path (only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs import it).

Each function restates, in plain torch-on-CPU / Python integer arithmetic, what one piece of the
reference computes (citations are paths inside the reference repository):

  matmul_oracle            matmul_kernel            tritonix/ops/matmul.py:42-108
  matmul_blocked_oracle    the same, k-block by k-block in the kernel's summation order
  splitk_reference_oracle  gemm_splitk_kernel       tritonix/ops/matmul.py:147-202 (slices own
                           interleaved k-blocks; each partial is rounded to the output type and
                           the roundings are added in that type, as the atomic_add of :202 does)
  splitk_oracle            the deterministic variant the CUDA kernel implements (contiguous
                           k ranges, fp32 partials summed in slice order, one rounding)
  glu_oracle               glu_kernel               tritonix/ops/swiglu.py:24-110
  swiglu_mlp_oracle        what swiglu_kernel (tritonix/ops/swiglu.py:113-230) intends
  swizzle2d / grouped_launch / serpentine   tile remaps, tritonix/ops/matmul.py:9-27,70,111-130
  tuning_key               _tuning_key              tritonix/dispatcher.py:18-30

The arithmetic core (tl.dot, tl.sigmoid, tl.swizzle2d) lives in a third-party dependency of the
reference — Triton, `triton >=3.4.0,<4.0.0` in its pyproject.toml, no lock file; 3.6.0 is the
version installed here — so these functions restate the published semantics: fp32-accumulated
dot products and one round-to-nearest-even cast to the output type.

Pinning: tests/test_oracle.py checks every function against the golden outputs in
tests/golden/, which tests/golden/make_golden.py produced by running the reference's own
kernels on CPU under Triton's interpreter (fp16 and fp32; bf16 is not usable there), and
against the reference's own tests for the host logic (tests/test_trie.py, the Hilbert tests
in playground/test_hilbert_swizzle.py).
"""
from __future__ import annotations

from typing import Tuple

import torch

ERR_TOLERANCE = {torch.float16: 2e-3, torch.bfloat16: 8e-3, torch.float32: 1e-5}


def rel_err(out: torch.Tensor, ref: torch.Tensor) -> float:
    """max|out - ref| / max|ref| — the metric every parity test uses."""
    ref = ref.double()
    denom = ref.abs().max().item()
    if denom == 0.0:
        return (out.double() - ref).abs().max().item()
    return ((out.double() - ref).abs().max() / denom).item()


# ---------------------------------------------------------------------------- GEMM
def matmul_oracle(a: torch.Tensor, b: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """C = A.B with fp32 accumulation and one cast (tritonix/ops/matmul.py:90-102)."""
    out_dtype = out_dtype or a.dtype
    return (a.float().cpu() @ b.float().cpu()).to(out_dtype)


def matmul_blocked_oracle(a: torch.Tensor, b: torch.Tensor, block_k: int = 64,
                          out_dtype=None) -> torch.Tensor:
    """Same result up to fp32 summation order, accumulating k-block after k-block as the
    kernel's loop does (tritonix/ops/matmul.py:91-100); masked K tail = zero padding."""
    out_dtype = out_dtype or a.dtype
    a32, b32 = a.float().cpu(), b.float().cpu()
    k = a32.shape[1]
    acc = torch.zeros(a32.shape[0], b32.shape[1], dtype=torch.float32)
    for k0 in range(0, k, block_k):
        acc += a32[:, k0:k0 + block_k] @ b32[k0:k0 + block_k]
    return acc.to(out_dtype)


def splitk_reference_oracle(a: torch.Tensor, b: torch.Tensor, split_k: int, block_k: int = 32,
                            out_dtype=None) -> torch.Tensor:
    """gemm_splitk_kernel: slice s owns k-blocks s, s+S, s+2S, ... (tritonix/ops/matmul.py:176,
    192-193); its fp32 partial is rounded to the output type (:195) and added into a zeroed C
    in that type (:202).  The order of the adds is unspecified on a GPU; slice order is used."""
    out_dtype = out_dtype or a.dtype
    a32, b32 = a.float().cpu(), b.float().cpu()
    m, k = a32.shape
    n = b32.shape[1]
    c = torch.zeros(m, n, dtype=out_dtype)
    for s in range(split_k):
        acc = torch.zeros(m, n, dtype=torch.float32)
        for k0 in range(s * block_k, k, block_k * split_k):
            acc += a32[:, k0:k0 + block_k] @ b32[k0:k0 + block_k]
        c = (c.float() + acc.to(out_dtype).float()).to(out_dtype)
    return c


def splitk_oracle(a: torch.Tensor, b: torch.Tensor, split_k: int, tile_k: int = 64,
                  out_dtype=None) -> torch.Tensor:
    """The deterministic split-K of the CUDA kernel: slice s owns the contiguous k-blocks
    [s*per, (s+1)*per), per = ceil(ceil(K/tile_k)/S); fp32 partials are added in slice order and
    rounded once."""
    out_dtype = out_dtype or a.dtype
    a32, b32 = a.float().cpu(), b.float().cpu()
    m, k = a32.shape
    n = b32.shape[1]
    num_kb = -(-k // tile_k)
    per = -(-num_kb // max(1, min(split_k, num_kb)))
    total = torch.zeros(m, n, dtype=torch.float32)
    for s in range(-(-num_kb // per)):
        k0, k1 = s * per * tile_k, min((s + 1) * per * tile_k, k)
        total += a32[:, k0:k1] @ b32[k0:k1]
    return total.to(out_dtype)


# ---------------------------------------------------------------------------- GLU
def _gate(g: torch.Tensor, activation: str) -> torch.Tensor:
    if activation == "silu":
        return torch.sigmoid(g) * g  # silu() of tritonix/ops/swiglu.py:7-9
    if activation == "sigmoid":
        return torch.sigmoid(g)
    return g  # any other value: no activation (tritonix/ops/swiglu.py:100-102)


def glu_oracle(x: torch.Tensor, w12: torch.Tensor, activation: str = "silu",
               out_dtype=None) -> torch.Tensor:
    """Z = act(X.W1) * (X.W2) with W1 = W12[:, 0::2], W2 = W12[:, 1::2]; everything before the
    final cast in fp32 (tritonix/ops/swiglu.py:82-104)."""
    out_dtype = out_dtype or x.dtype
    acc = x.float().cpu() @ w12.float().cpu()
    return (_gate(acc[:, 0::2], activation) * acc[:, 1::2]).to(out_dtype)


def swiglu_mlp_oracle(x, w12, w_down, out_dtype=None, hidden_dtype=None) -> torch.Tensor:
    """(silu(X.W1) * (X.W2)).W_down.  ``hidden_dtype`` rounds the intermediate the way a
    two-launch implementation stores it (default: no rounding, pure fp32)."""
    out_dtype = out_dtype or x.dtype
    h = glu_oracle(x, w12, "silu", out_dtype=torch.float32)
    if hidden_dtype is not None:
        h = h.to(hidden_dtype).float()
    return (h @ w_down.float().cpu()).to(out_dtype)


# ---------------------------------------------------------------------------- tile orders
def swizzle2d(i: int, j: int, size_i: int, size_j: int, size_g: int) -> Tuple[int, int]:
    """tl.swizzle2d as the reference's kernels call it (tritonix/ops/matmul.py:70): the row-major
    tile id i*size_j + j is re-read band by band (size_g rows), column-major inside a band."""
    ij = i * size_j + j
    per_band = size_g * size_j
    band = ij // per_band
    off_i = band * size_g
    rows = min(size_i - off_i, size_g)
    r = ij % per_band
    return off_i + r % rows, r // rows


def grouped_launch(pid: int, m: int, n: int, block_m: int, block_n: int, group_m: int):
    """1-D form of the same remap (tritonix/ops/matmul.py:111-130)."""
    grid_m, grid_n = -(-m // block_m), -(-n // block_n)
    width = group_m * grid_n
    group_id = pid // width
    group_size = min(grid_m - group_id * group_m, group_m)
    return group_id * group_m + (pid % group_size), (pid % width) // group_size


def serpentine(t: int, size_i: int, size_j: int, size_g: int) -> Tuple[int, int]:
    """Boustrophedon walk of the banded order: odd columns bottom-up, odd bands right-to-left.
    This is what swizzle2d_rows (tritonix/ops/matmul.py:9-27, never called by the reference)
    describes; its `(start - pid_n) % 2` takes different signs under Triton's compiler and its
    interpreter for even bands, so the unambiguous intent is restated here."""
    i, j = swizzle2d(t // size_j, t % size_j, size_i, size_j, size_g)
    band = i // size_g
    off_i = band * size_g
    rows = min(size_i - off_i, size_g)
    if j % 2 == 1:
        i = off_i + rows - 1 - (i - off_i)
    if band % 2 == 1:
        j = size_j - 1 - j
    return i, j


# ---------------------------------------------------------------------------- dispatcher key
def tuning_key(key_names, args, kwargs, arg_names) -> tuple:
    """_tuning_key (tritonix/dispatcher.py:18-30)."""
    bound = dict(zip(arg_names, args))
    bound.update(kwargs)
    parts = []
    for name in key_names:
        if name in bound:
            v = bound[name]
            parts += [*v.shape, str(v.dtype)] if isinstance(v, torch.Tensor) else [v]
    for name, v in bound.items():
        if name not in key_names and isinstance(v, torch.Tensor):
            parts += [*v.shape, str(v.dtype)]
    return tuple(parts)
