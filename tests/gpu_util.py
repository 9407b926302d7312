"""Helpers shared by the GPU parity tests.  Every launch goes through the C ABI
(tritonix_b200._cabi -> ctypes -> libtritonix_b200.so) and is followed by a status-word check."""
import torch

from oracle import contraction as O
from tritonix_b200 import _cabi

TOL = {torch.float16: 2e-3, torch.bfloat16: 8e-3, torch.float32: 1e-5}
DEV = "cuda"


def seeded(m, k, n, dtype, seed=0, a_scale=1.0, b_scale=None):
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(m, k, generator=g) * a_scale).to(dtype)
    b = (torch.randn(k, n, generator=g) * (k ** -0.5 if b_scale is None else b_scale)).to(dtype)
    return a, b


def run_gemm(a_cpu, b_cpu, cfg=None, epilogue=_cabi.EPI_NONE, poison=True):
    a, b = a_cpu.to(DEV), b_cpu.to(DEV)
    n_out = b.shape[1] // 2 if epilogue else b.shape[1]
    c = torch.empty(a.shape[0], n_out, device=DEV, dtype=a.dtype)
    if poison:
        c.fill_(float("nan"))
    res = _cabi.launch(a, b, c, cfg, epilogue)
    _cabi.check_status(c.device)
    return c.cpu(), res


def assert_close(out, ref, dtype, scale=1.0):
    assert out.shape == ref.shape and out.dtype == ref.dtype
    assert not torch.isnan(out.float()).any(), "output has unwritten / NaN elements"
    err = O.rel_err(out, ref)
    assert err <= TOL[dtype] * scale, f"max|err|/max|ref| = {err:.3e} > {TOL[dtype] * scale:.1e}"
    return err
