"""The allocation-free split-K entry point, `tnx_gemm_splitk_static`.

Some embedders of the library must not allocate device memory once they are running — a serving
runtime that owns all of it through its own arena, or a latency-critical loop that cannot risk
the device-wide stall an allocation may cause.  For them the split-K scratch is a fixed array
inside the library.  This test calls that entry point through the C ABI twice in a row and
checks both results against the regular entry point (`tnx_gemm`, caller-owned workspace) and
against the CPU oracle; the second call runs on the scratch contents the first one left behind.

The file name sorts last so that a `-x` run has executed every other test before this one.
"""
import ctypes

import pytest
import torch

from oracle import contraction as O
from tests.gpu_util import DEV, assert_close, seeded
from tritonix_b200 import _cabi

pytestmark = pytest.mark.gpu
f16, bf16 = torch.float16, torch.bfloat16


def call_static(a, b, c, cfg, epilogue=_cabi.EPI_NONE):
    """Straight through ctypes: problem/config structs, raw pointers, the current stream."""
    problem = _cabi.make_problem(a.shape[0], b.shape[1], a.shape[1], a.dtype,
                                 (*a.stride(), *b.stride(), *c.stride()), epilogue)
    config = _cabi.make_config(cfg)
    stream = torch.cuda.current_stream(a.device).cuda_stream
    return _cabi.lib.tnx_gemm_splitk_static(ctypes.byref(problem), ctypes.byref(config), a.data_ptr(),
                                            b.data_ptr(), c.data_ptr(),
                                            _cabi.status_word(a.device).data_ptr(), stream)


@pytest.mark.parametrize("m,n,k,dtype,cfg", [
    (64, 1024, 3584, f16, {"tile_n": 128, "tile_k": 128, "split_k": 6, "stages": 3}),
    (200, 520, 1000, bf16, {"tile_n": 64, "split_k": 3}),
])
def test_matches_regular_entry_point_twice_in_a_row(m, n, k, dtype, cfg):
    a_cpu, b_cpu = seeded(m, k, n, dtype, seed=n)
    a, b = a_cpu.to(DEV), b_cpu.to(DEV)
    expected = torch.empty(m, n, device=DEV, dtype=dtype)
    _cabi.launch(a, b, expected, {"kernel": "tcgen05", **cfg})     # tnx_gemm, caller-owned workspace
    _cabi.check_status(a.device)
    oracle = O.splitk_oracle(a_cpu, b_cpu, cfg["split_k"], cfg.get("tile_k", 64))
    assert_close(expected.cpu(), oracle, dtype)

    first = torch.full((m, n), float("nan"), device=DEV, dtype=dtype)
    second = torch.full((m, n), float("nan"), device=DEV, dtype=dtype)
    assert call_static(a, b, first, cfg) == _cabi.OK, _cabi.last_error()
    assert call_static(a, b, second, cfg) == _cabi.OK, _cabi.last_error()
    _cabi.check_status(a.device)
    for out in (first, second):
        assert_close(out.cpu(), expected.cpu(), dtype)   # within the suite's tolerance ...
        assert torch.equal(out, expected)                # ... and in fact bit-identical
        assert_close(out.cpu(), oracle, dtype)


def test_a_different_problem_reuses_the_same_scratch():
    x_cpu, w_cpu = seeded(256, 1024, 2 * 192, bf16, seed=5, b_scale=0.04)
    x, w = x_cpu.to(DEV), w_cpu.to(DEV)
    z = torch.full((256, 192), float("nan"), device=DEV, dtype=bf16)
    _cabi.launch_splitk_static(x, w, z, {"tile_n": 128, "split_k": 4}, _cabi.EPI_GLU_SILU)
    _cabi.check_status(x.device)
    assert_close(z.cpu(), O.glu_oracle(x_cpu, w_cpu, "silu"), bf16)


def test_rejects_what_does_not_fit_or_qualify():
    a = torch.zeros(4096, 4096, device=DEV, dtype=bf16)
    c = torch.empty(4096, 4096, device=DEV, dtype=bf16)
    rc = call_static(a, a, c, {"tile_n": 256, "split_k": 8})       # needs ~134 MB of scratch
    assert rc == _cabi.ERR_INVALID
    msg = _cabi.last_error()
    assert "built-in scratch holds" in msg and str(_cabi.STATIC_SCRATCH_BYTES) in msg
    with pytest.raises(ValueError, match="built-in scratch"):
        _cabi.launch_splitk_static(a, a, c, {"tile_n": 256, "split_k": 8})
    odd = torch.zeros(100, 70, device=DEV, dtype=f16)               # not TMA-legal: strided family
    rc = call_static(odd, torch.zeros(70, 90, device=DEV, dtype=f16),
                     torch.empty(100, 90, device=DEV, dtype=f16), {"split_k": 2})
    assert rc == _cabi.ERR_INVALID and "tcgen05 kernel only" in _cabi.last_error()


def test_python_wrapper_validates_operands():
    a = torch.zeros(128, 256, device=DEV, dtype=f16)
    b = torch.zeros(256, 128, device=DEV, dtype=f16)
    c = torch.empty(128, 128, device=DEV, dtype=f16)
    with pytest.raises(ValueError, match="inner dimensions"):
        _cabi.launch_splitk_static(a, b[:128], c, {"split_k": 2})
    with pytest.raises(ValueError, match="output must be"):
        _cabi.launch_splitk_static(a, b, c[:64], {"split_k": 2})
    with pytest.raises(ValueError, match="dtype mismatch"):
        _cabi.launch_splitk_static(a, b.to(bf16), c, {"split_k": 2})
