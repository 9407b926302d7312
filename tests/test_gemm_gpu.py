"""GEMM parity on a B200: CUDA kernels (through the C ABI) against the CPU oracle, against the
committed outputs of the reference's own Triton kernel, and at full size through sampled rows.
Tolerance: max|err|/max|ref| <= 2e-3 (fp16), 8e-3 (bf16), 1e-5 (fp32)."""
import pytest
import torch

from oracle import contraction as O
from tests.golden_cases import case_ids, inputs_and_reference
from tests.gpu_util import DEV, TOL, assert_close, run_gemm, seeded
from tritonix_b200 import _cabi

pytestmark = pytest.mark.gpu
bf16, f16, f32 = torch.bfloat16, torch.float16, torch.float32
T = {"kernel": "tcgen05"}


@pytest.mark.parametrize("name", case_ids("matmul"))
def test_matches_reference_kernel_outputs(golden, name):
    a, b, ref, case = inputs_and_reference(golden, name)
    out, _ = run_gemm(a, b)
    assert_close(out, ref, a.dtype)
    assert_close(out, O.matmul_oracle(a, b), a.dtype)


@pytest.mark.parametrize("m,n,k,dtype,cfg", [
    (128, 128, 64, bf16, {"tile_n": 128, "stages": 2}),
    (128, 64, 256, f16, {"tile_n": 64, "stages": 4}),
    (128, 256, 256, bf16, {"tile_n": 256, "stages": 4}),
    (256, 256, 512, bf16, {"tile_n": 128, "tile_k": 128, "stages": 3}),
    (512, 512, 512, bf16, {"tile_n": 128, "acc_stages": 1}),
    (1024, 768, 512, f16, {}),                                    # README quick start shape
    (200, 136, 72, f16, {"tile_n": 128}),                         # ragged in M, N and K
    (1000, 1000, 1000, bf16, {"tile_n": 256}),
    (1, 8, 8, f16, {"tile_n": 64}),                               # smallest TMA-legal problem
    (129, 264, 1032, bf16, {"tile_n": 256, "stages": 3}),         # one row / 8 columns past a tile
    (1024, 1024, 256, bf16, {"tile_n": 128, "tile_order": "serpentine", "group_m": 4}),
    (1280, 1536, 256, f16, {"tile_n": 128, "tile_order": "hilbert"}),
    (1536, 1024, 512, bf16, {"tile_n": 256, "group_m": 3}),
    (256, 256, 256, bf16, {"tile_n": 256, "cta_group": 2, "stages": 4}),
    (2048, 2048, 2048, bf16, {"tile_n": 256, "cta_group": 2}),
    (1000, 1000, 1000, f16, {"tile_n": 256, "cta_group": 2}),    # ragged, CTA pairs
    (300, 520, 264, bf16, {"tile_n": 128, "cta_group": 2, "tile_k": 128, "stages": 3}),
    (2048, 512, 1024, f16, {"tile_n": 256, "cta_group": 2, "tile_order": "hilbert"}),
    (4096, 4096, 4096, bf16, {"tile_n": 256, "max_ctas": 32}),   # many tiles per CTA
])
def test_tcgen05_against_oracle(m, n, k, dtype, cfg):
    a, b = seeded(m, k, n, dtype, seed=m + n + k)
    out, res = run_gemm(a, b, {**T, **cfg})
    assert res.kernel == _cabi.KERNEL_TCGEN05
    assert_close(out, O.matmul_oracle(a, b), dtype)


WIDE = {"tile_n": 512, "cta_group": 2, "tile_k": 64, "stages": 4}


@pytest.mark.parametrize("m,n,k,dtype,cfg", [
    (512, 1024, 512, bf16, WIDE),
    (256, 512, 64, f16, WIDE),                                    # a single K block
    (256, 512, 192, bf16, WIDE),                                  # fewer K blocks than ring slots
    (1000, 1296, 1000, bf16, WIDE),                               # ragged; six 256-column tiles
    (384, 768, 2048, f16, WIDE),                                  # the last double tile has no right half
    (300, 264, 520, bf16, WIDE),                                  # one double tile, right half 8 columns
    (2048, 2048, 2048, bf16, {**WIDE, "stages": 3, "group_m": 4}),
    (1024, 1024, 4096, bf16, {**WIDE, "tile_order": "serpentine", "group_m": 2}),
    (4096, 4096, 1024, bf16, {**WIDE, "max_ctas": 24}),           # many double tiles per CTA pair
    (1024, 2048, 512, f16, {**WIDE, "tile_k": 128, "stages": 2}),
])
def test_double_tiles_against_oracle_and_single_tiles(m, n, k, dtype, cfg):
    """tile_n = 512: a CTA pair computes two column-adjacent 256-column tiles from one stream of
    A.  The K order of every output is that of the 256-column configuration, so the two must
    agree bit for bit."""
    a, b = seeded(m, k, n, dtype, seed=m + n + k)
    out, res = run_gemm(a, b, {**T, **cfg})
    assert res.kernel == _cabi.KERNEL_TCGEN05 and res.tmem_columns == 512
    assert_close(out, O.matmul_oracle(a, b), dtype)
    single, _ = run_gemm(a, b, {**T, "tile_n": 256, "cta_group": 2, "tile_k": cfg["tile_k"]})
    assert torch.equal(out, single)


@pytest.mark.parametrize("m,n,k,dtype", [(100, 70, 90, f16), (100, 70, 90, bf16), (96, 80, 72, f32),
                                         (33, 1, 17, f32), (5, 3, 0, f16), (257, 129, 65, f32)])
def test_strided_kernel_against_oracle(m, n, k, dtype):
    a, b = seeded(m, k, n, dtype, seed=7, b_scale=1.0 if k == 0 else None)
    out, res = run_gemm(a, b)
    assert res.kernel == _cabi.KERNEL_STRIDED
    assert_close(out, O.matmul_oracle(a, b), dtype, scale=4 if dtype == f32 else 1)


def test_arbitrary_strides_like_the_reference_accepts():
    """Transposed and column-sliced views: the reference's kernels take any strides
    (tritonix/ops/matmul.py:50-55)."""
    a0, b0 = seeded(192, 160, 224, f16, seed=11)
    a = a0.to(DEV).t().contiguous().t()          # column-major A: no TMA layout for it
    b = b0.to(DEV).t().contiguous().t()          # column-major B
    c_full = torch.full((192, 448), float("nan"), device=DEV, dtype=f16)
    c = c_full[:, ::2]                           # output with column stride 2
    res = _cabi.launch(a, b, c, None)
    _cabi.check_status(c.device)
    assert res.kernel == _cabi.KERNEL_STRIDED
    assert_close(c.cpu(), O.matmul_oracle(a0, b0), f16)
    assert torch.isnan(c_full[:, 1::2]).all()    # nothing written between the strided columns
    # row-sliced operands stay on the tcgen05 path (pitch > row length)
    big = torch.randn(300, 512, device=DEV).to(bf16)
    a_view = big[10:266, 64:320]
    bmat = (torch.randn(256, 128, device=DEV) * 0.06).to(bf16)
    c2 = torch.empty(256, 128, device=DEV, dtype=bf16)
    res = _cabi.launch(a_view, bmat, c2, None)
    _cabi.check_status(c2.device)
    assert res.kernel == _cabi.KERNEL_TCGEN05
    assert_close(c2.cpu(), O.matmul_oracle(a_view.cpu(), bmat.cpu()), bf16)


@pytest.mark.parametrize("m,n,k,dtype,cfg,epi", [
    (256, 384, 512, bf16, {"tile_n": 128}, 0),
    (1000, 520, 264, f16, {"tile_n": 256, "tile_k": 128, "stages": 2}, 0),
    (2048, 1024, 1024, bf16, {"tile_n": 256, "cta_group": 2, "tile_k": 128, "stages": 3}, 0),
    (512, 768, 512, bf16, {"tile_n": 128, "cta_group": 2}, 0),
    (64, 1024, 2048, f16, {"tile_n": 128, "split_k": 4}, 0),
    (300, 512, 512, bf16, {"tile_n": 256}, _cabi.EPI_GLU_SILU),
])
def test_transposed_b_operand(m, n, k, dtype, cfg, epi):
    """B given as the transpose of an (N, K) row-major tensor — the usual layout of a linear
    layer's weight — runs on the tcgen05 kernel as a K-major operand, without a copy."""
    a, b = seeded(m, k, n, dtype, seed=n + 1, b_scale=0.05 if epi else None)
    bt = b.t().contiguous().to(DEV)          # stored (N, K)
    b_view = bt.t()                          # logical (K, N), strides (1, K)
    assert b_view.stride() == (1, k)
    n_out = n // 2 if epi else n
    c = torch.full((m, n_out), float("nan"), device=DEV, dtype=dtype)
    res = _cabi.launch(a.to(DEV), b_view, c, {**T, **cfg}, epi)
    _cabi.check_status(c.device)
    assert res.kernel == _cabi.KERNEL_TCGEN05
    ref = O.glu_oracle(a, b, "silu") if epi else O.matmul_oracle(a, b)
    assert_close(c.cpu(), ref, dtype)


@pytest.mark.parametrize("m,n,k,dtype,cfg,b_transposed", [
    (256, 384, 512, bf16, {"tile_n": 128}, False),
    (1000, 520, 264, f16, {"tile_n": 256, "tile_k": 128, "stages": 2}, False),
    (2048, 1024, 1024, bf16, {"tile_n": 256, "cta_group": 2, "tile_k": 128, "stages": 3}, True),
    (64, 1024, 2048, f16, {"tile_n": 128, "split_k": 4}, False),
    (200, 256, 320, bf16, {"tile_n": 64, "split_k": 2}, True),
    (1024, 1024, 768, bf16, {"tile_n": 512, "cta_group": 2, "tile_k": 64, "stages": 4}, False),  # double tiles
])
def test_transposed_a_operand(m, n, k, dtype, cfg, b_transposed):
    """A given as the transpose of a (K, M) row-major tensor (as in a weight-gradient product
    X^T . dY) runs on the tcgen05 kernel as an M-major operand, without a copy."""
    a, b = seeded(m, k, n, dtype, seed=m + 3)
    a_view = a.t().contiguous().to(DEV).t()            # logical (M, K), strides (1, M)
    assert a_view.stride() == (1, m)
    b_dev = b.t().contiguous().to(DEV).t() if b_transposed else b.to(DEV)
    c = torch.full((m, n), float("nan"), device=DEV, dtype=dtype)
    res = _cabi.launch(a_view, b_dev, c, {**T, **cfg})
    _cabi.check_status(c.device)
    assert res.kernel == _cabi.KERNEL_TCGEN05
    assert_close(c.cpu(), O.matmul_oracle(a, b), dtype)


def test_output_tails_are_not_overwritten():
    """Canary rows/columns around C: the TMA store clips at the tensor bounds."""
    a, b = seeded(200, 72, 136, f16, seed=5)
    canvas = torch.full((200 + 16, 136 + 16), 777.0, device=DEV, dtype=f16)
    c = canvas[8:208, 8:144]
    _cabi.launch(a.to(DEV), b.to(DEV), c, T)
    _cabi.check_status(c.device)
    assert_close(c.cpu(), O.matmul_oracle(a, b), f16)
    mask = torch.ones_like(canvas, dtype=torch.bool)
    mask[8:208, 8:144] = False
    assert (canvas[mask] == 777.0).all()


def test_empty_problem_is_a_no_op():
    a = torch.empty(0, 64, device=DEV, dtype=f16)
    b = torch.empty(64, 32, device=DEV, dtype=f16)
    c = torch.empty(0, 32, device=DEV, dtype=f16)
    _cabi.launch(a, b, c, None)
    _cabi.check_status(c.device)


def test_full_size_square_gemm_by_sampled_rows():
    """bf16 8192^3 (entries N(0,1)/sqrt(K), outputs O(1)): 48 sampled rows against the oracle,
    bit-identical results from two runs of one configuration, and agreement between the
    one-SM and the CTA-pair kernels."""
    m = n = k = 8192
    g = torch.Generator(device=DEV).manual_seed(0)
    a = (torch.randn(m, k, device=DEV, generator=g) / k ** 0.5).to(bf16)
    b = (torch.randn(k, n, device=DEV, generator=g) / k ** 0.5).to(bf16)
    c = torch.empty(m, n, device=DEV, dtype=bf16)
    cfg = {**T, "tile_n": 256, "cta_group": 2, "tile_k": 128, "stages": 3, "group_m": 16}
    _cabi.launch(a, b, c, cfg)
    _cabi.check_status(c.device)
    rows = torch.randint(0, m, (48,), generator=torch.Generator().manual_seed(1)).tolist() + [0, m - 1]
    ref = O.matmul_oracle(a[rows].cpu(), b.cpu())
    assert_close(c[rows].cpu(), ref, bf16)
    c2 = torch.empty_like(c)
    _cabi.launch(a, b, c2, cfg)
    assert torch.equal(c, c2)
    c3 = torch.empty_like(c)
    _cabi.launch(a, b, c3, {**T, "tile_n": 256, "cta_group": 1, "stages": 4})
    _cabi.check_status(c.device)
    assert_close(c3[rows].cpu(), ref, bf16)
    assert O.rel_err(c3.float().cpu()[::64], c.float().cpu()[::64]) <= 8e-3


def test_invalid_launches_raise():
    a, b = seeded(128, 128, 128, f16)
    a, b = a.to(DEV), b.to(DEV)
    c = torch.empty(128, 128, device=DEV, dtype=f16)
    with pytest.raises(ValueError, match="inner dimensions"):
        _cabi.launch(a, b[:64], c)
    with pytest.raises(ValueError, match="dtype mismatch"):
        _cabi.launch(a, b.float(), c)
    with pytest.raises(ValueError, match="output must be"):
        _cabi.launch(a, b, c[:, :64])
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        _cabi.launch(a.cpu(), b, c)
    from tritonix_b200 import OutOfResources
    with pytest.raises(OutOfResources):
        _cabi.launch(a, b, c, {"tile_n": 256, "stages": 9})
    with pytest.raises(ValueError):
        _cabi.launch(a[:, 1:], b[1:], c, T)  # misaligned base address for TMA


def test_auto_kernel_takes_views_at_odd_offsets():
    """With the kernel family left open, a view whose storage offset is not a multiple of 16
    bytes runs on the strided kernel (the reference accepts any pointer,
    tritonix/ops/matmul.py:50-55); forcing the tcgen05 family on it is an error."""
    import tritonix_b200 as tnx
    g = torch.Generator().manual_seed(11)
    big = torch.randn(256, 520, generator=g).to(bf16)
    b_cpu = (torch.randn(512, 256, generator=g) / 512 ** 0.5).to(bf16)
    big_d, b = big.to(DEV), b_cpu.to(DEV)
    view = big_d[:, 4:516]                      # 8-byte offset, pitch 520 elements (16-byte multiple)
    assert view.data_ptr() % 16 == 8
    ref = O.matmul_oracle(big[:, 4:516], b_cpu)
    c = torch.full((256, 256), float("nan"), device=DEV, dtype=bf16)
    res = _cabi.launch(view, b, c)
    _cabi.check_status(c.device)
    assert_close(c.cpu(), ref, bf16)
    with pytest.raises(ValueError, match="16-byte aligned"):
        _cabi.launch(view, b, c, T)
    # the public entry point: first call (general path) and second call (prepared call)
    for _ in range(2):
        out = tnx.cuda_matmul(view, b)
        _cabi.check_status(c.device)
        assert_close(out.cpu(), ref, bf16)
