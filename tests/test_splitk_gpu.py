"""Split-K parity and determinism.  The reference's kernel adds fp16-rounded partials with
atomics (tritonix/ops/matmul.py:195-202) and is neither deterministic nor exact to one rounding;
the CUDA kernel sums fp32 partials in slice order, so it must agree with the oracle within the
fp16 tolerance for every split factor and be bit-identical from run to run."""
import pytest
import torch

from oracle import contraction as O
from tests.golden_cases import case_ids, inputs_and_reference
from tests.gpu_util import DEV, assert_close, run_gemm, seeded
from tritonix_b200 import _cabi

pytestmark = pytest.mark.gpu
bf16, f16 = torch.bfloat16, torch.float16
T = {"kernel": "tcgen05"}


@pytest.mark.parametrize("name", case_ids("splitk"))
def test_matches_reference_kernel_outputs(golden, name):
    a, b, ref, case = inputs_and_reference(golden, name)
    out, res = run_gemm(a, b, {**T, "tile_n": 64, "split_k": case[6]["split_k"]})
    assert_close(out, ref, a.dtype)
    assert_close(out, O.splitk_oracle(a, b, case[6]["split_k"]), a.dtype)


@pytest.mark.parametrize("split_k", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("tile_n,tile_k", [(128, 64), (64, 128)])
def test_skinny_decode_shape_scaled(split_k, tile_n, tile_k):
    """M=64 against a tall B (the decode-like configuration at 1/4 of its K and N)."""
    a, b = seeded(64, 3584, 1024, f16, seed=split_k, a_scale=3584 ** -0.5, b_scale=1.0)
    out, res = run_gemm(a, b, {**T, "tile_n": tile_n, "tile_k": tile_k, "split_k": split_k, "stages": 3})
    num_kb = -(-3584 // tile_k)
    per = -(-num_kb // split_k)
    assert res.split_k == -(-num_kb // per)  # the requested split, unless a slice would be empty
    assert_close(out, O.splitk_oracle(a, b, res.split_k, tile_k), f16)


@pytest.mark.parametrize("m,n,k,dtype,cfg", [
    (200, 520, 1000, bf16, {"tile_n": 64, "split_k": 3}),
    (128, 128, 512, f16, {"tile_n": 128, "split_k": 2}),
    (256, 512, 2048, bf16, {"tile_n": 128, "cta_group": 2, "split_k": 4}),
    (130, 264, 200, f16, {"tile_n": 256, "split_k": 8}),   # split clamps to the 4 k-blocks
    (64, 4096, 14336, f16, {"tile_n": 128, "split_k": 4, "tile_k": 128, "stages": 3}),  # full size
])
def test_general_shapes(m, n, k, dtype, cfg):
    a, b = seeded(m, k, n, dtype, seed=k)
    out, res = run_gemm(a, b, {**T, **cfg})
    assert_close(out, O.matmul_oracle(a, b), dtype)


def test_bit_deterministic_and_workspace_reusable():
    a, b = seeded(64, 14336, 4096, f16, seed=3)
    a, b = a.to(DEV), b.to(DEV)
    outs = []
    for i in range(4):
        c = torch.empty(64, 4096, device=DEV, dtype=f16)
        _cabi.launch(a, b, c, {**T, "tile_n": 128, "split_k": 8, "stages": 6})
        outs.append(c)
    _cabi.check_status(a.device)
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    # the tile counters are left at zero: the same workspace serves a different shape next
    a2, b2 = seeded(256, 1024, 384, bf16, seed=4)
    out, _ = run_gemm(a2, b2, {**T, "tile_n": 128, "split_k": 4})
    assert_close(out, O.matmul_oracle(a2, b2), bf16)
    ws = next(iter(_cabi._workspaces.values()))
    assert int(ws[:_cabi.COUNTER_BYTES].view(torch.int32).abs().sum()) == 0


def test_split_changes_only_the_summation_order():
    a, b = seeded(128, 2048, 256, f16, seed=9)
    ref = O.matmul_oracle(a, b)
    errs = []
    for s in (1, 2, 4, 8, 16):
        out, _ = run_gemm(a, b, {**T, "tile_n": 128, "split_k": s})
        errs.append(O.rel_err(out, ref))
    assert max(errs) <= 2e-3 and max(errs) - min(errs) < 5e-4  # no growth with the split factor


@pytest.mark.parametrize("split_k", [1, 3])
@pytest.mark.parametrize("n", [104, 100, 98, 9])
def test_column_counts_inside_pitched_views(split_k, n):
    """Column-sliced views: TMA clips in 16-byte units, so only N % 8 == 0 may take the tcgen05
    path; other widths go to the strided kernel.  Either way nothing is written past column n."""
    g = torch.Generator().manual_seed(n)
    a = (torch.randn(72, 320, generator=g) * 320 ** -0.5).to(f16)
    b_full = torch.randn(320, 128, generator=g).to(f16)
    a_d, b_d = a.to(DEV), b_full.to(DEV)[:, :n]
    c_full = torch.full((72, 104), float("nan"), device=DEV, dtype=f16)
    c = c_full[:, :n]
    res = _cabi.launch(a_d, b_d, c, {"tile_n": 64, "split_k": split_k})
    _cabi.check_status(c.device)
    assert res.kernel == (_cabi.KERNEL_TCGEN05 if n % 8 == 0 else _cabi.KERNEL_STRIDED)
    assert_close(c.cpu(), O.matmul_oracle(a, b_full[:, :n]), f16)
    assert torch.isnan(c_full[:, n:]).all()  # nothing written past column n


def test_split_k_with_glu_epilogue():
    x, w12 = seeded(200, 1024, 2 * 88, bf16, seed=21, b_scale=0.04)
    w_d = torch.zeros(1024, 192, dtype=bf16)
    w_d[:, :176] = w12
    out = torch.full((200, 96), float("nan"), device=DEV, dtype=bf16)
    z = out[:, :88]
    res = _cabi.launch(x.to(DEV), w_d.to(DEV)[:, :176], z, {**T, "tile_n": 128, "split_k": 4}, _cabi.EPI_GLU_SILU)
    _cabi.check_status(z.device)
    assert res.split_k == 4
    assert_close(z.cpu(), O.glu_oracle(x, w12, "silu"), bf16)
    assert torch.isnan(out[:, 88:]).all()


@pytest.mark.parametrize("m,n,k,split_k,tile_n", [(64, 1024, 2048, 4, 128), (64, 512, 4096, 8, 128), (8, 256, 1024, 2, 256),
                                                  (128, 256, 2048, 4, 64), (40, 136, 1024, 4, 128), (300, 192, 1536, 2, 64),
                                                  (64, 1024, 4096, 8, 256), (48, 512, 2048, 4, 256)])
def test_cluster_exchange_matches_workspace_path(m, n, k, split_k, tile_n, monkeypatch):
    """2, 4 or 8 slices of a small tile exchange partials through cluster shared memory; the
    result must be bit-identical to the workspace path (same fp32 sum, same order)."""
    a, b = seeded(m, k, n, f16, seed=m + n)
    cfg = {**T, "tile_n": tile_n, "split_k": split_k}
    prob = _cabi.make_problem(m, n, k, f16, (k, 1, n, 1, n, 1))
    assert _cabi.query(prob, _cabi.make_config(cfg)).workspace_bytes == 0   # cluster exchange
    out_cluster, _ = run_gemm(a, b, cfg)
    out_cluster2, _ = run_gemm(a, b, cfg)
    assert_close(out_cluster, O.splitk_oracle(a, b, split_k), f16)
    assert torch.equal(out_cluster, out_cluster2)
    monkeypatch.setenv("TNX_NO_CLUSTER_SPLITK", "1")
    _cabi._plans.clear()
    try:
        assert _cabi.query(prob, _cabi.make_config(cfg)).workspace_bytes > 0
        out_ws, _ = run_gemm(a, b, cfg)
    finally:
        monkeypatch.delenv("TNX_NO_CLUSTER_SPLITK")
        _cabi._plans.clear()
    assert torch.equal(out_cluster, out_ws)
