"""Pins the CPU oracle to outputs of the reference's own kernels (tests/golden)."""
import pytest
import torch

from oracle import contraction as O
from tests.golden_cases import case_ids, inputs_and_reference

TOL = {"float16": 2e-3, "float32": 1e-5}


@pytest.mark.parametrize("name", case_ids("matmul"))
def test_matmul_oracle_matches_reference_kernel(golden, name):
    a, b, ref, case = inputs_and_reference(golden, name)
    out = O.matmul_oracle(a, b)
    assert out.dtype == ref.dtype and out.shape == ref.shape
    assert O.rel_err(out, ref) <= TOL[case[5]]
    blocked = O.matmul_blocked_oracle(a, b, block_k=case[6]["block_k"])
    # same summation order as the kernel's k loop: agreement to the last rounding
    assert O.rel_err(blocked, ref) <= (1e-3 if case[5] == "float16" else 2e-6)


@pytest.mark.parametrize("name", case_ids("splitk"))
def test_splitk_oracles_match_reference_kernel(golden, name):
    a, b, ref, case = inputs_and_reference(golden, name)
    cfg = case[6]
    restated = O.splitk_reference_oracle(a, b, cfg["split_k"], cfg["block_k"])
    # the reference rounds every slice's partial to fp16 and adds in fp16
    assert O.rel_err(restated, ref) <= 1.5e-3
    ours = O.splitk_oracle(a, b, cfg["split_k"])
    assert O.rel_err(ours, ref) <= 2e-3
    # one rounding instead of S: closer to the exact product than the reference is
    exact = a.double() @ b.double()
    assert O.rel_err(ours, exact) <= O.rel_err(ref, exact) + 1e-6


@pytest.mark.parametrize("name", case_ids("glu"))
def test_glu_oracle_matches_reference_kernel(golden, name):
    a, b, ref, case = inputs_and_reference(golden, name)
    out = O.glu_oracle(a, b, case[7]["activation"])
    assert out.shape == ref.shape
    assert O.rel_err(out, ref) <= TOL[case[5]] * (10 if case[5] == "float32" else 1)


def test_glu_activations_differ_as_defined():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(8, 16, generator=g)
    w = torch.randn(16, 12, generator=g)
    acc = x @ w
    gate, up = acc[:, 0::2], acc[:, 1::2]
    assert torch.allclose(O.glu_oracle(x, w, "silu"), torch.nn.functional.silu(gate) * up, atol=1e-6)
    assert torch.allclose(O.glu_oracle(x, w, "sigmoid"), torch.sigmoid(gate) * up, atol=1e-6)
    assert torch.allclose(O.glu_oracle(x, w, "none"), gate * up, atol=1e-6)
    assert torch.allclose(O.glu_oracle(x, w, "anything-else"), gate * up, atol=1e-6)


def test_mlp_oracle_is_composition():
    g = torch.Generator().manual_seed(4)
    x, w12, wd = torch.randn(8, 16, generator=g), torch.randn(16, 24, generator=g), torch.randn(12, 5, generator=g)
    ref = (torch.nn.functional.silu((x @ w12)[:, 0::2]) * (x @ w12)[:, 1::2]) @ wd
    assert torch.allclose(O.swiglu_mlp_oracle(x, w12, wd), ref, atol=1e-5)


@pytest.mark.parametrize("gm,gn,g", [(1, 1, 4), (5, 7, 4), (8, 8, 8), (9, 3, 4), (64, 64, 8), (3, 11, 16)])
def test_tile_orders_are_bijections_and_agree(gm, gn, g):
    from tritonix_b200.utils.tile_order import grouped_order, serpentine_order
    seen_g, seen_s = set(), set()
    prev = None
    for t in range(gm * gn):
        i, j = divmod(t, gn)
        o = O.swizzle2d(i, j, gm, gn, g)
        assert o == O.grouped_launch(t, gm * 32, gn * 32, 32, 32, g) == grouped_order(t, gm, gn, g)
        s = O.serpentine(t, gm, gn, g)
        assert s == serpentine_order(t, gm, gn, g)
        seen_g.add(o)
        seen_s.add(s)
        if prev is not None:  # consecutive serpentine tiles share a row or a column of tiles
            assert prev[0] == s[0] or prev[1] == s[1]
        prev = s
    full = {(i, j) for i in range(gm) for j in range(gn)}
    assert seen_g == full and seen_s == full


def test_tuning_key_example():
    a = torch.empty(1024, 512, dtype=torch.float16)
    b = torch.empty(512, 768, dtype=torch.float16)
    from tritonix_b200.dispatcher import _tuning_key
    expect = (1024, 512, "torch.float16", 512, 768, "torch.float16")
    assert O.tuning_key(["a", "b"], (a, b), {}, ["a", "b"]) == expect
    assert _tuning_key(["a", "b"], (a, b), {}, ["a", "b"]) == expect
    assert _tuning_key(["a"], (a,), {"b": b, "flag": 3}, ["a", "b", "flag"]) == expect
    assert _tuning_key(["flag"], (a, b, 3), {}, ["a", "b", "flag"]) == (3,) + expect
