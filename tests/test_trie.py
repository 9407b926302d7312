"""Behaviour of the out-of-resources trie and the unimodality pruner; the cases follow the
reference's tests/test_trie.py:10-104 (same shapes, same expected sets) and add the
generators and pruner rules that file leaves untested."""
import pytest

from tritonix_b200.utils.pruners import (CoordinateMonotonicFunction, CoordinateUnimodalFunction,
                                         MonotonicCascadeTrie)
from tritonix_b200.utils.spaces import Choice, SpaceConfig


def make_trie(*dims):
    return MonotonicCascadeTrie(SpaceConfig({str(i): Choice(range(d)) for i, d in enumerate(dims)}))


def test_shape_and_empty_axis():
    assert make_trie(4, 5, 3).shape == (4, 5, 3)
    with pytest.raises(ValueError):
        make_trie(4, 0, 3)


def test_prune_dominates_upwards_only():
    t = make_trie(4, 4, 4, 4)
    assert not t.is_pruned((2, 2, 1, 0))
    t.prune((2, 2, 0, 0))
    assert t.is_pruned((2, 2, 0, 0)) and t.is_pruned((3, 3, 3, 3))
    assert not t.is_pruned((2, 1, 3, 3))
    with pytest.raises(ValueError):
        t.is_pruned((1, 1))


def test_minimal_failure_set_is_maintained():
    t = make_trie(4, 4, 4, 4)
    t.prune((2, 2, 2, 2))
    t.prune((1, 1, 1, 1))
    assert t._minimal_failures == [(1, 1, 1, 1)]
    t = make_trie(4, 4, 4, 4)
    for f in [(1, 4, 4, 1), (3, 3, 3, 0), (0, 4, 0, 1), (1, 3, 0, 0)]:
        t.prune(f)
    assert set(t._minimal_failures) == {(1, 3, 0, 0), (0, 4, 0, 1)}
    t = make_trie(4, 4, 3)
    t.prune((2, 1, 0))
    t.prune((1, 2, 1))
    assert not t.is_pruned((1, 2, 0)) and t.is_pruned((1, 3, 1))
    assert not t.is_pruned((1, 3, 2)[:2] + (0,))
    t.prune((1, 2, 0))
    assert (1, 2, 0) in t._minimal_failures and (1, 2, 1) not in t._minimal_failures
    assert t.is_pruned((1, 2, 1))
    before = list(t._minimal_failures)
    t.prune((3, 3, 2))  # already dominated: no change
    assert t._minimal_failures == before


def test_prefix_doom():
    t = make_trie(4, 4, 4, 4)
    assert not t._is_prefix_doomed(())
    t.prune((1, 2, 0, 1))
    assert not t._is_prefix_doomed((1, 2)) and not t._is_prefix_doomed((1, 2, 0))
    t.prune((1, 2, 0, 0))
    assert t._is_prefix_doomed((1, 2)) and t._is_prefix_doomed((1, 2, 0))
    assert not t._is_prefix_doomed((1, 1))


def test_generators():
    t = make_trie(3, 3, 3)
    t.prune((1, 1, 0))
    got = list(t.generate_all_unpruned())
    assert len(got) == 15 and got == sorted(got)
    assert (1, 1, 0) not in got and (2, 2, 2) not in got and (1, 0, 2) in got and (0, 2, 1) in got
    mid = list(t.generate_all_unpruned_midpoint())
    assert sorted(mid) == got
    assert mid[0] == (1, 0, 1)  # axis order is mid, mid-1, mid+1; (1,1,*) is pruned
    t = make_trie(4, 4, 3)
    t.prune((2, 1, 0))
    t.prune((1, 2, 0))
    for _ in range(20):
        cfg = t.get_random_unpruned()
        assert cfg is not None and not t.is_pruned(cfg)
    assert t.get_mid_point_unpruned() == (2, 0, 1)
    t = make_trie(2, 2)
    t.prune((0, 0))
    assert t.get_random_unpruned() is None and t.get_mid_point_unpruned() is None
    assert list(t.generate_all_unpruned()) == [] and list(t.generate_all_unpruned_midpoint()) == []


def test_midpoint_axis_order_and_lazy_pruning():
    t = make_trie(5)
    assert [c[0] for c in t.generate_all_unpruned_midpoint()] == [2, 1, 3, 0, 4]
    t = make_trie(4)
    assert [c[0] for c in t.generate_all_unpruned_midpoint()] == [2, 1, 3, 0]
    # a prune made while iterating removes configurations not yet visited
    t = make_trie(5)
    seen = []
    for c in t.generate_all_unpruned_midpoint():
        seen.append(c[0])
        if c[0] == 2:
            t.prune((3,))
    assert seen == [2, 1, 0]


def test_custom_comparison_functions():
    sp = SpaceConfig({"a": Choice(range(4)), "b": Choice(range(4))})
    # "failure spreads downwards" instead of upwards
    t = MonotonicCascadeTrie(sp, config_comparison_func=lambda f, c: all(x <= y for x, y in zip(c, f)),
                             dimension_comparison_func=lambda f, c, rank=0: c <= f)
    t.prune((1, 2))
    assert t.is_pruned((0, 0)) and t.is_pruned((1, 2)) and not t.is_pruned((2, 2))


def test_unimodal_pruner_rules():
    assert CoordinateMonotonicFunction is CoordinateUnimodalFunction
    sp = SpaceConfig({"x": Choice(range(5)), "y": Choice(range(2))})
    p = CoordinateUnimodalFunction(sp)
    p.record((1, 0), 1.0)
    assert not any(p.is_pruned((i, j)) for i in range(5) for j in range(2))
    p.record((2, 0), 2.0)  # worse to the right of the best: x >= 2 is cut on the line y = 0
    assert [p.is_pruned((i, 0)) for i in range(5)] == [False, False, True, True, True]
    assert not any(p.is_pruned((i, 1)) for i in range(5))
    p.record((0, 0), 3.0)  # worse to the left: x <= 0 is cut as well
    assert [p.is_pruned((i, 0)) for i in range(5)] == [True, False, True, True, True]
    q = CoordinateUnimodalFunction(sp)
    q.record((3, 1), 5.0)
    q.record((1, 1), 4.0)
    q.record((2, 1), 4.5)  # nearest worse point right of the best (x=1) is x=2
    assert [q.is_pruned((i, 1)) for i in range(5)] == [False, False, True, True, True]
    q.record((1, 0), 1.0)  # along y at x = 1: y=1 is worse than y=0
    assert q.is_pruned((1, 1)) and not q.is_pruned((1, 0))
