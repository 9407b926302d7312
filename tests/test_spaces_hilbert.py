import pytest

from tritonix_b200 import Choice, ConfigSpace, PowerOfTwo, Range, SpaceConfig
from tritonix_b200.utils.hilbert import (hilbert_d2xy, hilbert_inverse_permutation,
                                         hilbert_permutation, hilbert_rect_coords,
                                         hilbert_swizzled_coords, hilbert_tile_table)


def test_axis_types():
    assert PowerOfTwo(32, 256).values() == [32, 64, 128, 256]
    assert PowerOfTwo(16, 100).values() == [16, 32, 64] and len(PowerOfTwo(16, 100)) == 3
    assert PowerOfTwo(32, 256)[1] == 64
    assert Range(2, 5).values() == [2, 3, 4, 5]  # inclusive (tritonix/utils/spaces.py:37)
    assert Range(2, 8, 2).values() == [2, 4, 6, 8] and Range(2, 8, 2)[3] == 8 and len(Range(2, 9, 2)) == 4
    c = Choice((4, 8))
    assert c.values() == [4, 8] and c[1] == 8 and len(c) == 2 and c.options == [4, 8]
    assert Choice([4, 8]) == Choice([4, 8]) and Range(1, 2) == Range(1, 2, 1)


def test_space_config():
    assert ConfigSpace is SpaceConfig
    sp = SpaceConfig({"a": PowerOfTwo(32, 128), "b": Range(2, 5), "c": Choice(["x", "y"])})
    assert sp.shape == (3, 4, 2) and len(sp) == 24
    assert sp[(1, 3, 0)] == [64, 5, "x"]
    with pytest.raises(ValueError):
        SpaceConfig({"a": Range(3, 2)})
    with pytest.raises(AssertionError):
        sp[(0, 0)]


def test_hilbert_small_known_prefix():
    assert hilbert_rect_coords(4, 4)[:5] == [(0, 0), (0, 1), (1, 1), (1, 0), (2, 0)]
    assert hilbert_rect_coords(0, 3) == []
    with pytest.raises(ValueError):
        hilbert_d2xy(6, 0)


def test_hilbert_covers_rectangle():
    coords = hilbert_rect_coords(3, 5)
    assert len(coords) == 15 == len(set(coords))
    assert all(0 <= i < 3 and 0 <= j < 5 for i, j in coords)
    m, n = 4, 7
    assert len(set(hilbert_swizzled_coords(m, n))) == m * n


@pytest.mark.parametrize("m,n", [(1, 1), (2, 2), (3, 4), (4, 3), (5, 5), (32, 32), (7, 64)])
def test_hilbert_permutation_roundtrip(m, n):
    p, inv = hilbert_permutation(m, n), hilbert_inverse_permutation(m, n)
    assert sorted(p) == list(range(m * n))
    assert all(inv[h] == r for r, h in enumerate(p))


def test_hilbert_square_steps_are_adjacent():
    c = hilbert_rect_coords(8, 8)
    assert all(abs(a[0] - b[0]) + abs(a[1] - b[1]) == 1 for a, b in zip(c, c[1:]))


def test_tile_table_packing():
    table = hilbert_tile_table(3, 5)
    assert [(v >> 16, v & 0xFFFF) for v in table] == hilbert_rect_coords(3, 5)
