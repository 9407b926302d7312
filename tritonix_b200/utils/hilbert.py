"""Hilbert-curve orderings of a rectangular tile grid.

Behaviour of the reference's tritonix/utils/hilbert.py:10-98: the m x n rectangle is embedded
in the enclosing power-of-two square, the square's Hilbert curve is walked, and cells outside
the rectangle are skipped, which yields a bijection on the rectangle.  Here the order is also
exported as the packed int32 table the CUDA kernels consume (``hilbert_tile_table``).
"""
from __future__ import annotations

from functools import lru_cache
from typing import List, Tuple


def hilbert_d2xy(n: int, d: int) -> Tuple[int, int]:
    """(x, y) of the d-th cell of the Hilbert curve over an n x n grid, n a power of two."""
    if n <= 0 or n & (n - 1):
        raise ValueError(f"n must be a power of two, got {n}")
    x = y = 0
    side = 1
    rest = d
    while side < n:
        quad = rest & 3          # which quadrant at this level (2 bits of d)
        rx = quad >> 1
        ry = (quad ^ rx) & 1
        if ry == 0:              # rotate / reflect the sub-square
            if rx:
                x, y = side - 1 - x, side - 1 - y
            x, y = y, x
        x += side * rx
        y += side * ry
        rest >>= 2
        side <<= 1
    return x, y


def hilbert_rect_coords(m: int, n: int) -> List[Tuple[int, int]]:
    """(row, col) of every cell of an m x n grid, in Hilbert order."""
    if m <= 0 or n <= 0:
        return []
    side = 1 << (max(m, n) - 1).bit_length()
    out: List[Tuple[int, int]] = []
    want = m * n
    for d in range(side * side):
        x, y = hilbert_d2xy(side, d)
        if y < m and x < n:
            out.append((y, x))
            if len(out) == want:
                break
    return out


def hilbert_permutation(m: int, n: int) -> List[int]:
    """P with P[i*n + j] = rank of cell (i, j) along the curve."""
    perm = [0] * (m * n)
    for rank, (i, j) in enumerate(hilbert_rect_coords(m, n)):
        perm[i * n + j] = rank
    return perm


def hilbert_inverse_permutation(m: int, n: int) -> List[int]:
    """I with I[rank] = row-major index of the rank-th cell, so I[P[r]] == r."""
    return [i * n + j for i, j in hilbert_rect_coords(m, n)]


def hilbert_swizzled_coords(m: int, n: int) -> List[Tuple[int, int]]:
    """Alias of ``hilbert_rect_coords`` (name used when re-ordering MMA tile coordinates)."""
    return hilbert_rect_coords(m, n)


@lru_cache(maxsize=64)
def hilbert_tile_table(tiles_m: int, tiles_n: int) -> tuple[int, ...]:
    """The order as packed words ``(tile_row << 16) | tile_col`` — the ``tile_table`` argument
    of ``tnx_gemm`` when ``tile_order`` is TNX_ORDER_TABLE."""
    if tiles_m > 0xFFFF or tiles_n > 0xFFFF:
        raise ValueError("tile grid too large for the packed table")
    return tuple((i << 16) | j for i, j in hilbert_rect_coords(tiles_m, tiles_n))
