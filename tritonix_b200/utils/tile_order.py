"""Host-side statement of the orders in which the persistent CTAs visit the output tiles.
These functions mirror, index for index, what the CUDA kernels compute on the device
(``tile_coords`` in csrc/tnx_umma_gemm.cu), so tests can check the device order on the host.
"""
from __future__ import annotations

from typing import List, Tuple

from tritonix_b200.utils.hilbert import hilbert_rect_coords


def grouped_order(t: int, tiles_m: int, tiles_n: int, group_m: int) -> Tuple[int, int]:
    """Tile visited t-th: bands of ``group_m`` tile rows, column by column inside a band —
    the remap ``tl.swizzle2d`` applies in the reference's kernels (tritonix/ops/matmul.py:70;
    1-D form ``grouped_launch`` at :111-130)."""
    band_tiles = group_m * tiles_n
    band, r = divmod(t, band_tiles)
    first_row = band * group_m
    rows = min(tiles_m - first_row, group_m)
    col, row_in_band = divmod(r, rows)
    return first_row + row_in_band, col


def serpentine_order(t: int, tiles_m: int, tiles_n: int, group_m: int) -> Tuple[int, int]:
    """Boustrophedon variant: odd columns of a band run bottom-up and odd bands run right to
    left, so consecutive tiles always share an A panel or a B panel (the intent of the
    reference's unused ``swizzle2d_rows``, tritonix/ops/matmul.py:9-27)."""
    band_tiles = group_m * tiles_n
    band, r = divmod(t, band_tiles)
    first_row = band * group_m
    rows = min(tiles_m - first_row, group_m)
    col, row_in_band = divmod(r, rows)
    if col & 1:
        row_in_band = rows - 1 - row_in_band
    if band & 1:
        col = tiles_n - 1 - col
    return first_row + row_in_band, col


def tile_sequence(order: str, tiles_m: int, tiles_n: int, group_m: int = 8) -> List[Tuple[int, int]]:
    """All tiles in visiting order for ``order`` in {"grouped", "serpentine", "hilbert"}."""
    if order == "hilbert":
        return hilbert_rect_coords(tiles_m, tiles_n)
    fn = {"grouped": grouped_order, "serpentine": serpentine_order}[order]
    return [fn(t, tiles_m, tiles_n, group_m) for t in range(tiles_m * tiles_n)]
