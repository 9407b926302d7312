"""Host-side checks of the one-launch SwiGLU MLP (tnx_swiglu_mlp): struct layouts, the resource
query, and the property its freedom from deadlock rests on — in the fixed global order of work
units, everything a unit waits for comes EARLIER in the order:
  * an output tile D(t, .) needs every hidden tile G(t, .) of its row tile;
  * a hidden tile G(t, .) that reuses a ring slot needs every D(t', .) of the row tile t' that
    held the slot before (t' = t - ring_bands * band).
The order is produced by the library itself (tnx_swiglu_mlp_unit_order, the same function the
kernel calls on the device), on the host, without a GPU."""
import ctypes
import re

import pytest
import torch

from tritonix_b200 import OutOfResources, _cabi
from tests.test_cabi_cpu import HEADER


def test_struct_layouts_match_header():
    text = open(HEADER).read()
    for struct, cls in (("tnx_mlp_problem", _cabi.MlpProblem), ("tnx_mlp_resources", _cabi.MlpResources)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), text, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if decl:
                fields += [f.strip() for f in decl.split(None, 1)[1].split(",")]
        assert fields == [n for n, _ in cls._fields_], struct
    assert ctypes.sizeof(_cabi.MlpProblem) == 56 and ctypes.sizeof(_cabi.MlpResources) == 40
    body = re.search(r"typedef struct tnx_mlp_exchange \{(.*?)\} tnx_mlp_exchange;", text, re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = [re.sub(r"[^a-z0-9_]", "", part.split()[-1]) for decl in body.split(";") if decl.strip()
             for part in decl.split(",")]
    assert names == [n for n, _ in _cabi.MlpExchange._fields_]
    assert ctypes.sizeof(_cabi.MlpExchange) == 64


def query(m, d, ff, n_out, cfg=None, dtype=_cabi.BF16):
    problem = _cabi.MlpProblem(m, d, ff, n_out, dtype, _cabi.EPI_GLU_SILU, d, 2 * ff, n_out, n_out)
    return _cabi.mlp_query(problem, _cabi.make_config(cfg))


def test_resource_query():
    r = query(32768, 4096, 14336, 4096, {"tile_k": 128, "stages": 3, "group_m": 4})
    assert (r.tiles_m, r.band_rows, r.num_bands, r.tmem_columns) == (128, 1024, 32, 512)
    assert r.smem_bytes == 3 * (128 + 128) * 128 * 2 + 2 * 16384 + 512 + 1024
    band = 1024 * 14336 * 2
    assert r.min_workspace_bytes == 1792 + 2 * band and r.workspace_bytes == r.min_workspace_bytes
    small = query(300, 512, 1024, 512)
    assert small.num_bands == 1 and small.min_workspace_bytes == small.workspace_bytes
    with pytest.raises(OutOfResources, match="shared memory"):
        query(4096, 4096, 14336, 4096, {"tile_k": 128, "stages": 4})
    with pytest.raises(ValueError, match="256 x 256"):
        query(4096, 4096, 14336, 4096, {"tile_n": 128})
    with pytest.raises(ValueError, match="multiples of 8"):
        query(4096, 4100, 14336, 4096)
    with pytest.raises(ValueError, match="fp16 or bf16"):
        query(4096, 4096, 14336, 4096, dtype=_cabi.F32)


@pytest.mark.parametrize("m,d,ff,n_out,group_m", [
    (32768, 4096, 14336, 4096, 4),     # the Llama-3-8B block
    (32768, 4096, 1792, 4096, 16),     # its 8-way tensor-parallel shard
    (2048, 512, 2048, 512, 4),
    (1000, 256, 520, 264, 2),          # ragged everywhere, last band short
    (256, 128, 128, 128, 4),           # one row tile
    (2304, 512, 640, 384, 4),          # nine row tiles: bands of 4, 4, 1
    (1536, 512, 640, 384, 1),          # bands of a single row tile
])
def test_every_wait_targets_an_earlier_unit(m, d, ff, n_out, group_m):
    order = _cabi.mlp_unit_order(m, d, ff, n_out, {"group_m": group_m})
    tiles_m, n_g, n_d = -(-m // 256), -(-2 * ff // 256), -(-n_out // 256)
    assert len(order) == tiles_m * (n_g + n_d)
    assert len(set(order)) == len(order)                       # every unit exactly once
    assert {(0, t, j) for t in range(tiles_m) for j in range(n_g)} | \
        {(1, t, j) for t in range(tiles_m) for j in range(n_d)} == set(order)
    pos = {unit: i for i, unit in enumerate(order)}
    band = min(group_m, tiles_m)
    for t in range(tiles_m):
        last_g = max(pos[(0, t, j)] for j in range(n_g))
        first_d = min(pos[(1, t, j)] for j in range(n_d))
        assert last_g < first_d
        for ring in (2, 3):
            prev = t - ring * band
            if prev >= 0:
                assert max(pos[(1, prev, j)] for j in range(n_d)) < min(pos[(0, t, j)] for j in range(n_g))


def test_neighbouring_units_share_a_weight_tile():
    """Inside a band units run column by column: consecutive positions differ in the row tile."""
    order = _cabi.mlp_unit_order(4096, 1024, 2048, 1024, {"group_m": 4})
    first_band = [u for u in order if u[0] == 0 and u[1] < 4][:8]
    assert [u[2] for u in first_band] == [0, 0, 0, 0, 1, 1, 1, 1]
    assert [u[1] for u in first_band] == [0, 1, 2, 3, 0, 1, 2, 3]
