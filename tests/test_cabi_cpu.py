"""The C-ABI library loads without a GPU, exports every symbol the public header declares, and
its host-side resource check answers without touching a device."""
import ctypes
import os
import re

import pytest
import torch

from tritonix_b200 import OutOfResources, _cabi

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(REPO, "include", "tritonix_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tnx_[a-z_0-9]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    names = declared_functions()
    assert {"tnx_gemm", "tnx_glu", "tnx_gemm_query", "tnx_version", "tnx_last_error",
            "tnx_read_status", "tnx_sm_count"} <= set(names)
    lib = ctypes.CDLL(str(_cabi._LIB_PATH))
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert set(_cabi.EXPORTS) <= set(names)


def test_struct_layouts_match_header():
    text = open(HEADER).read()
    for struct, cls in (("tnx_problem", _cabi.Problem), ("tnx_config", _cabi.Config),
                        ("tnx_resources", _cabi.Resources)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), text, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if decl:
                fields += [f.strip() for f in decl.split(None, 1)[1].split(",")]
        assert fields == [n for n, _ in cls._fields_], struct
    assert ctypes.sizeof(_cabi.Problem) == 72 and ctypes.sizeof(_cabi.Config) == 48
    assert ctypes.sizeof(_cabi.Resources) == 40


def test_version():
    assert _cabi.lib.tnx_version().decode() == "0.1.0"


def q(m, n, k, cfg=None, dtype=torch.bfloat16, strides=None, epilogue=0):
    strides = strides or (k, 1, n, 1, (n // 2 if epilogue else n), 1)
    return _cabi.query(_cabi.make_problem(m, n, k, dtype, strides, epilogue), _cabi.make_config(cfg))


def test_resource_query_budgets():
    r = q(8192, 8192, 8192, {"tile_n": 256, "cta_group": 2, "stages": 6})
    assert r.kernel == _cabi.KERNEL_TCGEN05 and r.tmem_columns == 512 and r.split_k == 1
    assert r.smem_bytes == 6 * (128 + 128) * 64 * 2 + 2 * 16384 + 512 + 1024 <= 232448
    assert (r.tiles_m, r.tiles_n, r.workspace_bytes) == (32, 32, 0)
    with pytest.raises(OutOfResources, match="shared memory"):
        q(8192, 8192, 8192, {"tile_n": 256, "cta_group": 1, "stages": 5})
    with pytest.raises(OutOfResources):
        q(8192, 8192, 8192, {"tile_n": 256, "cta_group": 2, "stages": 8})
    # memory use is monotone in every memory axis: once it fails it keeps failing
    for axis, bigger in (("stages", 6), ("tile_k", 128)):
        with pytest.raises(OutOfResources):
            q(4096, 4096, 4096, {"tile_n": 256, "cta_group": 1, "stages": 5, "tile_k": 64, axis: bigger})


def test_double_tile_resources():
    """tile_n = 512 = two 256-column tiles per CTA pair: both TMEM buffers are accumulators and a
    ring slot holds the B columns of both tiles."""
    r = q(8192, 8192, 8192, {"tile_n": 512, "cta_group": 2, "tile_k": 64, "stages": 4})
    assert r.kernel == _cabi.KERNEL_TCGEN05 and r.tmem_columns == 512
    assert r.smem_bytes == 4 * (128 + 256) * 64 * 2 + 2 * 16384 + 512 + 1024 <= 232448
    assert (r.tiles_m, r.tiles_n, r.grid) == (32, 16, 148)
    assert q(512, 768, 512, {"tile_n": 512, "cta_group": 2}).tiles_n == 2   # the last one is half empty
    with pytest.raises(OutOfResources, match="shared memory"):
        q(8192, 8192, 8192, {"tile_n": 512, "cta_group": 2, "tile_k": 64, "stages": 5})
    for bad in ({"cta_group": 1}, {"cta_group": 2, "split_k": 2}, {"cta_group": 2, "acc_stages": 1},
                {"cta_group": 2, "tile_order": "hilbert"}):
        with pytest.raises(ValueError, match="tile_n=512"):
            q(2048, 2048, 2048, {"tile_n": 512, **bad})
    with pytest.raises(ValueError, match="tile_n=512"):   # B stored N x K
        q(2048, 2048, 2048, {"tile_n": 512, "cta_group": 2}, strides=(2048, 1, 1, 2048, 2048, 1))


def test_invalid_and_unbuilt_configs_are_value_errors():
    with pytest.raises(ValueError, match="not built"):
        q(512, 512, 512, {"tile_k": 32})
    with pytest.raises(ValueError):
        q(512, 512, 512, {"tile_n": 64, "cta_group": 2})
    with pytest.raises(ValueError):
        q(512, 512, 512, {"tile_m": 64})
    with pytest.raises(ValueError, match="even"):
        q(512, 513, 512, {}, epilogue=_cabi.EPI_GLU_SILU, strides=(512, 1, 513, 1, 256, 1))
    with pytest.raises(ValueError, match="unknown kernel configuration key"):
        _cabi.make_config({"tile_q": 3})
    with pytest.raises(ValueError, match="unsupported dtype"):
        _cabi.make_problem(1, 1, 1, torch.int8, (1, 1, 1, 1, 1, 1))
    with pytest.raises(ValueError, match="unit stride"):
        q(512, 512, 512, {"kernel": "tcgen05"}, strides=(2, 1024, 512, 1, 512, 1))
    with pytest.raises(ValueError, match="unit stride"):
        q(512, 512, 512, {"kernel": "tcgen05"}, strides=(512, 1, 512, 1, 1, 512))   # column-major C
    # a transposed A (stored K x M) is a legal tcgen05 operand
    assert q(512, 512, 512, {"kernel": "tcgen05"}, strides=(1, 512, 512, 1, 512, 1)).kernel == _cabi.KERNEL_TCGEN05
    # a transposed B (stored N x K) is a legal tcgen05 operand
    assert q(512, 512, 512, {"kernel": "tcgen05"}, strides=(512, 1, 1, 512, 512, 1)).kernel == _cabi.KERNEL_TCGEN05


def test_family_selection_and_aliases():
    assert q(100, 70, 90, dtype=torch.float16).kernel == _cabi.KERNEL_STRIDED  # pitches not 16-byte multiples
    assert q(128, 128, 128, dtype=torch.float32, strides=(128, 1, 128, 1, 128, 1)).kernel == _cabi.KERNEL_STRIDED
    assert q(128, 128, 128, {"kernel": "strided"}).kernel == _cabi.KERNEL_STRIDED
    c = _cabi.make_config({"block_n": 128, "block_k": 64, "num_stages": 4, "num_warps": 8, "group_m": 4})
    assert (c.tile_n, c.tile_k, c.stages, c.group_m) == (128, 64, 4, 4)
    # a 256-row tile means a CTA pair (the reference's block_m axis carries the 1-SM / 2-SM choice)
    pair = q(4096, 4096, 4096, {"block_m": 256, "block_n": 256, "block_k": 64, "num_stages": 6})
    single = q(4096, 4096, 4096, {"block_m": 128, "block_n": 256, "block_k": 64, "num_stages": 4})
    assert (pair.tiles_m, single.tiles_m) == (16, 32) and pair.smem_bytes == 6 * 256 * 64 * 2 + 34304


def test_split_k_resources():
    # skinny M, 2/4/8 slices: the slices form a cluster and exchange partials through shared
    # memory, so no workspace is needed
    r = q(64, 4096, 14336, {"tile_n": 128, "split_k": 4, "stages": 6}, dtype=torch.float16)
    assert r.split_k == 4 and r.grid == 128 and r.workspace_bytes == 0
    # otherwise: 64 KiB of counters + one fp32 partial tile per (tile, slice)
    r = q(64, 4096, 14336, {"tile_n": 128, "split_k": 3, "stages": 6}, dtype=torch.float16)
    assert r.split_k == 3 and r.grid == 96
    assert r.workspace_bytes == 65536 + 32 * 3 * 128 * 128 * 4
    r = q(256, 4096, 14336, {"tile_n": 128, "split_k": 4}, dtype=torch.float16)
    assert r.workspace_bytes == 65536 + 2 * 32 * 4 * 128 * 128 * 4
    # never more slices than k-blocks, and no empty slice
    assert q(128, 128, 64 * 3, {"tile_n": 128, "split_k": 8}).split_k == 3
    assert q(128, 128, 64 * 5, {"tile_n": 128, "split_k": 4}).split_k == 3
