"""GEMM entry points: ``matmul_kernel`` / ``gemm_splitk_kernel`` handles, their launchers, the
per-shape tuned configuration caches, ``cuda_matmul`` (the reference's ``triton_matmul``),
``matmul_splitk`` and the ``matmul`` dispatcher — the surface of tritonix/ops/matmul.py:30-293.

Search space = the CUDA kernels' template and launch parameters, under the reference's key
names (tritonix/ops/matmul.py:33-39) so that launchers written against it keep working:
  block_m     rows of C per tile: 128 = one SM per tile, 256 = a CTA pair (tcgen05 cta_group::2)
  block_n     columns of B per tile (64 / 128 / 256)
  block_k     K elements per pipeline stage (64 / 128)
  num_stages  depth of the TMA -> shared-memory ring
  group_m     band height of the grouped tile order
  split_k     K slices per tile (split-K kernel only)
  acc_stages  TMEM accumulator buffers (2 overlaps a tile's epilogue with the next main loop)
The C ABI's own names (tile_m, tile_n, tile_k, stages, cta_group, ...) are accepted as well.
"out of resources" means num_stages x stage bytes (+ epilogue staging) exceeds the 227 KiB of
shared memory of an SM, or the accumulators exceed its 512 TMEM columns.
"""
from __future__ import annotations

import os

import torch

from tritonix_b200 import _cabi, tuning_cache
from tritonix_b200.autotune import Choice, PowerOfTwo, Range, tunable
from tritonix_b200.dispatcher import dynamic_dispatch
from tritonix_b200.ops._kernel_handle import CudaKernel

_MEMORY = {"block_m", "block_n", "block_k", "num_stages", "acc_stages"}
# A 256-row tile is shared by two CTAs, each loading half of the B columns: less shared memory
# per CTA than a 128-row tile, so this axis is ranked by descending value.
_RANK = {"block_m": lambda rows: -rows}

matmul_kernel = tunable(
    keys=["m", "n", "k"],
    space={
        "block_m": PowerOfTwo(128, 256),
        "block_n": PowerOfTwo(64, 512),   # 512: two 256-column tiles per CTA pair, sharing A
        "block_k": PowerOfTwo(64, 128),
        "group_m": Choice([4, 8, 16]),
        "split_k": Choice([1, 2, 4, 8]),
        "num_stages": Range(2, 8),
        "acc_stages": Choice([1, 2]),
    },
    memory_params=_MEMORY,
    memory_rank=_RANK,
)(CudaKernel("matmul_kernel", doc="C = A x B; A is (M, K), B is (K, N), C is (M, N); fp32 "
                                  "accumulation, result cast to the input type."))

gemm_splitk_kernel = tunable(
    keys=["m", "n", "k"],
    space={
        "block_m": Choice([128]),
        "block_n": PowerOfTwo(64, 256),
        "block_k": PowerOfTwo(64, 128),
        "group_m": Choice([8]),
        "split_k": Choice([1, 2, 4, 8, 16]),
        "num_stages": Range(3, 8),
        "acc_stages": Choice([1, 2]),
    },
    memory_params=_MEMORY,
    memory_rank=_RANK,
)(CudaKernel("gemm_splitk_kernel", doc="C = A x B with K cut into split_k slices per tile; the "
                                       "slices' fp32 partials are summed in a fixed order."))


def _strides(a, b, c):
    return (a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0), c.stride(1))


def _new_output(a, b, out):
    m, n = a.shape[0], b.shape[1]
    if out is None:
        return torch.empty((m, n), device=a.device, dtype=a.dtype)
    if tuple(out.shape) != (m, n) or out.dtype != a.dtype or out.device != a.device:
        raise ValueError(f"out must be a {(m, n)} {a.dtype} tensor on {a.device}")
    return out


def _launch_matmul(a: torch.Tensor, b: torch.Tensor, cfg: dict, out=None) -> torch.Tensor:
    """Allocates C (unless ``out`` is given) and runs ``matmul_kernel`` with ``cfg``
    (tritonix/ops/matmul.py:217-237)."""
    m, k = a.shape
    _, n = b.shape
    c = _new_output(a, b, out)
    matmul_kernel[(1,)](a, b, c, m, n, k, *_strides(a, b, c), **cfg)
    return c


def _launch_splitk(a: torch.Tensor, b: torch.Tensor, cfg: dict, out=None) -> torch.Tensor:
    """Split-K launch (tritonix/ops/matmul.py:240-264).  C needs no zero fill: nothing is
    accumulated into it, the last slice to finish writes the ordered sum."""
    m, k = a.shape
    _, n = b.shape
    c = _new_output(a, b, out)
    gemm_splitk_kernel[(1,)](a, b, c, m, n, k, *_strides(a, b, c), **cfg)
    return c


# ------------------------------------------------------------------------------------------
# configuration choice
# ------------------------------------------------------------------------------------------

def default_config(m: int, n: int, k: int, split_k: int | None = None) -> dict:
    """Configuration used when tuning is disabled (``TRITONIX_B200_TUNE=0``): the shapes that
    measured best on a B200 for large, skinny and small problems."""
    if split_k is not None:
        return {"block_m": 128, "block_n": 128 if n >= 1024 else 64, "block_k": 128, "group_m": 8,
                "split_k": int(split_k), "num_stages": 4 if m <= 64 else 3}
    # Large problems: 256 x 256 tiles on CTA pairs.  Problems that cannot give most SMs such a
    # tile take smaller single-SM tiles, and whatever still leaves SMs idle is split along K.
    def ctas(bm, bn):
        return -(-m // bm) * -(-n // bn) * (bm // 128)

    def wave_fill(pairs):
        return pairs / (-(-pairs // 74) * 74)

    if (m > 128 and n >= 512 and k >= 6144 and ctas(256, 512) >= 100
            and wave_fill(ctas(256, 512) // 2) >= wave_fill(ctas(256, 256) // 2) - 0.05):
        # two waves or more of double tiles and a K loop long enough to pay for their epilogue
        # (8192^3: +5 %, K = 14336: +10 %, K = 4096: -4 %): one stage of A feeds two accumulators
        cfg = {"block_m": 256, "block_n": 512, "block_k": 64, "group_m": 8, "num_stages": 4}
    elif m > 128 and n >= 256 and ctas(256, 256) >= 100:
        cfg = {"block_m": 256, "block_n": 256, "block_k": 128, "group_m": 16, "num_stages": 3}
    elif n > 64 and (m <= 128 or ctas(128, 128) >= 74):
        cfg = {"block_m": 128, "block_n": 128, "block_k": 128, "group_m": 8, "num_stages": 4}
    else:
        cfg = {"block_m": 128, "block_n": 64, "block_k": 128, "group_m": 8, "num_stages": 4}
    cfg["split_k"] = _auto_split(m, n, k, cfg)
    # deepest ring that fits next to the 34 KiB of epilogue staging and barriers (at most 6 slots)
    pair = cfg["block_m"] // 128
    a_rows = 128 if (m >= 128 or pair == 2) else -(-m // 8) * 8
    stage_bytes = (a_rows + cfg["block_n"] // pair) * cfg["block_k"] * 2
    cfg["num_stages"] = max(2, min(6, (232448 - 34304) // stage_bytes))
    return cfg


_SM_COUNT = 148  # B200


def _auto_split(m: int, n: int, k: int, cfg: dict) -> int:
    """K slices for a problem whose tiles cannot fill the GPU: the largest power of two (at most
    8) that still fits one wave of CTAs and leaves every slice at least 512 elements of K."""
    tiles = -(-m // cfg["block_m"]) * -(-n // cfg["block_n"]) * (cfg["block_m"] // 128)
    split = 1
    while split < 8 and tiles * split * 2 <= _SM_COUNT and k // (split * 2) >= 512:
        split *= 2
    return split


def _plausible_split(m: int, n: int, k: int):
    """Split factors worth timing: 1 always, larger ones only while one wave of CTAs holds them."""
    def keep(cfg):
        s = cfg.get("split_k", 1)
        if s == 1:
            return True
        tiles = -(-m // cfg["block_m"]) * -(-n // cfg["block_n"]) * (cfg["block_m"] // 128)
        return tiles * s <= _SM_COUNT and k // s >= 256
    return keep


def _tuning_enabled() -> bool:
    return os.environ.get("TRITONIX_B200_TUNE", "1") not in ("0", "false", "off")


def _plausible(m: int, n: int):
    """Drops configurations that cannot win for the shape, to keep the first call short."""
    def keep(cfg):
        if cfg.get("block_m", 128) == 256 and m <= 128:
            return False
        if cfg["block_n"] > 64 and cfg["block_n"] >= 2 * max(n, 64):
            return False
        if cfg["block_n"] == 512 and (cfg.get("block_m", 128) != 256 or cfg.get("split_k", 1) != 1
                                      or cfg.get("acc_stages", 2) != 2):
            return False  # a double tile needs a CTA pair, both accumulator buffers and all of K
        if cfg.get("acc_stages", 2) == 1:
            # a single accumulator only ties when no CTA ever gets a second tile
            tiles = -(-m // 128) * -(-n // cfg["block_n"]) * cfg.get("split_k", 1)
            if tiles > _SM_COUNT:
                return False
        return True
    return keep


def seed_configs(m: int, n: int, k: int, split_k: int | None = None) -> list:
    """Configurations timed before the sweep of the first call for a shape: the ones that
    measured best on a B200 for large, mid-sized and skinny problems.  They stand in for the
    reference's hand-picked lists (tritonix/utils/triton.py:34-90)."""
    if split_k is not None:
        return [dict(block_m=128, block_n=bn, block_k=128, group_m=8, split_k=int(split_k),
                     num_stages=st, acc_stages=2) for bn, st in ((128, 4), (64, 6), (256, 3))]
    seeds = []
    for bm, bn, bk, g, st in ((256, 512, 64, 8, 4), (256, 512, 64, 16, 4),
                              (256, 256, 128, 16, 3), (256, 256, 64, 16, 6), (256, 256, 128, 8, 3),
                              (128, 256, 64, 8, 4), (128, 128, 128, 8, 4), (128, 64, 128, 8, 4)):
        seeds.append(dict(block_m=bm, block_n=bn, block_k=bk, group_m=g, split_k=1, num_stages=st,
                          acc_stages=2))
    return seeds


_matmul_cfg: dict = {}
_splitk_cfg: dict = {}


def _disk_key(shape_key: tuple, a: torch.Tensor) -> str:
    return tuning_cache.make_key(shape_key, a.dtype, torch.cuda.get_device_name(a.device),
                                 _cabi.lib.tnx_version().decode())


def _tuned(kernel, launcher, shape_key: tuple, a: torch.Tensor, filter_fn, seeds=(), flops: float = 0.0):
    """Disk hit, else tune and persist.  Returns None when nothing could be run.  Kernels long
    enough to run into the power cap (>= 100 GFLOP) are timed on a GPU that has settled at its
    sustained clock, and the best three are re-timed in alternation."""
    key = _disk_key(shape_key, a)
    cfg = tuning_cache.load(kernel.kernel.__name__, key)
    if cfg is not None and set(cfg) != set(kernel.space):
        cfg = None  # written by a version with a different space
    if cfg is None:
        heavy = flops >= 1e11
        # (kernels that long differ by a few per cent between their best configurations, less
        # than the clock wanders during a sweep: five finalists, five alternating passes)
        cfg = kernel.tune(launcher, filter_fn=filter_fn, seeds=seeds, finalists=5 if heavy else 3,
                          steady_state_ms=300.0 if heavy else 0.0)
        # tuning has synchronised anyway: make sure no probed configuration gave up a device wait
        _cabi.check_status(a.device)
        tuning_cache.save(kernel.kernel.__name__, key, cfg)
    return cfg


# Call signatures seen before (shapes, dtypes, strides, devices) -> a closure that allocates C and
# goes straight to tnx_gemm with the structs prepared the first time: eager calls on small
# matrices are bound by the host, and this path costs about two thirds of the general one.
_FAST_MATMUL: dict = {}


def _prepare_fast_matmul(a, b, cfg):
    import ctypes

    m, k = a.shape
    n = b.shape[1]
    strides = (*a.stride(), *b.stride(), n, 1)
    problem, config, res = _cabi._plan(m, n, k, a.dtype, strides, cfg, _cabi.EPI_NONE)
    if config.tile_order == _cabi.ORDER_TABLE:
        return None  # needs a tile table: general path
    gemm = _cabi.lib.tnx_gemm
    problem_ref, config_ref = ctypes.byref(problem), ctypes.byref(config)
    device, dtype = a.device, a.dtype
    index = device.index if device.index is not None else torch.cuda.current_device()
    status_ptr = _cabi.status_word(device).data_ptr()
    ws_bytes = int(res.workspace_bytes)
    keep = (problem, config)  # the C structs must outlive the references above

    def call(a, b):
        if torch.cuda.current_device() != index:
            return None  # the general path switches devices
        c = torch.empty((m, n), device=device, dtype=dtype)
        ws_ptr = _cabi.workspace(device, ws_bytes).data_ptr() if ws_bytes else None
        rc = gemm(problem_ref, config_ref, a.data_ptr(), b.data_ptr(), c.data_ptr(), ws_ptr,
                  ws_bytes, None, status_ptr, torch.cuda.current_stream().cuda_stream)
        if rc:
            _cabi.raise_for(rc)
        return c

    call.keep = keep
    return call


def cuda_matmul(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``a @ b`` on the CUDA kernels, tuning once per (m, n, k)
    (the reference's ``triton_matmul``, tritonix/ops/matmul.py:271-277).  ``out`` optionally
    receives the result instead of a fresh tensor."""
    signature = None
    if out is None and not matmul_kernel.kernel._pre_hooks:
        signature = (a.shape, b.shape, a.dtype, b.dtype, a.stride(), b.stride(), a.device, b.device)
        fast = _FAST_MATMUL.get(signature)
        if fast is not None:
            c = fast(a, b)
            if c is not None:
                return c
    _cabi.require_cuda(a, b)
    m, k = a.shape
    _, n = b.shape
    key = (m, n, k)
    cfg = _matmul_cfg.get(key)
    if cfg is None:
        if _tuning_enabled() and _cabi.umma_eligible_tensors(a, b):
            keep_tile, keep_split = _plausible(m, n), _plausible_split(m, n, k)
            cfg = _tuned(matmul_kernel, lambda c: _launch_matmul(a, b, c), key, a,
                         lambda c: keep_tile(c) and keep_split(c), seed_configs(m, n, k),
                         2.0 * m * n * k)
        cfg = cfg or default_config(m, n, k)
        _matmul_cfg[key] = cfg
    c = _launch_matmul(a, b, cfg, out)
    if signature is not None and a.dim() == 2 and b.dim() == 2 and a.device == b.device:
        if len(_FAST_MATMUL) >= 4096:
            _FAST_MATMUL.clear()
        fast = _prepare_fast_matmul(a, b, cfg)
        if fast is not None:
            _FAST_MATMUL[signature] = fast
    return c


cuda_matmul.__name__ = "cuda_matmul"
triton_matmul = cuda_matmul  # name kept for callers of the reference API


def matmul_splitk(a: torch.Tensor, b: torch.Tensor, split_k: int = 4,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """Split-K GEMM (tritonix/ops/matmul.py:280-288).  Unlike the reference, where ``split_k``
    only keys the cache and the tuner picks the factor, the requested factor is the one used;
    the remaining parameters are tuned once per (m, n, k, split_k)."""
    _cabi.require_cuda(a, b)
    m, k = a.shape
    _, n = b.shape
    key = (m, n, k, split_k)
    cfg = _splitk_cfg.get(key)
    if cfg is None:
        if _tuning_enabled() and _cabi.umma_eligible_tensors(a, b):
            cfg = _tuned(gemm_splitk_kernel, lambda c: _launch_splitk(a, b, c), key, a,
                         lambda c: c["split_k"] == split_k and _plausible(m, n)(c),
                         seed_configs(m, n, k, split_k), 2.0 * m * n * k)
        cfg = cfg or default_config(m, n, k, split_k)
        _splitk_cfg[key] = cfg
    return _launch_splitk(a, b, cfg, out)


# A single backend: the dispatcher keeps its shape-keyed .cache / .timings and force_backend,
# but there is no Triton, PyTorch or CPU implementation behind it.
matmul = dynamic_dispatch({"cuda": cuda_matmul}, key=["a", "b"])
