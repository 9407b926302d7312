"""ctypes binding of libtritonix_b200.so (declared in include/tritonix_b200.h).

This module is the only place where Python touches the C ABI.  There is no fallback: if the
library is missing or fails to load, importing this module raises, and every op of the package
raises with it.
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path

import torch

import os

# TRITONIX_B200_LIB points at an alternative build of the library (e.g. a development build).
_LIB_PATH = Path(os.environ.get("TRITONIX_B200_LIB") or
                 Path(__file__).resolve().parent / "lib" / "libtritonix_b200.so")

# ---- constants mirrored from include/tritonix_b200.h
OK, ERR_INVALID, ERR_RESOURCES, ERR_NOT_BUILT, ERR_CUDA, ERR_DEVICE = range(6)
F16, BF16, F32 = 0, 1, 2
EPI_NONE, EPI_GLU_LINEAR, EPI_GLU_SILU, EPI_GLU_SIGMOID = 0, 1, 2, 3
ORDER_GROUPED, ORDER_SERPENTINE, ORDER_TABLE = 0, 1, 2
KERNEL_AUTO, KERNEL_TCGEN05, KERNEL_STRIDED = 0, 1, 2
COUNTER_BYTES = 65536

DTYPES = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}
ACTIVATIONS = {"none": EPI_GLU_LINEAR, "silu": EPI_GLU_SILU, "sigmoid": EPI_GLU_SIGMOID}
TILE_ORDERS = {"grouped": ORDER_GROUPED, "serpentine": ORDER_SERPENTINE, "hilbert": ORDER_TABLE,
               "table": ORDER_TABLE}
KERNELS = {"auto": KERNEL_AUTO, "tcgen05": KERNEL_TCGEN05, "strided": KERNEL_STRIDED}


class OutOfResources(Exception):
    """A kernel configuration exceeds the shared-memory or TMEM budget of one SM.

    Plays the role of ``triton.OutOfResources`` in the reference's tuner
    (tritonix/autotune.py:134-138): the tuner catches it and prunes every configuration that
    needs at least as much memory.
    """


class DeviceStatusError(RuntimeError):
    """A kernel gave up one of its bounded waits and reported it through the status word."""


class Problem(ctypes.Structure):
    _fields_ = [("m", ctypes.c_int32), ("n", ctypes.c_int32), ("k", ctypes.c_int32),
                ("dtype", ctypes.c_int32), ("epilogue", ctypes.c_int32),
                ("reserved0", ctypes.c_int32),
                ("stride_am", ctypes.c_int64), ("stride_ak", ctypes.c_int64),
                ("stride_bk", ctypes.c_int64), ("stride_bn", ctypes.c_int64),
                ("stride_cm", ctypes.c_int64), ("stride_cn", ctypes.c_int64)]


class Config(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "tile_m", "tile_n", "tile_k", "stages", "acc_stages", "cta_group", "split_k", "group_m",
        "tile_order", "kernel", "max_ctas", "reserved0")]


class Resources(ctypes.Structure):
    _fields_ = [("kernel", ctypes.c_int32), ("smem_bytes", ctypes.c_int32),
                ("tmem_columns", ctypes.c_int32), ("grid", ctypes.c_int32),
                ("tiles_m", ctypes.c_int32), ("tiles_n", ctypes.c_int32),
                ("split_k", ctypes.c_int32), ("reserved0", ctypes.c_int32),
                ("workspace_bytes", ctypes.c_int64)]


class ConvProblem(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "batch", "c_in", "h_in", "w_in", "c_out", "filter_h", "filter_w", "stride_h", "stride_w",
        "pad_h", "pad_w", "dil_h", "dil_w", "dtype", "has_bias", "input_layout", "output_layout",
        "weight_layout")]


class ConvResources(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "kernel", "h_out", "w_out", "tile_w", "tile_h", "smem_bytes", "tmem_columns", "grid")] + \
        [("workspace_bytes", ctypes.c_int64)]


class MlpProblem(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("m", "d_model", "d_ff", "n_out", "dtype", "activation")] + \
        [(n, ctypes.c_int64) for n in ("stride_xm", "stride_w12k", "stride_w3k", "stride_ym")]


class MlpResources(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("smem_bytes", "tmem_columns", "grid", "tiles_m",
                                              "band_rows", "num_bands")] + \
        [("min_workspace_bytes", ctypes.c_int64), ("workspace_bytes", ctypes.c_int64)]


class MlpExchange(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int32), ("rank", ctypes.c_int32), ("tile_split", ctypes.c_int32),
                ("epoch", ctypes.c_uint32), ("signal_tiles", ctypes.c_int32),
                ("reserved0", ctypes.c_int32), ("y_multicast", ctypes.c_void_p),
                ("partial_local", ctypes.c_void_p), ("partial_multicast", ctypes.c_void_p),
                ("signal_multicast", ctypes.c_void_p), ("signal_local", ctypes.c_void_p)]


LAYOUT_NCHW, LAYOUT_NHWC = 0, 1
WEIGHT_KCRS, WEIGHT_PACKED = 0, 1

EXPORTS = ("tnx_version", "tnx_last_error", "tnx_sm_count", "tnx_gemm_query", "tnx_gemm",
           "tnx_glu", "tnx_read_status", "tnx_gemm_splitk_static", "tnx_selftest_bounded_wait",
           "tnx_conv2d_query", "tnx_conv2d_forward", "tnx_conv2d_packed_weight_bytes",
           "tnx_conv2d_pack_weights", "tnx_swiglu_mlp_query", "tnx_swiglu_mlp",
           "tnx_swiglu_mlp_unit_order")
STATIC_SCRATCH_BYTES = 16 * 1024 * 1024 + 65536


def _load() -> ctypes.CDLL:
    if not _LIB_PATH.exists():
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python tritonix_b200/csrc/build.py` "
            "(needs nvcc). tritonix_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(str(_LIB_PATH))
    missing = [name for name in EXPORTS if not hasattr(lib, name)]
    if missing:
        raise ImportError(f"{_LIB_PATH} is out of date (no {', '.join(missing)}): rebuild it with "
                          "`python tritonix_b200/csrc/build.py`")
    lib.tnx_version.restype = ctypes.c_char_p
    lib.tnx_last_error.restype = ctypes.c_char_p
    lib.tnx_sm_count.restype = ctypes.c_int
    lib.tnx_gemm_query.restype = ctypes.c_int
    lib.tnx_gemm_query.argtypes = [ctypes.POINTER(Problem), ctypes.POINTER(Config),
                                   ctypes.POINTER(Resources)]
    lib.tnx_gemm.restype = ctypes.c_int
    lib.tnx_gemm.argtypes = [ctypes.POINTER(Problem), ctypes.POINTER(Config), ctypes.c_void_p,
                             ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                             ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.tnx_glu.restype = ctypes.c_int
    lib.tnx_glu.argtypes = [ctypes.POINTER(Problem), ctypes.POINTER(Config), ctypes.c_int,
                            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                            ctypes.c_void_p, ctypes.c_void_p]
    lib.tnx_gemm_splitk_static.restype = ctypes.c_int
    lib.tnx_gemm_splitk_static.argtypes = [ctypes.POINTER(Problem), ctypes.POINTER(Config),
                                           ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                           ctypes.c_void_p, ctypes.c_void_p]
    lib.tnx_selftest_bounded_wait.restype = ctypes.c_int
    lib.tnx_selftest_bounded_wait.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p]
    lib.tnx_read_status.restype = ctypes.c_int
    lib.tnx_read_status.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32),
                                    ctypes.c_void_p]
    lib.tnx_swiglu_mlp_query.restype = ctypes.c_int
    lib.tnx_swiglu_mlp_query.argtypes = [ctypes.POINTER(MlpProblem), ctypes.POINTER(Config),
                                         ctypes.POINTER(MlpResources)]
    lib.tnx_swiglu_mlp_unit_order.restype = ctypes.c_int
    lib.tnx_swiglu_mlp_unit_order.argtypes = [ctypes.POINTER(MlpProblem), ctypes.POINTER(Config),
                                              ctypes.POINTER(ctypes.c_int32), ctypes.c_int32]
    lib.tnx_swiglu_mlp.restype = ctypes.c_int
    lib.tnx_swiglu_mlp.argtypes = [ctypes.POINTER(MlpProblem), ctypes.POINTER(Config),
                                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                   ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(MlpExchange),
                                   ctypes.c_void_p, ctypes.c_void_p]
    lib.tnx_conv2d_query.restype = ctypes.c_int
    lib.tnx_conv2d_query.argtypes = [ctypes.POINTER(ConvProblem), ctypes.POINTER(Config),
                                     ctypes.POINTER(ConvResources)]
    lib.tnx_conv2d_packed_weight_bytes.restype = ctypes.c_int64
    lib.tnx_conv2d_packed_weight_bytes.argtypes = [ctypes.POINTER(ConvProblem)]
    lib.tnx_conv2d_pack_weights.restype = ctypes.c_int
    lib.tnx_conv2d_pack_weights.argtypes = [ctypes.POINTER(ConvProblem), ctypes.c_void_p,
                                            ctypes.c_void_p, ctypes.c_void_p]
    lib.tnx_conv2d_forward.restype = ctypes.c_int
    lib.tnx_conv2d_forward.argtypes = [ctypes.POINTER(ConvProblem), ctypes.POINTER(Config),
                                       ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                       ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                                       ctypes.c_void_p, ctypes.c_void_p]
    return lib


lib = _load()


def last_error() -> str:
    return lib.tnx_last_error().decode()


def raise_for(rc: int) -> None:
    """Maps a TNX_* status to the exception the reference's callers expect."""
    if rc == OK:
        return
    msg = last_error()
    if rc == ERR_RESOURCES:
        raise OutOfResources(msg)
    if rc in (ERR_INVALID, ERR_NOT_BUILT):
        raise ValueError(msg)  # the tuner skips ValueError (tritonix/autotune.py:130-133)
    if rc == ERR_DEVICE:
        raise DeviceStatusError(msg)
    raise RuntimeError(msg)


# Config keys: new names, with the reference's Triton names accepted as aliases
# (block_m/block_n/block_k/num_stages, tritonix/ops/matmul.py:33-38).  num_warps is a Triton
# launch option with no meaning here; it is accepted and ignored.
_ALIASES = {"block_m": "tile_m", "block_n": "tile_n", "block_k": "tile_k", "num_stages": "stages"}
_IGNORED = {"num_warps", "use_tf32", "activation", "num_ctas", "maxnreg"}
_CONFIG_FIELDS = {n for n, _ in Config._fields_} - {"reserved0"}


def make_config(cfg: dict | None) -> Config:
    c = Config()
    for key, value in (cfg or {}).items():
        name = _ALIASES.get(key, key)
        if name in _IGNORED or value is None:
            continue
        if name == "tile_order":
            value = TILE_ORDERS[value] if isinstance(value, str) else int(value)
        elif name == "kernel":
            value = KERNELS[value] if isinstance(value, str) else int(value)
        if name not in _CONFIG_FIELDS:
            raise ValueError(f"unknown kernel configuration key {key!r}")
        setattr(c, name, int(value))
    return c


def make_problem(m, n, k, dtype, strides, epilogue=EPI_NONE) -> Problem:
    if dtype not in DTYPES:
        raise ValueError(f"unsupported dtype {dtype}; expected float16, bfloat16 or float32")
    sam, sak, sbk, sbn, scm, scn = (int(s) for s in strides)
    return Problem(int(m), int(n), int(k), DTYPES[dtype], int(epilogue), 0,
                   sam, sak, sbk, sbn, scm, scn)


def query(problem: Problem, config: Config) -> Resources:
    res = Resources()
    raise_for(lib.tnx_gemm_query(ctypes.byref(problem), ctypes.byref(config), ctypes.byref(res)))
    return res


def require_cuda(*tensors: torch.Tensor) -> None:
    """The package has a single backend; host tensors are an error, never a fallback."""
    for t in tensors:
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise RuntimeError("tritonix_b200 operates on CUDA tensors only: there is no CPU, "
                               "Triton or PyTorch path to fall back to")


def umma_eligible_tensors(a: torch.Tensor, b: torch.Tensor) -> bool:
    """True when (a, b) can run on the TMA/tcgen05 kernels (the only ones worth tuning)."""
    if not (a.dtype in (torch.float16, torch.bfloat16) and a.dtype == b.dtype
            and a.dim() == 2 and b.dim() == 2
            and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0
            and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0):
        return False
    row_major_a = a.stride(1) == 1 and a.stride(0) % 8 == 0
    transposed_a = a.stride(0) == 1 and a.stride(1) % 8 == 0 and a.shape[0] % 8 == 0
    if not (row_major_a or transposed_a):
        return False
    row_major_b = b.stride(1) == 1 and b.stride(0) % 8 == 0
    transposed_b = b.stride(0) == 1 and b.stride(1) % 8 == 0   # e.g. weight.t()
    return row_major_b or transposed_b


# ---- per-device scratch owned by the Python layer (the C ABI never allocates)
_scratch_lock = threading.Lock()
_status_words: dict[int, torch.Tensor] = {}
_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        with _scratch_lock:
            w = _status_words.get(idx)
            if w is None:
                w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
                _status_words[idx] = w
    return w


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised split-K scratch, one per (device, stream), grown on demand.

    The kernel leaves the counter region zero after every launch, so the buffer is cleared
    only when it is (re)allocated.
    """
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, torch.cuda.current_stream(idx).cuda_stream)
    with _scratch_lock:
        w = _workspaces.get(key)
        if w is None or w.numel() < nbytes:
            size = max(nbytes, 2 * w.numel() if w is not None else 0)
            w = torch.zeros(size, dtype=torch.uint8, device=torch.device("cuda", idx))
            _workspaces[key] = w
        return w


def check_status(device: torch.device | None = None) -> None:
    """Synchronises the current stream and raises DeviceStatusError if a kernel gave up a wait."""
    device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    w = status_word(device)
    code = ctypes.c_int32(0)
    stream = torch.cuda.current_stream(w.device).cuda_stream
    rc = lib.tnx_read_status(w.data_ptr(), ctypes.byref(code), stream)
    if rc == ERR_DEVICE:
        # Slices of a split-K tile that gave up never bumped their tile counter, so the counters
        # of this device's scratch buffers may be left non-zero: clear them (after everything
        # queued on the device has drained) before any later launch trusts them.
        message = last_error()
        torch.cuda.synchronize(w.device)
        with _scratch_lock:
            for (idx, _), ws in _workspaces.items():
                if idx == w.device.index:
                    ws[:COUNTER_BYTES].zero_()
        torch.cuda.synchronize(w.device)
        raise DeviceStatusError(message)
    raise_for(rc)


_hilbert_tables: dict = {}


def hilbert_table(device: torch.device, tiles_m: int, tiles_n: int) -> torch.Tensor:
    """Device copy of the Hilbert tile order for a tiles_m x tiles_n grid (cached)."""
    from tritonix_b200.utils.hilbert import hilbert_tile_table
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, tiles_m, tiles_n)
    table = _hilbert_tables.get(key)
    if table is None:
        table = torch.tensor(hilbert_tile_table(tiles_m, tiles_n), dtype=torch.int32,
                             device=torch.device("cuda", idx))
        _hilbert_tables[key] = table
    return table


_plans: dict = {}


def _plan(m, n, k, dtype, strides, cfg, epilogue):
    """(problem, config, resources) for a launch signature; validated once, then reused."""
    key = (m, n, k, dtype, strides, epilogue, tuple(cfg.items()) if cfg else ())
    plan = _plans.get(key)
    if plan is None:
        problem = make_problem(m, n, k, dtype, strides, epilogue)
        config = make_config(cfg)
        plan = (problem, config, query(problem, config))
        if len(_plans) > 4096:
            _plans.clear()
        _plans[key] = plan
    return plan


def launch_raw(device: torch.device, dtype: torch.dtype, a_ptr: int, b_ptr: int, c_ptr: int,
               m: int, n: int, k: int, strides, cfg: dict | None = None,
               epilogue: int = EPI_NONE, tile_table=None) -> Resources:
    """Enqueues one contraction from raw pointers, sizes and element strides
    (stride_am, stride_ak, stride_bk, stride_bn, stride_cm, stride_cn) on torch's current
    stream of ``device``.  With ``tile_order="hilbert"`` the tile table is generated here;
    ``tile_order="table"`` takes it from ``tile_table`` (int32 CUDA tensor, one packed
    ``(row << 16) | col`` word per tile)."""
    problem, config, res = _plan(m, n, k, dtype, tuple(strides), cfg, epilogue)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    switch = idx != torch.cuda.current_device()
    if switch:
        previous = torch.cuda.current_device()
        torch.cuda.set_device(idx)
    try:
        ws_ptr, ws_bytes = None, 0
        if res.workspace_bytes > 0:
            ws = workspace(device, int(res.workspace_bytes))
            ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
        table_ptr = None
        if config.tile_order == ORDER_TABLE and res.kernel == KERNEL_TCGEN05:
            if tile_table is None and (cfg or {}).get("tile_order") == "hilbert":
                tile_table = hilbert_table(device, res.tiles_m, res.tiles_n)
            if tile_table is None or tile_table.dtype != torch.int32 or not tile_table.is_cuda:
                raise ValueError("tile_order='hilbert'/'table' needs an int32 CUDA tile table")
            if tile_table.numel() != res.tiles_m * res.tiles_n:
                raise ValueError("tile table length does not match the tile grid")
            table_ptr = tile_table.data_ptr()
        stream = torch.cuda.current_stream(idx).cuda_stream
        rc = lib.tnx_gemm(ctypes.byref(problem), ctypes.byref(config), a_ptr, b_ptr, c_ptr,
                          ws_ptr, ws_bytes, table_ptr, status_word(device).data_ptr(), stream)
    finally:
        if switch:
            torch.cuda.set_device(previous)
    if rc != OK:
        raise_for(rc)
    return res


def _check_operands(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, epilogue: int):
    """Shape, dtype and device checks shared by the launch functions; returns (m, n, k).  Without
    them a mismatched operand would make the tensor maps cover memory outside the caller's
    tensors."""
    if not (a.is_cuda and b.is_cuda and c.is_cuda):
        raise RuntimeError("tritonix_b200 runs on CUDA tensors only (there is no CPU path)")
    if a.dim() != 2 or b.dim() != 2 or c.dim() != 2:
        raise ValueError("a, b and c must be 2-D")
    if not (a.dtype == b.dtype == c.dtype):
        raise ValueError(f"dtype mismatch: {a.dtype}, {b.dtype}, {c.dtype}")
    if not (a.device == b.device == c.device):
        raise ValueError("a, b and c must live on the same device")
    m, k = a.shape
    kb, n = b.shape
    if kb != k:
        raise ValueError(f"inner dimensions differ: a is {tuple(a.shape)}, b is {tuple(b.shape)}")
    n_out = n // 2 if epilogue != EPI_NONE else n
    if tuple(c.shape) != (m, n_out):
        raise ValueError(f"output must be {(m, n_out)}, got {tuple(c.shape)}")
    return m, n, k


def launch(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, cfg: dict | None = None,
           epilogue: int = EPI_NONE, tile_table=None) -> Resources:
    """Enqueues C = epilogue(A.B) on torch's current stream.  a: M x K, b: K x N, c: M x N (or
    M x N/2 for a GLU epilogue); any strides.  Returns the resources the launch used."""
    m, n, k = _check_operands(a, b, c, epilogue)
    return launch_raw(a.device, a.dtype, a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k,
                      (*a.stride(), *b.stride(), *c.stride()), cfg, epilogue, tile_table)


def launch_splitk_static(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor,
                         cfg: dict | None = None, epilogue: int = EPI_NONE) -> None:
    """C = epilogue(A.B) through ``tnx_gemm_splitk_static``: the split-K scratch is the fixed
    array inside the library, so nothing is allocated by this call or by the library (``c`` is
    the caller's).  For hosts that must not allocate device memory while running; problems
    whose scratch exceeds ``STATIC_SCRATCH_BYTES`` raise ``ValueError``.  Calls on one device
    share the array and must be ordered on the GPU."""
    m, n, k = _check_operands(a, b, c, epilogue)
    problem = make_problem(m, n, k, a.dtype, (*a.stride(), *b.stride(), *c.stride()), epilogue)
    config = make_config(cfg)
    stream = torch.cuda.current_stream(a.device).cuda_stream
    with torch.cuda.device(a.device):
        rc = lib.tnx_gemm_splitk_static(ctypes.byref(problem), ctypes.byref(config), a.data_ptr(),
                                        b.data_ptr(), c.data_ptr(),
                                        status_word(a.device).data_ptr(), stream)
    raise_for(rc)


# ---------------------------------------------------------------------------------------------
# Fused SwiGLU MLP (one launch)
# ---------------------------------------------------------------------------------------------
_mlp_workspaces: dict = {}
_mlp_plans: dict = {}


def mlp_eligible(x: torch.Tensor, w12: torch.Tensor, w3: torch.Tensor, y: torch.Tensor | None = None) -> bool:
    """True when the one-launch MLP kernel can take these operands (16-bit type, contiguous rows,
    16-byte aligned bases and pitches, sizes that are multiples of 8)."""
    ts = [x, w12, w3] + ([y] if y is not None else [])
    if not all(t.is_cuda and t.dim() == 2 and t.dtype == x.dtype and t.stride(1) == 1
               and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 and t.shape[1] % 8 == 0 for t in ts):
        return False
    return (x.dtype in (torch.float16, torch.bfloat16) and w12.shape[0] == x.shape[1]
            and w12.shape[1] == 2 * w3.shape[0] and x.shape[0] >= 1)


def mlp_query(problem: MlpProblem, config: Config) -> MlpResources:
    res = MlpResources()
    raise_for(lib.tnx_swiglu_mlp_query(ctypes.byref(problem), ctypes.byref(config), ctypes.byref(res)))
    return res


def mlp_unit_order(m: int, d_model: int, d_ff: int, n_out: int, cfg: dict | None = None):
    """The kernel's global work-unit order as a list of (down, row_tile, column_tile); computed
    on the host by the library (no GPU needed)."""
    problem = MlpProblem(m, d_model, d_ff, n_out, BF16, EPI_GLU_SILU, d_model, 2 * d_ff, n_out, n_out)
    config = make_config(cfg)
    total = lib.tnx_swiglu_mlp_unit_order(ctypes.byref(problem), ctypes.byref(config), None, 0)
    if total < 0:
        raise_for(-total)
    buf = (ctypes.c_int32 * total)()
    lib.tnx_swiglu_mlp_unit_order(ctypes.byref(problem), ctypes.byref(config), buf, total)
    return [(v >> 30, (v >> 14) & 0xffff, v & 0x3fff) for v in buf]


def launch_mlp(x: torch.Tensor, w12: torch.Tensor, w3: torch.Tensor, y: torch.Tensor,
               cfg: dict | None = None, activation: int = EPI_GLU_SILU,
               workspace: torch.Tensor | None = None, ring_bands: int | None = None,
               exchange: MlpExchange | None = None) -> MlpResources:
    """Enqueues y = (act(x W1) * (x W2)) W3 as ONE kernel (``tnx_swiglu_mlp``) on torch's current
    stream.  The workspace (dependency counters + a ring of bands of the hidden activation) is a
    cached per-(device, stream) tensor unless one is passed; ``ring_bands`` sizes the cached one
    (default: the library's recommendation, two bands).  ``exchange`` describes the
    tensor-parallel sum of the ranks' partial outputs inside the kernel (``tnx_mlp_exchange``)."""
    require_cuda(x, w12, w3, y)
    if not mlp_eligible(x, w12, w3, y):
        raise ValueError("the one-launch MLP needs 2-D fp16/bf16 CUDA tensors with contiguous rows, "
                         "16-byte aligned bases and pitches, and w12 (K, 2F), w3 (F, N)")
    m, d_model = x.shape
    d_ff, n_out = w3.shape
    if tuple(y.shape) != (m, n_out):
        raise ValueError(f"output must be {(m, n_out)}, got {tuple(y.shape)}")
    key = (m, d_model, d_ff, n_out, x.dtype, activation, x.stride(0), w12.stride(0), w3.stride(0),
           y.stride(0), tuple(cfg.items()) if cfg else ())
    plan = _mlp_plans.get(key)
    if plan is None:
        problem = MlpProblem(m, d_model, d_ff, n_out, DTYPES[x.dtype], activation, x.stride(0),
                             w12.stride(0), w3.stride(0), y.stride(0))
        config = make_config(cfg)
        plan = _mlp_plans[key] = (problem, config, mlp_query(problem, config))
    problem, config, res = plan
    idx = x.device.index if x.device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(idx):
        stream = torch.cuda.current_stream(idx).cuda_stream
        ws_bytes = workspace.numel() if workspace is not None else 0
        if workspace is None:
            want = int(res.workspace_bytes)
            if ring_bands is not None and res.num_bands > 2:
                per_band = res.band_rows * d_ff * x.element_size()
                want = int(res.min_workspace_bytes) + (min(max(2, ring_bands), res.num_bands) - 2) * per_band
            wkey = (idx, stream)
            workspace = _mlp_workspaces.get(wkey)
            if workspace is None or workspace.numel() < want:
                workspace = torch.empty(want, dtype=torch.uint8, device=torch.device("cuda", idx))
                _mlp_workspaces[wkey] = workspace
            ws_bytes = want  # a larger cached buffer must not turn into a deeper ring
        rc = lib.tnx_swiglu_mlp(ctypes.byref(problem), ctypes.byref(config), x.data_ptr(), w12.data_ptr(),
                                w3.data_ptr(), y.data_ptr(), workspace.data_ptr(), ws_bytes,
                                ctypes.byref(exchange) if exchange is not None else None,
                                status_word(x.device).data_ptr(), stream)
    raise_for(rc)
    return res


# ---------------------------------------------------------------------------------------------
# Convolution
# ---------------------------------------------------------------------------------------------
_conv_workspaces: dict = {}


def conv_workspace(device: torch.device, nbytes: int, stream: int | None = None) -> torch.Tensor:
    """Scratch for the repacked input, weights and output of a convolution, one per (device,
    stream), grown on demand.  Not cleared: the library writes every byte it reads.  ``stream``
    is the raw handle of the stream the call will run on (default: torch's current one)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, torch.cuda.current_stream(idx).cuda_stream if stream is None else stream)
    w = _conv_workspaces.get(key)
    if w is not None and w.numel() >= nbytes:
        return w
    with _scratch_lock:
        w = _conv_workspaces.get(key)
        if w is None or w.numel() < nbytes:
            w = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=torch.device("cuda", idx))
            _conv_workspaces[key] = w
        return w


def make_conv_problem(batch, c_in, h_in, w_in, c_out, filter_h, filter_w, stride, padding, dilation,
                      dtype, has_bias, input_layout=LAYOUT_NCHW,
                      output_layout=LAYOUT_NCHW, weight_layout=WEIGHT_KCRS) -> ConvProblem:
    if dtype not in DTYPES:
        raise ValueError(f"unsupported dtype {dtype}")
    return ConvProblem(batch, c_in, h_in, w_in, c_out, filter_h, filter_w, stride[0], stride[1],
                       padding[0], padding[1], dilation[0], dilation[1], DTYPES[dtype],
                       1 if has_bias else 0, input_layout, output_layout, weight_layout)


def conv_query(problem: ConvProblem, config: Config | None = None) -> ConvResources:
    res = ConvResources()
    raise_for(lib.tnx_conv2d_query(ctypes.byref(problem),
                                   ctypes.byref(config) if config is not None else None,
                                   ctypes.byref(res)))
    return res


def conv_launch(problem: ConvProblem, config: Config | None, res: ConvResources,
                x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None,
                y: torch.Tensor) -> None:
    """Enqueues tnx_conv2d_forward on torch's current stream of x's device."""
    require_cuda(x, w, y)
    ws = conv_workspace(x.device, res.workspace_bytes) if res.workspace_bytes else None
    idx = x.device.index if x.device.index is not None else torch.cuda.current_device()
    switch = idx != torch.cuda.current_device()
    if switch:
        previous = torch.cuda.current_device()
        torch.cuda.set_device(idx)
    try:
        rc = lib.tnx_conv2d_forward(
            ctypes.byref(problem), ctypes.byref(config) if config is not None else None,
            x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None,
            y.data_ptr(), ws.data_ptr() if ws is not None else None,
            ws.numel() if ws is not None else 0, status_word(x.device).data_ptr(),
            torch.cuda.current_stream(idx).cuda_stream)
    finally:
        if switch:
            torch.cuda.set_device(previous)
    raise_for(rc)


def conv_pack_weights(problem: ConvProblem, weight: torch.Tensor) -> torch.Tensor:
    """The weights in the layout the tcgen05 kernel reads (tnx_conv2d_pack_weights), as a new
    uint8 tensor; enqueued on torch's current stream."""
    require_cuda(weight)
    nbytes = lib.tnx_conv2d_packed_weight_bytes(ctypes.byref(problem))
    if nbytes <= 0:
        raise ValueError("these weights have no packed form (fp32, or an invalid problem)")
    packed = torch.empty(nbytes, dtype=torch.uint8, device=weight.device)
    with torch.cuda.device(weight.device):
        raise_for(lib.tnx_conv2d_pack_weights(ctypes.byref(problem), weight.data_ptr(),
                                              packed.data_ptr(),
                                              torch.cuda.current_stream(weight.device).cuda_stream))
    return packed
