"""Device timing helper with the contract of ``triton.testing.do_bench`` (the function the
reference's tuner and dispatcher call at tritonix/autotune.py:119 and tritonix/dispatcher.py:85):
one run to estimate the cost, warm-up and repeat counts derived from time budgets in
milliseconds, the L2 cache flushed before every timed run, CUDA events per run, mean returned.
"""
from __future__ import annotations

import statistics
from typing import Callable, Sequence

import torch

_L2_FLUSH_BYTES = 256 * 1024 * 1024  # larger than the 126 MB L2 of a B200
_flush_buffers: dict[int, torch.Tensor] = {}


def l2_flush_buffer(device=None) -> torch.Tensor:
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    buf = _flush_buffers.get(idx)
    if buf is None:
        buf = torch.empty(_L2_FLUSH_BYTES, dtype=torch.int8, device=torch.device("cuda", idx))
        _flush_buffers[idx] = buf
    return buf


def _summarise(times: Sequence[float], quantiles, return_mode: str):
    if quantiles is not None:
        ts = torch.tensor(list(times), dtype=torch.float64)
        q = torch.quantile(ts, torch.tensor(list(quantiles), dtype=torch.float64)).tolist()
        return q[0] if len(q) == 1 else q
    if return_mode == "all":
        return list(times)
    fn = {"mean": statistics.fmean, "median": statistics.median, "min": min, "max": max}[return_mode]
    return fn(times)


def do_bench(fn: Callable[[], object], warmup: float = 25, rep: float = 100, quantiles=None,
             return_mode: str = "mean", flush_l2: bool = True):
    """Milliseconds per call of ``fn`` on the current CUDA stream.

    ``warmup`` and ``rep`` are time budgets in milliseconds (not iteration counts).  Exceptions
    raised by ``fn`` (``OutOfResources``, ``ValueError`` ...) propagate from the first call, which
    is what lets the tuner prune or skip a configuration before any time is spent on it.
    """
    if not torch.cuda.is_available():
        raise RuntimeError("do_bench needs a CUDA device")
    fn()
    torch.cuda.synchronize()
    cache = l2_flush_buffer() if flush_l2 else None

    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(5):
        if cache is not None:
            cache.zero_()
        fn()
    end.record()
    torch.cuda.synchronize()
    estimate = max(start.elapsed_time(end) / 5, 1e-6)
    n_warmup = max(1, int(warmup / estimate))
    n_repeat = max(1, int(rep / estimate))

    for _ in range(n_warmup):
        fn()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    for i in range(n_repeat):
        if cache is not None:
            cache.zero_()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    times = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    return _summarise(times, quantiles, return_mode)
