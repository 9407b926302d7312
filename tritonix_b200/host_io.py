"""Row-pipelined execution for operands that live in host memory.

A contraction whose left operand and result sit in (pinned) host memory is bound by the PCIe
copies, not by the kernel.  ``HostRowPipeline`` cuts the rows into chunks and runs three streams
— host-to-device copy, compute (the caller's current stream), device-to-host copy — so that chunk
i+1 is uploaded and chunk i-1 is downloaded while chunk i is computed.  The reference leaves
host/device traffic to the caller; this is a convenience on top of the same kernels.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch


class HostRowPipeline:
    """Reusable buffers and streams for ``out_host[r] = fn(x_host[r])`` over row chunks.

    ``fn(x_dev, out_dev)`` must enqueue its work on torch's current stream and write its result
    for the given rows into ``out_dev``.
    """

    def __init__(self, device: torch.device, in_cols: int, out_cols: int, dtype: torch.dtype,
                 rows_per_chunk: int = 1024, depth: int = 2):
        self.device = torch.device(device)
        self.rows = int(rows_per_chunk)
        self.depth = max(2, int(depth))
        self.x = [torch.empty((self.rows, in_cols), device=self.device, dtype=dtype)
                  for _ in range(self.depth)]
        self.out = [torch.empty((self.rows, out_cols), device=self.device, dtype=dtype)
                    for _ in range(self.depth)]
        self.h2d = torch.cuda.Stream(device=self.device)
        self.d2h = torch.cuda.Stream(device=self.device)
        self.loaded = [torch.cuda.Event() for _ in range(self.depth)]
        self.computed = [torch.cuda.Event() for _ in range(self.depth)]
        self.stored = [torch.cuda.Event() for _ in range(self.depth)]

    def run(self, fn: Callable[[torch.Tensor, torch.Tensor], None], x_host: torch.Tensor,
            out_host: torch.Tensor, before: Optional[Callable[[], None]] = None) -> None:
        """Processes every row of ``x_host``; returns once all work is enqueued.  The caller's
        current stream is made to wait for the last download, so synchronising it is enough.
        ``before()`` runs on the upload stream first (e.g. to upload a right-hand operand)."""
        m = x_host.shape[0]
        compute = torch.cuda.current_stream(self.device)
        self.h2d.wait_stream(compute)
        self.d2h.wait_stream(compute)
        if before is not None:
            with torch.cuda.stream(self.h2d):
                before()
        for i, lo in enumerate(range(0, m, self.rows)):
            hi = min(m, lo + self.rows)
            n, s = hi - lo, i % self.depth
            with torch.cuda.stream(self.h2d):
                if i >= self.depth:
                    self.h2d.wait_event(self.computed[s])   # the kernel that read x[s] is done
                self.x[s][:n].copy_(x_host[lo:hi], non_blocking=True)
                self.loaded[s].record(self.h2d)
            compute.wait_event(self.loaded[s])
            if i >= self.depth:
                compute.wait_event(self.stored[s])           # out[s] has been downloaded
            fn(self.x[s][:n], self.out[s][:n])
            self.computed[s].record(compute)
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(self.computed[s])
                out_host[lo:hi].copy_(self.out[s][:n], non_blocking=True)
                self.stored[s].record(self.d2h)
        compute.wait_stream(self.d2h)
        compute.wait_stream(self.h2d)


_pipelines: dict = {}


def matmul_from_host(a_host: torch.Tensor, b: torch.Tensor, out_host: torch.Tensor,
                     rows_per_chunk: int = 1024, b_device: Optional[torch.Tensor] = None,
                     device: Optional[torch.device] = None,
                     b_upload: Optional[Callable[[torch.Tensor], None]] = None) -> torch.Tensor:
    """``out_host[:] = a_host @ b`` with A and the result in pinned host memory.

    ``b`` may be a device tensor, or a host tensor that is uploaded (into ``b_device`` if given)
    ahead of the first chunk.  ``b_upload(b_device)``, if given, replaces the plain upload of a
    host ``b``: it runs on the upload stream and must leave all of B in ``b_device`` (e.g. ranks
    that hold the same B each upload a slice and all-gather the rest over NVLink).  Work is
    enqueued asynchronously; synchronise the current stream before reading ``out_host``.
    """
    from tritonix_b200.ops import cuda_matmul
    dev = torch.device(device) if device is not None else (
        b.device if b.is_cuda else torch.device("cuda", torch.cuda.current_device()))
    m, k = a_host.shape
    n = b.shape[1]
    key = (dev.index, k, n, a_host.dtype, rows_per_chunk)
    pipe = _pipelines.get(key)
    if pipe is None:
        pipe = _pipelines[key] = HostRowPipeline(dev, k, n, a_host.dtype, rows_per_chunk)
    before = None
    if not b.is_cuda:
        if b_device is None:
            b_device = torch.empty(b.shape, device=dev, dtype=b.dtype)
        b_src, b = b, b_device
        # uploaded on the same stream as A's chunks, so it is complete before the first kernel
        if b_upload is not None:
            before = lambda: b_upload(b_device)  # noqa: E731
        else:
            before = lambda: b_device.copy_(b_src, non_blocking=True)  # noqa: E731

    def step(x_dev, out_dev):
        cuda_matmul(x_dev, b, out=out_dev)

    pipe.run(step, a_host, out_host, before=before)
    return out_host
