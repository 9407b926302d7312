"""Multi-GPU use of the contraction kernels: one process per GPU, ``torch.distributed`` (NCCL
over NVLink) for the single exchange step.  The reference has no multi-device code; the two
layouts here are the ones its kernels shard into naturally.

* Large-M GEMM: rows of A (and of C) are split across ranks, B is replicated, no collective.
* SwiGLU MLP, tensor parallel: gate/up projections are column-parallel (rank r owns hidden
  units [r*F/p, (r+1)*F/p), i.e. interleaved W12 columns [2rF/p, 2(r+1)F/p)), the down
  projection is row-parallel, and ONE all-reduce sums the partial outputs.  The all-reduce is
  cut into row chunks and issued on a side stream so that it overlaps the next chunk's GEMMs.

No kernel of this package reads another GPU's memory; remote data only ever arrives through
the collective into local buffers.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(total: int, rank: int, world: int, multiple: int = 1) -> Tuple[int, int]:
    """[lo, hi) of ``rank``'s contiguous share of ``total`` items, in units of ``multiple``
    (the last ranks get one unit less when it does not divide evenly)."""
    if total % multiple:
        raise ValueError(f"{total} is not a multiple of {multiple}")
    units = total // multiple
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo * multiple, hi * multiple


def shard_rows(a: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rank's row block of A for the M-sharded GEMM (a view, no copy)."""
    lo, hi = shard_bounds(a.shape[0], rank, world)
    return a[lo:hi]


def sharded_matmul(a_rows: torch.Tensor, b: torch.Tensor, matmul_fn: Optional[Callable] = None):
    """C rows of this rank = its A rows times the replicated B.  No communication."""
    if matmul_fn is None:
        from tritonix_b200.ops import cuda_matmul as matmul_fn
    return matmul_fn(a_rows, b)


def shard_mlp_weights(w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, rank: int,
                      world: int, multiple: int = 128):
    """Slices global weights for ``rank`` and interleaves gate/up AFTER slicing, so that a shard
    boundary never separates a (gate_j, up_j) column pair.

    w_gate, w_up: (d_model, d_ff); w_down: (d_ff, d_model).
    Returns (w12_shard (d_model, 2*F_r), w_down_shard (F_r, d_model)).
    """
    d_ff = w_gate.shape[1]
    lo, hi = shard_bounds(d_ff, rank, world, multiple if d_ff % (multiple * world) == 0 else 1)
    g, u = w_gate[:, lo:hi], w_up[:, lo:hi]
    w12 = torch.stack((g, u), dim=2).reshape(g.shape[0], 2 * g.shape[1]).contiguous()
    return w12, w_down[lo:hi].contiguous()


class TensorParallelSwiGLU:
    """y = (silu(x W_gate) * (x W_up)) W_down with the hidden dimension split over the group.

    ``gate_up_fn(x, w12) -> h`` and ``down_fn(h, w_down, out=y_rows)`` (writes the partial
    output into ``out``) default to this package's CUDA kernels; they are parameters so that the partitioning and the chunked
    all-reduce schedule can be exercised by CPU (gloo) ranks in tests.

    ``comm_sms``: the GEMM kernels are persistent (one CTA per SM, nearly all of its shared
    memory), so a collective's kernel cannot slip in beside them; it only gets SMs as GEMM CTAs
    retire.  ``comm_sms > 0`` makes the default kernels leave that many SMs free (grid capped at
    SM count - comm_sms) so that NCCL's all-reduce of chunk i runs while chunk i+1 is computed.
    It pays off only when communication is a large share of the step: on 8 B200, 4 chunks with
    32 SMs left free take 1.48-1.54 ms per 32768-token step against 1.65-1.86 ms with none; with
    16 or 24 SMs NCCL loses bandwidth, and on 2 GPUs the slower GEMMs cost more than is hidden.
    ``None`` (default) picks 32 on 8 or more ranks and 0 otherwise.
    ``gate_up_cfg`` / ``down_cfg`` override the kernel configurations of the default kernels.
    """

    def __init__(self, w12_shard: torch.Tensor, w_down_shard: torch.Tensor,
                 group: Optional[dist.ProcessGroup] = None, chunks=4,
                 gate_up_fn: Optional[Callable] = None, down_fn: Optional[Callable] = None,
                 comm_sms: Optional[int] = None, gate_up_cfg: Optional[dict] = None,
                 down_cfg: Optional[dict] = None):
        if w12_shard.shape[1] != 2 * w_down_shard.shape[0]:
            raise ValueError("w12 shard must have twice as many columns as w_down shard has rows")
        self.w12 = w12_shard
        self.w_down = w_down_shard
        self.group = group
        # an int = that many equal chunks; a sequence of positive weights = chunks of those
        # relative sizes (a small last chunk shortens the one all-reduce nothing overlaps)
        if isinstance(chunks, (list, tuple)):
            self.chunk_weights = [float(w) for w in chunks if float(w) > 0] or [1.0]
            self.chunks = len(self.chunk_weights)
        else:
            self.chunks = max(1, int(chunks))
            self.chunk_weights = [1.0] * self.chunks
        if comm_sms is None:  # measured on 8 B200: 32 SMs left to NCCL; not worth it on fewer ranks
            comm_sms = 32 if self.world_size >= 8 else 0
        self.comm_sms = max(0, int(comm_sms))
        if gate_up_fn is None or down_fn is None:
            default_gate_up, default_down = self._default_kernels(gate_up_cfg, down_cfg)
            gate_up_fn = gate_up_fn or default_gate_up
            down_fn = down_fn or default_down
        self.gate_up_fn = gate_up_fn
        self.down_fn = down_fn
        self._comm_stream = None

    def _default_kernels(self, gate_up_cfg, down_cfg):
        """This package's fused gate/up and down-projection launches, with the grid cap that
        leaves SMs to the collective when there is one."""
        import sys

        import tritonix_b200.ops  # noqa: F401
        from tritonix_b200 import _cabi
        mm = sys.modules["tritonix_b200.ops.matmul"]
        sw = sys.modules["tritonix_b200.ops.swiglu"]
        cap = {}
        if self.world_size > 1 and self.comm_sms > 0 and self.w12.is_cuda:
            with torch.cuda.device(self.w12.device):
                sms = _cabi.lib.tnx_sm_count()
            if sms > self.comm_sms + 2:
                cap = {"max_ctas": (sms - self.comm_sms) // 2 * 2}
        d, two_f = self.w12.shape
        d_out = self.w_down.shape[1]

        def gate_up(x, w12):
            cfg = gate_up_cfg or sw.default_glu_config(x.shape[0], two_f, d)
            return sw._launch_glu(x, w12, {**cfg, **cap}, "silu")

        def down(h, w_down, out):
            cfg = down_cfg or mm.default_config(h.shape[0], d_out, two_f // 2)
            return mm._launch_matmul(h, w_down, {**cfg, **cap}, out)

        return gate_up, down

    @property
    def world_size(self) -> int:
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    def chunk_bounds(self, m: int) -> List[Tuple[int, int]]:
        """Row ranges of the all-reduce chunks: multiples of 256 rows where possible."""
        n = min(self.chunks, max(1, m // 256))
        mult = 256 if m % 256 == 0 else 1
        if len(set(self.chunk_weights[:n])) <= 1:
            return [shard_bounds(m, i, n, mult) for i in range(n)]
        weights = self.chunk_weights[:n]
        total, bounds, lo, acc = sum(weights), [], 0, 0.0
        for i, w in enumerate(weights):
            acc += w
            hi = m if i == n - 1 else min(m, max(lo, int(round(m * acc / total / mult)) * mult))
            if hi > lo:
                bounds.append((lo, hi))
            lo = hi
        return bounds

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        m = x.shape[0]
        y = out if out is not None else torch.empty((m, self.w_down.shape[1]), device=x.device,
                                                    dtype=x.dtype)
        world = self.world_size
        on_gpu = x.is_cuda
        if on_gpu and world > 1 and self._comm_stream is None:
            # high priority: the collective's blocks are placed as soon as SMs are free
            self._comm_stream = torch.cuda.Stream(device=x.device, priority=-1)
        pending = []
        for lo, hi in self.chunk_bounds(m):
            h = self.gate_up_fn(x[lo:hi], self.w12)
            self.down_fn(h, self.w_down, out=y[lo:hi])
            if world == 1:
                continue
            if on_gpu:
                # all-reduce of this chunk runs on the side stream while the main stream
                # computes the next chunk
                ready = torch.cuda.Event()
                ready.record(torch.cuda.current_stream(x.device))
                with torch.cuda.stream(self._comm_stream):
                    self._comm_stream.wait_event(ready)
                    dist.all_reduce(y[lo:hi], op=dist.ReduceOp.SUM, group=self.group)
            else:
                pending.append(dist.all_reduce(y[lo:hi], op=dist.ReduceOp.SUM, group=self.group,
                                               async_op=True))
        if world > 1:
            if on_gpu:
                torch.cuda.current_stream(x.device).wait_stream(self._comm_stream)
            for work in pending:
                work.wait()
        return y

    __call__ = forward


class FusedTensorParallelSwiGLU:
    """The tensor-parallel SwiGLU MLP as ONE kernel per rank and step: the one-launch MLP kernel
    (``tnx_swiglu_mlp``) computes this rank's hidden units and its partial output row tile by row
    tile, and two extra warps of every CTA sum the partial outputs across the ranks as the row
    tiles complete — ``multimem.ld_reduce`` / ``multimem.st`` through an NVLink multicast mapping
    — so the exchange is spread over the whole step and over all SMs instead of following the
    step.  ``tile_split`` crews share one row tile.  No collective library call is made in
    ``forward``.

    The output buffer, the exchange counters and (with ``fp32_partials``) the fp32 partial
    outputs live in symmetric memory
    (``torch.distributed._symmetric_memory``: the same allocation on every rank, bound to one
    multicast object).  ``forward`` returns a view of that buffer: it holds the full result on
    every rank and is overwritten by the next call.  Needs NVSwitch multicast support; when it
    is missing the constructor raises and ``TensorParallelSwiGLU`` (NCCL all-reduce) is the
    alternative.

    ``fp32_partials=True`` keeps every rank's partial output in fp32 until the cross-rank sum
    (one rounding, the single-GPU error at any world size) at twice the NVLink traffic;
    ``False`` (default) rounds the partial outputs to the output type and sums them in place
    with fp32 accumulation in the switch (about two roundings; measured 5.9e-3 against the
    oracle at world size 2 where one GPU gives 2.9e-3, tolerance 8e-3).

    Every rank must call ``forward`` the same number of times with the same token count.
    """

    def __init__(self, w12_shard: torch.Tensor, w_down_shard: torch.Tensor, max_tokens: int,
                 group: Optional[dist.ProcessGroup] = None, tile_split: int = 16,
                 cfg: Optional[dict] = None, fp32_partials: bool = False):
        import torch.distributed._symmetric_memory as symm

        from tritonix_b200 import _cabi
        if w12_shard.shape[1] != 2 * w_down_shard.shape[0]:
            raise ValueError("w12 shard must have twice as many columns as w_down shard has rows")
        self._cabi = _cabi
        self.w12, self.w_down = w12_shard, w_down_shard
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if 256 % self.world:
            raise ValueError("the in-kernel exchange splits 256-row tiles over the ranks: "
                             f"world size {self.world} does not divide 256")
        self.tile_split = int(tile_split)
        self.cfg = dict(cfg or {})
        if "group_m" not in self.cfg:
            # Bands of row tiles share a pass over the weights.  A shard whose weights stay in L2
            # anyway (8-way split of a Llama-3-8B block: 44 MB) gains from shorter bands, whose
            # partial outputs are complete, and exchanged, earlier (8 GPUs: 1.07 ms with bands
            # of 4 against 1.12 ms with 8); larger shards lose more in weight traffic (4 GPUs,
            # 88 MB: 2.11 ms against 2.00 ms).
            weight_bytes = (w12_shard.numel() + w_down_shard.numel()) * w12_shard.element_size()
            self.cfg["group_m"] = 4 if weight_bytes <= 48 * 1024 * 1024 else 8
        self.d_out = w_down_shard.shape[1]
        self.max_tokens = int(max_tokens)
        dev, dtype = w12_shard.device, w12_shard.dtype
        tiles = -(-self.max_tokens // 256)
        self._tiles = tiles
        self._y_bytes = tiles * 256 * self.d_out * dtype.itemsize
        self.fp32_partials = bool(fp32_partials)
        self._part_bytes = tiles * 256 * self.d_out * 4 if self.fp32_partials else 0
        sig_bytes = (tiles + 1) * 4
        total = self._y_bytes + self._part_bytes + -(-sig_bytes // 256) * 256
        import warnings
        with warnings.catch_warnings():  # older releases need the group enabled explicitly;
            warnings.simplefilter("ignore")  # newer ones deprecate the call
            try:
                symm.enable_symm_mem_for_group(self.group.group_name)
            except Exception:
                pass
        self._buf = symm.empty(total, dtype=torch.uint8, device=dev)
        self._handle = symm.rendezvous(self._buf, self.group.group_name)
        mc = int(getattr(self._handle, "multicast_ptr", 0) or 0)
        if mc == 0:
            raise RuntimeError("symmetric memory on this system has no multicast mapping (NVSwitch "
                               "multimem); use TensorParallelSwiGLU (NCCL all-reduce) instead")
        self._mc = mc
        self._epoch = 0
        self.reset()

    def reset(self) -> None:
        """Zeroes the exchange counters on every rank and restarts the call count (collective;
        needed after a call that raised ``DeviceStatusError``)."""
        torch.cuda.synchronize(self._buf.device)
        self._buf[self._y_bytes + self._part_bytes:].zero_()
        torch.cuda.synchronize(self._buf.device)
        self._handle.barrier()
        torch.cuda.synchronize(self._buf.device)
        self._epoch = 0

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        m = x.shape[0]
        if m > self.max_tokens:
            raise ValueError(f"{m} tokens exceed the {self.max_tokens} this instance was sized for")
        cabi = self._cabi
        y = self._buf[:m * self.d_out * x.element_size()].view(x.dtype).view(m, self.d_out)
        if (self._epoch + 1) * self.world >= 2 ** 31:
            self.reset()  # the counters count calls x ranks in 32 bits; every rank gets here at the same call
        self._epoch += 1
        local = self._buf.data_ptr()
        part, sig = self._y_bytes, self._y_bytes + self._part_bytes
        exchange = cabi.MlpExchange(self.world, self.rank, self.tile_split, self._epoch, self._tiles, 0,
                                    self._mc, (local + part) if self.fp32_partials else None,
                                    (self._mc + part) if self.fp32_partials else None,
                                    self._mc + sig, local + sig)
        cabi.launch_mlp(x, self.w12, self.w_down, y, self.cfg, cabi.EPI_GLU_SILU, exchange=exchange)
        return y

    __call__ = forward
