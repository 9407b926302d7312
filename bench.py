#!/usr/bin/env python
"""Benchmark of the dense-contraction path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload all|gemm|splitk|glu|mlp|conv] [--scaling weak|strong]

Headline (`value`): bf16 C = A.B with M = N = K = 8192, entries N(0,1)/sqrt(K), fp32 accumulation,
bf16 output — one step is one pass of the kernel over one such problem.  With N GPUs every rank
owns an 8192-row block of a (8192*N) x 8192 A and a replica of B (row-sharded, no collective):
per-GPU work is fixed, so scaling is "weak".

With the default `--workload all` the same JSON line carries, under "workloads", one entry per
remaining configuration, each measured to the same rules (device-timed value, roofline, e2e,
clocks):
  splitk       fp16 64 x 14336 x 4096, HBM-bound; every GPU runs its own replica
  glu          bf16 fused SwiGLU 8192x4096 . 4096x28672 (interleaved W12); replicas
  mlp          bf16 SwiGLU MLP d=4096, ff=14336, 32768 tokens, tensor parallel over the N GPUs
               with one all-reduce (strong scaling, tokens/s) + parity of sampled rows against the
               CPU oracle, computed outside the timed region
  gemm_strong  (N > 1) the 8192^3 problem itself split along M: 8192/N rows per GPU
and the gemm entry gains "sustained": at least 2 s of back-to-back launches under the power cap.
`--workload X` measures one of them alone (`conv`: bf16 conv2d forward, 64 x 256 x 28 x 28).

`value` is device-timed with the operands resident in HBM; `e2e` is the same metric through the
public API (`tritonix_b200.matmul_from_host`, ...) with the operands in pinned host memory and
the host<->device copies inside the timed region.  "comparators" (N = 1) times, on the same GPU
and operands, cuBLAS through torch.matmul and the reference's own Triton kernel run by
oracle/reference_gpu.py in a process of its own — comparisons only, never a backend.

`--impl reference` times the reference's CPU path for the same workload — tritonix.matmul under
force_backend("pytorch") on host tensors, i.e. torch.matmul on the host cores in fp32
(tritonix/ops/matmul.py:291-293) — through the oracle port, on the full problem for `gemm`.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024

WORKLOADS = {
    "gemm": dict(m=8192, n=8192, k=8192, dtype="bf16",
                 name="gemm_bf16_8192x8192x8192_per_gpu_rows_sharded_B_replicated"),
    "gemm_strong": dict(m=8192, n=8192, k=8192, dtype="bf16",
                        name="gemm_bf16_8192x8192x8192_total_rows_sharded_B_replicated"),
    "splitk": dict(m=64, n=4096, k=14336, dtype="f16", name="splitk_gemm_f16_64x14336x4096"),
    "glu": dict(m=8192, n=28672, k=4096, dtype="bf16",
                name="swiglu_bf16_x8192x4096_w12_4096x28672_interleaved"),
    "mlp": dict(m=32768, d=4096, ff=14336, dtype="bf16",
                name="swiglu_mlp_bf16_d4096_ff14336_tokens32768_tensor_parallel"),
    # a ResNet-50 stage-3 3x3 layer; m, n, k are the implicit GEMM's sizes
    "conv": dict(batch=64, c_in=256, h=28, w=28, c_out=256, r=3, s=3, stride=1, pad=1,
                 m=64 * 28 * 28, n=256, k=256 * 9, dtype="bf16",
                 name="conv2d_fwd_bf16_nchw_64x256x28x28_w256x256x3x3_s1_p1_per_gpu_batch_sharded"),
}

# tile_n 512 = two 256-column tiles per CTA pair fed by one stream of A: fewer operand bytes per
# flop, at the price of an epilogue that is only partly hidden; it pays for long K
GEMM_CFG = {"kernel": "tcgen05", "tile_n": 512, "tile_k": 64, "stages": 4, "cta_group": 2, "group_m": 8,
            "tile_order": "serpentine"}
GEMM_CFG_SHORT_K = {"kernel": "tcgen05", "tile_n": 256, "tile_k": 128, "stages": 3, "cta_group": 2, "group_m": 16}
SPLITK_CFG = {"kernel": "tcgen05", "tile_n": 128, "tile_k": 128, "stages": 4, "cta_group": 1, "split_k": 4}
GLU_CFG = {"kernel": "tcgen05", "tile_n": 256, "tile_k": 128, "stages": 3, "cta_group": 2, "group_m": 16}
CONFIG_SOURCE = "fixed in bench.py (the configurations that measured best on a B200)"

# DRAM traffic of the dominant kernel per launch, from the ncu captures summarised under
# profiles/ (None until a capture of that workload exists).
NCU_TRAFFIC_BYTES = {"gemm": 1_045_709_568, "gemm_strong": None, "splitk": 124_318_464,
                     "glu": 885_355_520, "mlp": None, "conv": 26_989_568}

# swiglu_mlp_kernel at 8192 tokens (d_model 4096, d_ff 14336): dram read + written per launch
MLP_ONE_LAUNCH_TRAFFIC_8192 = 2_526_534_000 + 299_845_376

# The reference's Triton kernels are timed with configurations from its own search space
# (tritonix/ops/matmul.py:33-38; the hand-picked list of tritonix/utils/triton.py:34-53 tops
# out at 128 x 128 x 64 tiles); the best of these is reported.
TRITON_REF_CONFIGS = [
    dict(block_m=128, block_n=128, block_k=64, group_m=8, num_stages=3, num_warps=8),
    dict(block_m=128, block_n=128, block_k=64, group_m=8, num_stages=4, num_warps=4),
    dict(block_m=128, block_n=128, block_k=32, group_m=8, num_stages=4, num_warps=4),
    dict(block_m=128, block_n=64, block_k=64, group_m=8, num_stages=4, num_warps=4),
]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], burst=p["bf16_tflops"], sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, burst=1590.0, sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML while a timed region runs."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.samples, self.power, self.reasons, self.max_mhz = [], [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
            self._period = period_s
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        names = {getattr(nv, n): n for n in dir(nv) if n.startswith("nvmlClocksThrottleReason")
                 and isinstance(getattr(nv, n), int)}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if bit and mask & bit and name not in ("nvmlClocksThrottleReasonAll",):
                        self.reasons.add(name.replace("nvmlClocksThrottleReason", ""))
            except Exception:
                pass
            self._stop.wait(self._period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        pretty = {"GpuIdle": "gpu_idle", "ApplicationsClocksSetting": "applications_clocks_setting",
                  "SwPowerCap": "sw_power_cap", "HwSlowdown": "hw_slowdown", "SyncBoost": "sync_boost",
                  "SwThermalSlowdown": "sw_thermal_slowdown", "HwThermalSlowdown": "hw_thermal_slowdown",
                  "HwPowerBrakeSlowdown": "hw_power_brake_slowdown", "DisplayClockSetting": "display_clock_setting",
                  "None": "none"}
        reasons = sorted(pretty.get(r, r) for r in self.reasons if r not in ("None", "GpuIdle"))
        out = {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
               "reasons": reasons, "samples": len(s)}
        if self.power:
            out["power_w_max"] = round(max(self.power), 1)
        return out


class Dist:
    """The few collective helpers the timing needs; no-ops on one GPU."""

    def __init__(self, world, dev):
        self.world, self.dev = world, dev

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()

    def max(self, value):
        if self.world == 1:
            return value
        import torch.distributed as dist
        t = torch.tensor([value], device=self.dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())


# ---------------------------------------------------------------------------------------------
# workloads: each setup returns (step_fn, e2e_step_fn, work dict)
# ---------------------------------------------------------------------------------------------
def torch_dtype(name):
    return {"bf16": torch.bfloat16, "f16": torch.float16}[name]


def randn(shape, dtype, device, seed, scale):
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(shape, device=device, generator=g, dtype=torch.float32) * scale).to(dtype)


def gemm_cfg_for_rows(m, n):
    """Double tiles unless their last wave over the 74 CTA pairs is much emptier than that of
    single tiles (4096 rows: 256 double tiles = 3.46 waves against 512 = 6.92)."""
    def wave_fill(tiles):
        return tiles / (-(-tiles // 74) * 74)
    rows = -(-m // 256)
    double, single = rows * -(-n // 512), rows * -(-n // 256)
    return GEMM_CFG if wave_fill(double) >= wave_fill(single) - 0.05 else GEMM_CFG_SHORT_K


def setup_contraction(workload, rank, world, dev):
    """gemm / gemm_strong / splitk / glu: one kernel launch per step."""
    from tritonix_b200 import _cabi
    import tritonix_b200 as tnx
    w = WORKLOADS[workload]
    m, n, k, dt = w["m"], w["n"], w["k"], torch_dtype(w["dtype"])
    if workload == "gemm_strong":
        m = m // world  # this rank's rows of the one 8192^3 problem
    glu = workload == "glu"
    epi = _cabi.EPI_GLU_SILU if glu else _cabi.EPI_NONE
    n_out = n // 2 if epi else n
    cfg = {"gemm": GEMM_CFG, "gemm_strong": gemm_cfg_for_rows(m, n), "splitk": SPLITK_CFG,
           "glu": GLU_CFG}[workload]
    algo_bytes = (m * k + k * n + m * n_out) * 2
    # operands smaller than L2 are rotated through enough copies to defeat it
    copies = 1 if algo_bytes > 2 * L2_BYTES else -(-3 * L2_BYTES // algo_bytes)
    a_scale = 1.0 if glu else k ** -0.5
    b_scale = 0.02 if glu else k ** -0.5
    a_dev = [randn((m, k), dt, dev, 1000 * rank + i, a_scale) for i in range(copies)]
    b_dev = [randn((k, n), dt, dev, 1 + 7 * i, b_scale) for i in range(copies)]  # B is replicated
    c_dev = torch.empty((m, n_out), device=dev, dtype=dt)
    state = {"i": 0}

    def step():
        i = state["i"] % copies
        state["i"] += 1
        _cabi.launch(a_dev[i], b_dev[i], c_dev, cfg, epi)

    # end to end through the public API, operands in pinned host memory
    a_host = a_dev[0].cpu().pin_memory()
    b_host = b_dev[0].cpu().pin_memory()
    c_host = torch.empty((m, n_out), dtype=dt).pin_memory()
    a_in, b_in = torch.empty_like(a_dev[0]), torch.empty_like(b_dev[0])
    mm = sys.modules["tritonix_b200.ops.matmul"]
    sw = sys.modules["tritonix_b200.ops.swiglu"]
    rows = min(1024, m)
    mm._matmul_cfg[(m, n, k)] = dict(GEMM_CFG)
    mm._matmul_cfg[(rows, n, k)] = dict(GEMM_CFG)   # row chunks of the host pipeline
    sw._glu_cfg[(rows, n, k)] = dict(GLU_CFG)
    mm._splitk_cfg[(m, n, k, SPLITK_CFG["split_k"])] = dict(SPLITK_CFG)
    sw._glu_cfg[(m, n, k)] = dict(GLU_CFG)
    pipe = tnx.HostRowPipeline(dev, k, n_out, dt, rows_per_chunk=rows) if glu else None

    # B is the same on every rank: on several GPUs each rank uploads 1/N of its rows and the
    # ranks all-gather the rest over NVLink, instead of N uploads of all of B through one host
    share_b = world > 1 and workload in ("gemm", "gemm_strong") and k % world == 0
    b_upload = None
    if share_b:
        import torch.distributed as dist
        rows_b = k // world
        b_slice_host = b_host[rank * rows_b:(rank + 1) * rows_b]

        def b_upload(b_device):
            mine = b_device[rank * rows_b:(rank + 1) * rows_b]
            mine.copy_(b_slice_host, non_blocking=True)
            dist.all_gather_into_tensor(b_device, mine)

    def e2e_step():
        # every step uploads A and B from pinned host memory and downloads the result; for the
        # large workloads the rows of A / C are pipelined against the kernel (public helpers)
        if workload in ("gemm", "gemm_strong"):
            tnx.matmul_from_host(a_host, b_host, c_host, rows_per_chunk=rows, b_device=b_in,
                                 b_upload=b_upload)
        elif glu:
            pipe.run(lambda xd, od: tnx.swiglu(xd, b_in, out=od), a_host, c_host,
                     before=lambda: b_in.copy_(b_host, non_blocking=True))
        else:
            a_in.copy_(a_host, non_blocking=True)
            b_in.copy_(b_host, non_blocking=True)
            out = tnx.matmul_splitk(a_in, b_in, split_k=SPLITK_CFG["split_k"])
            c_host.copy_(out, non_blocking=True)

    def e2e_check():
        """The end-to-end result (host buffer) against the device-resident one of the same
        operands: same kernel, same K order, so sampled rows must agree bit for bit."""
        if copies != 1 or workload not in ("gemm", "gemm_strong"):
            return None
        rows_s = sorted({0, m // 3, m - 1})
        return bool(torch.equal(c_host[rows_s], c_dev[rows_s].cpu()))

    work = dict(flops=2.0 * m * n * k, bytes=float(algo_bytes), units=None, launches=1, e2e_check=e2e_check,
                h2d=a_host.numel() * 2 + b_host.numel() * 2 // (world if share_b else 1),
                d2h=c_host.numel() * 2, copies=copies,
                cfg=cfg, operands=(a_dev, b_dev, c_dev), shape=(m, n, k), share_b=share_b)
    return step, e2e_step, work


def setup_conv(rank, world, dev, fixed_cfg=None):
    """conv: conv2d_forward through the public API on NCHW tensors (the reference's layout), so a
    step is the input repack, the implicit-GEMM kernel and the output repack; the weights are
    packed once (they do not change between steps)."""
    import tritonix_b200 as tnx
    w = WORKLOADS["conv"]
    dt = torch_dtype(w["dtype"])
    xshape = (w["batch"], w["c_in"], w["h"], w["w"])
    wt = randn((w["c_out"], w["c_in"], w["r"], w["s"]), dt, dev, 1, (w["c_in"] * w["r"] * w["s"]) ** -0.5)
    x_bytes = w["batch"] * w["c_in"] * w["h"] * w["w"] * 2
    algo_bytes = x_bytes + wt.numel() * 2 + w["m"] * w["n"] * 2
    copies = -(-3 * L2_BYTES // algo_bytes)
    xs = [randn(xshape, dt, dev, 1000 * rank + i, 1.0) for i in range(copies)]
    state = {"i": 0, "out": None}
    kw = dict(stride=w["stride"], padding=w["pad"])
    # --cfg fixes the configuration: no first-call tuning (e.g. for a profiler run)
    step_kw = dict(kw, config=dict(fixed_cfg)) if fixed_cfg else kw

    def step():
        i = state["i"] % copies
        state["i"] += 1
        state["out"] = tnx.conv2d_forward(xs[i], wt, None, **step_kw)

    step()  # first call: picks the configuration and packs the weights
    torch.cuda.synchronize(dev)
    x_host = xs[0].cpu().pin_memory()
    y_host = torch.empty(tuple(state["out"].shape), dtype=dt).pin_memory()
    x_in = torch.empty_like(xs[0])

    def e2e_step():
        x_in.copy_(x_host, non_blocking=True)
        y_host.copy_(tnx.conv2d_forward(x_in, wt, None, **step_kw), non_blocking=True)

    cfg = dict(fixed_cfg) if fixed_cfg else dict(next(iter(
        sys.modules["tritonix_b200.ops.conv2d"]._CONV_FWD_CONFIG_CACHE.values())))

    # the implicit-GEMM kernel alone (for the roofline): channels_last tensors need no repacking
    xs_cl = [x.contiguous(memory_format=torch.channels_last) for x in xs]

    def kernel_step():
        i = state["i"] % copies
        state["i"] += 1
        state["out"] = tnx.conv2d_forward(xs_cl[i], wt, None, config=cfg, **kw)

    work = dict(flops=2.0 * w["m"] * w["n"] * w["k"], bytes=float(algo_bytes), units=None, launches=3,
                h2d=x_host.numel() * 2, d2h=y_host.numel() * 2, copies=copies, cfg=cfg,
                kernel_step=kernel_step)
    return step, e2e_step, work


def _mlp_weight_blocks(dev, lo, hi):
    """Hidden units [lo, hi) of the global weights, generated per 128-unit block from
    (seed, block) so that every tensor-parallel degree slices the same global matrices."""
    d, dt = WORKLOADS["mlp"]["d"], torch.bfloat16
    blocks = range(lo // 128, hi // 128)
    wg = torch.cat([randn((d, 128), dt, dev, 10_000 + j, 0.02) for j in blocks], 1)
    wu = torch.cat([randn((d, 128), dt, dev, 20_000 + j, 0.02) for j in blocks], 1)
    wd = torch.cat([randn((128, d), dt, dev, 30_000 + j, 0.02) for j in blocks], 0)
    return wg, wu, wd


def setup_mlp(rank, world, dev, chunks=0, comm_sms=-1, mode="auto", tile_split=16, band=0, tokens=0,
              fp32_partials=False):
    """SwiGLU MLP, tensor parallel: hidden units split over the ranks (column-parallel gate/up,
    row-parallel down projection), partial outputs summed across the ranks.  Global weights come
    from fixed seeds and are sliced, so every world size computes the same function.
    Two implementations: "two_launch" = fused gate/up kernel + down GEMM per row chunk with a
    chunked NCCL all-reduce on a side stream; "one_launch" = the one-launch MLP kernel, which on
    several GPUs also sums the partial outputs itself (multimem over NVLink) while computing."""
    import tritonix_b200 as tnx
    from tritonix_b200.distributed import (FusedTensorParallelSwiGLU, TensorParallelSwiGLU,
                                           shard_bounds)
    comm_sms = (32 if world >= 8 else 0) if comm_sms < 0 else comm_sms
    w = WORKLOADS["mlp"]
    m, d, ff, dt = (tokens or w["m"]), w["d"], w["ff"], torch.bfloat16
    lo, hi = shard_bounds(ff, rank, world, 128)
    fr = hi - lo
    wg, wu, wd = _mlp_weight_blocks(dev, lo, hi)  # slice-then-interleave
    w12 = torch.stack((wg, wu), 2).reshape(d, 2 * fr).contiguous()
    del wg, wu
    x = randn((m, d), dt, dev, 5, 1.0)
    down_cfg = GEMM_CFG if fr >= 6144 else GEMM_CFG_SHORT_K   # K of the down projection = this rank's hidden units
    mlp = TensorParallelSwiGLU(
        w12, wd, chunks=chunks if (isinstance(chunks, list) or chunks > 0) else (1 if world == 1 else 4),
        comm_sms=comm_sms, gate_up_cfg=GLU_CFG, down_cfg=down_cfg)
    state = {}
    if band <= 0:  # bands of 8 row tiles; 4 where a rank's weights stay in L2 anyway (see the class)
        band = 4 if 3 * d * fr * 2 <= 48 * 1024 * 1024 else 8
    fused_cfg = {"tile_k": 128, "stages": 3, "group_m": band}
    fused = None
    fused_note = None
    if world > 1:
        try:
            fused = FusedTensorParallelSwiGLU(w12, wd, max_tokens=m, tile_split=tile_split, cfg=fused_cfg,
                                              fp32_partials=fp32_partials)
        except Exception as exc:  # no multicast mapping on this system: the NCCL path remains
            fused_note = f"{type(exc).__name__}: {exc}"[:200]

    def step_two_launch():
        state["y"] = mlp(x)

    def step_one_launch():
        if world > 1:
            state["y"] = fused(x)
        else:
            state["y"] = tnx.swiglu_mlp(x, w12, wd, fused=True, fused_cfg=fused_cfg)

    chosen_by = None
    if world > 1 and fused is not None and mode == "auto":
        # Before the in-kernel exchange is given the headline: one trial step whose result must
        # agree with the NCCL implementation's on every rank, then a short calibration of both.
        import torch.distributed as dist
        ok = torch.ones(1, device=dev)
        failure = None
        torch.cuda.synchronize(dev)
        dist.barrier()  # the ranks enter the first call together: its cross-rank waits are bounded
        try:
            y_one = fused(x).clone()
            torch.cuda.synchronize(dev)
            tnx.check_status(dev)
        except Exception as exc:
            failure = exc
        y_two = mlp(x)  # (every rank, whatever happened above: it holds a collective)
        torch.cuda.synchronize(dev)
        if failure is None:
            diff = (y_one.float() - y_two.float()).abs().max().item() / max(y_two.float().abs().max().item(), 1e-30)
            if not diff <= 1.5e-2:
                failure = RuntimeError("trial step differs from the NCCL implementation by %.3g" % diff)
        if failure is not None:
            ok.zero_()
            fused_note = f"trial step failed on rank {rank}: {type(failure).__name__}: {failure}"[:240]
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            fused = None
            fused_note = fused_note or "trial step failed on another rank"
        else:
            t_cal = {}
            for name, fn in (("one_launch", lambda: fused(x)), ("two_launch", lambda: mlp(x))):
                t = torch.tensor([time_steps(fn, 5, 2, dist.barrier)], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                t_cal[name] = t.item() / 5
            mode = min(t_cal, key=t_cal.get)
            chosen_by = "calibration of 5 steps each: " + ", ".join("%s %.3f ms" % kv for kv in sorted(t_cal.items()))
    one_launch_ok = world == 1 or fused is not None
    if mode == "auto":  # one GPU: two launches measure 5-9 % faster from the same rest
        mode = "one_launch" if (world > 1 and fused is not None) else "two_launch"
    if mode == "one_launch" and not one_launch_ok:
        raise RuntimeError("the one-launch tensor-parallel MLP is unavailable: " + str(fused_note))
    step = step_one_launch if mode == "one_launch" else step_two_launch
    other = None
    if mode == "one_launch":
        other = ("two_launch", step_two_launch)
    elif one_launch_ok:
        other = ("one_launch", step_one_launch)

    x_host = x.cpu().pin_memory()
    y_host = torch.empty((m, d), dtype=dt).pin_memory()
    pipe = tnx.HostRowPipeline(dev, d, d, dt, rows_per_chunk=4096)
    chunk_mlp = TensorParallelSwiGLU(w12, wd, chunks=1, comm_sms=comm_sms, gate_up_cfg=GLU_CFG,
                                     down_cfg=down_cfg)

    e2e_rows = 4096
    share_io = world > 1 and e2e_rows % world == 0 and m % e2e_rows == 0
    if share_io:
        # x and y are the same on every rank: each rank uploads 1/N of the rows of every chunk
        # (the ranks all-gather the chunk over NVLink) and downloads 1/N of the chunk's result,
        # instead of N copies of both crossing the one host's PCIe links
        import torch.distributed as dist
        per = e2e_rows // world
        x_host = x.view(m // e2e_rows, world, per, d)[:, rank].reshape(-1, d).cpu().pin_memory()
        y_host = torch.empty((m // world, d), dtype=dt).pin_memory()
        pipe = tnx.HostRowPipeline(dev, d, d, dt, rows_per_chunk=per)
        x_full = torch.empty((e2e_rows, d), device=dev, dtype=dt)
        y_full = torch.empty((e2e_rows, d), device=dev, dtype=dt)

        def chunk_fn(xd, yd):
            dist.all_gather_into_tensor(x_full, xd)
            chunk_mlp(x_full, out=y_full)
            yd.copy_(y_full[rank * per:(rank + 1) * per])
    else:
        def chunk_fn(xd, yd):
            chunk_mlp(xd, out=yd)

    def e2e_step():
        # rows of x stream in, rows of y stream out, 4096 rows (one all-reduce) at a time
        pipe.run(chunk_fn, x_host, y_host)

    def e2e_check():
        """Sampled rows of the end-to-end result against the device-timed implementation's
        (another chunking or another implementation of the same function: not bit-equal)."""
        if "y" not in state:
            return None
        if share_io:
            mine = [c * e2e_rows + rank * per + r for c in (0, m // e2e_rows - 1) for r in (0, per - 1)]
            got = y_host.view(m // e2e_rows, per, d)[[0, 0, -1, -1], [0, per - 1, 0, per - 1]].float()
        else:
            mine = [0, m // 2, m - 1]
            got = y_host[mine].float()
        want = state["y"][mine].float().cpu()
        return bool(((got - want).abs().max() / want.abs().max().clamp_min(1e-30)).item() <= 1.5e-2)

    def parity():
        """max|err|/max|ref| of sampled tokens of the last step's output against the CPU oracle
        applied to the GLOBAL weights (rank 0 rebuilds them; outside any timed region)."""
        from oracle import contraction as O
        rows = sorted(set([0, m - 1] + torch.randint(0, m, (14,), generator=torch.Generator().manual_seed(3)).tolist()))
        y_rows = state["y"][rows].cpu()
        if rank != 0:
            return None
        g, u, dn = _mlp_weight_blocks(dev, 0, ff)
        w12_cpu = torch.stack((g, u), 2).reshape(d, 2 * ff).cpu()
        dn_cpu = dn.cpu()
        del g, u, dn
        ref = O.swiglu_mlp_oracle(x[rows].cpu(), w12_cpu, dn_cpu, out_dtype=torch.float32,
                                  hidden_dtype=torch.bfloat16)
        return O.rel_err(y_rows, ref)

    flops = 2.0 * m * d * (2 * ff) + 2.0 * m * ff * d
    nchunks = len(mlp.chunk_bounds(m))
    if mode == "one_launch":
        cfg = {"one_launch": dict(fused_cfg, tile_m=256, tile_n=256, cta_group=2)}
        launches = 1
        exchange = ("inside the kernel: %s partial outputs summed with multimem.ld_reduce / multimem.st per "
                    "256-row tile by two extra warps of every CTA, %d crews per tile"
                    % ("fp32" if fp32_partials else "bf16", tile_split)) \
            if world > 1 else "none (one GPU)"
    else:
        cfg = {"gate_up": GLU_CFG, "down": down_cfg}
        launches = 2 * nchunks
        exchange = ("NCCL all-reduce per row chunk on a side stream (%d chunks, %d SMs left to it)"
                    % (nchunks, comm_sms)) if world > 1 else "none (one GPU)"
    work = dict(flops=flops, bytes=None, units=float(m), launches=launches, h2d=x_host.numel() * 2,
                d2h=y_host.numel() * 2, copies=1, cfg=cfg, chunks=nchunks, comm_sms=comm_sms,
                e2e_check=e2e_check, share_io=share_io,
                parity=parity, mode=mode, exchange=exchange, other=other, fused_note=fused_note,
                chosen_by=chosen_by)
    return step, e2e_step, work


# ---------------------------------------------------------------------------------------------
def time_steps(fn, steps, warmup, barrier, graph=False):
    """Device time of exactly `steps` calls of fn.  With graph=True the `steps` launches are
    captured once into a CUDA graph (the way a decode loop issues a short, launch-latency-bound
    kernel) and the timed region is one replay of that graph."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(steps):
                    fn()
            g.replay()  # warm-up replay
            torch.cuda.synchronize()
            barrier()
            start.record(side)
            g.replay()
            end.record(side)
        torch.cuda.synchronize()
        barrier()
        return start.elapsed_time(end)
    barrier()
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    barrier()
    return start.elapsed_time(end)  # ms, on the launching (current) stream


def sustained_leg(step, flops, local_rank, seconds, peaks):
    """At least `seconds` of back-to-back launches: the chip settles at the clock its power cap
    allows.  Launches are issued in batches sized from a first estimate; the timed region is the
    whole run (CUDA events), the clock is NVML-sampled during it."""
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        step()
    e1.record()
    e1.synchronize()
    per = max(e0.elapsed_time(e1) / 10, 1e-3)
    launches = int(seconds * 1000.0 / per * 1.05) + 1
    with ClockSampler(local_rank, period_s=0.02) as clocks:
        e0.record()
        for _ in range(launches):
            step()
        e1.record()
        e1.synchronize()
    ms = e0.elapsed_time(e1)
    c = clocks.summary()
    tf = flops * launches / (ms * 1e-3) / 1e12
    ms_launch = ms / launches
    return {"seconds": ms * 1e-3, "launches": launches, "ms_per_launch": ms_launch, "value": tf,
            "unit": "TFLOP/s", "peak": peaks["sustained"], "frac": tf / peaks["sustained"],
            "peak_source": peaks["source"] + " sustained cuBLAS bf16", "clocks": c,
            "ms_x_mhz": ms_launch * c["sm_mhz"] if c.get("sm_mhz") else None}


def metric_of(workload):
    if workload == "mlp":
        return "SwiGLU MLP tokens/s", "tokens/s"
    if workload == "conv":
        return "conv2d forward TFLOP/s", "TFLOP/s"
    return "GEMM TFLOP/s", "TFLOP/s"


def to_metric(workload, work_flops, units, ms):
    if workload == "mlp":
        return units / (ms * 1e-3)
    return work_flops / (ms * 1e-3) / 1e12


def measure(workload, args, rank, local_rank, world, dev, D, peaks):
    """One workload, measured to the contract's rules.  Returns the entry (rank 0's view)."""
    import tritonix_b200 as tnx
    if workload == "mlp":
        chunks = [float(v) for v in args.chunk_weights.split(",")] if args.chunk_weights else args.chunks
        step, e2e_step, work = setup_mlp(rank, world, dev, chunks, args.comm_sms, args.mlp_mode,
                                         args.tile_split, args.mlp_band, args.mlp_tokens, args.fp32_partials)
    elif workload == "conv":
        step, e2e_step, work = setup_conv(rank, world, dev, json.loads(args.cfg) if args.cfg else None)
    else:
        step, e2e_step, work = setup_contraction(workload, rank, world, dev)

    # ---- device-timed value (operands resident in HBM)
    use_graph = args.launch == "graph" or (args.launch == "auto" and workload == "splitk")
    if workload == "mlp":
        torch.cuda.synchronize()
        time.sleep(1.0)  # (see the variants below: same rest before either implementation is timed)
    with ClockSampler(local_rank) as clocks:
        ms_total = time_steps(step, args.steps, args.warmup, D.barrier, graph=use_graph)
    tnx.check_status(dev)
    ms_total = D.max(ms_total)
    ms_step = ms_total / args.steps

    # ---- end to end through the public API, host buffers
    ms_e2e = None
    if not args.no_e2e:
        e2e_steps = max(3, min(args.steps, 10))
        ms_e2e = D.max(time_steps(e2e_step, e2e_steps, 3, D.barrier)) / e2e_steps
        tnx.check_status(dev)

    e2e_ok = None
    if ms_e2e is not None and work.get("e2e_check") is not None:
        torch.cuda.synchronize(dev)
        e2e_ok = work["e2e_check"]()
    strong = workload in ("mlp", "gemm_strong")
    # weak scaling: every rank does the whole per-GPU problem; gemm_strong: each rank 1/N of it
    scale = 1 if workload == "mlp" else world
    metric, unit = metric_of(workload)
    units = work["units"]
    value = to_metric(workload, work["flops"] * scale, units, ms_step)
    e2e_value = to_metric(workload, work["flops"] * scale, units, ms_e2e) if ms_e2e else None

    # ---- roofline of the dominant kernel (per launch, per GPU)
    if workload == "splitk":
        achieved = work["bytes"] / (ms_step * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                "frac": achieved / peaks["hbm"], "traffic": NCU_TRAFFIC_BYTES["splitk"],
                "peak_source": peaks["source"] + " copy bandwidth",
                "frac_of_nominal_8000": achieved / 8000.0}
    else:
        per_gpu_flops = work["flops"] / (world if workload == "mlp" else 1)
        ms_kernel = ms_step
        if work.get("kernel_step") is not None:
            # a step has several launches: time the dominant kernel on its own
            ms_kernel = D.max(time_steps(work["kernel_step"], args.steps, args.warmup,
                                         D.barrier, graph=True)) / args.steps
            tnx.check_status(dev)
        achieved = per_gpu_flops / (ms_kernel * 1e-3) / 1e12
        long_run = ms_total > 1000.0
        peak = peaks["sustained"] if long_run else peaks["burst"]
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES[workload],
                "peak_source": peaks["source"] + (" sustained" if long_run else " burst") + " cuBLAS bf16",
                "frac_of_nominal_2250": achieved / 2250.0}
        if workload == "mlp":
            roof["note"] = ("whole step (fused gate/up GEMM + down GEMM"
                            + (" + cross-rank sum" if world > 1 else "") + ") against the tensor peak")
            if world == 1:
                # captures exist for a quarter of the tokens (8192); traffic grows with the tokens
                scale_m = work["units"] / 8192.0
                if work["mode"] == "one_launch":
                    roof["traffic"] = int(MLP_ONE_LAUNCH_TRAFFIC_8192 * scale_m)
                    roof["traffic_note"] = "swiglu_mlp_kernel captured at 8192 tokens, scaled by the tokens"
                else:
                    roof["traffic"] = int(NCU_TRAFFIC_BYTES["glu"] * scale_m)
                    roof["traffic_note"] = ("dominant kernel (fused gate/up GEMM) captured at 8192 tokens "
                                            "(the glu workload), scaled by the tokens")
        if work.get("kernel_step") is not None:
            roof["kernel_ms"] = ms_kernel
            roof["note"] = ("dominant kernel timed alone on channels_last tensors, launches replayed "
                            "as one CUDA graph; a step on NCHW tensors adds the two repacking passes")

    parallelism = {"mlp": "tp%d", "conv": "batch_sharded_x%d", "splitk": "replicas_x%d",
                   "glu": "replicas_x%d"}.get(workload, "rows_sharded_x%d") % world
    entry = {
        "metric": metric, "value": value, "unit": unit, "ms_per_step": ms_step,
        "scaling": "strong" if strong else "weak", "dtype": WORKLOADS[workload]["dtype"],
        "config": {"workload": WORKLOADS[workload]["name"], "kernel_config": work["cfg"],
                   "kernel_config_source": CONFIG_SOURCE,
                   **({"implementation": work["mode"], "exchange": work["exchange"]}
                      if workload == "mlp" else {}),
                   **({"implementation_chosen_by": work["chosen_by"]}
                      if workload == "mlp" and work.get("chosen_by") else {}),
                   **({"tokens": args.mlp_tokens} if workload == "mlp" and args.mlp_tokens else {}),
                   **({"allreduce_chunks": work["chunks"], "comm_sms": work["comm_sms"]}
                      if workload == "mlp" and world > 1 and work["mode"] == "two_launch" else {}),
                   "parallelism": parallelism,
                   "launch": "cuda_graph_of_%d_steps" % args.steps if use_graph else "eager",
                   "l2": ("operands rotate through %d copies (> 3x L2)" % work["copies"]) if work["copies"] > 1
                   else "operands exceed the 126 MB L2"},
        "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": work["h2d"],
                "d2h_bytes_per_step": work["d2h"], "ms_per_step": ms_e2e,
                **({("agrees_with_device_result" if workload == "mlp" else "equals_device_result"): e2e_ok}
                   if e2e_ok is not None else {}),
                **({"note": "bytes per rank; B is identical on every rank: each uploads 1/%d of it "
                            "and the ranks all-gather the rest over NVLink" % world}
                   if work.get("share_b") else {}),
                **({"note": "bytes per rank; x and y are identical on every rank: each uploads 1/%d of "
                            "every 4096-row chunk (all-gathered over NVLink) and downloads 1/%d of its "
                            "result" % (world, world)}
                   if work.get("share_io") else {})},
        "gpu_launches": work["launches"] * args.steps,
        "clocks": clocks.summary(),
        "roofline": roof,
    }
    if workload == "mlp" and work["other"] is not None:
        # the other implementation of the same step, timed the same way (a comparison: `value`
        # is the implementation named in config.implementation)
        name, other_step = work["other"]
        time.sleep(1.0)  # both implementations start from a GPU that has had a moment to cool
        ms_other = D.max(time_steps(other_step, args.steps, args.warmup, D.barrier)) / args.steps
        tnx.check_status(dev)
        entry["variants"] = {work["mode"]: {"ms_per_step": ms_step, "value": value},
                             name: {"ms_per_step": ms_other, "value": units / (ms_other * 1e-3)}}
    if workload == "mlp" and work.get("fused_note"):
        entry["one_launch_unavailable"] = work["fused_note"]
    if workload == "mlp":
        step()  # one more step outside any timed region; its output is what parity checks
        torch.cuda.synchronize(dev)
        err = work["parity"]()
        if err is not None:
            entry["parity_err"] = err
            entry["parity"] = ("max|err|/max|ref| over 16 sampled tokens against the CPU oracle "
                               "(fp32, intermediate rounded to bf16) on the global weights; tolerance 8e-3")
        tnx.check_status(dev)
    if workload == "gemm" and not args.no_sustained:
        entry["sustained"] = sustained_leg(step, work["flops"], local_rank, args.sustained_seconds, peaks)
        tnx.check_status(dev)
    if workload == "gemm" and world == 1 and not args.no_drop_in:
        entry["drop_in"] = drop_in_leg(work, args, dev)
    if workload in ("gemm", "glu", "splitk") and world == 1 and rank == 0 and not args.no_comparators:
        entry["comparators"] = comparators(workload, work, args, dev)
    return entry


def drop_in_leg(work, args, dev):
    """The call a user of the reference makes — `matmul(a, b)` with nothing configured — on the
    same operands: its first call tunes (seeded grid search with out-of-resources pruning, no
    disk cache), later calls go through the dispatcher to the tuned kernel and allocate C."""
    import tritonix_b200 as tnx
    mm = sys.modules["tritonix_b200.ops.matmul"]
    a_all, b_all, _ = work["operands"]
    a, b = a_all[0], b_all[0]
    m, n, k = work["shape"]
    keep = {key: os.environ.get(key) for key in ("TRITONIX_B200_TUNE_CACHE", "TRITONIX_B200_TUNE")}
    os.environ["TRITONIX_B200_TUNE_CACHE"], os.environ["TRITONIX_B200_TUNE"] = "0", "1"
    mm._matmul_cfg.pop((m, n, k), None)
    mm._FAST_MATMUL.clear()
    tnx.matmul.clear_cache()
    try:
        t0 = time.perf_counter()
        tnx.matmul(a, b)
        torch.cuda.synchronize(dev)
        first = time.perf_counter() - t0
        cfg = dict(mm._matmul_cfg[(m, n, k)])
        time.sleep(1.0)
        steps = max(5, min(args.steps, 20))
        ms = time_steps(lambda: tnx.matmul(a, b), steps, 3, lambda: None) / steps
        tnx.check_status(dev)
    finally:
        for key, value in keep.items():
            if value is None:
                os.environ.pop(key, None)
            else:
                os.environ[key] = value
        mm._matmul_cfg[(m, n, k)] = dict(GEMM_CFG)
    return {"call": "tritonix_b200.matmul(a, b), untuned process, no disk cache", "first_call_seconds": first,
            "tuned_config": cfg, "ms_per_step": ms, "value": work["flops"] / (ms * 1e-3) / 1e12,
            "unit": "TFLOP/s"}


# ---------------------------------------------------------------------------------------------
# comparisons on the same GPU (never a backend of the product)
# ---------------------------------------------------------------------------------------------
def comparators(workload, work, args, dev):
    out = {}
    a_all, b_all, c = work["operands"]
    m, n, k = work["shape"]
    steps = max(5, min(args.steps, 20))
    noop = lambda: None  # noqa: E731
    state = {"i": 0}
    if workload == "glu":
        a, b = a_all[0], b_all[0]
        w1, w2 = b[:, 0::2].contiguous(), b[:, 1::2].contiguous()
        fn = lambda: torch.nn.functional.silu(a @ w1) * (a @ w2)  # noqa: E731
        label = "unfused F.silu(x @ W1) * (x @ W2), cuBLAS + elementwise kernels"
    else:
        def fn():  # the same rotation through operand copies as the kernel under test
            i = state["i"] % len(a_all)
            state["i"] += 1
            torch.matmul(a_all[i], b_all[i], out=c)
        label = "torch.matmul (cuBLAS), same operands"
    ms = time_steps(fn, steps, 3, noop, graph=(workload == "splitk")) / steps
    out["cublas"] = {"what": label, "ms_per_step": ms, "value": work["flops"] / (ms * 1e-3) / 1e12,
                     "unit": "TFLOP/s"}
    if workload == "glu":
        del w1, w2
    out["triton_ref"] = triton_reference_timing(workload, m, n, k)
    return out


def triton_reference_timing(workload, m, n, k):
    """The reference's own Triton kernel on this GPU, in a process of its own (its package name
    collides with this one's alias, and its JIT should not share this context)."""
    if not os.path.isdir(os.path.join(ROOT, "oracle", "_ref", "tritonix")):
        return {"unavailable": "the reference package is not staged under oracle/_ref "
                               "(python oracle/make_ref.py <reference tree>)"}
    kind = {"gemm": "matmul", "splitk": "splitk", "glu": "glu"}[workload]
    dtype = "float16" if workload == "splitk" else "bfloat16"
    cases = []
    for i, cfg in enumerate(TRITON_REF_CONFIGS[:4 if workload == "gemm" else 2]):
        cfg = dict(cfg)
        if kind == "splitk":
            cfg.update(block_m=64, split_k=4)
        cases.append(dict(name=f"cfg{i}", kind=kind, m=m, n=n, k=k, dtype=dtype, seed=i,
                          a_scale=1.0 if kind == "glu" else k ** -0.5,
                          b_scale=0.02 if kind == "glu" else k ** -0.5, cfg=cfg, rows=[0], time=True,
                          reps=10, activation="silu"))
    try:
        with tempfile.TemporaryDirectory() as tmp:
            spec, raw = os.path.join(tmp, "spec.json"), os.path.join(tmp, "raw.npz")
            with open(spec, "w") as f:
                json.dump(cases, f)
            env = {k_: v for k_, v in os.environ.items() if k_ != "TRITON_INTERPRET"}
            done = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "reference_gpu.py"),
                                   "--spec", spec, "--out", raw], env=env, capture_output=True,
                                  text=True, timeout=600)
            if done.returncode != 0:
                return {"unavailable": "reference kernels failed to run: " + done.stderr.strip()[-300:]}
            import numpy as np
            got = np.load(raw)
            best = min(range(len(cases)), key=lambda i: float(got[f"cfg{i}/ms"][0]))
            ms = float(got[f"cfg{best}/ms"][0])
    except Exception as exc:  # a comparison that cannot run must not take the benchmark down
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
    return {"what": "the reference's Triton kernel (JIT for this GPU), best of %d configurations of its own "
                    "search space, mean of 10 launches with L2 flushed" % len(cases),
            "config": cases[best]["cfg"], "ms_per_step": ms, "value": 2.0 * m * n * k / (ms * 1e-3) / 1e12,
            "unit": "TFLOP/s"}


# ---------------------------------------------------------------------------------------------
# the reference's CPU path
# ---------------------------------------------------------------------------------------------
def cpu_baseline_sample(workload, seconds_target=15.0, full=False):
    """The reference's CPU path on the workload (or a bounded sample of it), all host threads."""
    from oracle import contraction as O
    if torch.get_num_threads() < (os.cpu_count() or 1):
        torch.set_num_threads(os.cpu_count() or 1)
    threads = torch.get_num_threads()
    g = torch.Generator().manual_seed(0)
    w = WORKLOADS[workload]
    if workload == "mlp":
        m_s, d, ff = 256, w["d"], w["ff"]
        x = torch.randn(m_s, d, generator=g)
        w12 = torch.randn(d, 2 * ff, generator=g) * 0.02
        wd = torch.randn(ff, d, generator=g) * 0.02
        fn = lambda: O.swiglu_mlp_oracle(x, w12, wd, out_dtype=torch.float32)  # noqa: E731
        flops = 2.0 * m_s * d * 2 * ff + 2.0 * m_s * ff * d
        sample = f"{m_s} of {w['m']} tokens, fp32 torch on host"
        units = float(m_s)
    elif workload == "conv":
        from oracle import conv2d as OC
        b_s = 4
        x = torch.randn(b_s, w["c_in"], w["h"], w["w"], generator=g)
        wt = torch.randn(w["c_out"], w["c_in"], w["r"], w["s"], generator=g) * 0.02
        fn = lambda: OC.conv2d_oracle(x, wt, None, (w["stride"],) * 2, (w["pad"],) * 2)  # noqa: E731
        flops = 2.0 * (w["m"] // w["batch"] * b_s) * w["n"] * w["k"]
        sample = f"{b_s} of {w['batch']} images, fp32 im2col + torch.matmul on host"
        units = None
    else:
        m, n, k = w["m"], w["n"], w["k"]
        m_s = m if full else min(m, 512 if workload == "glu" else 1024)
        a = torch.randn(m_s, k, generator=g)
        b = torch.randn(k, n, generator=g) * (0.02 if workload == "glu" else k ** -0.5)
        if workload == "glu":
            fn = lambda: O.glu_oracle(a, b, "silu", out_dtype=torch.float32)  # noqa: E731
        else:
            fn = lambda: O.matmul_oracle(a, b, out_dtype=torch.float32)  # noqa: E731
        flops = 2.0 * m_s * n * k
        sample = (f"the full problem ({m} x {k} . {k} x {n})" if m_s == m else
                  f"{m_s} of {m} rows of A against the full B") + ", fp32 torch.matmul on host"
        units = None
    fn()  # warm-up
    t0 = time.perf_counter()
    fn()
    one = time.perf_counter() - t0
    reps = max(1, min(20, int(seconds_target / max(one, 1e-3))))
    best = one
    for _ in range(reps - 1):
        t0 = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t0)
    return dict(flops=flops, seconds=best, threads=threads, sample=sample, units=units, fn=fn)


def run_reference(args, rank):
    """CPU arm: rank 0 only.  For the headline workload every step is one pass over the FULL
    8192^3 problem (about half a second on 16 cores); the others use a bounded sample."""
    if rank != 0:
        return
    # launchers such as torchrun pin OMP_NUM_THREADS=1; the CPU arm uses every host core
    torch.set_num_threads(os.cpu_count() or 1)
    workload = "gemm" if args.workload == "all" else args.workload
    metric, unit = metric_of(workload)
    base = cpu_baseline_sample(workload, seconds_target=1.0, full=(workload == "gemm"))
    fn = base["fn"]
    for _ in range(max(0, args.warmup - 2)):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    sec = (time.perf_counter() - t0) / args.steps
    value = base["units"] / sec if workload == "mlp" else base["flops"] / sec / 1e12
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong" if workload == "mlp" else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOADS[workload]["name"]},
        "cpu_baseline": {"value": value, "unit": unit, "cores": base["threads"], "kind": "port",
                         "sample": base["sample"]},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", choices=["all"] + list(WORKLOADS), default="all")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak",
                    help="--workload gemm on N GPUs: weak = 8192 rows per GPU, strong = 8192/N rows "
                         "per GPU of the one 8192^3 problem")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sustained", action="store_true")
    ap.add_argument("--no-comparators", action="store_true")
    ap.add_argument("--no-drop-in", action="store_true",
                    help="gemm on one GPU: skip the leg that tunes and times the plain matmul(a, b) call")
    ap.add_argument("--sustained-seconds", type=float, default=2.0)
    ap.add_argument("--cfg", type=str, default=None,
                    help="JSON object overriding kernel-config keys of the workload, e.g. "
                         "'{\"group_m\": 8}'")
    ap.add_argument("--chunk-weights", default="",
                    help="mlp: comma-separated relative sizes of the row chunks (overrides --chunks), "
                         "e.g. 3,3,2,1 for a short last chunk")
    ap.add_argument("--chunks", type=int, default=0,
                    help="mlp: row chunks whose all-reduce overlaps the next chunk's GEMMs "
                         "(default: 1 on one GPU, 4 otherwise)")
    ap.add_argument("--comm-sms", type=int, default=-1,
                    help="mlp on >1 GPU: SMs the GEMM grids leave free for the all-reduce kernel "
                         "(-1: 32 on 8 or more GPUs, else 0)")
    ap.add_argument("--mlp-mode", choices=["auto", "two_launch", "one_launch"], default="auto",
                    help="mlp: which implementation `value` times (auto: two_launch on one GPU, one_launch "
                         "on several when the NVLink multicast mapping is available); the other one is "
                         "timed too, from the same rest, and reported under `variants`")
    ap.add_argument("--fp32-partials", action="store_true",
                    help="mlp one_launch on >1 GPU: exchange fp32 partial outputs (one rounding) instead of bf16")
    ap.add_argument("--tile-split", type=int, default=16,
                    help="mlp one_launch on >1 GPU: CTAs whose spare warps share one row tile's exchange")
    ap.add_argument("--mlp-band", type=int, default=0,
                    help="mlp one_launch: 256-row tiles per band (0: 8, or 4 when a rank's weights are under 48 MB)")
    ap.add_argument("--mlp-tokens", type=int, default=0,
                    help="mlp: token count, if not the 32768 of the benchmark configuration (a smaller "
                         "case for a profiler capture; the line then names it in config.tokens)")
    ap.add_argument("--launch", choices=["auto", "eager", "graph"], default="auto",
                    help="how the timed steps are issued: one by one, or as one CUDA graph of "
                         "`steps` launches (auto: graph for the launch-latency-bound splitk workload)")
    ap.add_argument("--no-e2e", action="store_true",
                    help="skip the host-buffer leg (used for profiler captures of the kernel)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch.distributed as dist
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    everything = args.workload == "all"
    headline = "gemm" if everything else args.workload
    if headline == "gemm" and args.scaling == "strong":
        headline = "gemm_strong"
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        pg_options = None
        reserve = (32 if world >= 8 else 0) if args.comm_sms < 0 else args.comm_sms
        if (everything or headline == "mlp") and reserve > 0:
            try:  # keep the all-reduce inside the SMs that the GEMM grids leave free
                pg_options = dist.ProcessGroupNCCL.Options()
                pg_options.config.max_ctas = reserve
            except Exception:
                pg_options = None
        dist.init_process_group("nccl", device_id=dev, pg_options=pg_options)
    D = Dist(world, dev)

    import tritonix_b200 as tnx  # noqa: F401
    if args.cfg and headline != "conv":
        override = json.loads(args.cfg)
        for base in (GEMM_CFG, SPLITK_CFG, GLU_CFG):
            base.update(override)
    peaks = measured_peaks()

    entry = measure(headline, args, rank, local_rank, world, dev, D, peaks)
    line = {
        "metric": entry["metric"], "value": entry["value"], "unit": entry["unit"], "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": entry["ms_per_step"],
        "higher_is_better": True, "scaling": entry["scaling"], "vs_baseline": None,
        "dtype": entry["dtype"], "data": "synthetic", "config": entry["config"], "e2e": entry["e2e"],
        "gpu_launches": entry["gpu_launches"], "clocks": entry["clocks"], "roofline": entry["roofline"],
    }
    for extra in ("sustained", "drop_in", "comparators", "parity_err", "parity", "variants",
                  "one_launch_unavailable"):
        if extra in entry:
            line[extra] = entry[extra]
    if rank == 0 and not args.no_cpu_baseline and world == 1:
        wl = "gemm" if headline == "gemm_strong" else headline
        base = cpu_baseline_sample(wl)
        v = base["units"] / base["seconds"] if wl == "mlp" else base["flops"] / base["seconds"] / 1e12
        line["cpu_baseline"] = {"value": v, "unit": entry["unit"], "cores": base["threads"],
                                "kind": "port", "sample": base["sample"]}
    if everything:
        line["workloads"] = {}
        others = ["splitk", "glu", "mlp"] + (["gemm_strong"] if world > 1 else [])
        for wl in others:
            torch.cuda.empty_cache()
            sub = measure(wl, args, rank, local_rank, world, dev, D, peaks)
            sub["steps"], sub["warmup"], sub["n_gpus"] = args.steps, args.warmup, world
            line["workloads"][wl] = sub
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
