#!/usr/bin/env python
"""Benchmark of the dense-contraction path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload gemm|splitk|glu|mlp|conv]
                    [--impl ours|reference]

Default workload (`gemm`): bf16 C = A.B with M = N = K = 8192, entries N(0,1)/sqrt(K), fp32
accumulation, bf16 output — one step is one pass of the kernel over one such problem.  With N
GPUs every rank owns an 8192-row block of a (8192*N) x 8192 A and a replica of B (row-sharded,
no collective): per-GPU work is fixed, so scaling is "weak".
Other workloads: `splitk` (fp16 64 x 14336 x 4096, HBM-bound), `glu` (bf16 fused SwiGLU
8192x4096 . 4096x28672), `mlp` (bf16 SwiGLU MLP d=4096, ff=14336, 32768 tokens, tensor parallel
over the N GPUs with one chunked NCCL all-reduce; strong scaling), `conv` (bf16 conv2d forward,
64 x 256 x 28 x 28 NCHW with 256 3x3 filters through `conv2d_forward`; batch-sharded, weak).

One JSON line is printed by rank 0.  `value` is device-timed with the operands resident in HBM;
`e2e` is the same metric through the public API (`tritonix_b200.matmul`, ...) with the operands
in pinned host memory, host<->device copies inside the timed region.

`--impl reference` times the reference's CPU path for the same workload — tritonix.matmul under
force_backend("pytorch") on host tensors, i.e. torch.matmul on the host cores in fp32
(tritonix/ops/matmul.py:291-293) — through the oracle port, on a bounded sample per step.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024

WORKLOADS = {
    # name: (m, n, k, dtype, description)
    "gemm": dict(m=8192, n=8192, k=8192, dtype="bf16",
                 name="gemm_bf16_8192x8192x8192_per_gpu_rows_sharded_B_replicated"),
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

GEMM_CFG = {"kernel": "tcgen05", "tile_n": 256, "tile_k": 128, "stages": 3, "cta_group": 2, "group_m": 16}
SPLITK_CFG = {"kernel": "tcgen05", "tile_n": 128, "tile_k": 128, "stages": 4, "cta_group": 1, "split_k": 4}
GLU_CFG = {"kernel": "tcgen05", "tile_n": 256, "tile_k": 128, "stages": 3, "cta_group": 2, "group_m": 16}

# DRAM traffic of the dominant kernel per launch, from the ncu captures summarised under
# profiles/ (None until a capture of that workload exists).
NCU_TRAFFIC_BYTES = {"gemm": 1_389_138_048, "splitk": 125_974_528, "glu": 885_355_520, "mlp": None,
                     "conv": 26_989_568}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], burst=p["bf16_tflops"], sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, burst=1590.0, sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.samples, self.reasons, self.max_mhz = [], set(), None
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
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(s)}


# ---------------------------------------------------------------------------------------------
# workloads: each returns (step_fn, e2e_step_fn, work dict)
# ---------------------------------------------------------------------------------------------
def torch_dtype(name):
    return {"bf16": torch.bfloat16, "f16": torch.float16}[name]


def randn(shape, dtype, device, seed, scale):
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(shape, device=device, generator=g, dtype=torch.float32) * scale).to(dtype)


def setup_contraction(workload, rank, world, dev):
    """gemm / splitk / glu: one kernel launch per step."""
    from tritonix_b200 import _cabi
    import tritonix_b200 as tnx
    w = WORKLOADS[workload]
    m, n, k, dt = w["m"], w["n"], w["k"], torch_dtype(w["dtype"])
    epi = _cabi.EPI_GLU_SILU if workload == "glu" else _cabi.EPI_NONE
    n_out = n // 2 if epi else n
    cfg = {"gemm": GEMM_CFG, "splitk": SPLITK_CFG, "glu": GLU_CFG}[workload]
    algo_bytes = (m * k + k * n + m * n_out) * 2
    # operands smaller than L2 are rotated through enough copies to defeat it
    copies = 1 if algo_bytes > 2 * L2_BYTES else -(-3 * L2_BYTES // algo_bytes)
    a_scale = 1.0 if workload == "glu" else k ** -0.5
    b_scale = 0.02 if workload == "glu" else k ** -0.5
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
    mm._matmul_cfg[(m, n, k)] = {x: v for x, v in GEMM_CFG.items()}
    mm._matmul_cfg[(1024, n, k)] = dict(GEMM_CFG)   # row chunks of the host pipeline
    sw._glu_cfg[(1024, n, k)] = dict(GLU_CFG)
    mm._splitk_cfg[(m, n, k, SPLITK_CFG["split_k"])] = dict(SPLITK_CFG)
    sw._glu_cfg[(m, n, k)] = dict(GLU_CFG)
    if workload == "gemm":
        tnx.matmul.cache[(m, k, str(dt), k, n, str(dt))] = "cuda"  # skip the first-call timing

    rows = 1024
    pipe = tnx.HostRowPipeline(dev, k, n_out, dt, rows_per_chunk=rows) if workload == "glu" else None

    def e2e_step():
        # every step uploads A and B from pinned host memory and downloads the result; for the
        # two large workloads the rows of A / C are pipelined against the kernel (public helpers)
        if workload == "gemm":
            tnx.matmul_from_host(a_host, b_host, c_host, rows_per_chunk=rows, b_device=b_in)
        elif workload == "glu":
            pipe.run(lambda xd, od: tnx.swiglu(xd, b_in, out=od), a_host, c_host,
                     before=lambda: b_in.copy_(b_host, non_blocking=True))
        else:
            a_in.copy_(a_host, non_blocking=True)
            b_in.copy_(b_host, non_blocking=True)
            out = tnx.matmul_splitk(a_in, b_in, split_k=SPLITK_CFG["split_k"])
            c_host.copy_(out, non_blocking=True)

    work = dict(flops=2.0 * m * n * k, bytes=float(algo_bytes), units=None, launches=1,
                h2d=a_host.numel() * 2 + b_host.numel() * 2, d2h=c_host.numel() * 2, copies=copies,
                cfg=cfg, out=c_dev, check=(a_dev[0], b_dev[0], epi))
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
                h2d=x_host.numel() * 2, d2h=y_host.numel() * 2, copies=copies, cfg=cfg, out=None,
                check=None, kernel_step=kernel_step)
    return step, e2e_step, work


def setup_mlp(rank, world, dev, chunks=0, comm_sms=-1):
    comm_sms = (32 if world >= 8 else 0) if comm_sms < 0 else comm_sms
    """SwiGLU MLP, tensor parallel: column-parallel fused gate/up, row-parallel down, one
    all-reduce.  Global weights come from fixed seeds and are sliced, so every world size
    computes the same function."""
    import tritonix_b200 as tnx
    from tritonix_b200.distributed import TensorParallelSwiGLU, shard_bounds
    w = WORKLOADS["mlp"]
    m, d, ff, dt = w["m"], w["d"], w["ff"], torch.bfloat16
    lo, hi = shard_bounds(ff, rank, world, 128)
    fr = hi - lo
    # slice-then-interleave; generating the shard's columns directly from (seed, column block)
    wg = torch.cat([randn((d, 128), dt, dev, 10_000 + j, 0.02) for j in range(lo // 128, hi // 128)], 1)
    wu = torch.cat([randn((d, 128), dt, dev, 20_000 + j, 0.02) for j in range(lo // 128, hi // 128)], 1)
    wd = torch.cat([randn((128, d), dt, dev, 30_000 + j, 0.02) for j in range(lo // 128, hi // 128)], 0)
    w12 = torch.stack((wg, wu), 2).reshape(d, 2 * fr).contiguous()
    del wg, wu
    x = randn((m, d), dt, dev, 5, 1.0)
    sw = sys.modules["tritonix_b200.ops.swiglu"]
    mm = sys.modules["tritonix_b200.ops.matmul"]
    mlp = TensorParallelSwiGLU(
        w12, wd, chunks=chunks if (isinstance(chunks, list) or chunks > 0) else (1 if world == 1 else 4),
        comm_sms=comm_sms,
        gate_up_cfg=GLU_CFG, down_cfg=GEMM_CFG)
    state = {}

    def step():
        state["y"] = mlp(x)

    x_host = x.cpu().pin_memory()
    y_host = torch.empty((m, d), dtype=dt).pin_memory()

    pipe = tnx.HostRowPipeline(dev, d, d, dt, rows_per_chunk=4096)
    chunk_mlp = TensorParallelSwiGLU(w12, wd, chunks=1, comm_sms=comm_sms, gate_up_cfg=GLU_CFG,
                                     down_cfg=GEMM_CFG)

    def e2e_step():
        # rows of x stream in, rows of y stream out, 4096 rows (one all-reduce) at a time
        pipe.run(lambda xd, yd: chunk_mlp(xd, out=yd), x_host, y_host)

    flops = 2.0 * m * d * (2 * ff) + 2.0 * m * ff * d
    nchunks = len(mlp.chunk_bounds(m))
    work = dict(flops=flops, bytes=None, units=float(m), launches=2 * nchunks, h2d=x_host.numel() * 2,
                d2h=y_host.numel() * 2, copies=1, cfg={"gate_up": GLU_CFG, "down": GEMM_CFG},
                out=None, check=None, chunks=nchunks, comm_sms=comm_sms)
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


def cpu_baseline_sample(workload, seconds_target=15.0):
    """The reference's CPU path on a bounded sample of the workload, all host threads."""
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
        m_s = min(m, 512 if workload == "glu" else 1024)
        a = torch.randn(m_s, k, generator=g)
        b = torch.randn(k, n, generator=g) * (0.02 if workload == "glu" else k ** -0.5)
        if workload == "glu":
            fn = lambda: O.glu_oracle(a, b, "silu", out_dtype=torch.float32)  # noqa: E731
        else:
            fn = lambda: O.matmul_oracle(a, b, out_dtype=torch.float32)  # noqa: E731
        flops = 2.0 * m_s * n * k
        sample = f"{m_s} of {m} rows of A against the full B, fp32 torch.matmul on host"
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


def run_reference(args, rank):
    """CPU arm: rank 0 only; every step is one pass over the bounded sample."""
    if rank != 0:
        return
    # launchers such as torchrun pin OMP_NUM_THREADS=1; the CPU arm uses every host core
    torch.set_num_threads(os.cpu_count() or 1)
    metric, unit = metric_of(args.workload)
    base = cpu_baseline_sample(args.workload, seconds_target=2.0)
    fn = base["fn"]
    for _ in range(max(0, args.warmup - 1)):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    sec = (time.perf_counter() - t0) / args.steps
    value = base["units"] / sec if args.workload == "mlp" else base["flops"] / sec / 1e12
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.workload == "mlp" else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOADS[args.workload]["name"]},
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
    ap.add_argument("--workload", choices=list(WORKLOADS), default="gemm")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        pg_options = None
        reserve = (32 if world >= 8 else 0) if args.comm_sms < 0 else args.comm_sms
        if args.workload == "mlp" and reserve > 0:
            try:  # keep the all-reduce inside the SMs that the GEMM grids leave free
                pg_options = dist.ProcessGroupNCCL.Options()
                pg_options.config.max_ctas = reserve
            except Exception:
                pg_options = None
        dist.init_process_group("nccl", device_id=dev, pg_options=pg_options)

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    import tritonix_b200 as tnx
    if args.cfg:
        override = json.loads(args.cfg)
        for base in (GEMM_CFG, SPLITK_CFG, GLU_CFG):
            base.update(override)
    if args.workload == "mlp":
        chunks = [float(v) for v in args.chunk_weights.split(",")] if args.chunk_weights else args.chunks
        step, e2e_step, work = setup_mlp(rank, world, dev, chunks, args.comm_sms)
    elif args.workload == "conv":
        step, e2e_step, work = setup_conv(rank, world, dev, json.loads(args.cfg) if args.cfg else None)
    else:
        step, e2e_step, work = setup_contraction(args.workload, rank, world, dev)

    # ---- device-timed value (operands resident in HBM)
    use_graph = args.launch == "graph" or (args.launch == "auto" and args.workload == "splitk")
    with ClockSampler(local_rank) as clocks:
        ms_total = time_steps(step, args.steps, args.warmup, barrier, graph=use_graph)
    tnx.check_status(dev)
    ms_total = max_over_ranks(ms_total)
    ms_step = ms_total / args.steps

    # ---- end to end through the public API, host buffers
    ms_e2e = None
    if not args.no_e2e:
        e2e_steps = max(3, min(args.steps, 10))
        ms_e2e = max_over_ranks(time_steps(e2e_step, e2e_steps, 3, barrier)) / e2e_steps
        tnx.check_status(dev)

    strong = args.workload == "mlp"
    scale = 1 if strong else world  # weak scaling: every rank does the whole per-GPU problem
    metric, unit = metric_of(args.workload)
    units = work["units"]
    value = to_metric(args.workload, work["flops"] * scale, units, ms_step)
    e2e_value = to_metric(args.workload, work["flops"] * scale, units, ms_e2e) if ms_e2e else None

    # ---- roofline of the dominant kernel (per launch, per GPU)
    peaks = measured_peaks()
    launches_per_step = work["launches"]
    if args.workload == "splitk":
        achieved = work["bytes"] / (ms_step * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                "frac": achieved / peaks["hbm"], "traffic": NCU_TRAFFIC_BYTES["splitk"],
                "peak_source": peaks["source"] + " copy bandwidth"}
    else:
        per_gpu_flops = work["flops"] / (world if strong else 1)
        ms_kernel = ms_step
        if work.get("kernel_step") is not None:
            # a step has several launches: time the dominant kernel on its own
            ms_kernel = max_over_ranks(time_steps(work["kernel_step"], args.steps, args.warmup,
                                                  barrier, graph=True)) / args.steps
            tnx.check_status(dev)
        achieved = per_gpu_flops / (ms_kernel * 1e-3) / 1e12
        long_run = ms_total > 1000.0
        peak = peaks["sustained"] if long_run else peaks["burst"]
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES[args.workload],
                "peak_source": peaks["source"] + (" sustained" if long_run else " burst") + " cuBLAS bf16",
                "frac_of_nominal_2250": achieved / 2250.0}
        if work.get("kernel_step") is not None:
            roof["kernel_ms"] = ms_kernel
            roof["note"] = ("dominant kernel timed alone on channels_last tensors, launches replayed "
                            "as one CUDA graph; a step on NCHW tensors adds the two repacking passes")

    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": WORKLOADS[args.workload]["dtype"],
        "data": "synthetic",
        "config": {"workload": WORKLOADS[args.workload]["name"], "kernel_config": work["cfg"],
                   **({"allreduce_chunks": work["chunks"], "comm_sms": work["comm_sms"]}
                      if args.workload == "mlp" and world > 1 else {}),
                   "parallelism": ("tp%d" % world) if strong else
                   (("batch_sharded_x%d" if args.workload == "conv" else "rows_sharded_x%d") % world),
                   "launch": "cuda_graph_of_%d_steps" % args.steps if use_graph else "eager",
                   "l2": ("operands rotate through %d copies (> 3x L2)" % work["copies"]) if work["copies"] > 1
                   else "operands exceed the 126 MB L2"},
        "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": work["h2d"],
                "d2h_bytes_per_step": work["d2h"], "ms_per_step": ms_e2e},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks.summary(),
        "roofline": roof,
    }
    if rank == 0 and world >= 1 and not args.no_cpu_baseline and args.gpus == 1:
        base = cpu_baseline_sample(args.workload)
        v = base["units"] / base["seconds"] if strong else base["flops"] / base["seconds"] / 1e12
        line["cpu_baseline"] = {"value": v, "unit": unit, "cores": base["threads"], "kind": "port",
                                "sample": base["sample"]}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
