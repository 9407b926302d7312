"""Tuner walk-through on the CUDA kernels: grid search with out-of-resources and unimodality
pruning, the auto-tuned entry point, and the dispatcher's cache — the scenario of the
reference's examples/tune_matmul.py, with this package's names.

    python examples/tune_matmul.py [M N K]
"""
import sys
import time

import torch

import tritonix_b200 as tritonix
from tritonix_b200.ops.matmul import cuda_matmul, matmul, matmul_kernel

DTYPE = torch.bfloat16
M, N, K = (int(v) for v in sys.argv[1:4]) if len(sys.argv) >= 4 else (512, 2048, 4096)


def make_launcher(a, b):
    m, k = a.shape
    _, n = b.shape

    def launcher(cfg):
        c = torch.empty((m, n), device=a.device, dtype=a.dtype)
        grid = (-(-m // cfg["block_m"]), -(-n // cfg["block_n"]))  # ignored: the kernel is persistent
        matmul_kernel[grid](a, b, c, m, n, k, a.stride(0), a.stride(1), b.stride(0), b.stride(1),
                            c.stride(0), c.stride(1), **cfg)
        return c

    return launcher


def tflops(ms):
    return 2.0 * M * N * K / (ms * 1e-3) / 1e12


def main():
    a = torch.randn((M, K), device="cuda", dtype=DTYPE)
    b = torch.randn((K, N), device="cuda", dtype=DTYPE)
    launcher = make_launcher(a, b)
    print(f"Problem   : {M}x{K} @ {K}x{N}  dtype={DTYPE}")
    print(f"Space     : {len(matmul_kernel.configs())} configs")
    print(f"Mem params: {sorted(matmul_kernel.memory_params)}\n")

    print("Grid search (out-of-resources trie + unimodality pruning) ...")
    t0 = time.perf_counter()
    best = matmul_kernel.tune(launcher, method="grid", warmup=5, rep=20, verbose=True)
    tune_s = time.perf_counter() - t0

    ms_best = tritonix.do_bench(lambda: launcher(best), warmup=25, rep=100)
    ms_auto = tritonix.do_bench(lambda: cuda_matmul(a, b), warmup=25, rep=100)
    ms_torch = tritonix.do_bench(lambda: torch.matmul(a, b), warmup=25, rep=100)
    print(f"\n{'method':<22}{'ms':>9}{'TFLOP/s':>10}")
    print(f"{'grid search':<22}{ms_best:>9.3f}{tflops(ms_best):>10.1f}   ({tune_s:.1f} s of tuning) {best}")
    print(f"{'cuda_matmul (auto)':<22}{ms_auto:>9.3f}{tflops(ms_auto):>10.1f}")
    print(f"{'torch.matmul (cuBLAS)':<22}{ms_torch:>9.3f}{tflops(ms_torch):>10.1f}   (comparison only, not a backend)")

    matmul.clear_cache()
    matmul(a, b)
    key, winner = next(iter(matmul.cache.items()))
    print(f"\ndispatcher: key={key} winner={winner} timings={matmul.timings[key]}")
    tritonix.check_status()


if __name__ == "__main__":
    main()
