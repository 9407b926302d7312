"""The SwiGLU MLP block  y = (silu(x W1) * (x W2)) W3  three ways on a B200:

    python examples/swiglu_mlp.py                          # one GPU: two launches vs one launch
    torchrun --nproc-per-node 2 examples/swiglu_mlp.py     # tensor parallel, exchange inside the kernel

W1 and W2 are stored column-interleaved as one matrix W12 (column 2j = W1[:, j], 2j+1 = W2[:, j]),
the layout the reference's glu_kernel / swiglu_kernel read (tritonix/ops/swiglu.py:12-230).
"""
import os

import torch

import tritonix_b200 as tnx


def main():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    tokens, d_model, d_ff = 8192, 4096, 14336
    g = torch.Generator().manual_seed(0)          # the same global weights on every rank
    x = torch.randn(tokens, d_model, generator=g).to(torch.bfloat16).to(dev)
    w1 = (torch.randn(d_model, d_ff, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(d_model, d_ff, generator=g) * 0.02).to(torch.bfloat16)
    w3 = (torch.randn(d_ff, d_model, generator=g) * 0.02).to(torch.bfloat16)

    if world == 1:
        w12 = tnx.interleave_weights(w1, w2).to(dev)
        w3 = w3.to(dev)
        y_two = tnx.swiglu_mlp(x, w12, w3)                 # fused gate/up kernel, then the down GEMM
        y_one = tnx.swiglu_mlp(x, w12, w3, fused=True)     # the whole block in one launch
        tnx.check_status(dev)
        print("max |one launch - two launches| =", (y_one.float() - y_two.float()).abs().max().item())
        return

    import torch.distributed as dist
    from tritonix_b200.distributed import FusedTensorParallelSwiGLU, shard_mlp_weights
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    w12_shard, w3_shard = shard_mlp_weights(w1, w2, w3, rank, world)   # slice, then interleave
    mlp = FusedTensorParallelSwiGLU(w12_shard.to(dev), w3_shard.to(dev), max_tokens=tokens)
    y = mlp(x)        # every rank gets the full sum; the partial outputs were summed inside the kernel
    tnx.check_status(dev)
    if rank == 0:
        ref = (torch.nn.functional.silu(x.float() @ w1.float().to(dev)) * (x.float() @ w2.float().to(dev))) @ w3.float().to(dev)
        print("max|err|/max|ref| =", ((y.float() - ref).abs().max() / ref.abs().max()).item())
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
