"""Sharding arithmetic and the chunked all-reduce schedule of the multi-GPU layouts, run as two
gloo ranks on CPU.  The local contractions are supplied by the oracle here (the product's own
kernels need a GPU); what is under test is the partitioning and the exchange step."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tritonix_b200.distributed import (TensorParallelSwiGLU, shard_bounds, shard_mlp_weights,
                                       shard_rows, sharded_matmul)


def test_shard_bounds_cover_exactly():
    for total, world, mult in [(8192, 8, 1), (14336, 8, 128), (14336, 4, 256), (10, 3, 1), (7, 8, 1), (1024, 3, 128)]:
        spans = [shard_bounds(total, r, world, mult) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(lo % mult == 0 and hi % mult == 0 for lo, hi in spans)
        sizes = [hi - lo for lo, hi in spans]
        assert max(sizes) - min(sizes) <= mult
    with pytest.raises(ValueError):
        shard_bounds(100, 0, 2, 64)


def test_weight_shards_keep_gate_up_pairs_together():
    g = torch.Generator().manual_seed(0)
    d, ff, world = 16, 1024, 4
    wg, wu, wd = torch.randn(d, ff, generator=g), torch.randn(d, ff, generator=g), torch.randn(ff, d, generator=g)
    x = torch.randn(8, d, generator=g)
    full = (torch.nn.functional.silu(x @ wg) * (x @ wu)) @ wd
    total = torch.zeros_like(full)
    for r in range(world):
        w12, wdr = shard_mlp_weights(wg, wu, wd, r, world)
        lo, hi = shard_bounds(ff, r, world, 128)
        assert torch.equal(w12[:, 0::2], wg[:, lo:hi]) and torch.equal(w12[:, 1::2], wu[:, lo:hi])
        acc = x @ w12
        total += (torch.nn.functional.silu(acc[:, 0::2]) * acc[:, 1::2]) @ wdr
    assert torch.allclose(total, full, atol=1e-3)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import contraction as O
        g = torch.Generator().manual_seed(1234)  # same global tensors on every rank
        d, ff, m = 64, 512, 1024
        x = torch.randn(m, d, generator=g)
        wg = torch.randn(d, ff, generator=g) * 0.05
        wu = torch.randn(d, ff, generator=g) * 0.05
        wd = torch.randn(ff, d, generator=g) * 0.05
        w12, wdr = shard_mlp_weights(wg, wu, wd, rank, world)

        def down(h, w, out):
            out.copy_(O.matmul_oracle(h, w))
        mlp = TensorParallelSwiGLU(w12, wdr, chunks=4,
                                   gate_up_fn=lambda xx, ww: O.glu_oracle(xx, ww, "silu"), down_fn=down)
        assert mlp.world_size == world and len(mlp.chunk_bounds(m)) == 4
        y = mlp(x)
        w12_full = torch.stack((wg, wu), 2).reshape(d, 2 * ff)
        ref = O.swiglu_mlp_oracle(x, w12_full, wd)
        err = O.rel_err(y, ref)
        # M-sharded GEMM: every rank computes its own rows, no collective
        b = torch.randn(d, 96, generator=g)
        rows = shard_rows(x, rank, world)
        c_rows = sharded_matmul(rows, b, matmul_fn=O.matmul_oracle)
        lo, hi = shard_bounds(m, rank, world)
        err2 = O.rel_err(c_rows, O.matmul_oracle(x, b)[lo:hi])
        torch.save({"err": err, "err2": err2, "rows": (lo, hi)}, os.path.join(result_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_mlp_and_row_sharded_gemm(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    assert all(r["err"] < 1e-5 and r["err2"] < 1e-6 for r in res), res
    assert [r["rows"] for r in res] == [(0, 512), (512, 1024)]


def test_weighted_chunk_bounds_cover_the_rows():
    """chunks may be a list of relative sizes: contiguous, non-empty, 256-row aligned ranges."""
    import torch
    from tritonix_b200.distributed import TensorParallelSwiGLU
    ident = dict(gate_up_fn=lambda x, w: x, down_fn=lambda h, w, out=None: h)
    w12, wd = torch.zeros(8, 16), torch.zeros(8, 8)
    for chunks in (4, [3, 3, 2, 1], [1, 1, 1, 1, 0.5], [5, 0, 1], [1]):
        tp = TensorParallelSwiGLU(w12, wd, chunks=chunks, **ident)
        for m in (32768, 4096, 1000, 300):
            b = tp.chunk_bounds(m)
            assert b[0][0] == 0 and b[-1][1] == m
            assert all(b[i][1] == b[i + 1][0] for i in range(len(b) - 1))
            assert all(hi > lo for lo, hi in b)
            if m % 256 == 0:
                assert all(lo % 256 == 0 for lo, _ in b)
    tp = TensorParallelSwiGLU(w12, wd, chunks=[3, 3, 2, 1], **ident)
    sizes = [hi - lo for lo, hi in tp.chunk_bounds(32768)]
    assert sizes[-1] < sizes[0] and sizes[-1] == 3584
