"""The reference-facing Python surface on a GPU: matmul / matmul_splitk / glu entry points,
kernel handles with Triton's launch syntax, TunableKernel.tune on the real kernels, the
single-backend dispatcher, the torch custom ops, and the device status word.
The first three tests follow the reference's tests/test_matmul.py:9-52."""
import pytest
import torch

import tritonix_b200 as tnx
from oracle import contraction as O
from tests.gpu_util import DEV, assert_close, seeded
from tritonix_b200 import _cabi

pytestmark = pytest.mark.gpu
f16, bf16, f32 = torch.float16, torch.bfloat16, torch.float32


@pytest.fixture(autouse=True)
def quick_tuning(monkeypatch):
    """Keep first-call tuning short: a handful of configurations, short timing budgets."""
    real = tnx.TunableKernel.tune

    def tune(self, launcher, **kw):
        kw.setdefault("max_configs", 6)
        kw.update(warmup=1, rep=3)
        return real(self, launcher, **kw)
    monkeypatch.setattr(tnx.TunableKernel, "tune", tune)
    mm = __import__("sys").modules["tritonix_b200.ops.matmul"]
    mm._matmul_cfg.clear()
    mm._FAST_MATMUL.clear()
    mm._splitk_cfg.clear()
    yield


@pytest.mark.parametrize("M,N,K", [(512, 512, 512), (1024, 2048, 512), (2048, 2048, 2048)])
def test_matmul_correctness(M, N, K):
    a = torch.randn(M, K, device=DEV, dtype=f16)
    b = torch.randn(K, N, device=DEV, dtype=f16)
    out = tnx.triton_matmul(a, b)
    tnx.check_status()
    ref = torch.matmul(a, b)
    assert torch.allclose(ref, out, atol=1.0, rtol=1e-2)          # the reference's own bar
    assert_close(out.cpu(), O.matmul_oracle(a.cpu(), b.cpu()), f16)  # this package's bar


def test_dispatch_correctness_and_single_backend():
    a = torch.randn(512, 512, device=DEV, dtype=f16)
    b = torch.randn(512, 512, device=DEV, dtype=f16)
    with tnx.matmul.force_backend("cuda"):
        out = tnx.matmul(a, b)
    assert_close(out.cpu(), O.matmul_oracle(a.cpu(), b.cpu()), f16)
    for name in ("triton", "pytorch"):
        with pytest.raises(KeyError):
            with tnx.matmul.force_backend(name):
                pass


def test_dispatch_caches_winner(tmp_path):
    tnx.matmul.clear_cache()
    a = torch.randn(1024, 1024, device=DEV, dtype=f16)
    b = torch.randn(1024, 1024, device=DEV, dtype=f16)
    out1 = tnx.matmul(a, b)
    assert len(tnx.matmul.cache) == 1
    key = (1024, 1024, "torch.float16", 1024, 1024, "torch.float16")
    assert tnx.matmul.cache[key] == "cuda" and set(tnx.matmul.timings[key]) == {"cuda"}
    assert tnx.matmul.timings[key]["cuda"] > 0
    out2 = tnx.matmul(a, b)
    assert torch.equal(out1, out2)
    tnx.matmul.clear_cache()


def test_quick_start_shape_with_fp32_reference():
    """A 1024x512, B 512x768, N(0,1) entries, fp16 in / fp32 accumulate / fp16 out."""
    a, b = seeded(1024, 512, 768, f16, seed=0, b_scale=1.0)
    out = tnx.matmul(a.to(DEV), b.to(DEV))
    tnx.check_status()
    assert_close(out.cpu(), O.matmul_oracle(a, b), f16)


def test_matmul_splitk_uses_requested_factor():
    a, b = seeded(64, 2048, 1024, f16, seed=1)
    a, b = a.to(DEV), b.to(DEV)
    for s in (2, 4):
        out = tnx.matmul_splitk(a, b, split_k=s)
        tnx.check_status()
        assert_close(out.cpu(), O.splitk_oracle(a.cpu(), b.cpu(), s), f16)
        mm = __import__("sys").modules["tritonix_b200.ops.matmul"]
        assert mm._splitk_cfg[(64, 1024, 2048, s)]["split_k"] == s


def test_kernel_handle_launch_syntax():
    """kernel[grid](ptr args, sizes, strides, **cfg) with the reference's config names."""
    a, b = seeded(256, 128, 192, f16, seed=2)
    a, b = a.to(DEV), b.to(DEV)
    c = torch.empty(256, 192, device=DEV, dtype=f16)
    grid = (2, 2)
    tnx.matmul_kernel[grid](a, b, c, 256, 192, 128, a.stride(0), a.stride(1), b.stride(0), b.stride(1),
                            c.stride(0), c.stride(1), block_m=128, block_n=128, block_k=64, group_m=8,
                            num_stages=3, num_warps=8)
    tnx.check_status()
    assert_close(c.cpu(), O.matmul_oracle(a.cpu(), b.cpu()), f16)
    # GLU handle: n counts the interleaved columns (2F), output is M x F
    x, w12 = seeded(128, 256, 2 * 96, f16, seed=3, b_scale=0.05)
    x, w12 = x.to(DEV), w12.to(DEV)
    for act in ("silu", "none", "sigmoid"):
        z = torch.empty(128, 96, device=DEV, dtype=f16)
        tnx.glu_kernel[(1, 2)](x, w12, z, 128, 192, 256, x.stride(0), x.stride(1), w12.stride(0),
                               w12.stride(1), z.stride(0), z.stride(1), block_m=128, block_n=128,
                               block_k=64, group_m=4, activation=act)
        tnx.check_status()
        assert_close(z.cpu(), O.glu_oracle(x.cpu(), w12.cpu(), act), f16)
    # pre-run hooks fire with the launch arguments
    seen = []
    tnx.gemm_splitk_kernel.add_pre_run_hook(lambda *args, **kw: seen.append(kw.get("split_k")))
    try:
        tnx.gemm_splitk_kernel[(1,)](a, b, c, 256, 192, 128, a.stride(0), a.stride(1), b.stride(0),
                                     b.stride(1), c.stride(0), c.stride(1), tile_n=64, split_k=2)
        tnx.check_status()
    finally:
        tnx.gemm_splitk_kernel.kernel._pre_hooks.clear()
    assert seen == [2]
    assert_close(c.cpu(), O.matmul_oracle(a.cpu(), b.cpu()), f16)


def test_swiglu_mlp_kernel_signature():
    """swiglu_kernel[grid](x, w12, w3, z, m, n, k, f, strides...) = (silu(xW1)*(xW2)) W3."""
    g = torch.Generator().manual_seed(4)
    x = torch.randn(256, 512, generator=g).to(bf16)
    w12 = (torch.randn(512, 2 * 384, generator=g) * 0.04).to(bf16)
    w3 = (torch.randn(384, 256, generator=g) * 0.05).to(bf16)
    xd, wd, w3d = x.to(DEV), w12.to(DEV), w3.to(DEV)
    z = torch.empty(256, 256, device=DEV, dtype=bf16)
    tnx.swiglu_kernel[(2, 3)](xd, wd, w3d, z, 256, 768, 512, 256, xd.stride(0), xd.stride(1),
                              wd.stride(0), wd.stride(1), w3d.stride(0), w3d.stride(1), z.stride(0),
                              z.stride(1), block_m=128, block_n=128, block_k=64, group_m=4, block_l=64)
    tnx.check_status()
    assert_close(z.cpu(), O.swiglu_mlp_oracle(x, w12, w3, hidden_dtype=bf16), bf16)
    y = tnx.swiglu_mlp(xd, wd, w3d, cfg={"tile_n": 128}, down_cfg={"tile_n": 128})
    tnx.check_status()
    assert_close(y.cpu(), O.swiglu_mlp_oracle(x, w12, w3, hidden_dtype=bf16), bf16)


def test_tuner_on_real_kernels_prunes_out_of_resources():
    a, b = seeded(512, 512, 1024, bf16, seed=5)
    a, b = a.to(DEV), b.to(DEV)
    mm = __import__("sys").modules["tritonix_b200.ops.matmul"]
    events = []

    def launcher(cfg):
        try:
            return mm._launch_matmul(a, b, cfg)
        except tnx.OutOfResources:
            events.append(("oom", dict(cfg)))
            raise
        except ValueError:
            events.append(("skip", dict(cfg)))
            raise
    best = tnx.matmul_kernel.tune(launcher, max_configs=40,
                                  filter_fn=lambda c: c["group_m"] == 8 and c["block_k"] == 64)
    tnx.check_status()
    assert best is not None and set(best) == set(tnx.matmul_kernel.space)
    ooms = [c for kind, c in events if kind == "oom"]
    assert ooms, "the 7- and 8-stage configurations of the 256-wide tile cannot fit in shared memory"
    # nothing that needs at least as much memory as a failed configuration was tried afterwards
    for i, (kind, c) in enumerate(events):
        if kind != "oom":
            continue
        for kind2, c2 in events[i + 1:]:
            assert not (c2["block_n"] >= c["block_n"] and c2["num_stages"] >= c["num_stages"]
                        and c2["block_m"] <= c["block_m"] and c2["block_k"] >= c["block_k"]
                        and c2["acc_stages"] >= c["acc_stages"])
    out = mm._launch_matmul(a, b, best)
    assert_close(out.cpu(), O.matmul_oracle(a.cpu(), b.cpu()), bf16)


def test_torch_custom_ops():
    a, b = seeded(256, 256, 512, bf16, seed=6)
    a, b = a.to(DEV), b.to(DEV)
    c = torch.ops.tritonix.gemm(a, b, [])
    assert_close(c.cpu(), O.matmul_oracle(a.cpu(), b.cpu()), bf16)
    c = torch.ops.tritonix.gemm_splitk(a, b, 2, [0, 128])
    assert_close(c.cpu(), O.matmul_oracle(a.cpu(), b.cpu()), bf16)
    z = torch.ops.tritonix.glu(a, b, _cabi.EPI_GLU_SILU, [0, 256, 64, 4, 2, 1])
    assert_close(z.cpu(), O.glu_oracle(a.cpu(), b.cpu(), "silu"), bf16)
    tnx.check_status()
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        fa, fb = torch.empty(64, 32, dtype=bf16, device=DEV), torch.empty(32, 48, dtype=bf16, device=DEV)
        assert torch.ops.tritonix.gemm(fa, fb, []).shape == (64, 48)
        assert torch.ops.tritonix.glu(fa, fb, 2, []).shape == (64, 24)


def test_do_bench_returns_positive_ms():
    a, b = seeded(1024, 1024, 1024, bf16)
    a, b = a.to(DEV), b.to(DEV)
    c = torch.empty(1024, 1024, device=DEV, dtype=bf16)
    ms = tnx.do_bench(lambda: _cabi.launch(a, b, c, None), warmup=2, rep=10)
    med = tnx.do_bench(lambda: _cabi.launch(a, b, c, None), warmup=2, rep=10, return_mode="median")
    assert 0 < ms < 5 and 0 < med < 5


def test_expired_wait_is_reported_not_fatal():
    """A device wait that nothing satisfies gives up after its limit, the kernel returns, the
    status word carries a code, Python raises DeviceStatusError, and the context keeps working."""
    dev = torch.device(DEV, torch.cuda.current_device())
    word = _cabi.status_word(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    assert _cabi.lib.tnx_selftest_bounded_wait(word.data_ptr(), 50, stream) == _cabi.OK
    with pytest.raises(tnx.DeviceStatusError, match="0x1ff"):
        tnx.check_status(dev)
    tnx.check_status(dev)  # the word was reset; nothing else is wrong
    a, b = seeded(128, 128, 128, f16)
    c = torch.empty(128, 128, device=DEV, dtype=f16)
    _cabi.launch(a.to(DEV), b.to(DEV), c, None)
    tnx.check_status(dev)
    assert_close(c.cpu(), O.matmul_oracle(a, b), f16)
    assert _cabi.lib.tnx_selftest_bounded_wait(None, 50, stream) == _cabi.ERR_INVALID


def test_status_word_reports_clean_after_all_launches():
    tnx.check_status()
    w = _cabi.status_word(torch.device(DEV, torch.cuda.current_device()))
    assert int(w.item()) == 0


def test_tuned_configuration_is_persisted(tmp_path, monkeypatch):
    """The winner of the first call's tuning is written to disk and reused by a fresh cache."""
    monkeypatch.setenv("TRITONIX_B200_CACHE_DIR", str(tmp_path))
    mm = __import__("sys").modules["tritonix_b200.ops.matmul"]
    a = torch.randn(384, 512, device=DEV, dtype=bf16)
    b = torch.randn(512, 640, device=DEV, dtype=bf16)
    out1 = tnx.triton_matmul(a, b)
    files = list((tmp_path / "tuned").glob("matmul_kernel.json"))
    assert len(files) == 1
    stored = __import__("json").loads(files[0].read_text())
    (key, cfg), = stored.items()
    assert key.startswith("384,640,512|torch.bfloat16|") and cfg == mm._matmul_cfg[(384, 640, 512)]
    mm._matmul_cfg.clear()
    mm._FAST_MATMUL.clear()

    def no_tuning(self, *args, **kwargs):
        raise AssertionError("the stored configuration should have been used")
    monkeypatch.setattr(tnx.TunableKernel, "tune", no_tuning)
    out2 = tnx.triton_matmul(a, b)
    assert torch.equal(out1, out2) and mm._matmul_cfg[(384, 640, 512)] == cfg


def test_matmul_from_host_pipelines_rows(monkeypatch):
    """A and the result in pinned host memory, B uploaded once: rows are pipelined through
    upload / compute / download streams and the result equals the one-shot product."""
    monkeypatch.setenv("TRITONIX_B200_TUNE", "0")
    a, b = seeded(1000, 512, 384, bf16, seed=8)
    a_host, b_host = a.pin_memory(), b.pin_memory()
    out_host = torch.full((1000, 384), float("nan"), dtype=bf16).pin_memory()
    tnx.matmul_from_host(a_host, b_host, out_host, rows_per_chunk=256)   # 3 full chunks + 232 rows
    torch.cuda.synchronize()
    tnx.check_status()
    assert_close(out_host, O.matmul_oracle(a, b), bf16)
    # device-resident B, second call reuses the pipeline's buffers
    out2 = torch.empty_like(out_host).pin_memory()
    tnx.matmul_from_host(a_host, b.to(DEV), out2, rows_per_chunk=256)
    torch.cuda.synchronize()
    assert torch.equal(out2, out_host)
