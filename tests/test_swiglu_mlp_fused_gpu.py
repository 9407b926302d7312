"""The one-launch SwiGLU MLP (tnx_swiglu_mlp through the C ABI) against the CPU oracle of what the
reference's swiglu_kernel intends (tritonix/ops/swiglu.py:113-230): Y = (act(X.W1) * (X.W2)) . W3
with the hidden activation rounded to the operand type.  Tolerance 2e-3 (fp16) / 8e-3 (bf16).
Also: bit equality with the two-launch composition of the same tiles, bit-identical repeats,
grids far smaller than the work (every dependency wait is exercised), ring slots reused."""
import pytest
import torch

from oracle import contraction as O
from tests.gpu_util import DEV, assert_close
from tritonix_b200 import _cabi

pytestmark = pytest.mark.gpu
bf16, f16 = torch.bfloat16, torch.float16
EPI = {"none": _cabi.EPI_GLU_LINEAR, "silu": _cabi.EPI_GLU_SILU, "sigmoid": _cabi.EPI_GLU_SIGMOID}


def seeded_mlp(m, d, ff, n_out, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, d, generator=g).to(dtype)
    w12 = (torch.randn(d, 2 * ff, generator=g) * d ** -0.5).to(dtype)
    w3 = (torch.randn(ff, n_out, generator=g) * ff ** -0.5).to(dtype)
    return x, w12, w3


def oracle(x, w12, w3, act):
    h = O.glu_oracle(x, w12, act, out_dtype=x.dtype)
    return O.matmul_oracle(h, w3)


def run_fused(x, w12, w3, cfg=None, act="silu", workspace_bands=None):
    xd, wd, w3d = x.to(DEV), w12.to(DEV), w3.to(DEV)
    y = torch.full((x.shape[0], w3.shape[1]), float("nan"), device=DEV, dtype=x.dtype)
    ws = None
    if workspace_bands is not None:
        problem = _cabi.MlpProblem(x.shape[0], x.shape[1], w3.shape[0], w3.shape[1], _cabi.DTYPES[x.dtype],
                                   EPI[act], x.shape[1], w12.shape[1], w3.shape[1], w3.shape[1])
        res = _cabi.mlp_query(problem, _cabi.make_config(cfg))
        band_bytes = res.band_rows * w3.shape[0] * 2
        counters = res.min_workspace_bytes - min(2, res.num_bands) * band_bytes
        ws = torch.empty(counters + workspace_bands * band_bytes, dtype=torch.uint8, device=DEV)
    res = _cabi.launch_mlp(xd, wd, w3d, y, cfg, EPI[act], workspace=ws)
    _cabi.check_status(y.device)
    return y, res


@pytest.mark.parametrize("act", ["silu", "sigmoid", "none"])
@pytest.mark.parametrize("m,d,ff,n_out,dtype,cfg", [
    (256, 256, 256, 256, bf16, None),                                  # one unit of each kind per column
    (512, 512, 1024, 512, bf16, {"tile_k": 64}),
    (2048, 512, 2048, 512, f16, {"tile_k": 128, "stages": 3, "group_m": 2}),
    (1000, 264, 520, 200, bf16, {"group_m": 2}),                       # ragged in every dimension
    (1536, 512, 640, 384, f16, {"group_m": 1}),
])
def test_against_oracle(act, m, d, ff, n_out, dtype, cfg):
    x, w12, w3 = seeded_mlp(m, d, ff, n_out, dtype, seed=m + ff)
    y, res = run_fused(x, w12, w3, cfg, act)
    assert y.shape == (m, n_out)
    assert_close(y.cpu(), oracle(x, w12, w3, act), dtype)


@pytest.mark.parametrize("max_ctas", [2, 6, 30])
def test_tiny_grids_wait_on_every_dependency(max_ctas):
    """With a handful of clusters the units of a row tile are spread over many rounds, so output
    tiles really wait for hidden tiles, and with two ring slots for five bands the writers of a
    slot really wait for its previous readers."""
    x, w12, w3 = seeded_mlp(2304, 512, 1280, 768, bf16, seed=max_ctas)
    y, res = run_fused(x, w12, w3, {"group_m": 2, "max_ctas": max_ctas}, workspace_bands=2)
    assert res.grid == max_ctas and res.num_bands == 5
    ref = oracle(x, w12, w3, "silu")
    assert_close(y.cpu(), ref, bf16)
    y2, _ = run_fused(x, w12, w3, {"group_m": 2}, workspace_bands=5)   # no slot reused at all
    assert torch.equal(y, y2)


def test_bit_identical_to_the_two_launch_composition_and_repeatable():
    import tritonix_b200 as tnx
    x, w12, w3 = seeded_mlp(4096, 1024, 3584, 1024, bf16, seed=3)
    xd, wd, w3d = x.to(DEV), w12.to(DEV), w3.to(DEV)
    tiles = {"kernel": "tcgen05", "tile_n": 256, "cta_group": 2, "tile_k": 128, "stages": 3}
    two = tnx.swiglu_mlp(xd, wd, w3d, cfg=tiles, down_cfg=tiles)
    one = tnx.swiglu_mlp(xd, wd, w3d, fused=True, fused_cfg={"tile_k": 128, "stages": 3})
    again = tnx.swiglu_mlp(xd, wd, w3d, fused=True, fused_cfg={"tile_k": 128, "stages": 3, "group_m": 8})
    _cabi.check_status(one.device)
    assert torch.equal(one, two) and torch.equal(one, again)
    rows = [0, 1, 255, 256, 2047, 4095]
    assert_close(one[rows].cpu(), oracle(x[rows], w12, w3, "silu"), bf16)


def test_reference_launch_syntax_is_one_launch(monkeypatch):
    """swiglu_kernel[grid](x, w12, w3, z, m, n, k, f, strides...) — the reference's argument list —
    goes to the one-launch kernel; operands it cannot take fall back to two launches."""
    import tritonix_b200 as tnx
    x, w12, w3 = seeded_mlp(512, 512, 384, 256, bf16, seed=8)
    xd, wd, w3d = x.to(DEV), w12.to(DEV), w3.to(DEV)
    calls = []
    real = _cabi.launch_mlp
    monkeypatch.setattr(_cabi, "launch_mlp", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    z = torch.full((512, 256), float("nan"), device=DEV, dtype=bf16)
    tnx.swiglu_kernel[(4, 3)](xd, wd, w3d, z, 512, 768, 512, 256, xd.stride(0), xd.stride(1), wd.stride(0),
                              wd.stride(1), w3d.stride(0), w3d.stride(1), z.stride(0), z.stride(1),
                              block_m=256, block_n=256, block_k=64, block_l=64, group_m=4, num_stages=4)
    _cabi.check_status(z.device)
    assert calls == [1]
    assert_close(z.cpu(), oracle(x, w12, w3, "silu"), bf16)
    # fp32 operands: not served by the fused kernel -> two launches on the strided kernels
    xf, wf, w3f = xd.float()[:64], wd.float(), w3d.float()
    zf = torch.empty(64, 256, device=DEV, dtype=torch.float32)
    tnx.swiglu_kernel[(1, 1)](xf, wf, w3f, zf, 64, 768, 512, 256, xf.stride(0), xf.stride(1), wf.stride(0),
                              wf.stride(1), w3f.stride(0), w3f.stride(1), zf.stride(0), zf.stride(1))
    _cabi.check_status(z.device)
    assert calls == [1]
    ref = O.swiglu_mlp_oracle(x[:64].float(), w12.float(), w3.float(), out_dtype=torch.float32)
    assert O.rel_err(zf.cpu(), ref) <= 1e-4


def test_llama_block_at_full_size_in_one_launch():
    """d = 4096, ff = 14336, 32768 tokens, bf16: 64 sampled tokens against the oracle, and the
    whole output bit-identical to the two-launch path."""
    import tritonix_b200 as tnx
    m, d, ff = 32768, 4096, 14336
    g = torch.Generator(device=DEV).manual_seed(50)
    x = torch.randn(m, d, device=DEV, generator=g).to(bf16)
    w12 = (torch.randn(d, 2 * ff, device=DEV, generator=g) * 0.02).to(bf16)
    w3 = (torch.randn(ff, d, device=DEV, generator=g) * 0.02).to(bf16)
    y = tnx.swiglu_mlp(x, w12, w3, fused=True, fused_cfg={"tile_k": 128, "stages": 3, "group_m": 4})
    _cabi.check_status(y.device)
    rows = sorted(set(torch.randint(0, m, (62,), generator=torch.Generator().manual_seed(7)).tolist()
                      + [0, m - 1]))
    ref = O.swiglu_mlp_oracle(x[rows].cpu(), w12.cpu(), w3.cpu(), hidden_dtype=bf16)
    assert_close(y[rows].cpu(), ref, bf16)
    tiles = {"kernel": "tcgen05", "tile_n": 256, "cta_group": 2, "tile_k": 128, "stages": 3, "group_m": 16}
    assert torch.equal(y, tnx.swiglu_mlp(x, w12, w3, cfg=tiles, down_cfg=tiles))


def test_invalid_calls():
    x, w12, w3 = seeded_mlp(256, 256, 256, 256, bf16, seed=1)
    xd, wd, w3d = x.to(DEV), w12.to(DEV), w3.to(DEV)
    y = torch.empty(256, 256, device=DEV, dtype=bf16)
    with pytest.raises(ValueError, match="output must be"):
        _cabi.launch_mlp(xd, wd, w3d, y[:128])
    with pytest.raises(ValueError, match="one-launch MLP needs"):
        _cabi.launch_mlp(xd, wd[:, :256], w3d, y)
    with pytest.raises(ValueError, match="workspace of at least"):
        _cabi.launch_mlp(xd, wd, w3d, y, workspace=torch.empty(1024, dtype=torch.uint8, device=DEV))
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        _cabi.launch_mlp(x, wd, w3d, y)
