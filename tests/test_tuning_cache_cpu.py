"""Persisted tuned configurations: round trip, corruption tolerance, opt-out."""
import json

from tritonix_b200 import tuning_cache as tc


def test_roundtrip_and_isolation(tmp_path, monkeypatch):
    monkeypatch.setenv("TRITONIX_B200_CACHE_DIR", str(tmp_path))
    key = tc.make_key((8192, 8192, 8192), "torch.bfloat16", "NVIDIA B200", "0.1.0")
    assert key == "8192,8192,8192|torch.bfloat16|NVIDIA B200|0.1.0"
    assert tc.load("matmul_kernel", key) is None
    cfg = {"tile_n": 256, "tile_k": 128, "stages": 3, "cta_group": 2, "group_m": 16}
    tc.save("matmul_kernel", key, cfg)
    tc.save("matmul_kernel", key + "x", {"tile_n": 64})
    assert tc.load("matmul_kernel", key) == cfg
    assert tc.load("glu_kernel", key) is None
    data = json.loads((tmp_path / "tuned" / "matmul_kernel.json").read_text())
    assert set(data) == {key, key + "x"}
    tc.save("matmul_kernel", key, None)  # "nothing could be run" is not persisted
    assert tc.load("matmul_kernel", key) == cfg


def test_corrupted_file_is_a_miss_and_gets_replaced(tmp_path, monkeypatch):
    monkeypatch.setenv("TRITONIX_B200_CACHE_DIR", str(tmp_path))
    (tmp_path / "tuned").mkdir()
    (tmp_path / "tuned" / "k.json").write_text("{broken")
    assert tc.load("k", "a") is None
    tc.save("k", "a", {"x": 1})
    assert tc.load("k", "a") == {"x": 1}


def test_opt_out(tmp_path, monkeypatch):
    monkeypatch.setenv("TRITONIX_B200_CACHE_DIR", str(tmp_path))
    monkeypatch.setenv("TRITONIX_B200_TUNE_CACHE", "0")
    tc.save("k", "a", {"x": 1})
    assert not (tmp_path / "tuned").exists() and tc.load("k", "a") is None
