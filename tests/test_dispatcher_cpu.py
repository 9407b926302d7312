"""DynamicDispatcher semantics (tritonix/dispatcher.py:38-175) with a fake timer: selection,
.cache/.timings, force_backend, error handling, disk persistence."""
import json
import logging
import os

import pytest
import torch

import tritonix_b200.dispatcher as D
from tritonix_b200 import DynamicDispatcher, dynamic_dispatch

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = json.load(open(os.path.join(HERE, "golden", "host_logic.json")))


@pytest.fixture
def timer(monkeypatch):
    cost = {}

    def fake(fn, warmup=None, rep=None, **kw):
        out = fn()
        return cost[out]
    monkeypatch.setattr(D, "do_bench", fake)
    return cost


def test_keys_match_reference():
    a, b = torch.empty(1024, 512, dtype=torch.float16), torch.empty(512, 768, dtype=torch.float16)
    key = D._tuning_key(["a", "b"], (a, b), {}, ["a", "b"])
    assert list(key) == GOLD["dispatch"]["tuning_key"]
    assert D._disk_key("triton_matmul", ["triton", "pytorch"], key) == GOLD["dispatch"]["disk_key"]
    assert D._disk_key("cuda_matmul", ["cuda"], key) == GOLD["dispatch"]["disk_key_cuda"]


def test_picks_fastest_and_caches(timer):
    timer.update({"fast": 1.0, "slow": 2.0})
    calls = []

    def slow(a, b):
        calls.append("slow")
        return "slow"

    def fast(a, b):
        calls.append("fast")
        return "fast"
    d = dynamic_dispatch({"slow": slow, "fast": fast}, key=["a", "b"], use_disk_cache=False)
    assert d.__name__ == "slow"  # name of the first backend (dispatcher.py:58,166-167)
    a, b = torch.empty(4, 8), torch.empty(8, 2)
    assert d(a, b) == "fast"
    key = (4, 8, "torch.float32", 8, 2, "torch.float32")
    assert d.cache == {key: "fast"} and d.timings == {key: {"slow": 2.0, "fast": 1.0}}
    assert d.best_config() == {key: "fast"}
    calls.clear()
    assert d(a, b) == "fast" and calls == ["fast"]  # no re-benchmark
    d(torch.empty(5, 8), b)
    assert len(d.cache) == 2
    d.clear_cache()
    assert d.cache == {} and d.timings == {}


def test_force_backend(timer):
    timer.update({"x": 1.0, "y": 2.0})
    d = dynamic_dispatch({"x": lambda a: "x", "y": lambda a: "y"}, key=["a"], use_disk_cache=False)
    with d.force_backend("y"):
        assert d(torch.empty(1)) == "y"
        assert d.cache == {}  # forced calls do not benchmark
    assert d(torch.empty(1)) == "x"
    with pytest.raises(KeyError):
        with d.force_backend("pytorch"):
            pass
    with pytest.raises(ValueError):
        with d.force_backend("x"):
            raise ValueError("inside")
    assert d.forced is None


def test_failing_backends(timer, caplog):
    timer.update({"ok": 1.0})

    def bad(a):
        raise RuntimeError("broken backend")
    d = dynamic_dispatch({"bad": bad, "ok": lambda a: "ok"}, key=["a"], use_disk_cache=False)
    with caplog.at_level(logging.DEBUG, logger="tritonix.dispatcher"):
        assert d(torch.empty(2)) == "ok"
    assert any("skipped" in r.message for r in caplog.records)
    assert list(d.timings.values()) == [{"ok": 1.0}]
    only_bad = dynamic_dispatch({"bad": bad}, key=["a"], use_disk_cache=False)
    with pytest.raises(RuntimeError, match="all backends failed"):
        only_bad(torch.empty(2))
    empty = DynamicDispatcher(lambda a: a, key=["a"], arg_names=["a"])
    with pytest.raises(RuntimeError, match="no backends registered"):
        empty(torch.empty(1))


def test_decorator_mode_and_register_chain(timer):
    timer.update({"r": 1.0})

    @dynamic_dispatch(key=["a"], use_disk_cache=False)
    def op(a, scale=1):
        """doc"""
    assert isinstance(op, DynamicDispatcher) and op.__name__ == "op" and op.__doc__ == "doc"
    assert op.register("r", lambda a, scale=1: "r") is op
    assert op(torch.empty(3), scale=2) == "r"
    assert list(op.cache) == [(3, "torch.float32")]  # non-tensor, non-key kwargs are not in the key


def test_disk_cache_roundtrip(timer, tmp_path, monkeypatch):
    monkeypatch.setenv("TRITONIX_B200_CACHE_DIR", str(tmp_path / "c"))
    timer.update({"p": 3.0, "q": 2.0})
    mk = lambda: dynamic_dispatch({"p": lambda a: "p", "q": lambda a: "q"}, key=["a"])  # noqa: E731
    d1 = mk()
    a = torch.empty(7, 7)
    assert d1(a) == "q"
    files = list((tmp_path / "c").rglob("backend_dispatch.json"))
    assert len(files) == 1
    payload = json.loads(files[0].read_text())
    assert payload == {"op": "<lambda>", "key": [7, 7, "torch.float32"], "winner": "q",
                       "timings": {"p": 3.0, "q": 2.0}}
    # a new process-alike instance loads the winner without timing anything
    timer.clear()
    d2 = mk()
    assert d2(a) == "q" and d2.timings[(7, 7, "torch.float32")] == {"p": 3.0, "q": 2.0}
    # corrupted file -> treated as a miss, re-benchmarked
    files[0].write_text("{not json")
    timer.update({"p": 1.0, "q": 2.0})
    d3 = mk()
    assert d3(a) == "p"


def test_unwritable_cache_dir_is_not_fatal(timer, tmp_path, monkeypatch, caplog):
    blocker = tmp_path / "file"
    blocker.write_text("x")
    monkeypatch.setenv("TRITONIX_B200_CACHE_DIR", str(blocker / "sub"))
    timer.update({"p": 1.0})
    d = dynamic_dispatch({"p": lambda a: "p"}, key=["a"])
    with caplog.at_level(logging.WARNING, logger="tritonix.dispatcher"):
        assert d(torch.empty(1)) == "p"
    assert any("disk write failed" in r.message for r in caplog.records)


def test_matmul_dispatcher_surface():
    import tritonix_b200 as t
    assert isinstance(t.matmul, DynamicDispatcher)
    assert t.matmul.__name__ == "cuda_matmul" and t.matmul.backends == ["cuda"]
    with pytest.raises(KeyError):
        with t.matmul.force_backend("pytorch"):
            pass
    with pytest.raises(KeyError):
        with t.matmul.force_backend("triton"):
            pass
    # no CPU path: host tensors are rejected loudly, not computed elsewhere
    with t.matmul.force_backend("cuda"):
        with pytest.raises(RuntimeError, match="CUDA tensors"):
            t.matmul(torch.zeros(8, 8, dtype=torch.float16), torch.zeros(8, 8, dtype=torch.float16))
