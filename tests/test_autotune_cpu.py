"""Tuner behaviour without a GPU: the timer is replaced by a synthetic cost model.  The
expected visiting orders, pruning decisions and winners in tests/golden/host_logic.json were
recorded from the reference's own TunableKernel (tests/golden/make_host_golden.py)."""
import json
import os

import pytest

import tritonix_b200.autotune as autotune
from tritonix_b200 import Choice, OutOfResources, PowerOfTwo, Range, TunableKernel, tunable

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = json.load(open(os.path.join(HERE, "golden", "host_logic.json")))


@pytest.fixture(autouse=True)
def fake_timer(monkeypatch):
    monkeypatch.setattr(autotune, "do_bench", lambda fn, warmup=None, rep=None, **kw: fn())


def make_launcher(log, model):
    def launcher(cfg):
        r = model(cfg)
        log.append([dict(cfg), r])
        if r == "OOM":
            raise OutOfResources("does not fit")
        if r == "SKIP":
            raise ValueError("invalid")
        return r
    return launcher


def golden_cost_model():
    import importlib.util
    spec = importlib.util.spec_from_file_location("mhg", os.path.join(HERE, "golden", "make_host_golden.py"))
    src = open(spec.origin).read()
    ns = {}
    start = src.index("def cost_model")
    end = src.index("def main")
    exec(src[start:end], ns)  # only the pure cost function, none of the reference imports
    return ns["cost_model"]


@pytest.mark.parametrize("run", GOLD["tuner"], ids=[r["label"] for r in GOLD["tuner"]])
def test_grid_search_replays_reference(run):
    order = run["memory_axes_order"]
    names = order + [n for n in run["space"] if n not in order]
    space = {n: Choice(run["space"][n]) for n in names}
    mem = set(order)

    class Kernel:
        pass

    tk = tunable(keys=["m", "n", "k"], space=space, memory_params=mem)(Kernel())
    assert isinstance(tk, TunableKernel) and tk.kernel.specialize_keys == ["m", "n", "k"]
    log = []
    filt = (lambda c: c["block_k"] >= 32) if run["filter"] else None
    best = tk.tune(make_launcher(log, golden_cost_model()), max_configs=run["max_configs"], filter_fn=filt)
    assert best == run["best"]
    assert log == run["visited"]


def test_configs_cross_product_order():
    class Kernel:
        pass
    run = GOLD["tuner"][0]
    tk = tunable(keys=[], space={n: Choice(v) for n, v in run["space"].items()})(Kernel())
    cfgs = tk.configs()
    assert len(cfgs) == run["n_configs"] and cfgs[:5] == run["first_configs"]
    assert len(tk.configs(lambda c: c["group_m"] == 8)) == run["n_configs"] // 2


def test_num_stages_is_always_a_memory_axis_and_delegation():
    class Kernel:
        tag = "k"

        def __getitem__(self, grid):
            return ("launch", grid)

    tk = tunable(keys=["m"], space={"stages": Range(2, 4), "x": Choice([1])})(Kernel())
    assert {"num_stages", "stages"} <= tk.memory_params
    assert tk.tag == "k" and tk[(2, 3)] == ("launch", (2, 3))
    assert TunableKernel(tk, ["m"], tk.space, tk.memory_params).kernel is tk.kernel  # unwraps


def test_memory_rank_orders_a_decreasing_axis():
    """cta_group=2 needs less shared memory per CTA than cta_group=1: with memory_rank the trie
    visits 2 before 1 and an out-of-resources at cta_group=1 does not hide cta_group=2."""
    class Kernel:
        pass
    tk = tunable(keys=[], space={"stages": Range(2, 6), "cta_group": Choice([1, 2])},
                 memory_params={"cta_group"}, memory_rank={"cta_group": lambda g: -g})(Kernel())
    log = []

    def model(cfg):
        need = cfg["stages"] * (2 if cfg["cta_group"] == 1 else 1)
        return "OOM" if need > 6 else 10.0 / cfg["stages"] + (0.1 if cfg["cta_group"] == 1 else 0.0)
    best = tk.tune(make_launcher(log, model))
    assert best == {"stages": 6, "cta_group": 2}
    tried = [(c["stages"], c["cta_group"]) for c, _ in log]
    assert (4, 1) in tried and (5, 1) not in tried  # pruned above the first failure
    assert (6, 2) in tried


def test_all_failing_returns_none_and_other_errors_propagate():
    class Kernel:
        pass
    tk = tunable(keys=[], space={"stages": Range(2, 3)})(Kernel())
    assert tk.tune(make_launcher([], lambda c: "SKIP")) is None
    assert tk.tune(make_launcher([], lambda c: "OOM")) is None

    def boom(cfg):
        raise RuntimeError("device fault")
    with pytest.raises(RuntimeError):
        tk.tune(boom)


def test_bayesian_needs_ax():
    class Kernel:
        pass
    tk = tunable(keys=[], space={"stages": Range(2, 3)})(Kernel())
    try:
        import ax  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError):
            tk.tune(lambda c: 1.0, method="bayesian", max_evals=2)


def test_shipped_kernel_spaces_are_consistent():
    import tritonix_b200 as t
    for tk in (t.matmul_kernel, t.gemm_splitk_kernel, t.glu_kernel, t.swiglu_kernel):
        assert isinstance(tk, TunableKernel) and tk.keys == ["m", "n", "k"]
        names, values = tk._memory_axes()
        # the reference's memory axes plus the TMEM accumulator count
        assert set(names) == {"block_m", "block_n", "block_k", "num_stages", "acc_stages"}
        assert values[names.index("block_m")][0] == max(tk.space["block_m"].values())
    assert len(t.matmul_kernel.configs()) == 2 * 4 * 2 * 3 * 4 * 7 * 2


def test_seeds_steady_state_and_finalists():
    """Seeds are timed first (and only if they are points of the space), the sweep still covers
    the rest, and the final alternating round can overturn the sweep's ranking."""
    from tritonix_b200 import autotune as A
    calls = []

    class Kernel:
        pass
    tk = tunable(keys=[], space={"a": Choice([1, 2, 3]), "stages": Range(2, 4)})(Kernel())
    cost = {(1, 2): 5.0, (2, 2): 4.0, (3, 2): 6.0, (1, 3): 5.5, (2, 3): 3.0, (3, 3): 7.0,
            (1, 4): 5.2, (2, 4): 3.5, (3, 4): 8.0}
    state = {"final": False}

    def fake_bench(fn, warmup=None, rep=None, **kw):
        cfg = fn()
        key = (cfg["a"], cfg["stages"])
        calls.append(key)
        # in the final round (short budgets) the sweep's runner-up turns out to be faster
        if rep is not None and rep <= 30 and key == (2, 4):
            return 2.5
        return cost[key]
    old = A.do_bench
    A.do_bench = fake_bench
    try:
        best = tk.tune(lambda c: c, seeds=[{"a": 3, "stages": 4}, {"a": 9, "stages": 2}, {"a": 1}])
        assert best == {"a": 2, "stages": 3}
        assert calls[0] == (3, 4)                       # the valid seed came first, the others were dropped
        assert len(calls) == len(set(calls))            # and it was not timed twice
        calls.clear()
        best = tk.tune(lambda c: c, finalists=3)
        assert best == {"a": 2, "stages": 4}
        assert calls[-9:].count((2, 4)) == 3 and calls[-9:].count((2, 3)) == 3
    finally:
        A.do_bench = old
