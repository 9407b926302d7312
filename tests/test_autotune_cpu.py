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
        assert set(names) == {"block_m", "block_n", "block_k", "num_stages"}  # the reference's axes
        assert values[names.index("block_m")][0] == max(tk.space["block_m"].values())
    assert len(t.matmul_kernel.configs()) == 2 * 3 * 2 * 3 * 4 * 7
