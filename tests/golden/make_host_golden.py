"""Generates tests/golden/host_logic.json by running the REFERENCE's host-side code
(ayghri/tritonix: MonotonicCascadeTrie, CoordinateUnimodalFunction, TunableKernel, the Hilbert
helpers, the dispatcher's key functions) on fixed scenarios.  Run where the reference tree is
mounted:

    python tests/golden/make_host_golden.py <path to the reference source tree>

The tuner is driven with a deterministic cost model in place of the GPU timer
(triton.testing.do_bench is replaced for the run), so the recorded visiting order, the
pruning decisions and the winner are exactly the reference's.
"""
from __future__ import annotations

import json
import os
import sys

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, REPO)
os.environ["TRITON_INTERPRET"] = "1"

import importlib  # noqa: E402

from oracle.ref_loader import load_reference  # noqa: E402


def cost_model(cfg):
    """Synthetic kernel: returns milliseconds, raises for configs that do not fit / are invalid."""
    smem = cfg.get("num_stages", 2) * (cfg["block_m"] * cfg["block_k"] + cfg["block_k"] * cfg["block_n"]) * 2
    if smem > 96 * 1024:
        return "OOM"
    if cfg["block_m"] == 32 and cfg["block_n"] == 128:
        return "SKIP"
    t = 10.0 / (cfg["block_m"] * cfg["block_n"]) ** 0.5 + abs(cfg["block_k"] - 32) * 0.01
    t += abs(cfg.get("num_stages", 2) - 3) * 0.05 + (0.02 if cfg.get("group_m", 8) == 4 else 0.0)
    return round(t, 6)


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python " + sys.argv[0] + " <path to the reference source tree>")
    root = sys.argv[1]
    load_reference(root)
    import triton
    rp = importlib.import_module("tritonix.utils.pruners")
    rs = importlib.import_module("tritonix.utils.spaces")
    rh = importlib.import_module("tritonix.utils.hilbert")
    ra = importlib.import_module("tritonix.autotune")
    rd = importlib.import_module("tritonix.dispatcher")
    out = {}

    # ---- trie scenarios
    tries = []
    for dims, prunes in [((3, 3, 3), [(1, 1, 0)]), ((4, 4, 4, 4), [(1, 4, 4, 1), (3, 3, 3, 0), (0, 4, 0, 1), (1, 3, 0, 0)]),
                         ((4, 4, 3), [(2, 1, 0), (1, 2, 0)]), ((5, 2, 6), [(4, 1, 3), (2, 0, 5), (3, 1, 1)]), ((2, 2), [(0, 0)])]:
        t = rp.MonotonicCascadeTrie(rs.SpaceConfig({str(i): rs.Choice(range(d)) for i, d in enumerate(dims)}))
        for f in prunes:
            t.prune(f)
        tries.append({"dims": dims, "prunes": prunes, "minimal": t._minimal_failures,
                      "all": list(t.generate_all_unpruned()),
                      "midpoint": list(t.generate_all_unpruned_midpoint()),
                      "first_midpoint": t.get_mid_point_unpruned()})
    out["tries"] = tries

    # ---- unimodal pruner
    uni = []
    for dims, records in [((5, 2), [((1, 0), 1.0), ((2, 0), 2.0), ((0, 0), 3.0), ((1, 1), 0.5)]),
                          ((4, 3, 2), [((0, 0, 0), 3.0), ((1, 0, 0), 2.0), ((2, 0, 0), 2.5), ((1, 1, 0), 1.0), ((1, 2, 0), 4.0), ((1, 1, 1), 0.9)])]:
        p = rp.CoordinateUnimodalFunction(rs.SpaceConfig({str(i): rs.Choice(range(d)) for i, d in enumerate(dims)}))
        steps = []
        import itertools
        allc = list(itertools.product(*[range(d) for d in dims]))
        for idx, val in records:
            p.record(idx, val)
            steps.append({"record": [idx, val], "pruned": [c for c in allc if p.is_pruned(c)]})
        uni.append({"dims": dims, "steps": steps})
    out["unimodal"] = uni

    # ---- tuner runs with the synthetic cost model
    log = []

    def fake_bench(fn, warmup=None, rep=None, **kw):
        return fn()

    triton.testing.do_bench = fake_bench
    runs = []
    for label, space, mem, kw in [
        ("one_memory_axis", {"block_m": rs.Choice([64]), "block_n": rs.PowerOfTwo(32, 128), "block_k": rs.Choice([32]),
                             "group_m": rs.Choice([4, 8]), "num_stages": rs.Range(2, 5)}, None, {}),
        ("capped", {"block_m": rs.Choice([64]), "block_n": rs.PowerOfTwo(32, 128), "block_k": rs.Choice([32]),
                    "group_m": rs.Choice([4, 8]), "num_stages": rs.Range(2, 5)}, None, {"max_configs": 5}),
        ("filtered", {"block_m": rs.Choice([128]), "block_n": rs.PowerOfTwo(32, 256), "block_k": rs.PowerOfTwo(16, 128),
                      "group_m": rs.Choice([8]), "num_stages": rs.Range(2, 6)}, None, {"filter": "block_k>=32"}),
        ("three_memory_axes", {"block_m": rs.Choice([128]), "block_n": rs.PowerOfTwo(32, 256), "block_k": rs.PowerOfTwo(16, 128),
                               "group_m": rs.Choice([4, 8]), "num_stages": rs.Range(2, 5)}, {"block_n", "block_k"}, {}),
    ]:
        class K:  # stands in for the jitted kernel object
            pass
        tk = ra.tunable(keys=["m", "n", "k"], space=space, memory_params=mem)(K())
        trie, trie_names, _ = tk._build_trie()
        log.clear()

        def launcher(cfg):
            r = cost_model(cfg)
            log.append([dict(cfg), r])
            if r == "OOM":
                raise triton.OutOfResources(1, 1, "smem")
            if r == "SKIP":
                raise ValueError("invalid")
            return r

        filt = (lambda c: c["block_k"] >= 32) if kw.get("filter") else None
        best = tk.tune(launcher, max_configs=kw.get("max_configs"), filter_fn=filt)
        runs.append({"label": label, "space": {k: v.values() for k, v in space.items()},
                     "memory_axes_order": trie_names, "max_configs": kw.get("max_configs"),
                     "filter": kw.get("filter"), "visited": list(log), "best": best,
                     "n_configs": len(tk.configs()), "first_configs": tk.configs()[:5]})
    out["tuner"] = runs

    # ---- hilbert
    out["hilbert"] = {f"{m}x{n}": rh.hilbert_rect_coords(m, n) for m, n in [(4, 4), (3, 5), (7, 2), (8, 8), (5, 12)]}
    out["hilbert_perm_3x4"] = rh.hilbert_permutation(3, 4)

    # ---- dispatcher keys
    import torch
    a, b = torch.empty(1024, 512, dtype=torch.float16), torch.empty(512, 768, dtype=torch.float16)
    key = rd._tuning_key(["a", "b"], (a, b), {}, ["a", "b"])
    out["dispatch"] = {"tuning_key": list(key),
                       "disk_key": rd._disk_key("triton_matmul", ["triton", "pytorch"], key),
                       "disk_key_cuda": rd._disk_key("cuda_matmul", ["cuda"], key)}

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "host_logic.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1, default=list)
    print("wrote", path, os.path.getsize(path))


if __name__ == "__main__":
    main()
