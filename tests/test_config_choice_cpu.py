"""Host-side choice of kernel configurations (no GPU): the defaults used when tuning is off, the
filter that keeps hopeless configurations out of the first call's sweep, and the seeds."""
import sys

import tritonix_b200  # noqa: F401  (loads the package; the ops module is reached through sys.modules)

mm = sys.modules["tritonix_b200.ops.matmul"]


def test_double_tiles_are_the_default_for_long_k_and_full_waves():
    big = mm.default_config(8192, 8192, 8192)
    assert (big["block_m"], big["block_n"], big["block_k"], big["num_stages"]) == (256, 512, 64, 4)
    assert mm.default_config(32768, 4096, 14336)["block_n"] == 512        # the MLP's down projection
    assert mm.default_config(8192, 28672, 4096)["block_n"] == 256         # K too short to pay for it
    # 4096 rows: 256 double tiles = 3.46 waves over 74 CTA pairs, 512 single tiles = 6.92
    assert mm.default_config(4096, 8192, 8192)["block_n"] == 256
    assert mm.default_config(2048, 8192, 8192)["block_n"] == 512
    small = mm.default_config(512, 512, 8192)
    assert small["block_m"] == 128 and small["split_k"] > 1                # too few tiles: split K


def test_sweep_filter_knows_what_a_double_tile_needs():
    keep = mm._plausible(8192, 8192)
    base = dict(block_m=256, block_n=512, block_k=64, group_m=8, split_k=1, num_stages=4, acc_stages=2)
    assert keep(base)
    assert not keep({**base, "block_m": 128})
    assert not keep({**base, "split_k": 2})
    assert not keep({**base, "acc_stages": 1})
    assert not mm._plausible(8192, 256)(base)                             # wider than the problem
    assert not keep({**base, "block_n": 256, "acc_stages": 1})            # more tiles than SMs


def test_seeds_start_with_the_double_tile_and_fit_the_space():
    seeds = mm.seed_configs(8192, 8192, 8192)
    assert seeds[0]["block_n"] == 512 and seeds[0]["block_m"] == 256
    space = mm.matmul_kernel.space
    for cfg in seeds + mm.seed_configs(64, 4096, 14336, split_k=4):
        assert set(cfg) == set(space)
        assert all(cfg[k] in space[k].values() for k in cfg), cfg
