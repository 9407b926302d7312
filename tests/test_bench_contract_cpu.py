"""bench.py's CPU arm prints one JSON line with the agreed keys (no GPU needed)."""
import json
import os
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_json_line():
    out = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference",
                          "--steps", "1", "--warmup", "1", "--workload", "splitk"],
                         capture_output=True, text=True, timeout=300, cwd=REPO)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "GEMM TFLOP/s" and d["unit"] == "TFLOP/s"
    assert d["higher_is_better"] is True and d["vs_baseline"] is None and d["data"] == "synthetic"
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["steps"] == 1
    assert d["config"]["workload"] == "splitk_gemm_f16_64x14336x4096"
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]


def test_reference_arm_other_ranks_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference",
                          "--gpus", "2", "--steps", "1"], capture_output=True, text=True,
                         timeout=120, cwd=REPO, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_tile_choice_for_row_shards():
    """Strong scaling cuts the 8192 rows of the GEMM into N blocks: double tiles unless their last
    wave over the 74 CTA pairs is much emptier than that of single tiles."""
    sys.path.insert(0, REPO)
    import bench
    assert bench.gemm_cfg_for_rows(8192, 8192) is bench.GEMM_CFG and bench.GEMM_CFG["tile_n"] == 512
    assert bench.gemm_cfg_for_rows(4096, 8192) is bench.GEMM_CFG_SHORT_K     # 3.46 waves against 6.92
    assert bench.gemm_cfg_for_rows(2048, 8192) is bench.GEMM_CFG
    assert bench.gemm_cfg_for_rows(1024, 8192) is bench.GEMM_CFG
