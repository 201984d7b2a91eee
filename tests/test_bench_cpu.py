"""bench.py's CPU-only pieces: the FLOP accounting and the reference arm (the reference's CPU path timed on a
bounded sample), which must run on a machine without a GPU and print the contract's JSON line."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def test_visible_pairs_matches_the_mask(oracle):
    import bench
    assert bench.visible_pairs(100, 0) == 100 * 100
    for seq, block in ((54, 6), (54, 18), (100, 7), (32760, 4680)):
        if seq <= 200:
            want = sum(1 for q in range(seq) for k in range(seq) if oracle.block_causal_allows(block, 0, 0, q, k))
        else:
            want = 4680 * 4680 * 28  # 7 chunks: 1 + 2 + ... + 7 chunk pairs
        assert bench.visible_pairs(seq, block) == want
    # the work figures the roofline is computed from
    assert abs(4.0 * 40 * bench.visible_pairs(75600, 0) * 128 / 1e12 - 117.05) < 0.01
    assert abs(4.0 * 24 * bench.visible_pairs(32760, 0) * 128 / 1e12 - 13.188) < 0.001
    assert abs(4.0 * 12 * bench.visible_pairs(32760, 4680) * 128 / 1e12 - 3.768) < 0.001


def test_reference_arm_prints_the_contract_line(oracle):
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "tiny", "--steps", "2",
                          "--warmup", "1", "--cpu-rows", "16", "--cpu-heads", "2", "--cpu-tokens", "64"],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "tiny" in line["config"]["workload"]


def test_reference_arm_non_zero_ranks_do_nothing(oracle):
    import os
    env = {**os.environ, "RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--workload", "tiny"],
                         capture_output=True, text=True, timeout=120, env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""
