"""CPU check of the bench's reference arm: it runs without a GPU, prints exactly one JSON line and
that line carries the keys the measurement contract asks for."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "images/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["n_gpus"] == 1 and d["steps"] == 1
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"] == {"value": d["value"], "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and d["vs_baseline"] is None


def test_layer_byte_formulas_match_the_tabulated_totals():
    sys.path.insert(0, ROOT)
    import bench
    # fwd+bwd algorithmic MB at batch 128, fp16: every tensor read or written once per pass
    want = {(96, 112, 1): 1714.8, (96, 112, 2): 1122.3, (144, 56, 1): 621.4, (144, 56, 2): 415.5, (192, 28, 1): 203.5,
            (192, 28, 2): 137.6, (384, 14, 1): 99.1, (384, 14, 2): 68.2, (960, 7, 1): 61.0, (960, 7, 2): 44.3}
    for (c, hw, s), mb in want.items():
        f, b = bench.layer_bytes(128, c, hw, s)
        assert abs((f + b) / 1e6 - mb) < 0.06 * mb / 100 + 0.1, (c, hw, s, (f + b) / 1e6)
