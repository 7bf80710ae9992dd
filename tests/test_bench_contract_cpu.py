"""bench.py's reference arm (the CPU port of the path on the host cores) runs without a GPU and prints
one JSON line with the agreed keys; the helpers that size the roofline numerators agree with the
closed-form figures of the scope table."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "cfg1",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tok/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["n_gpus"] == 1 and line["steps"] == 1
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in line["config"] and "model" not in line["config"]


def test_algorithmic_bytes_match_the_closed_forms():
    sys.path.insert(0, ROOT)
    import bench

    assert bench.gemv_bytes(5120, 27648, 12) == pytest.approx(5120 * 27648 * 0.5625 + 4 * 27648 + 4 * 5120)
    assert bench.gemv_bytes(152064, 5120, 14, M=8) == pytest.approx(152064 * 5120 * 210 / 256 + 8 * 4 * (5120 + 152064))
    w = bench.WORKLOADS["cfg2"]
    per_token = bench.step_gemv_bytes(w, 0, w["n_layer"], True)
    assert 19.3e9 < per_token < 19.6e9  # 19.40 GB of weights per token for the 32B shape
    w3 = bench.WORKLOADS["cfg3"]
    assert 41.5e9 < bench.step_gemv_bytes(w3, 0, w3["n_layer"], True) < 42.3e9
    moe = bench.WORKLOADS["cfg4"]
    active = bench.step_gemv_bytes(moe, 0, moe["n_layer"], True)
    assert 1.5e9 < active < 2.2e9  # 8 of 128 experts per token
