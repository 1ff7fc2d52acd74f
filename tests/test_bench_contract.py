"""CPU test of bench.py's reference arm: it runs without a GPU and prints one JSON line with the contract's keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    # the arm must not load the product library: point the package at a library that does not exist, so that
    # importing it would fail
    env = dict(os.environ, LIGHTOP_B200_LIB=os.path.join(ROOT, "no_such_library.so"))
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--cpu-sample-experts", "2"], capture_output=True, text=True, timeout=600,
                         cwd=ROOT, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, res.stdout
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "fused_moe_w8a8_block_int8_tokens_per_s"
    assert d["unit"] == "tokens/s" and d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 1
    assert d["value"] > 0 and d["ms_per_step"] > 0
    assert d["config"]["workload"] == "c1_dsv3_prefill" and d["config"]["M"] == 4096 and d["config"]["E"] == 256
    # "reference" when a checkout of the reference is found ($LIGHTOP_REF, baseline/_ref), else the restatement
    assert d["cpu_baseline"]["kind"] in ("port", "reference")
    assert d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert set(d["config"]) == {"workload", "E", "top_k", "M", "hidden", "intermediate", "parallelism", "l2"}
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
