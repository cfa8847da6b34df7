"""The benchmark driver contract that can be checked without a GPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_unavailable_line_and_exits_zero():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1",
                        "--steps", "2", "--warmup", "3"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-1000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


def test_bench_serving_config1_reduced_matches_oracle():
    r = subprocess.run([sys.executable, "-m", "oxide_tech_llm_engine_b200.bench_serving", "--config", "1", "--layers", "1",
                        "--prompt-len", "24", "--output-len", "6"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["config"] == 1 and out["reduced"] and out["generated"] == 6
    assert out["oracle_max_gap_sigma"] < 0.3
