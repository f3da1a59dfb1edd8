"""The reference arm of bench.py runs on the host alone (no GPU, nothing of the CUDA library loaded) and prints the
contract's JSON line. The check runs it on a 4-layer cut so that it takes seconds; the arm itself times the 64-layer model."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "3", "--layers", "4"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["higher_is_better"] is True
    assert line["n_gpus"] == 1 and line["steps"] == 1 and 1 <= line["warmup"] <= 3 and line["vs_baseline"] is None
    assert line["value"] > 0 and line["ms_per_step"] > 0
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and "4-layer cut of the 64-layer" in cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in line["config"] and "model" not in line["config"]


def test_reference_arm_does_not_load_the_cuda_library():
    src = open(os.path.join(ROOT, "bench.py")).read()
    body = src[src.index("def cpu_rounds"):src.index("def dense_config")]
    assert "hipster_b200" not in body and "import torch" not in body
