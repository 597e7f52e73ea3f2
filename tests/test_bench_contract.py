"""The JSON line of bench.py's reference arm (the arm that runs without a GPU): keys and invariants the benchmark contract
names. The GPU arm prints the same keys plus roofline / clocks / gpu_launches; it is exercised on a B200 by running bench.py."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_reference(*extra):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "3", *extra],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, "exactly one JSON line"
    return json.loads(lines[0])


def test_reference_arm_prints_the_contract_keys():
    d = run_reference()
    assert d["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["unit"] == "tokens/s" and d["higher_is_better"] is True and d["vs_baseline"] is None
    assert d["warmup"] >= 3 and d["value"] > 0 and d["ms_per_step"] > 0
    assert d["config"]["workload"] == "serve64" and d["config"]["tokens"] == 64 and d["config"]["layers"] == 40
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["sample"] and cb["value"] == d["value"]
    e = d["e2e"]
    assert e["value"] == d["value"] and e["unit"] == d["unit"] and e["h2d_bytes_per_step"] == 0 and e["d2h_bytes_per_step"] == 0


def test_reference_arm_of_another_workload_names_it():
    d = run_reference("--workload", "mtp4")
    assert d["config"]["workload"] == "mtp4" and d["config"]["tokens"] == 4
