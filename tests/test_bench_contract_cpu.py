"""The parts of bench.py's contract that need no GPU: the reference arm's JSON line, and that under a multi-rank launch
only rank 0 of that arm prints."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _run(extra_env=None, *args):
    env = dict(os.environ, **(extra_env or {}))
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "c1",
                           "--steps", "2", "--warmup", "1", *args], capture_output=True, text=True, timeout=300, env=env)


def test_reference_arm_prints_one_contract_line():
    r = _run()
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "spmv_gflops" and d["unit"] == "GFLOP/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 2 and d["value"] > 0
    assert d["dtype"] == "f64" and d["data"] == "synthetic" and d["vs_baseline"] is None
    assert d["config"]["workload"].startswith("c1")
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    e = d["e2e"]
    assert e["value"] == d["value"] and e["unit"] == d["unit"]
    assert e["h2d_bytes_per_step"] == 0 and e["d2h_bytes_per_step"] == 0
    # the same `config` keys as the GPU arm prints, and none of the GPU library mapped into the process
    assert {"workload", "tau", "n", "nnz", "scaling", "l2", "parallelism"} <= set(d["config"])
    assert d["config"]["n"] == 10000 and d["config"]["nnz"] > 0
    assert d["native_libs"] and not [p for p in d["native_libs"] if "libmatxtract_b200" in p or "libMatXtract" in p]
    assert any(p.startswith("oracle/") for p in d["native_libs"])


def test_reference_arm_is_silent_on_other_ranks():
    r = _run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}, "--gpus", "2")
    assert r.returncode == 0 and not [l for l in r.stdout.splitlines() if l.startswith("{")]
