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


def test_traffic_comes_from_the_tracked_table_and_names_a_stale_capture(tmp_path, monkeypatch):
    """roofline.traffic is read from profiles/dram_traffic.md, never typed into the benchmark: a row captured on the
    current kernel sources says so, a row captured on other sources is flagged, a capture of fewer rows is scaled by
    the row count, and a workload without a row yields None."""
    sys.path.insert(0, str(ROOT))
    import bench
    from matxtract_b200.build import source_hash

    (tmp_path / "profiles").mkdir()
    (tmp_path / "profiles" / "dram_traffic.md").write_text(
        "| workload | tau | kernel | rows | bytes per launch | source hash | summary |\n|---|---|---|---|---|---|---|\n"
        f"| c5 | 0,0 | k | 1000 | 5000 | {source_hash()} | a.md |\n"
        "| c2 | 0.46,0.33 | k | 2000 | 7000 | 0123456789ab | b.md |\n")
    monkeypatch.setattr(bench, "ROOT", tmp_path)
    b, note = bench.profiled_traffic("c5", "k", (0.0, 0.0), 1000)
    assert b == 5000 and "unchanged" in note
    b, note = bench.profiled_traffic("c5", "k", (0.0, 0.0), 4000)
    assert b == 20000 and "scaled to 4000 rows" in note
    b, note = bench.profiled_traffic("c2", "k", (0.46, 0.33), 2000)
    assert b == 7000 and "CHANGED" in note
    assert bench.profiled_traffic("c3", "k", (0.5, 0.5), 10)[0] is None
    # the committed table has a row for the default workload
    monkeypatch.setattr(bench, "ROOT", ROOT)
    b, _ = bench.profiled_traffic("c5", "resid_kernel(+fixup) column-slab passes + k_combine", (0.0, 0.0), 64_000_000)
    assert b and b > 1e10
