"""The drop-in command-line driver: argument rules without a GPU; on a GPU, the phrases the reference's scripts grep,
and the REFERENCE's own driver source (compiled unmodified, oracle/_ref/reference_driver_*) running on this library."""
import json
import subprocess
from pathlib import Path

import numpy as np
import pytest

import oracle

from cases import small_cases

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "matxtract_b200" / "lib"
CLI = {"fp64": LIB / "matxtract_perftest_fp64", "fp16": LIB / "matxtract_perftest_fp16"}
REFDRV = {"fp64": ROOT / "oracle" / "_ref" / "reference_driver_fp64", "fp16": ROOT / "oracle" / "_ref" / "reference_driver_fp16"}


def run(cmd):
    return subprocess.run([str(c) for c in cmd], capture_output=True, text=True, timeout=600)


@pytest.mark.parametrize("tag", ["fp64", "fp16"])
def test_argument_rules_match_the_reference(tag):
    # reference test/test_autotc_spmv.cpp:1052-1076 — all of these return before any CUDA call
    r = run([CLI[tag]])
    assert r.returncode == 1 and "Run the code by './matxtract_perftest (col_frac) (hot_frac) matrix.mtx'." in r.stdout
    r = run([CLI[tag], "0.25", "0.5", "nothing.mtx"])
    assert r.returncode == 1 and "Error: col_frac must be greater than hot_frac." in r.stdout
    r = run([CLI[tag], "0.5", "0.25", "extra", "nothing.mtx"])
    assert r.returncode == 1 and "Error: Too many arguments provided." in r.stdout


@pytest.fixture(scope="module")
def mtx(tmp_path_factory):
    name, n, rp, ci = small_cases()[2]  # skew300
    path = tmp_path_factory.mktemp("mtx") / f"{name}.mtx"
    oracle.write_mtx(path, n, n, rp, ci)
    return path


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ["fp64", "fp16"])
@pytest.mark.parametrize("tau", [(), ("0.5", "0.25"), ("0.75", "0.75")])
def test_cli_prints_the_phrases_the_reference_scripts_grep(tag, tau, mtx):
    r = run([CLI[tag], *tau, mtx])
    assert r.returncode == 0, r.stderr
    out = r.stdout
    assert f" Processing the {mtx} graph in {'FP64' if tag == 'fp64' else 'FP16'}" in out
    assert "MatXtract time = " in out and " ms" in out
    assert "Success! All values match within the tolerance for 300 elements." in out
    assert "MatXtract GFLOPS= " in out
    if tau:
        assert "cols_ratio = " in out and "TC_nnz_ratio = " in out
    rec = json.loads(out.strip().splitlines()[-1])
    assert rec["rows"] == 300 and rec["cpu_cores_used"] == 1


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ["fp64", "fp16"])
@pytest.mark.parametrize("tau", [(), ("0.5", "0.25")])
def test_reference_driver_source_runs_on_this_library(tag, tau, mtx):
    if not REFDRV[tag].exists():
        pytest.skip("oracle/_ref/reference_driver_* not built (needs the reference sources)")
    r = run([REFDRV[tag], *tau, mtx])
    assert r.returncode == 0, r.stderr
    assert "Success! All values match within the tolerance for 300 elements." in r.stdout
    assert "MatXtract time = " in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ["fp64", "fp16"])
def test_reference_cdspmv_driver_source_runs_on_this_library(tag, mtx):
    """The reference's second driver (test/test_cdspmv.cpp, its cuda_perftest target: cdspmv timed beside cuSPARSE and
    checked against its serial product), compiled unmodified and linked against this library's cdspmv."""
    exe = ROOT / "oracle" / "_ref" / f"reference_cdspmv_{tag}"
    if not exe.exists():
        pytest.skip("oracle/_ref/reference_cdspmv_* not built (needs the reference sources)")
    r = run([exe, mtx])
    assert r.returncode == 0, r.stderr
    assert "cd_perf:" in r.stdout and "our_pre:" in r.stdout and "cusparse_perf:" in r.stdout
    assert "Success! All values match within the tolerance for 300 elements." in r.stdout


def test_extract_features_usage_without_arguments():
    r = run([LIB / "extract_features"])
    assert r.returncode == 1 and "<mtx_root_folder> <output_csv>" in r.stderr


@pytest.mark.gpu
def test_extract_features_writes_the_reference_csv(tmp_path):
    """ML/extract_features.cpp:95-217: one row per <root>/<name>/<name>.mtx, the reference's header, default stream
    formatting (6 significant digits)."""
    import csv

    cases = {c[0]: c for c in small_cases()}
    root = tmp_path / "root"
    for name in ("skew300", "powerlaw500"):
        _, n, rp, ci = cases[name]
        (root / name).mkdir(parents=True)
        oracle.write_mtx(root / name / f"{name}.mtx", n, n, rp, ci)
    (root / "stray.txt").write_text("not a folder")
    out = tmp_path / "features.csv"
    r = run([LIB / "extract_features", root, out])
    assert r.returncode == 0, r.stderr
    assert f"Feature extraction done. Results saved to {out}" in r.stdout
    rows = list(csv.reader(out.open()))
    header = rows[0]
    assert header[:9] == ["MatrixName", "nrows", "ncols", "nnz", "rowMean", "rowStd", "rowMin", "rowMax", "rowPRatio"]
    assert len(header) == 4 + 48 and header[-1] == "colHot90" and header[28] == "colMean"
    got = {r[0]: r for r in rows[1:]}
    assert set(got) == {"skew300", "powerlaw500"}
    for name, rec in got.items():
        _, n, rp, ci = cases[name]
        o = oracle.matrix_features(n, n, rp, ci)
        assert [int(v) for v in rec[1:4]] == [n, n, len(ci)]
        np.testing.assert_allclose([float(v) for v in rec[4:28]], o["row"], rtol=1e-5, atol=1e-12)
        np.testing.assert_allclose([float(v) for v in rec[28:52]], o["col"], rtol=1e-5, atol=1e-12)
