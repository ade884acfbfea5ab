"""The reference's ML feature vector (ML/extract_features.cpp:19-93).  CPU: the oracle's restatement against golden
vectors made by the reference's own computeDistStats, and against that function itself where oracle/_ref is built.
GPU: mx_features against the oracle - identical doubles except the standard deviation (computed from exact integer
moments on the device side; relative tolerance 1e-12)."""
from pathlib import Path

import numpy as np
import pytest

import matxtract_b200 as mx
import oracle
from matxtract_b200 import FP16, FP64, synth

from cases import small_cases, values
from feature_cases import distributions

GOLDEN = np.load(Path(__file__).parent / "golden" / "features" / "features.npz")
DISTS = list(distributions())


@pytest.mark.parametrize("name,counts", DISTS, ids=[d[0] for d in DISTS])
def test_oracle_reproduces_reference_golden(name, counts):
    np.testing.assert_array_equal(oracle.dist_stats(counts).view(np.uint64), GOLDEN[name].view(np.uint64))


@pytest.mark.skipif(not oracle.ref_available(), reason="oracle/_ref not built (needs the reference sources)")
def test_oracle_matches_reference_function_on_random_distributions():
    rng = np.random.default_rng(5)
    for _ in range(40):
        n = int(rng.integers(1, 3000))
        counts = rng.integers(0, int(rng.integers(1, 500)), n) * (rng.random(n) < rng.random())
        np.testing.assert_array_equal(oracle.dist_stats(counts).view(np.uint64),
                                      oracle.ref_dist_stats(counts).view(np.uint64))


def _check(f, n_rows, n_cols, rp, ci):
    o = oracle.matrix_features(n_rows, n_cols, rp, ci)
    assert (f.rows, f.cols, f.nnz) == (n_rows, n_cols, len(ci))
    for got, want in ((f.row.as_array(), o["row"]), (f.col.as_array(), o["col"])):
        exact = [i for i in range(24) if i != 1]
        np.testing.assert_array_equal(got[exact].view(np.uint64), want[exact].view(np.uint64))
        assert got[1] == pytest.approx(want[1], rel=1e-12, abs=0)


@pytest.mark.gpu
@pytest.mark.parametrize("case", small_cases(), ids=[c[0] for c in small_cases()])
def test_device_features_match_oracle_small(case):
    name, n, rp, ci = case
    h = mx.MatXtract(FP64)
    h.upload_csr(n, n, rp, ci, values(FP64, len(ci), 1))
    _check(h.features(), n, n, rp, ci)
    h.close()


@pytest.mark.gpu
@pytest.mark.parametrize("name,n", [("c2", 300_000), ("c3", 8 * 20_000), ("c4", 400_000), ("c5", 500_000)])
def test_device_features_match_oracle_benchmark_shapes(name, n):
    m = synth.generate(name, n=n)
    h = mx.MatXtract(m["dtype"])
    h.upload_csr(n, n, m["row_ptr"], m["col_ind"], m["val"])
    _check(h.features(), n, n, m["row_ptr"], m["col_ind"])
    h.close()


@pytest.mark.gpu
def test_device_features_rectangular_and_empty():
    rng = np.random.default_rng(3)
    rows, cols = 700, 90
    lens = rng.integers(0, 12, rows)
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ci = np.concatenate([np.sort(rng.choice(cols, k, replace=False)) for k in lens]).astype(np.int32)
    h = mx.MatXtract(FP16)
    h.upload_csr(rows, cols, rp, ci, values(FP16, len(ci), 2))
    _check(h.features(), rows, cols, rp, ci)
    h.close()
    h = mx.MatXtract(FP64)
    h.upload_csr(5, 5, np.zeros(6, np.int32), np.zeros(0, np.int32), np.zeros(0))
    _check(h.features(), 5, 5, np.zeros(6, np.int32), np.zeros(0, np.int32))
    h.close()
