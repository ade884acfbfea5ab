"""Small matrices shared by the oracle, golden and GPU parity tests."""
from __future__ import annotations

import numpy as np

from matxtract_b200 import FP16, FP64, synth


def random_csr(n, mean_len, seed, sort_rows=True, empty_rows=0.0, skew=False):
    """Square CSR with distinct columns per row; optional empty rows, skewed columns, unsorted rows."""
    rng = np.random.default_rng(seed)
    lens = rng.poisson(mean_len, n)
    lens = np.minimum(lens, n)
    if empty_rows:
        lens[rng.random(n) < empty_rows] = 0
    if skew:  # a few very long rows
        for r in rng.choice(n, max(1, n // 50), replace=False):
            lens[r] = min(n, int(lens[r] * 12 + 30))
    row_ptr = np.zeros(n + 1, np.int32)
    np.cumsum(lens, out=row_ptr[1:])
    cols = np.empty(row_ptr[-1], np.int32)
    w = 1.0 / (1.0 + np.arange(n)) ** 0.9 if skew else None
    if w is not None:
        w = w[rng.permutation(n)]
        w /= w.sum()
    for r in range(n):
        c = rng.choice(n, lens[r], replace=False, p=w)
        cols[row_ptr[r]:row_ptr[r + 1]] = np.sort(c) if sort_rows else c
    return row_ptr, cols


def values(dtype, nnz, seed, kind="uniform"):
    rng = np.random.default_rng(seed + 7)
    v = rng.uniform(-1, 1, nnz) if kind == "uniform" else rng.standard_normal(nnz)
    return v.astype(np.float64 if dtype == FP64 else np.float16)


def small_cases():
    """(name, n, row_ptr, col_ind) — structures exercising ties, empty rows, long rows, ragged panels."""
    out = []
    out.append(("poisson64", 64) + random_csr(64, 6, 1))
    out.append(("poisson257_empty", 257) + random_csr(257, 5, 2, empty_rows=0.2))
    out.append(("skew300", 300) + random_csr(300, 4, 3, skew=True))
    out.append(("unsorted120", 120) + random_csr(120, 7, 4, sort_rows=False))
    m = synth.generate("c3", n=8 * 40)
    out.append(("block320", m["n"], m["row_ptr"], m["col_ind"]))
    m = synth.generate("c2", n=500)
    out.append(("powerlaw500", m["n"], m["row_ptr"], m["col_ind"]))
    m = synth.generate("c4", n=600)
    out.append(("hotcol600", m["n"], m["row_ptr"], m["col_ind"]))
    # identity-like: every column count equal -> all ties
    n = 40
    out.append(("diag40", n, np.arange(n + 1, dtype=np.int32), np.arange(n, dtype=np.int32)))
    return out


TAUS = [(0.46, 0.33), (0.5, 0.5), (0.75, 0.25), (0.25, 0.0), (1.0, 0.0), (0.9, 0.9), (0.5, 0.25)]
