"""The benchmark configurations at FULL size: bit-exact partition against the CPU oracle where the oracle finishes in
about a minute (C2, C3, C4), and size-independent properties (exactly accumulated product, linearity, determinism,
conservation of entries) for the large power-law shape."""
import numpy as np
import pytest

import matxtract_b200 as mx
import oracle
from matxtract_b200 import FP16, FP64, synth

from test_gpu_parity import TOL, _bits, assert_partition_equal, check_y

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,tau", [("c2", (0.46, 0.33)), ("c3", (0.5, 0.5)), ("c4", (0.5, 0.25))])
def test_full_size_partition_is_bit_exact(name, tau):
    m = synth.generate(name)
    dtype, n, rp, ci, val, x = m["dtype"], m["n"], m["row_ptr"], m["col_ind"], m["val"], m["x"]
    h = mx.MatXtract(dtype)
    h.upload_csr(n, n, rp, ci, val)
    s = h.partition(*tau)
    o = oracle.partition(dtype, n, n, rp, ci, val, *tau)
    assert_partition_equal(dtype, h, o)
    # conservation: every entry is in exactly one half
    assert s.nnzRowD + s.nnzCD == m["nnz"] and s.dCols + s.sCols == n and s.dRows + s.sRows == n
    for mode in (mx.DD_TILE, mx.DD_CSR):
        h.set_dd_executor(mode)
        y = h.spmv_host(x)
        check_y(dtype, y, rp, ci, val, x)
        np.testing.assert_array_equal(_bits(y), _bits(h.spmv_host(x)))
    assert h.device_error() == 0
    h.close()


def test_large_powerlaw_properties():
    """C5's shape at 16 M rows (≈2.4e8 non-zeros, x larger than L2), tau = (0,0) and a tuned tau."""
    n = 16_000_000
    m = synth.generate("c5", n=n)
    rp, ci, val, x = m["row_ptr"], m["col_ind"], m["val"], m["x"]
    exact = oracle.exact_spmv(rp, ci, val, x)
    absrow = oracle.exact_spmv(rp, ci, np.abs(val), np.abs(x)).max()
    h = mx.MatXtract(FP64)
    h.upload_csr(n, n, rp, ci, val)
    h.partition(0.0, 0.0)
    y0 = h.spmv_host(x)
    assert np.abs(y0 - exact).max() / absrow <= TOL[FP64]
    np.testing.assert_array_equal(_bits(y0), _bits(h.spmv_host(x)))  # bit-reproducible
    # linearity: A(x + z) = Ax + Az up to rounding
    z = np.roll(x, 12345)
    yz, yxz = h.spmv_host(z), h.spmv_host(x + z)
    assert np.abs(yxz - (y0 + yz)).max() / (2 * absrow) <= 1e-12
    # the split execution gives the same product
    s = h.partition(0.7, 0.5)
    assert s.nnzRowD + s.nnzCD == m["nnz"]
    y1 = h.spmv_host(x)
    assert np.abs(y1 - exact).max() / absrow <= TOL[FP64]
    assert h.device_error() == 0
    h.close()


def test_one_billion_nonzeros_with_an_active_partition():
    """The 64 M-row, ~1e9-non-zero configuration at FULL size, extracted with a non-zero tau (int32 offsets up to
    ~2^30, fragment slots counted in 64 bits): conservation of entries, determinism of the extraction and of the
    product, and y against an exactly accumulated product on rows sampled from the whole matrix.  Also the plain
    product through the column-slab passes, which this size selects by itself."""
    n = 64_000_000
    m = synth.generate("c5", n=n)
    rp, ci, val, x = m["row_ptr"], m["col_ind"], m["val"], m["x"]
    nnz = m["nnz"]
    assert 9e8 < nnz < 2**31
    rng = np.random.default_rng(7)
    starts = np.sort(rng.integers(0, n - 2048, 64))
    sample = np.unique(np.concatenate([np.arange(s, s + 2048) for s in starts] + [np.arange(0, 4096),
                                                                                   np.arange(n - 4096, n)]))

    def exact_rows(rows):
        out = np.empty(len(rows))
        scale = 0.0
        for k, r in enumerate(rows):
            a, b = rp[r], rp[r + 1]
            out[k] = float(np.sum(val[a:b] * x[ci[a:b]]))
            scale = max(scale, float(np.sum(np.abs(val[a:b]) * np.abs(x[ci[a:b]]))))
        return out, scale

    want, scale = exact_rows(sample)
    h = mx.MatXtract(FP64)
    h.upload_csr(n, n, rp, ci, val)
    s0 = h.partition(0.0, 0.0)
    assert s0.active == 0 and h.column_slabs[0] >= 2  # x (512 MB) is far larger than L2: slab passes chosen by timing
    y0 = h.spmv_host(x)
    assert np.abs(y0[sample] - want).max() / scale <= TOL[FP64]
    np.testing.assert_array_equal(_bits(y0), _bits(h.spmv_host(x)))
    s1 = h.partition(0.3, 0.1)
    assert s1.active == 1 and s1.nnzRowD + s1.nnzCD == nnz and s1.dCols + s1.sCols == n and s1.dRows + s1.sRows == n
    assert s1.nnzColD + s1.nnzColS == nnz and s1.nnzRowD + s1.nnzRowS == s1.nnzColD
    assert s1.nnzColD >= int(np.float32(nnz) * np.float32(0.3)) and s1.nnzRowD >= int(np.float32(nnz) * np.float32(0.1))
    y1 = h.spmv_host(x)
    assert np.abs(y1[sample] - want).max() / scale <= TOL[FP64]
    np.testing.assert_array_equal(_bits(y1), _bits(h.spmv_host(x)))
    s2 = h.partition(0.3, 0.1)  # the same extraction again: same counts, same product bits
    for k in ("dCols", "nnzColD", "dRows", "nnzRowD", "chunkNum", "totalFrags", "nnzCD"):
        assert getattr(s1, k) == getattr(s2, k), k
    np.testing.assert_array_equal(_bits(y1), _bits(h.spmv_host(x)))
    assert h.device_error() == 0
    h.close()
