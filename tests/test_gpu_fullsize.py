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
