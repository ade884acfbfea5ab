"""Inputs are checked before any kernel dereferences them: a matrix with a bad index, or a stored partition with a
corrupted array, is refused with MX_ERR_INVALID and nothing is launched on it."""
import numpy as np
import pytest

import matxtract_b200 as mx
from matxtract_b200 import FP16, FP64, synth

from conftest import has_gpu

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not has_gpu(), reason="needs a CUDA device")]


@pytest.mark.parametrize("dtype", [FP64, FP16])
def test_matrix_with_a_bad_index_is_refused_at_upload(dtype):
    m = synth.generate("c2", n=4000, dtype=dtype)
    n, rp, ci, val = m["n"], m["row_ptr"], m["col_ind"].copy(), m["val"]
    h = mx.MatXtract(dtype)
    for bad_value in (n, -1, 2**31 - 1):
        bad = ci.copy()
        bad[len(bad) // 2] = bad_value
        with pytest.raises(mx.MxError) as e:
            h.upload_csr(n, n, rp, bad, val)
        assert e.value.status == 1
        # nothing was kept: no extraction, no product, no launches on the refused matrix
        with pytest.raises(mx.MxError) as e:
            h.partition(0.0, 0.0)
        assert e.value.status == 4
        assert h.launches_per_spmv == 0 and h.device_error() == 0
    rp_bad = rp.copy()
    rp_bad[10], rp_bad[11] = rp[11] + 3, rp[10]  # decreases, ends unchanged
    with pytest.raises(mx.MxError) as e:
        h.upload_csr(n, n, rp_bad, ci, val)
    assert e.value.status == 1
    # the handle is still usable with a good matrix
    h.upload_csr(n, n, rp, ci, val)
    h.partition(0.46, 0.33)
    y = h.spmv_host(m["x"])
    assert np.isfinite(y.astype(np.float64)).all()
    h.close()


def test_corrupted_stored_partition_is_refused_before_upload(tmp_path):
    m = synth.generate("c4", n=20_000, dtype=FP64)
    n = m["n"]
    a = mx.MatXtract(FP64)
    a.upload_csr(n, n, m["row_ptr"], m["col_ind"], m["val"])
    st = a.partition(0.5, 0.25)
    path = tmp_path / "p.mxp"
    a.save_partition(path)
    data = bytearray(path.read_bytes())
    # the first array behind the 88-byte header is xperm ([u64 size][n ints]): point one entry far outside
    off = 88 + 8 + 4 * 7
    data[off:off + 4] = (2**30).to_bytes(4, "little")
    bad = tmp_path / "bad.mxp"
    bad.write_bytes(bytes(data))
    b = mx.MatXtract(FP64)
    with pytest.raises(mx.MxError) as e:
        b.load_partition(bad)
    assert e.value.status == 1 and "xperm" in str(e.value)
    assert b.launches_per_spmv == 0
    b.load_partition(path)  # the intact file still loads into the same handle
    assert b.stats.dRows == st.dRows
    for h in (a, b):
        h.close()
