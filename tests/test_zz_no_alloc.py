"""The allocation-free entry point `mx_csr_spmv_static`, for callers that cannot request device memory at call time
(a solver confined to a fixed arena, a real-time loop that must not block on the driver's allocator).  It has to give
exactly what the handle-based path gives, call after call, although every call reuses the same fixed scratch array.

Collected last on purpose: a failure here cannot hide the result of any other test."""
import numpy as np
import pytest
import torch

import matxtract_b200 as mx
from matxtract_b200 import capi, synth

from cases import random_csr, values

pytestmark = pytest.mark.gpu


def _reference_y(dtype, n, rp, ci, val, x_dev):
    """The existing entry point: a handle without extraction (tau = (0,0)) and mx_spmv."""
    h = mx.MatXtract(dtype)
    h.upload_csr(n, n, rp, ci, val)
    h.partition(0.0, 0.0)
    y = torch.empty(n, dtype=x_dev.dtype, device="cuda")
    h.spmv(x_dev, y)
    h.sync()
    out = y.cpu().numpy().copy()
    del y
    torch.cuda.synchronize()
    h.close()
    return out


def _dev(a, view=None):
    t = torch.from_numpy(np.ascontiguousarray(a).view(view) if view else np.ascontiguousarray(a))
    return t.cuda()


def _static_y(dtype, n, rp, ci, val, x_dev):
    tdt = torch.float64 if dtype == mx.FP64 else torch.float16
    d_rp, d_ci = _dev(rp.astype(np.int32)), _dev(ci.astype(np.int32))
    d_val = _dev(val, np.int16 if dtype == mx.FP16 else None)
    if dtype == mx.FP16:
        d_val = d_val.view(torch.float16)
    y = torch.full((n,), float("nan"), dtype=tdt, device="cuda")  # every row must be written by the call
    torch.cuda.synchronize()
    capi.csr_spmv_static(dtype, n, n, len(ci), d_rp, d_ci, d_val, x_dev, y, stream=0)
    torch.cuda.synchronize()
    return y.cpu().numpy()


@pytest.mark.parametrize("dtype", [mx.FP64, mx.FP16])
def test_static_entry_point_matches_the_handle_path_on_consecutive_calls(dtype):
    tdt = torch.float64 if dtype == mx.FP64 else torch.float16
    # call 1: power-law rows (some span several tiles); call 2: a different, smaller matrix with empty rows, so
    # anything left over in the shared scratch from call 1 would show; call 3: the first matrix again
    m = synth.generate("c2", n=60_000, dtype=dtype)
    rp2, ci2 = random_csr(3_000, 5, 17, empty_rows=0.3)
    mats = [(m["n"], m["row_ptr"], m["col_ind"], m["val"], m["x"]),
            (3_000, rp2, ci2, values(dtype, len(ci2), 5), values(dtype, 3_000, 6)),
            (m["n"], m["row_ptr"], m["col_ind"], m["val"], values(dtype, m["n"], 7))]
    for n, rp, ci, val, x in mats:
        x_dev = _dev(x, np.int16 if dtype == mx.FP16 else None)
        x_dev = x_dev.view(tdt) if dtype == mx.FP16 else x_dev
        want = _reference_y(dtype, n, rp, ci, val, x_dev)
        got = _static_y(dtype, n, rp, ci, val, x_dev)
        # same kernels, same summation order: the two entry points agree bit for bit
        np.testing.assert_array_equal(got.view(np.uint8), want.view(np.uint8))


def test_static_entry_point_rejects_what_does_not_fit():
    t = torch.zeros(8, dtype=torch.int32, device="cuda")
    v = torch.zeros(8, dtype=torch.float64, device="cuda")
    with pytest.raises(mx.MxError) as e:
        capi.csr_spmv_static(mx.FP64, (1 << 20) + 1, 8, 4, t, t, v, v, v)
    assert e.value.status == 9
    with pytest.raises(mx.MxError) as e:
        capi.csr_spmv_static(mx.FP64, 8, 8, -1, t, t, v, v, v)
    assert e.value.status == 1


def test_static_entry_point_takes_no_device_memory():
    """After a first call (which looks up the scratch array's address), repeated calls leave the amount of free device
    memory unchanged: nothing is allocated, from the driver or from a pool, at call time."""
    m = synth.generate("c5", n=40_000)
    n, rp, ci, val = m["n"], m["row_ptr"], m["col_ind"], m["val"]
    d_rp, d_ci, d_val = _dev(rp.astype(np.int32)), _dev(ci.astype(np.int32)), _dev(val)
    x_dev = _dev(m["x"])
    y = torch.zeros(n, dtype=torch.float64, device="cuda")
    capi.csr_spmv_static(mx.FP64, n, n, len(ci), d_rp, d_ci, d_val, x_dev, y, stream=0)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        capi.csr_spmv_static(mx.FP64, n, n, len(ci), d_rp, d_ci, d_val, x_dev, y, stream=0)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
