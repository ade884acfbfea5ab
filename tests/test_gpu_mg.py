"""The multi-GPU entry of the C ABI (mx_mg_*): one process drives the GPUs of the box.  With one GPU the exchange is
empty but every call is exercised; with two or more, the fused peer-store exchange and the NCCL exchange must give the
same bits, and every GPU must hold the same y."""
import numpy as np
import pytest

import matxtract_b200 as mx
import oracle
from matxtract_b200 import FP16, FP64, synth

from conftest import has_gpu

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not has_gpu(), reason="needs a CUDA device")]


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint8)


def _gpus():
    import torch

    return torch.cuda.device_count()


@pytest.mark.parametrize("name,n,tau", [("c5", 120_000, (0.0, 0.0)), ("c2", 90_000, (0.46, 0.33)),
                                        ("c3", 8 * 6000, (0.5, 0.5)), ("c4", 80_000, (0.5, 0.25))])
def test_single_process_multi_gpu_product(name, n, tau):
    m = synth.generate(name, n=n)
    dtype, rp, ci, val, x = m["dtype"], m["row_ptr"], m["col_ind"], m["val"], m["x"]
    y_ref = oracle.spmv_serial(dtype, rp, ci, val, x)
    tol = 1e-12 if dtype == FP64 else 2e-3
    for world in sorted({1, min(2, _gpus()), min(4, _gpus())}):
        g = mx.MultiGpu(dtype, world)
        g.upload_csr(n, n, rp, ci, val)
        np.testing.assert_array_equal(g.bounds, mx.mg_partition_rows(rp, world))
        stats = g.partition(*tau)
        assert len(stats) == world and all(s.active == (1 if tau != (0.0, 0.0) else 0) for s in stats)
        if world > 1 and tau != (0.0, 0.0):
            # the rankings are those of the whole matrix: every slab has the same hot columns, and the slabs' hot
            # rows add up to the whole matrix's (a slab that owns none still extracts one row)
            whole = oracle.partition(dtype, n, n, rp, ci, val, *tau)["stats"]
            assert {s.dCols for s in stats} == {whole["dCols"]}
            assert whole["dRows"] <= sum(s.dRows for s in stats) <= whole["dRows"] + world
        y = g.spmv(x)
        assert oracle.y_error(dtype, y, y_ref, rp, ci, val, x) <= tol
        y2 = g.spmv(x)  # the second product lands in the other buffer
        np.testing.assert_array_equal(_bits(y), _bits(y2))
        for d in range(world):
            np.testing.assert_array_equal(_bits(g.y_of(d)), _bits(y))
        if world > 1:
            g.set_exchange(mx.capi.MG_EXCHANGE_NCCL)
            np.testing.assert_array_equal(_bits(g.spmv(x)), _bits(y))
            g.set_exchange(mx.capi.MG_EXCHANGE_PEER)
            np.testing.assert_array_equal(_bits(g.spmv(x)), _bits(y))
        assert g.spmv_timed(x, warm=2, iters=5) > 0
        g.close()


def test_multi_gpu_handle_refuses_bad_arguments():
    with pytest.raises(mx.MxError):
        mx.MultiGpu(FP64, 0)
    with pytest.raises(mx.MxError):
        mx.MultiGpu(FP64, 2, devices=[0, 0])  # two slabs must not share a GPU
    g = mx.MultiGpu(FP64, 1)
    with pytest.raises(mx.MxError) as e:
        g.spmv(np.zeros(4))
    assert e.value.status == 4
    g.close()
