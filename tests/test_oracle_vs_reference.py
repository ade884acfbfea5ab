"""Pins the CPU oracle (oracle/cpu_oracle.cpp) against the REFERENCE's own host code, compiled unmodified from its
sources into oracle/_ref (see oracle/ref_shim.cpp for what is the reference's and what is a stand-in).

The reference's main() is run on Matrix Market files; every array it hands to its GPU API (the complete partition)
is captured and compared bit-for-bit with the oracle's.  Skipped where oracle/_ref was not built."""
import numpy as np
import pytest

import oracle
from matxtract_b200 import FP16, FP64

from cases import TAUS, small_cases, values

pytestmark = pytest.mark.skipif(not oracle.ref_available(), reason="oracle/_ref not built (needs the reference sources)")

CASES = small_cases()


def _run_ref(dtype, tmp_path, case, tau):
    name, n, row_ptr, col_ind = case
    path = tmp_path / f"{name}.mtx"
    oracle.write_mtx(path, n, n, row_ptr, col_ind)
    m, nn, rp, ci, _ = oracle.ref_read_mtx(dtype, path)
    assert (m, nn) == (n, n)
    val = oracle.init_vec(dtype, len(ci))  # the driver overwrites the values with i % 15
    ref = oracle.ref_run_main(dtype, path, *tau)
    return rp, ci, val, ref


@pytest.mark.parametrize("dtype", [FP64, FP16])
@pytest.mark.parametrize("tau", TAUS)
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_partition_matches_reference_main(dtype, tau, case, tmp_path):
    n = case[1]
    rp, ci, val, ref = _run_ref(dtype, tmp_path, case, tau)
    assert ref["rc"] == 0
    nnz = len(ci)
    if int(np.float32(nnz) * np.float32(tau[0])) > nnz:
        pytest.skip("threshold above nnz: the reference itself runs into undefined behaviour")
    x = oracle.init_vec(dtype, n)
    o = oracle.partition(dtype, n, n, rp, ci, val, *tau)
    st = o["stats"]
    # residual CSR and permuted x, exactly what the reference passes to cdspmv
    assert list(ref["cd_dims"]) == [n, n, st["nnzCD"]]
    np.testing.assert_array_equal(ref["rowPtr_CD"], o["rowPtr_CD"])
    np.testing.assert_array_equal(ref["colInd_CD"], o["colInd_CD"])
    np.testing.assert_array_equal(ref["val_CD"].view(np.uint8), o["val_CD"].view(np.uint8))
    np.testing.assert_array_equal(ref["x_CD"].view(np.uint8), x[o["xperm"]].view(np.uint8))
    # the core-dense block (small inputs take the reference's sparse-encode branch, which receives dd as CSR)
    assert "rowPtr_dd" in ref, "expected the se branch at these sizes"
    assert list(ref["se_dims"]) == [st["dRows"], st["dCols"], st["nnzRowD"]]
    np.testing.assert_array_equal(ref["rowPtr_dd"], o["rowPtr_dd"])
    np.testing.assert_array_equal(ref["colInd_dd"], o["colInd_dd"])
    np.testing.assert_array_equal(ref["val_dd"].view(np.uint8), o["val_dd"].view(np.uint8))
    np.testing.assert_array_equal(ref["x_d"].view(np.uint8), x[o["xperm"][:st["dCols"]]].view(np.uint8))
    # tiles: the reference's ecrPreprocess_opt1 + generateFormat_opt[_fp16] on that block
    t = oracle.ref_build_tiles(dtype, ref["rowPtr_dd"], ref["colInd_dd"], ref["val_dd"], st["dCols"])
    for k in ("chunkPtr", "AToX", "fragPtr", "fragBit"):
        np.testing.assert_array_equal(t[k], o[k], err_msg=k)
    np.testing.assert_array_equal(t["tcVal"].view(np.uint8), o["tcVal"].view(np.uint8))
    # end result of the reference run (its own serial stand-ins): tile half scattered by rId, residual added on top
    y_hot = oracle.spmv_serial(dtype, o["rowPtr_dd"], o["colInd_dd"], o["val_dd"], x[o["xperm"][:st["dCols"]]])
    y = np.zeros(n, y_hot.dtype)
    y[o["rId"]] = y_hot
    np.testing.assert_array_equal(ref["y_before_cd"].view(np.uint8), y.view(np.uint8))
    y = oracle.spmv_serial(dtype, o["rowPtr_CD"], o["colInd_CD"], o["val_CD"], x[o["xperm"]], y0=y)
    np.testing.assert_array_equal(ref["y_final"].view(np.uint8), y.view(np.uint8))


@pytest.mark.parametrize("dtype", [FP64, FP16])
def test_tau_zero_takes_the_plain_csr_branch(dtype, tmp_path):
    case = CASES[0]
    rp, ci, val, ref = _run_ref(dtype, tmp_path, case, (0.0, 0.0))
    assert "rowPtr_dd" not in ref and "chunkPtr" not in ref
    np.testing.assert_array_equal(ref["rowPtr_CD"], rp)  # cdspmv received the input matrix itself
    np.testing.assert_array_equal(ref["colInd_CD"], ci)


@pytest.mark.parametrize("dtype", [FP64, FP16])
def test_reference_rejects_tau_c_below_tau_r(dtype, tmp_path):
    case = CASES[0]
    path = tmp_path / "a.mtx"
    oracle.write_mtx(path, case[1], case[1], case[2], case[3])
    assert oracle.ref_run_main(dtype, path, 0.25, 0.5)["rc"] == 1
    with pytest.raises(oracle.OracleError) as e:
        oracle.partition(dtype, case[1], case[1], case[2], case[3], values(dtype, len(case[3]), 0), 0.25, 0.5)
    assert e.value.status == 3


@pytest.mark.parametrize("dtype", [FP64, FP16])
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_spmv_serial_is_bit_identical(dtype, case):
    name, n, rp, ci = case
    val = values(dtype, len(ci), 11)
    x = values(dtype, n, 12)
    y0 = values(dtype, n, 13)
    a = oracle.ref_spmv_serial(dtype, rp, ci, val, x, y0)
    b = oracle.spmv_serial(dtype, rp, ci, val, x, y0)
    np.testing.assert_array_equal(a.view(np.uint8), b.view(np.uint8))


@pytest.mark.parametrize("tau", TAUS[:4])
@pytest.mark.parametrize("case", CASES[:4], ids=[c[0] for c in CASES[:4]])
def test_tile_builders_and_tile_spmv_with_random_values(tau, case):
    """Function level, FP64 and FP16, with random values (main() only ever sees i % 15)."""
    name, n, rp, ci = case
    for dtype in (FP64, FP16):
        val = values(dtype, len(ci), 21)
        o = oracle.partition(dtype, n, n, rp, ci, val, *tau)
        st = o["stats"]
        t = oracle.ref_build_tiles(dtype, o["rowPtr_dd"], o["colInd_dd"], o["val_dd"], st["dCols"])
        for k in ("chunkPtr", "AToX", "fragPtr", "fragBit"):
            np.testing.assert_array_equal(t[k], o[k], err_msg=k)
        np.testing.assert_array_equal(t["tcVal"].view(np.uint8), o["tcVal"].view(np.uint8))
        x_d = values(dtype, st["dCols"], 22)
        mine = oracle.tile_spmv_serial(dtype, x_d, o["chunkPtr"], o["fragPtr"], o["fragBit"], o["tcVal"], o["AToX"],
                                       st["dRows"])
        if dtype == FP64:
            theirs = oracle.ref_tcspmv_serial(x_d, o["chunkPtr"], o["fragPtr"], o["fragBit"], o["tcVal"], o["AToX"],
                                              st["dRows"], st["dCols"])
            np.testing.assert_array_equal(mine, theirs)
        # and the format means what the CSR means
        direct = oracle.spmv_serial(dtype, o["rowPtr_dd"], o["colInd_dd"], o["val_dd"], x_d)
        np.testing.assert_array_equal(mine.view(np.uint8), direct.view(np.uint8))
