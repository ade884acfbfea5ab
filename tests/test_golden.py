"""The CPU oracle against golden vectors produced by the reference's own host code (tests/golden/make_golden.py).
Runs anywhere: needs neither the reference sources nor a GPU."""
from pathlib import Path

import numpy as np
import pytest

import oracle

FILES = sorted((Path(__file__).parent / "golden").glob("*.npz"))


def _eq(a, b, what):
    np.testing.assert_array_equal(np.asarray(a).view(np.uint8), np.asarray(b).view(np.uint8), err_msg=what)


@pytest.mark.parametrize("path", FILES, ids=[f.stem for f in FILES])
def test_oracle_reproduces_golden(path):
    g = np.load(path)
    dtype, n = int(g["dtype"]), int(g["n"])
    tau = tuple(g["tau"])
    val = oracle.init_vec(dtype, len(g["col_ind"]))
    x = oracle.init_vec(dtype, n)
    o = oracle.partition(dtype, n, n, g["row_ptr"], g["col_ind"], val, *tau)
    st = o["stats"]
    assert list(g["ref_se_dims"]) == [st["dRows"], st["dCols"], st["nnzRowD"]]
    assert list(g["ref_cd_dims"]) == [n, n, st["nnzCD"]]
    for k in ("rowPtr_CD", "colInd_CD", "val_CD", "rowPtr_dd", "colInd_dd", "val_dd", "chunkPtr", "AToX", "fragPtr",
              "fragBit", "tcVal"):
        _eq(g["ref_" + k], o[k], k)
    _eq(g["ref_x_CD"], x[o["xperm"]], "x_CD")
    _eq(g["ref_x_d"], x[o["xperm"][:st["dCols"]]], "x_d")
    y_hot = oracle.tile_spmv_serial(dtype, x[o["xperm"][:st["dCols"]]], o["chunkPtr"], o["fragPtr"], o["fragBit"],
                                    o["tcVal"], o["AToX"], st["dRows"])
    y = np.zeros(n, y_hot.dtype)
    y[o["rId"]] = y_hot
    _eq(g["ref_y_before_cd"], y, "tile half")
    y = oracle.spmv_serial(dtype, o["rowPtr_CD"], o["colInd_CD"], o["val_CD"], x[o["xperm"]], y0=y)
    _eq(g["ref_y_final"], y, "y")
    # and the split result equals the plain serial CSR product the reference checks against
    y_plain = oracle.spmv_serial(dtype, g["row_ptr"], g["col_ind"], val, x)
    assert oracle.eqcheck(dtype, y_plain, y) == -1


def test_golden_files_present():
    assert len(FILES) >= 16
