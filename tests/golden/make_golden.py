"""Generates tests/golden/*.npz from the REFERENCE's own host code (oracle/_ref, built from the reference sources by
oracle/Makefile).  Run in a checkout that has the reference sources:  python tests/golden/make_golden.py

Each file holds one small matrix, one (tau_c, tau_r), one precision, and every array the reference's main() handed to
its GPU API for it (residual CSR, permuted x, core-dense block, final y), plus the tile arrays its
ecrPreprocess_opt1 + generateFormat_opt[_fp16] build from that block.  Values are the driver's own i % 15.
"""
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

import oracle  # noqa: E402
from cases import small_cases  # noqa: E402

GOLDEN = [("poisson64", (0.46, 0.33)), ("poisson257_empty", (0.5, 0.5)), ("skew300", (0.75, 0.25)),
          ("unsorted120", (0.5, 0.25)), ("block320", (0.5, 0.5)), ("powerlaw500", (0.46, 0.33)),
          ("hotcol600", (0.25, 0.0)), ("diag40", (0.5, 0.5)), ("hotcol600", (0.75, 0.5))]


def main():
    cases = {c[0]: c for c in small_cases()}
    with tempfile.TemporaryDirectory() as tmp:
        for name, tau in GOLDEN:
            _, n, row_ptr, col_ind = cases[name]
            path = Path(tmp) / f"{name}.mtx"
            oracle.write_mtx(path, n, n, row_ptr, col_ind)
            for dtype, tag in ((oracle.FP64, "fp64"), (oracle.FP16, "fp16")):
                m, nn, rp, ci, _ = oracle.ref_read_mtx(dtype, path)
                ref = oracle.ref_run_main(dtype, path, *tau)
                assert ref["rc"] == 0
                tiles = oracle.ref_build_tiles(dtype, ref["rowPtr_dd"], ref["colInd_dd"], ref["val_dd"],
                                               int(ref["se_dims"][1]))
                out = {"n": n, "tau": np.array(tau), "dtype": dtype, "row_ptr": rp, "col_ind": ci}
                for k in ("rowPtr_CD", "colInd_CD", "val_CD", "x_CD", "rowPtr_dd", "colInd_dd", "val_dd", "x_d",
                          "se_dims", "cd_dims", "y_before_cd", "y_final"):
                    out["ref_" + k] = ref[k]
                for k, v in tiles.items():
                    out["ref_" + k] = v
                f = HERE / f"{name}_{tau[0]}_{tau[1]}_{tag}.npz"
                np.savez_compressed(f, **out)
                print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
