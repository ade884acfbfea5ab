"""Generates tests/golden/mtx/*.npz: the CSR the REFERENCE's Matrix Market reader (utilities/mmio.cpp, compiled
unmodified into oracle/_ref) produces for each hand-written tests/golden/mtx/*.mtx, in both value types.
Run in a checkout that has the reference sources:  python tests/golden/make_mtx_golden.py"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

import oracle  # noqa: E402


def main():
    for path in sorted((HERE / "mtx").glob("*.mtx")):
        out = {}
        for dtype, tag in ((oracle.FP64, "fp64"), (oracle.FP16, "fp16")):
            m, n, rp, ci, val = oracle.ref_read_mtx(dtype, path)
            out.update({f"rows_{tag}": m, f"cols_{tag}": n, f"row_ptr_{tag}": rp, f"col_ind_{tag}": ci,
                        f"val_{tag}": val.view(np.uint8)})
        f = path.with_suffix(".npz")
        np.savez_compressed(f, **out)
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
