"""The stored-partition loader's host-side check (mx_check_partition_file), without a GPU: a file written from the
oracle's partition passes; a file with one corrupted field, of the right size, is refused with a message."""
import struct

import numpy as np
import pytest

import oracle
from matxtract_b200 import FP16, FP64, capi

from cases import random_csr, values

ORDER = ("xperm", "rId", "rowPtr_dd", "colInd_dd", "val_dd", "chunkPtr", "AToX", "fragPtr", "fragBit", "tcVal",
         "rowPtr_CD", "colInd_CD", "val_CD")
HEADER = "<8s5i12iid"  # magic, version, dtype, n_rows, n_cols, nnz, 12 counts, reserved, tc_nnz_ratio


def write_partition_file(path, dtype, n, nnz, o, patch=None, header_patch=None):
    """Mirror of the layout mx_save_partition writes (header, then every array behind its byte count)."""
    arrays = {k: np.ascontiguousarray(o[k]).copy() for k in ORDER}
    if patch:
        patch(arrays)
    counts = [int(o["stats"][k]) for k in ("dCols", "nnzColD", "sCols", "nnzColS", "dRows", "nnzRowD", "sRows", "nnzRowS",
                                  "chunkNum", "totalFrags", "nnzCD")]
    hd = dict(version=2, dtype=dtype, n_rows=n, n_cols=n, nnz=nnz, counts=counts, fragK=4 if dtype == FP64 else 8)
    if header_patch:
        header_patch(hd)
    with open(path, "wb") as f:
        f.write(struct.pack(HEADER, b"MXPART02", hd["version"], hd["dtype"], hd["n_rows"], hd["n_cols"], hd["nnz"],
                            *hd["counts"], hd["fragK"], 0, float(o["stats"]["tc_nnz_ratio"])))
        for k in ORDER:
            b = arrays[k].tobytes()
            f.write(struct.pack("<Q", len(b)))
            f.write(b)


@pytest.fixture(scope="module", params=[FP64, FP16])
def part(request):
    dtype = request.param
    n = 300
    rp, ci = random_csr(n, 6, 11, empty_rows=0.1, skew=True)
    val = values(dtype, len(ci), 11)
    o = oracle.partition(dtype, n, n, rp, ci, val, 0.5, 0.25)
    return dtype, n, len(ci), o


def test_file_from_the_oracle_partition_passes(part, tmp_path):
    dtype, n, nnz, o = part
    p = tmp_path / "ok.mxp"
    write_partition_file(p, dtype, n, nnz, o)
    assert capi.check_partition_file(p, dtype) == ""
    assert "other value type" in capi.check_partition_file(p, FP16 if dtype == FP64 else FP64)


def _set(name, idx, value):
    def f(a):
        a[name][idx] = value
    return f


CORRUPTIONS = [
    ("rId out of range", _set("rId", 0, 10**6), "rId"),
    ("rId repeated", lambda a: a["rId"].__setitem__(1, a["rId"][0]), "rId"),
    ("xperm not a permutation", lambda a: a["xperm"].__setitem__(0, a["xperm"][1]), "xperm"),
    ("xperm negative", _set("xperm", 3, -1), "xperm"),
    ("rowPtr_dd decreases", lambda a: a["rowPtr_dd"].__setitem__(1, a["rowPtr_dd"][-1] + 5), "rowPtr_dd"),
    ("colInd_dd out of range", _set("colInd_dd", 0, 2**30), "colInd_dd"),
    ("chunkPtr wrong end", lambda a: a["chunkPtr"].__setitem__(-1, a["chunkPtr"][-1] + 1), "chunkPtr"),
    ("AToX out of range", _set("AToX", 0, 2**30), "AToX"),
    ("fragPtr vs bitmap", lambda a: a["fragBit"].__setitem__(0, a["fragBit"][0] ^ 1), "population count"),
    ("fragPtr first", _set("fragPtr", 0, 1), "fragPtr"),
    ("rowPtr_CD decreases", lambda a: a["rowPtr_CD"].__setitem__(2, -7), "rowPtr_CD"),
    ("colInd_CD out of range", _set("colInd_CD", 5, 300), "colInd_CD"),
]


@pytest.mark.parametrize("name,patch,needle", CORRUPTIONS, ids=[c[0] for c in CORRUPTIONS])
def test_corrupted_array_of_the_right_size_is_refused(part, tmp_path, name, patch, needle):
    dtype, n, nnz, o = part
    p = tmp_path / "bad.mxp"
    write_partition_file(p, dtype, n, nnz, o, patch=patch)
    msg = capi.check_partition_file(p, dtype)
    assert msg and needle in msg, msg


def test_inconsistent_headers_are_refused(part, tmp_path):
    dtype, n, nnz, o = part
    p = tmp_path / "hdr.mxp"
    for patch in (lambda h: h.__setitem__("version", 1), lambda h: h.__setitem__("fragK", 5),
                  lambda h: h.__setitem__("n_rows", -1), lambda h: h["counts"].__setitem__(0, 0),       # dCols = 0
                  lambda h: h["counts"].__setitem__(8, h["counts"][8] + 1),                              # chunkNum
                  lambda h: h["counts"].__setitem__(10, h["counts"][10] + 1)):                           # nnzCD
        write_partition_file(p, dtype, n, nnz, o, header_patch=patch)
        assert capi.check_partition_file(p, dtype) != ""
    # truncated file, and something that is not a partition at all
    write_partition_file(p, dtype, n, nnz, o)
    data = p.read_bytes()
    p.write_bytes(data[: len(data) - 10])
    assert "truncated" in capi.check_partition_file(p, dtype)
    p.write_bytes(b"not a partition")
    assert capi.check_partition_file(p, dtype) != ""
    assert "cannot open" in capi.check_partition_file(tmp_path / "missing", dtype)
