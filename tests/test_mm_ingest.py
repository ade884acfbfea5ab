"""The parallel Matrix Market reader (mx_read_matrix_market, host-only) against the reference's mmio_allinone:
committed golden vectors made by the reference reader, and - where oracle/_ref is built - the reference reader itself
on generated files large enough to be cut into several pieces."""
from pathlib import Path

import numpy as np
import pytest

import matxtract_b200 as mx
import oracle
from matxtract_b200 import FP16, FP64

MTX = sorted((Path(__file__).parent / "golden" / "mtx").glob("*.mtx"))
TAG = {FP64: "fp64", FP16: "fp16"}


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint8)


@pytest.mark.parametrize("dtype", [FP64, FP16])
@pytest.mark.parametrize("threads", [1, 3, 0])
@pytest.mark.parametrize("path", MTX, ids=[p.stem for p in MTX])
def test_reader_reproduces_reference_golden(path, threads, dtype):
    g = np.load(path.with_suffix(".npz"))
    t = TAG[dtype]
    m, n, rp, ci, val, sym = mx.read_matrix_market(path, dtype, threads)
    assert (m, n) == (int(g[f"rows_{t}"]), int(g[f"cols_{t}"]))
    np.testing.assert_array_equal(rp, g[f"row_ptr_{t}"])
    np.testing.assert_array_equal(ci, g[f"col_ind_{t}"])
    np.testing.assert_array_equal(_bits(val), g[f"val_{t}"])
    banner = path.read_text().splitlines()[0].lower()
    assert sym == (banner.endswith(" symmetric") or banner.endswith("hermitian"))


def test_fp16_values_are_rounded_once():
    """1.0004882814 lies just above the midpoint of two halves: double -> half gives 1 + 2^-10, while a detour
    through float would land on the midpoint and round to 1.0."""
    path = [p for p in MTX if p.stem == "real_general"][0]
    _, _, rp, ci, val, _ = mx.read_matrix_market(path, FP16)
    assert np.float16(1.0009765625) in val[rp[4]:rp[5]]


def _write_random(path, rng, rows, cols, entries, field, symmetry):
    r = rng.integers(1, rows + 1, entries)
    c = rng.integers(1, cols + 1, entries)
    if symmetry != "general":
        r, c = np.maximum(r, c), np.minimum(r, c)  # lower triangle
    with open(path, "w") as f:
        f.write(f"%%MatrixMarket matrix coordinate {field} {symmetry}\n% generated\n{rows} {cols} {entries}\n")
        if field == "pattern":
            np.savetxt(f, np.stack([r, c], 1), fmt="%d")
        elif field == "integer":
            np.savetxt(f, np.stack([r, c, rng.integers(-50, 50, entries)], 1), fmt="%d")
        elif field == "complex":
            v = rng.standard_normal((entries, 2))
            np.savetxt(f, np.column_stack([r, c, v]), fmt="%d %d %.17g %.17g")
        else:
            v = rng.standard_normal(entries) * 10.0 ** rng.integers(-6, 4, entries)
            np.savetxt(f, np.column_stack([r, c, v]), fmt="%d %d %.17g")


@pytest.mark.skipif(not oracle.ref_available(), reason="oracle/_ref not built (needs the reference sources)")
@pytest.mark.parametrize("dtype", [FP64, FP16])
@pytest.mark.parametrize("field,symmetry", [("real", "general"), ("real", "symmetric"), ("pattern", "symmetric"),
                                            ("integer", "general"), ("complex", "hermitian"),
                                            ("real", "skew-symmetric")])
def test_reader_matches_reference_reader_on_files_cut_into_pieces(field, symmetry, dtype, tmp_path):
    rng = np.random.default_rng(11)
    path = tmp_path / "a.mtx"
    _write_random(path, rng, 3000, 3000, 40_000, field, symmetry)  # ~0.5-1.5 MB: 8 or more pieces
    m, n, rp_r, ci_r, val_r = oracle.ref_read_mtx(dtype, path)
    for threads in (1, 7, 0):
        mm, nn, rp, ci, val, _ = mx.read_matrix_market(path, dtype, threads)
        assert (mm, nn) == (m, n)
        np.testing.assert_array_equal(rp, rp_r)
        np.testing.assert_array_equal(ci, ci_r)
        np.testing.assert_array_equal(_bits(val), _bits(val_r))


def test_reader_errors_follow_the_reference_codes(tmp_path):
    with pytest.raises(mx.MxError) as e:
        mx.read_matrix_market(tmp_path / "missing.mtx", FP64)
    assert e.value.status == -1
    bad = tmp_path / "bad.mtx"
    bad.write_text("%%NotMatrixMarket matrix coordinate real general\n1 1 1\n1 1 1.0\n")
    with pytest.raises(mx.MxError) as e:
        mx.read_matrix_market(bad, FP64)
    assert e.value.status == -2
    dense = tmp_path / "dense.mtx"
    dense.write_text("%%MatrixMarket matrix array real general\n1 1\n1.0\n")
    with pytest.raises(mx.MxError) as e:
        mx.read_matrix_market(dense, FP64)
    assert e.value.status == -2
    short = tmp_path / "short.mtx"
    short.write_text("%%MatrixMarket matrix coordinate real general\n2 2 3\n1 1 1.0\n")
    with pytest.raises(mx.MxError) as e:
        mx.read_matrix_market(short, FP64)
    assert e.value.status == -4
    outside = tmp_path / "outside.mtx"
    outside.write_text("%%MatrixMarket matrix coordinate real general\n2 2 1\n3 1 1.0\n")
    with pytest.raises(mx.MxError) as e:
        mx.read_matrix_market(outside, FP64)
    assert e.value.status == -4


def test_empty_matrix_and_trailing_lines(tmp_path):
    p = tmp_path / "e.mtx"
    p.write_text("%%MatrixMarket matrix coordinate real general\n3 4 0\n")
    m, n, rp, ci, val, sym = mx.read_matrix_market(p, FP64)
    assert (m, n, list(rp), len(ci), len(val), sym) == (3, 4, [0, 0, 0, 0], 0, 0, False)
    p.write_text("%%MatrixMarket matrix coordinate real general\n2 2 1\n2 1 4.0\n1 1 9.0\n")  # one line too many
    m, n, rp, ci, val, _ = mx.read_matrix_market(p, FP64)
    assert (list(rp), list(ci), list(val)) == ([0, 0, 1], [0], [4.0])


@pytest.mark.skipif(not oracle.ref_available(), reason="oracle/_ref not built (needs the reference sources)")
@pytest.mark.parametrize("body", ["3 3 3\r\n1 1 1.5\r\n2 3 -2\r\n3 2 4e1\r\n", "3 3 3\n1 1 1.5\n2 3 -2\n3 2 4e1",
                                  "  3\t3   3 \n   1 1   1.5\n\n2\t3 -2\n3 2 4e1\n\n"],
                         ids=["crlf", "no_trailing_newline", "blank_lines_tabs_spaces"])
def test_reader_line_ending_and_spacing_variants_match_reference(body, tmp_path):
    p = tmp_path / "v.mtx"
    p.write_bytes(("%%MatrixMarket matrix coordinate real general\n% c\n" + body).encode())
    m, n, rp_r, ci_r, val_r = oracle.ref_read_mtx(FP64, p)
    mm, nn, rp, ci, val, _ = mx.read_matrix_market(p, FP64, 2)
    assert (mm, nn) == (m, n)
    np.testing.assert_array_equal(rp, rp_r)
    np.testing.assert_array_equal(ci, ci_r)
    np.testing.assert_array_equal(_bits(val), _bits(val_r))
