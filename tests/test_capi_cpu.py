"""Host-side checks that need no GPU: the C ABI library loads and exports every symbol include/mx_capi.h declares,
argument validation, and the loud failure without a device."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import matxtract_b200 as mx
from matxtract_b200 import capi, synth

from conftest import has_gpu

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "mx_capi.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)  # declarations only, not the comments
    declared = set(re.findall(r"\b(mx_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    L = capi.lib()
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} declared in mx_capi.h but not exported"
    assert declared == set(capi.SYMBOLS), "ctypes table and header disagree"


def test_version_and_status_strings():
    L = capi.lib()
    assert L.mx_version() >= 100
    assert L.mx_status_string(0) == b"ok"
    assert b"no CUDA device" in L.mx_status_string(8)


@pytest.mark.skipif(has_gpu(), reason="only meaningful on a machine without a GPU")
def test_no_device_fails_loudly():
    with pytest.raises(mx.MxError) as e:
        mx.MatXtract(mx.FP64)
    assert e.value.status == 8
    with pytest.raises(mx.MxError):
        mx.cdspmv(mx.FP64, np.ones(1), np.array([0, 1]), np.array([0]), np.ones(1), np.zeros(1))


def test_invalid_arguments_do_not_reach_cuda():
    L = capi.lib()
    h = C.c_void_p()
    assert L.mx_create(None, 0, 0) == 1
    assert L.mx_create(C.byref(h), 0, 7) == 1
    assert L.mx_destroy(None) == 1
    assert L.mx_spmv(None, None, None) == 1
    ms = C.c_double()
    assert L.mx_cdspmv(5, None, None, None, None, None, 1, 1, 1, 0, 0, C.byref(ms), C.byref(ms)) == 1


def test_generators_are_deterministic_and_range_independent():
    a = synth.generate("c2", n=3000)
    b = synth.generate("c2", n=3000)
    np.testing.assert_array_equal(a["col_ind"], b["col_ind"])
    np.testing.assert_array_equal(a["val"].view(np.uint16), b["val"].view(np.uint16))
    part = synth.generate("c2", n=3000, rows=(1000, 2000))
    lo, hi = a["row_ptr"][1000], a["row_ptr"][2000]
    np.testing.assert_array_equal(part["col_ind"], a["col_ind"][lo:hi])
    np.testing.assert_array_equal(part["val"].view(np.uint16), a["val"][lo:hi].view(np.uint16))
    np.testing.assert_array_equal(part["row_ptr"], a["row_ptr"][1000:2001] - lo)
    np.testing.assert_array_equal(part["x"].view(np.uint16), a["x"].view(np.uint16))


@pytest.mark.parametrize("name,n", [("c1", 10000), ("c2", 20000), ("c3", 8000), ("c4", 20000), ("c5", 20000)])
def test_generator_shapes(name, n):
    m = synth.generate(name, n=n)
    rp, ci = m["row_ptr"], m["col_ind"]
    assert rp[0] == 0 and rp[-1] == len(ci) and np.all(np.diff(rp) >= 0)
    assert ci.min() >= 0 and ci.max() < n
    rows = np.repeat(np.arange(n), np.diff(rp))
    key = rows.astype(np.int64) * n + ci
    assert np.all(np.diff(key) > 0), "columns must be distinct and ascending inside a row"
    lens = np.diff(rp)
    cfg = synth.CONFIGS[name]
    if name == "c1":
        assert abs(lens.mean() - 10) < 0.3
    if name == "c3":
        assert np.all(lens == 64)
        blocks = ci.reshape(-1, 8)
        assert np.all(blocks[:, 0] % 8 == 0) and np.all(np.diff(blocks, axis=1) == 1)
    if name == "c4":
        assert abs(lens.mean() - 12) < 0.5
        cnt = np.bincount(ci, minlength=n)
        top = np.sort(cnt)[::-1][: int(0.02 * n)].sum()
        assert 0.35 < top / len(ci) < 0.5
    if cfg.kind == synth.POWERLAW:
        assert lens.min() >= 1 and lens.max() <= min(cfg.max_len, n)


def test_algorithmic_bytes_formula():
    # reference test/test_cdspmv.cpp:214: (nnz + cols + rows)*sizeof(val) + nnz*4 + (rows+1)*4
    assert synth.algorithmic_bytes(10, 10, 100, mx.FP64) == (100 + 10 + 10) * 8 + 100 * 4 + 11 * 4
    assert synth.algorithmic_bytes(10, 10, 100, mx.FP16) == (100 + 10 + 10) * 2 + 100 * 4 + 11 * 4


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: include/mx_capi.h must compile as C99 on its own, and its two plain structs must have
    the layout the ctypes mirror assumes."""
    import subprocess

    src = tmp_path / "t.c"
    src.write_text('#include "mx_capi.h"\n#include <stdio.h>\nint main(void){printf("%zu %zu %zu\\n", '
                   "sizeof(mx_partition_stats), sizeof(mx_dist_features), sizeof(mx_matrix_features)); return 0;}\n")
    exe = tmp_path / "t"
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", f"-I{ROOT / 'include'}",
                        str(src), "-o", str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    sizes = [int(v) for v in subprocess.run([str(exe)], capture_output=True, text=True).stdout.split()]
    assert sizes == [C.sizeof(capi.PartitionStats), C.sizeof(capi.DistFeatures), C.sizeof(capi.MatrixFeatures)]


def test_fragment_count_overflow_rule():
    """The int32 limit of the fragment format (fragment ids and fragK x-index slots per fragment), on the host."""
    L = capi.lib()
    int_max = 2**31 - 1
    for dtype, k in ((mx.FP64, 4), (mx.FP16, 8)):
        assert L.mx_fragment_count_status(0, dtype) == 0
        assert L.mx_fragment_count_status(int_max // k, dtype) == 0          # last total whose slots still fit
        assert L.mx_fragment_count_status(int_max // k + 1, dtype) == 5      # MX_ERR_OVERFLOW
        assert L.mx_fragment_count_status(2**40, dtype) == 5
        assert L.mx_fragment_count_status(-1, dtype) == 5
    assert L.mx_fragment_count_status(1, 7) == 1                             # unknown value type
