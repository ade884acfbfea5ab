"""ctypes view of oracle/_build/liboracle.so (the CPU restatement, cpu_oracle.cpp) and of oracle/_ref/libref_*.so
(the reference's own host code compiled from its sources; see ref_shim.cpp).  Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
FP64, FP16 = 0, 1
_vp = C.c_void_p


def build(quiet: bool = True):
    """Builds liboracle.so and, when the reference sources are present, oracle/_ref/libref_*.so."""
    r = subprocess.run(["make", "-C", str(HERE), "-j4"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(r.stdout + r.stderr)
    if not quiet:
        print(r.stdout)


def _p(a):
    return a.ctypes.data_as(_vp)


def _vdt(dtype):
    return np.float64 if dtype == FP64 else np.float16


_olib = None


def olib():
    global _olib
    if _olib is None:
        path = HERE / "_build" / "liboracle.so"
        if not path.exists():
            build()
        L = C.CDLL(str(path))
        L.mxo_partition.restype = _vp
        L.mxo_partition.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp, C.c_float, C.c_float,
                                    C.POINTER(C.c_int)]
        L.mxo_error.restype = C.c_char_p
        L.mxo_error.argtypes = [_vp]
        L.mxo_get_ints.restype = C.c_long
        L.mxo_get_ints.argtypes = [_vp, C.c_char_p, C.POINTER(_vp)]
        L.mxo_get_bytes.restype = C.c_long
        L.mxo_get_bytes.argtypes = [_vp, C.c_char_p, C.POINTER(_vp)]
        L.mxo_get_scalar.restype = C.c_double
        L.mxo_get_scalar.argtypes = [_vp, C.c_char_p]
        L.mxo_free.argtypes = [_vp]
        L.mxo_spmv_serial.argtypes = [C.c_int, _vp, _vp, _vp, _vp, _vp, C.c_int]
        L.mxo_tile_spmv_serial.argtypes = [C.c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_int]
        L.mxo_init_vec.argtypes = [C.c_int, _vp, C.c_int]
        L.mxo_eqcheck.restype = C.c_int
        L.mxo_eqcheck.argtypes = [C.c_int, _vp, _vp, C.c_int]
        L.mxo_dist_stats.restype = None
        L.mxo_dist_stats.argtypes = [_vp, C.c_longlong, _vp]
        L.mxo_abs_rowsum_max.restype = C.c_double
        L.mxo_abs_rowsum_max.argtypes = [C.c_int, _vp, _vp, _vp, _vp, C.c_int]
        _olib = L
    return _olib


STAT_NAMES = ("dCols", "nnzColD", "sCols", "nnzColS", "dRows", "nnzRowD", "sRows", "nnzRowS", "chunkNum",
              "totalFrags", "nnzCD")
INT_ARRAYS = ("xperm", "rId", "rowPtr_dd", "colInd_dd", "chunkPtr", "AToX", "fragPtr", "rowPtr_CD", "colInd_CD")
VAL_ARRAYS = ("val_dd", "tcVal", "val_CD")


class OracleError(RuntimeError):
    def __init__(self, status, msg):
        self.status = status
        super().__init__(f"oracle status {status}: {msg}")


def partition(dtype, n_rows, n_cols, row_ptr, col_ind, val, tau_c, tau_r) -> dict:
    """The whole extraction on the CPU; arrays named as in include/mx_capi.h (mx_partition_arrays)."""
    L = olib()
    row_ptr = np.ascontiguousarray(row_ptr, np.int32)
    col_ind = np.ascontiguousarray(col_ind, np.int32)
    val = np.ascontiguousarray(val, _vdt(dtype))
    st = C.c_int()
    h = L.mxo_partition(dtype, n_rows, n_cols, len(col_ind), _p(row_ptr), _p(col_ind), _p(val),
                        C.c_float(np.float32(tau_c)), C.c_float(np.float32(tau_r)), C.byref(st))
    try:
        if st.value != 0:
            raise OracleError(st.value, L.mxo_error(h).decode())
        out = {}
        ptr = _vp()
        n = L.mxo_get_ints(h, b"stats", C.byref(ptr))
        stats = np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_int)), (n,)).copy()
        out["stats"] = dict(zip(STAT_NAMES, (int(v) for v in stats)))
        out["stats"]["tc_nnz_ratio"] = L.mxo_get_scalar(h, b"tc_nnz_ratio")
        for name in INT_ARRAYS:
            n = L.mxo_get_ints(h, name.encode(), C.byref(ptr))
            out[name] = (np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_int)), (n,)).copy() if n > 0
                         else np.empty(0, np.int32))
        bdt = np.uint32 if dtype == FP64 else np.uint64
        for name, dt in [(v, _vdt(dtype)) for v in VAL_ARRAYS] + [("fragBit", bdt)]:
            n = L.mxo_get_bytes(h, name.encode(), C.byref(ptr))
            out[name] = (np.frombuffer(C.string_at(ptr, n), dtype=dt).copy() if n > 0 else np.empty(0, dt))
        return out
    finally:
        L.mxo_free(h)


def spmv_serial(dtype, row_ptr, col_ind, val, x, y0=None):
    """Serial CSR SpMV in valT arithmetic, y0 + A x (reference spmv_serial semantics)."""
    vdt = _vdt(dtype)
    row_ptr = np.ascontiguousarray(row_ptr, np.int32)
    col_ind = np.ascontiguousarray(col_ind, np.int32)
    val, x = np.ascontiguousarray(val, vdt), np.ascontiguousarray(x, vdt)
    y = np.zeros(len(row_ptr) - 1, vdt) if y0 is None else np.array(y0, vdt, copy=True)
    olib().mxo_spmv_serial(dtype, _p(val), _p(row_ptr), _p(col_ind), _p(x), _p(y), len(row_ptr) - 1)
    return y


def tile_spmv_serial(dtype, x_d, chunkPtr, fragPtr, fragBit, tcVal, AToX, dRows):
    vdt = _vdt(dtype)
    bdt = np.uint32 if dtype == FP64 else np.uint64
    x_d, tcVal = np.ascontiguousarray(x_d, vdt), np.ascontiguousarray(tcVal, vdt)
    chunkPtr, fragPtr, AToX = (np.ascontiguousarray(a, np.int32) for a in (chunkPtr, fragPtr, AToX))
    fragBit = np.ascontiguousarray(fragBit, bdt)
    y = np.zeros(dRows, vdt)
    olib().mxo_tile_spmv_serial(dtype, _p(x_d), _p(y), _p(chunkPtr), _p(fragPtr), _p(fragBit), _p(tcVal), _p(AToX), dRows)
    return y


def init_vec(dtype, n):
    v = np.empty(n, _vdt(dtype))
    olib().mxo_init_vec(dtype, _p(v), n)
    return v


def eqcheck(dtype, a, b):
    """Index of the first element failing the reference's relative check, or -1."""
    vdt = _vdt(dtype)
    a, b = np.ascontiguousarray(a, vdt), np.ascontiguousarray(b, vdt)
    return olib().mxo_eqcheck(dtype, _p(a), _p(b), len(a))


def abs_rowsum_max(dtype, row_ptr, col_ind, val, x):
    vdt = _vdt(dtype)
    row_ptr = np.ascontiguousarray(row_ptr, np.int32)
    col_ind = np.ascontiguousarray(col_ind, np.int32)
    val, x = np.ascontiguousarray(val, vdt), np.ascontiguousarray(x, vdt)
    return olib().mxo_abs_rowsum_max(dtype, _p(val), _p(row_ptr), _p(col_ind), _p(x), len(row_ptr) - 1)


def y_error(dtype, y, y_ref, row_ptr, col_ind, val, x):
    """max|y - y_ref| / max_i(sum_j |a_ij||x_j|): the tolerance statistic (1e-12 FP64, 2e-3 FP16)."""
    denom = abs_rowsum_max(dtype, row_ptr, col_ind, val, x)
    num = float(np.max(np.abs(np.asarray(y, np.float64) - np.asarray(y_ref, np.float64)))) if len(y) else 0.0
    return num / denom if denom > 0 else num


def exact_spmv(row_ptr, col_ind, val, x):
    """float64-accumulated y (numpy), the 'truth' both precisions are compared to."""
    row_ptr = np.asarray(row_ptr, np.int64)
    prod = np.asarray(val, np.float64) * np.asarray(x, np.float64)[np.asarray(col_ind, np.int64)]
    y = np.zeros(len(row_ptr) - 1)
    nz = row_ptr[1:] > row_ptr[:-1]
    if prod.size:
        y[nz] = np.add.reduceat(prod, row_ptr[:-1][nz])
    return y


# ---------------------------------------------------------------------------------------------------
# The reference's own host code (oracle/_ref).  Only available where it was built (needs the reference sources).
# ---------------------------------------------------------------------------------------------------
_rlibs = {}


FEATURE_NAMES = (["Mean", "Std", "Min", "Max", "PRatio"] + [f"Top{k}" for k in (1, 2, 3, 4, 5, 10, 50, 100, 200, 300)]
                 + [f"Hot{p}" for p in range(10, 100, 10)])


def dist_stats(counts) -> np.ndarray:
    """The 24 statistics of one count distribution, in the order of FEATURE_NAMES (ML/extract_features.cpp:19-93)."""
    a = np.ascontiguousarray(counts, np.int64)
    out = np.zeros(24, np.float64)
    olib().mxo_dist_stats(_p(a), len(a), _p(out))
    return out


def matrix_features(n_rows, n_cols, row_ptr, col_ind) -> dict:
    """Row and column distributions formed as in ML/extract_features.cpp:155-170."""
    rows = np.diff(np.asarray(row_ptr, np.int64))[:n_rows]
    cols = np.bincount(np.asarray(col_ind, np.int64), minlength=n_cols)[:n_cols] if n_cols else np.zeros(0, np.int64)
    return {"row": dist_stats(rows), "col": dist_stats(cols)}


def ref_dist_stats(counts) -> np.ndarray:
    """The reference's own computeDistStats (compiled from its source into oracle/_ref)."""
    L = rlib(FP64)
    L.ref_dist_stats.restype = None
    L.ref_dist_stats.argtypes = [_vp, C.c_longlong, _vp]
    a = np.ascontiguousarray(counts, np.int64)
    out = np.zeros(24, np.float64)
    L.ref_dist_stats(_p(a), len(a), _p(out))
    return out


def ref_available() -> bool:
    return (HERE / "_ref" / "libref_fp64.so").exists() and (HERE / "_ref" / "libref_fp16.so").exists()


def rlib(dtype):
    if dtype not in _rlibs:
        path = HERE / "_ref" / ("libref_fp64.so" if dtype == FP64 else "libref_fp16.so")
        L = C.CDLL(str(path))
        L.ref_run_main.restype = C.c_int
        L.ref_run_main.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p]
        L.ref_get_ints.restype = C.c_long
        L.ref_get_ints.argtypes = [C.c_char_p, C.POINTER(_vp)]
        L.ref_get_bytes.restype = C.c_long
        L.ref_get_bytes.argtypes = [C.c_char_p, C.POINTER(_vp)]
        L.ref_read_mtx.restype = C.c_int
        L.ref_read_mtx.argtypes = [C.c_char_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]
        L.ref_spmv_serial.argtypes = [_vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int]
        L.ref_eqcheck.restype = C.c_int
        L.ref_eqcheck.argtypes = [_vp, _vp, C.c_int]
        L.ref_build_tiles.restype = C.c_int
        L.ref_build_tiles.argtypes = [_vp, _vp, _vp, C.c_int, C.c_int]
        if dtype == FP64:
            L.ref_tcspmv_serial.argtypes = [_vp, _vp, _vp, _vp, C.c_int, _vp, _vp, C.c_int, _vp, C.c_int, C.c_int]
        assert L.ref_value_bytes() == (8 if dtype == FP64 else 2)
        _rlibs[dtype] = L
    return _rlibs[dtype]


def _ref_ints(L, name):
    ptr = _vp()
    n = L.ref_get_ints(name.encode(), C.byref(ptr))
    if n < 0:
        return None
    return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_int)), (n,)).copy() if n else np.empty(0, np.int32)


def _ref_bytes(L, name, dt):
    ptr = _vp()
    n = L.ref_get_bytes(name.encode(), C.byref(ptr))
    if n < 0:
        return None
    return np.frombuffer(C.string_at(ptr, n), dtype=dt).copy() if n else np.empty(0, dt)


def write_mtx(path, n_rows, n_cols, row_ptr, col_ind):
    """Matrix Market 'pattern general' file (the reference driver overwrites values with i % 15 anyway)."""
    rows = np.repeat(np.arange(n_rows), np.diff(row_ptr))
    with open(path, "w") as f:
        f.write("%%MatrixMarket matrix coordinate pattern general\n")
        f.write(f"{n_rows} {n_cols} {len(col_ind)}\n")
        np.savetxt(f, np.stack([rows + 1, np.asarray(col_ind) + 1], 1), fmt="%d")


def ref_run_main(dtype, mtx_path, tau_c=None, tau_r=None) -> dict:
    """Runs the reference's main() on a Matrix Market file and returns every array it handed to its GPU API."""
    L = rlib(dtype)
    rc = L.ref_run_main(None if tau_c is None else str(tau_c).encode(), None if tau_r is None else str(tau_r).encode(),
                        str(mtx_path).encode())
    out = {"rc": rc}
    vdt = _vdt(dtype)
    bdt = np.uint32 if dtype == FP64 else np.uint64
    for name in ("dcsrRowPtr", "dcsrColInd", "dcsr_dims", "scsrRowPtr", "scsrColInd", "scsr_dims", "rowPtr_CD",
                 "colInd_CD", "cd_dims", "chunkPtr", "fragPtr", "AToX", "rId", "du_dims", "rowPtr_dd", "colInd_dd",
                 "se_dims"):
        v = _ref_ints(L, name)
        if v is not None:
            out[name] = v
    for name in ("val_CD", "x_CD", "y_before_cd", "y_final", "tcVal", "x_d", "val_dd"):
        v = _ref_bytes(L, name, vdt)
        if v is not None:
            out[name] = v
    v = _ref_bytes(L, "fragBit", bdt)
    if v is not None:
        out["fragBit"] = v
    return out


def ref_read_mtx(dtype, path):
    L = rlib(dtype)
    m, n, nnz = C.c_int(), C.c_int(), C.c_int()
    rc = L.ref_read_mtx(str(path).encode(), C.byref(m), C.byref(n), C.byref(nnz))
    if rc != 0:
        raise RuntimeError(f"mmio_allinone failed: {rc}")
    return m.value, n.value, _ref_ints(L, "mm_rowPtr"), _ref_ints(L, "mm_colInd"), _ref_bytes(L, "mm_val", _vdt(dtype))


def ref_spmv_serial(dtype, row_ptr, col_ind, val, x, y0=None):
    vdt = _vdt(dtype)
    row_ptr = np.ascontiguousarray(row_ptr, np.int32)
    col_ind = np.ascontiguousarray(col_ind, np.int32)
    val, x = np.ascontiguousarray(val, vdt), np.ascontiguousarray(x, vdt)
    y = np.zeros(len(row_ptr) - 1, vdt) if y0 is None else np.array(y0, vdt, copy=True)
    rlib(dtype).ref_spmv_serial(_p(val), _p(row_ptr), _p(col_ind), _p(x), _p(y), len(row_ptr) - 1, len(x), len(col_ind))
    return y


def ref_build_tiles(dtype, rowPtr_dd, colInd_dd, val_dd, dCols) -> dict:
    """The reference's ecrPreprocess_opt1 + generateFormat_opt[_fp16] on a dd block."""
    L = rlib(dtype)
    vdt = _vdt(dtype)
    rowPtr_dd = np.ascontiguousarray(rowPtr_dd, np.int32)
    colInd_dd = np.ascontiguousarray(colInd_dd, np.int32)
    val_dd = np.ascontiguousarray(val_dd, vdt)
    L.ref_build_tiles(_p(val_dd), _p(rowPtr_dd), _p(colInd_dd), len(rowPtr_dd) - 1, dCols)
    bdt = np.uint32 if dtype == FP64 else np.uint64
    return {"chunkPtr": _ref_ints(L, "chunkPtr"), "AToX": _ref_ints(L, "AToX"), "fragPtr": _ref_ints(L, "fragPtr"),
            "fragBit": _ref_bytes(L, "fragBit", bdt), "tcVal": _ref_bytes(L, "tcVal", vdt)}


def ref_tcspmv_serial(x_d, chunkPtr, fragPtr, fragBit, tcVal, AToX, dRows, dCols):
    """FP64 only: the reference's serial statement of the fragment format."""
    L = rlib(FP64)
    x_d, tcVal = np.ascontiguousarray(x_d, np.float64), np.ascontiguousarray(tcVal, np.float64)
    chunkPtr, fragPtr, AToX = (np.ascontiguousarray(a, np.int32) for a in (chunkPtr, fragPtr, AToX))
    fragBit = np.ascontiguousarray(fragBit, np.uint32)
    y = np.zeros(dRows)
    L.ref_tcspmv_serial(_p(x_d), _p(y), _p(chunkPtr), _p(fragPtr), len(fragBit), _p(fragBit), _p(tcVal), len(tcVal),
                        _p(AToX), dRows, dCols)
    return y
