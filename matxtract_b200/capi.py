"""ctypes binding of the C ABI in ``include/mx_capi.h`` (the same stub a foreign host language would write)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

FP64, FP16 = 0, 1
DD_AUTO, DD_TILE, DD_CSR, DD_SE = 0, 1, 2, 3
COLSPACE_AUTO, COLSPACE_PERMUTED, COLSPACE_ORIGINAL = 0, 1, 2
HOT_AUTO, HOT_OFF, HOT_ON = 0, 1, 2

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libmatxtract_b200.so"

STATUS = {0: "MX_OK", 1: "MX_ERR_INVALID", 2: "MX_ERR_CUDA", 3: "MX_ERR_TAU", 4: "MX_ERR_STATE", 5: "MX_ERR_OVERFLOW",
          6: "MX_ERR_TIMEOUT", 7: "MX_ERR_NOMEM", 8: "MX_ERR_NO_DEVICE", 9: "MX_ERR_TOO_LARGE"}


class MxError(RuntimeError):
    def __init__(self, status: int, msg: str = ""):
        self.status = status
        super().__init__(f"{STATUS.get(status, status)}: {msg}")


class DistFeatures(C.Structure):
    _fields_ = [("mean", C.c_double), ("std_dev", C.c_double), ("min", C.c_longlong), ("max", C.c_longlong),
                ("p_ratio", C.c_double), ("top", C.c_double * 10), ("hot", C.c_double * 9)]

    def as_array(self) -> np.ndarray:
        """mean, std, min, max, pRatio, top1..top300, hot10..hot90: the reference's CSV column order."""
        return np.array([self.mean, self.std_dev, float(self.min), float(self.max), self.p_ratio,
                         *self.top, *self.hot], np.float64)


class MatrixFeatures(C.Structure):
    _fields_ = [("rows", C.c_longlong), ("cols", C.c_longlong), ("nnz", C.c_longlong),
                ("row", DistFeatures), ("col", DistFeatures)]


class PartitionStats(C.Structure):
    _fields_ = [("dCols", C.c_int), ("nnzColD", C.c_int), ("sCols", C.c_int), ("nnzColS", C.c_int),
                ("dRows", C.c_int), ("nnzRowD", C.c_int), ("sRows", C.c_int), ("nnzRowS", C.c_int),
                ("chunkNum", C.c_int), ("totalFrags", C.c_int), ("nnzCD", C.c_int), ("fragK", C.c_int),
                ("tc_nnz_ratio", C.c_double), ("preprocess_ms", C.c_float), ("active", C.c_int),
                ("tuning_ms", C.c_float)]

    def as_dict(self):
        return {k: getattr(self, k) for k, _ in self._fields_}


class _PartitionArrays(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("xperm", "rId", "rowPtr_dd", "colInd_dd", "val_dd", "chunkPtr", "AToX",
                                           "fragPtr", "fragBit", "tcVal", "rowPtr_CD", "colInd_CD", "val_CD")]


# every symbol include/mx_capi.h declares: name -> (restype, argtypes)
_vp, _i, _d = C.c_void_p, C.c_int, C.c_double
_ip = C.POINTER(C.c_int)
SYMBOLS = {
    "mx_version": (_i, []),
    "mx_status_string": (C.c_char_p, [_i]),
    "mx_create": (_i, [C.POINTER(_vp), _i, _i]),
    "mx_destroy": (_i, [_vp]),
    "mx_last_error_string": (C.c_char_p, [_vp]),
    "mx_stream": (_vp, [_vp]),
    "mx_sync": (_i, [_vp]),
    "mx_upload_csr": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp]),
    "mx_partition": (_i, [_vp, _d, _d, C.POINTER(PartitionStats)]),
    "mx_col_counts": (_i, [_vp, _vp]),
    "mx_row_counts_in_hot_columns": (_i, [_vp, _d, _vp, C.c_longlong, _vp]),
    "mx_rank_cut": (_i, [_vp, _vp, _i, C.c_longlong, C.POINTER(C.c_longlong * 4)]),
    "mx_partition_global": (_i, [_vp, _d, _d, _vp, C.c_longlong, _i, C.c_longlong, C.c_longlong,
                                 C.POINTER(PartitionStats)]),
    "mx_partition_stats_get": (_i, [_vp, C.POINTER(PartitionStats)]),
    "mx_save_partition": (_i, [_vp, C.c_char_p]),
    "mx_load_partition": (_i, [_vp, C.c_char_p, C.POINTER(PartitionStats)]),
    "mx_check_partition_file": (_i, [C.c_char_p, _i, C.c_char_p, _i]),
    "mx_autotune_tau": (_i, [_vp, _i, C.POINTER(_d), C.POINTER(_d), C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "mx_fragment_count_status": (_i, [C.c_longlong, _i]),
    "mx_dims": (_i, [_vp, _ip, _ip, _ip]),
    "mx_download_partition": (_i, [_vp, C.POINTER(_PartitionArrays)]),
    "mx_spmv": (_i, [_vp, _vp, _vp]),
    "mx_spmv_host": (_i, [_vp, _vp, _vp]),
    "mx_spmv_host_async": (_i, [_vp, _vp, _vp]),
    "mx_host_sync": (_i, [_vp]),
    "mx_spmv_peers": (_i, [_vp, _vp, C.POINTER(_vp), _i, C.c_longlong]),
    "mx_spmv_multicast": (_i, [_vp, _vp, C.POINTER(_vp), _i, _vp, C.c_longlong]),
    "mx_peer_push": (_i, [_i, C.POINTER(_vp), _i, _i, C.c_longlong, C.c_longlong, _vp, _vp]),
    "mx_mg_create": (_i, [C.POINTER(_vp), _i, _ip, _i]),
    "mx_mg_destroy": (_i, [_vp]),
    "mx_mg_last_error_string": (C.c_char_p, [_vp]),
    "mx_mg_set_exchange": (_i, [_vp, _i]),
    "mx_mg_partition_rows": (_i, [_vp, _i, _i, _vp]),
    "mx_mg_upload_csr": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp]),
    "mx_mg_partition": (_i, [_vp, _d, _d, C.POINTER(PartitionStats)]),
    "mx_mg_set_local_ranking": (_i, [_vp, _i]),
    "mx_mg_bounds": (_i, [_vp, _vp]),
    "mx_mg_devices": (_i, [_vp]),
    "mx_mg_handle": (_vp, [_vp, _i]),
    "mx_mg_spmv": (_i, [_vp, _vp, _vp]),
    "mx_mg_download_y": (_i, [_vp, _i, _vp]),
    "mx_mg_spmv_timed": (_i, [_vp, _vp, _i, _i, C.POINTER(C.c_float)]),
    "mx_read_matrix_market": (_i, [C.c_char_p, _i, _i, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                   C.POINTER(C.c_int), C.POINTER(C.POINTER(C.c_int)), C.POINTER(C.POINTER(C.c_int)),
                                   C.POINTER(_vp)]),
    "mx_host_free": (None, [_vp]),
    "mx_features": (_i, [_vp, _vp]),
    "mx_csr_prefetch": (_i, [_vp, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "mx_stream_gather_floor": (_i, [_vp, _vp, _i, _i, C.POINTER(C.c_float)]),
    "mx_spmv_timed": (_i, [_vp, _vp, _vp, _i, _i, C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "mx_spmv_launches": (_i, [_vp]),
    "mx_set_dd_executor": (_i, [_vp, _i]),
    "mx_dd_executor": (_i, [_vp]),
    "mx_set_column_space": (_i, [_vp, _i]),
    "mx_column_space": (_i, [_vp, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "mx_set_column_slabs": (_i, [_vp, _i]),
    "mx_set_row_offset": (_i, [_vp, C.c_longlong]),
    "mx_column_slabs": (_i, [_vp, _ip, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "mx_set_hot_prefix": (_i, [_vp, _i]),
    "mx_hot_prefix": (_i, [_vp, _ip, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "mx_device_error": (_i, [_vp, _ip]),
    "mx_cdspmv": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, C.POINTER(_d), C.POINTER(_d)]),
    "mx_du_tcspmv": (_i, [_i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, C.POINTER(_d)]),
    "mx_se_tcspmv": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _d, _i, _i, _i, C.POINTER(_d)]),
    "mx_dd_executor_times": (_i, [_vp, C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "mx_csr_spmv_static": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
}

_lib = None


def lib() -> C.CDLL:
    """Loads libmatxtract_b200.so (built in-tree by ``python -m matxtract_b200.build``).  No fallback."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise ImportError(f"{_LIB_PATH} is missing: run `python -m matxtract_b200.build` (there is no CPU path)")
        L = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def np_dtype(dtype: int):
    return np.float64 if dtype == FP64 else np.float16


def _ptr(a):
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return a.ctypes.data_as(C.c_void_p)
    if hasattr(a, "data_ptr"):  # torch tensor
        return C.c_void_p(a.data_ptr())
    return C.c_void_p(int(a))


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


class MatXtract:
    """One matrix on one GPU: upload, extract with (tau_c, tau_r), multiply.

    Mirrors what ``matxtract_perftest`` does inside its ``main()`` (reference test/test_autotc_spmv.cpp:1050-1669)
    as a reusable object.
    """

    def __init__(self, dtype: int = FP64, device: int = 0):
        self._h = C.c_void_p()
        self.dtype = dtype
        self.device = device
        st = lib().mx_create(C.byref(self._h), device, dtype)
        if st != 0:
            raise MxError(st, lib().mx_status_string(st).decode())
        self.n_rows = self.n_cols = self.nnz = 0
        self.stats = None
        self._peer_arrays = {}

    def _ck(self, st):
        if st != 0:
            raise MxError(st, lib().mx_last_error_string(self._h).decode())

    def close(self):
        if self._h:
            lib().mx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def upload_csr(self, n_rows, n_cols, row_ptr, col_ind, val):
        row_ptr, col_ind, val = _c(row_ptr, np.int32), _c(col_ind, np.int32), _c(val, np_dtype(self.dtype))
        nnz = int(col_ind.shape[0])
        self._ck(lib().mx_upload_csr(self._h, n_rows, n_cols, nnz, _ptr(row_ptr), _ptr(col_ind), _ptr(val)))
        self.n_rows, self.n_cols, self.nnz = n_rows, n_cols, nnz

    def partition(self, tau_c: float = 0.0, tau_r: float = 0.0) -> PartitionStats:
        st = PartitionStats()
        self._ck(lib().mx_partition(self._h, float(tau_c), float(tau_r), C.byref(st)))
        self.stats = st
        return st

    # ---- the whole matrix's rankings for a slab of a matrix spread over several GPUs (mx_partition_global) ----
    def col_counts(self, counts_dev):
        """Column histogram of this slab into a device int32 buffer of n_cols entries."""
        self._ck(lib().mx_col_counts(self._h, _ptr(counts_dev)))

    def row_counts_in_hot_columns(self, tau_c, global_col_counts_dev, global_nnz, row_counts_dev):
        self._ck(lib().mx_row_counts_in_hot_columns(self._h, float(tau_c), _ptr(global_col_counts_dev), int(global_nnz),
                                                    _ptr(row_counts_dev)))

    def rank_cut(self, counts_dev, n, threshold):
        """(k, sum, count of the k-th, index of the k-th) of the descending ranking of a device int32 array."""
        out = (C.c_longlong * 4)()
        self._ck(lib().mx_rank_cut(self._h, _ptr(counts_dev), int(n), int(threshold), C.byref(out)))
        return tuple(int(v) for v in out)

    def partition_global(self, tau_c, tau_r, global_col_counts_dev, global_nnz, row_cut_count, row_cut_index,
                         row_offset) -> PartitionStats:
        st = PartitionStats()
        self._ck(lib().mx_partition_global(self._h, float(tau_c), float(tau_r), _ptr(global_col_counts_dev),
                                           int(global_nnz), int(row_cut_count), int(row_cut_index), int(row_offset),
                                           C.byref(st)))
        self.stats = st
        return st

    def save_partition(self, path):
        self._ck(lib().mx_save_partition(self._h, str(path).encode()))

    def load_partition(self, path) -> PartitionStats:
        """Restores a stored partition; the handle is then ready for spmv without an uploaded matrix."""
        st = PartitionStats()
        self._ck(lib().mx_load_partition(self._h, str(path).encode(), C.byref(st)))
        self.stats = st
        r, c, z = C.c_int(), C.c_int(), C.c_int()
        self._ck(lib().mx_dims(self._h, C.byref(r), C.byref(c), C.byref(z)))
        self.n_rows, self.n_cols, self.nnz = r.value, c.value, z.value
        return st

    def autotune_tau(self, grid: int = 4):
        """Times every valid (tau_c, tau_r) of a grid on the device and installs the fastest.
        Returns (tau_c, tau_r, ms of the best, ms of tau = (0,0))."""
        tc, tr, mb, mp = C.c_double(), C.c_double(), C.c_float(), C.c_float()
        self._ck(lib().mx_autotune_tau(self._h, grid, C.byref(tc), C.byref(tr), C.byref(mb), C.byref(mp)))
        st = PartitionStats()
        self._ck(lib().mx_partition_stats_get(self._h, C.byref(st)))
        self.stats = st
        return tc.value, tr.value, mb.value, mp.value

    def download_partition(self) -> dict:
        s = self.stats
        vdt = np_dtype(self.dtype)
        bdt = np.uint32 if self.dtype == FP64 else np.uint64
        out = {
            "xperm": np.empty(self.n_cols, np.int32), "rId": np.empty(s.dRows, np.int32),
            "rowPtr_dd": np.empty(s.dRows + 1, np.int32), "colInd_dd": np.empty(s.nnzRowD, np.int32),
            "val_dd": np.empty(s.nnzRowD, vdt), "chunkPtr": np.empty(s.chunkNum + 1, np.int32),
            "AToX": np.empty(s.totalFrags * s.fragK, np.int32), "fragPtr": np.empty(s.totalFrags + 1, np.int32),
            "fragBit": np.empty(s.totalFrags, bdt), "tcVal": np.empty(s.nnzRowD, vdt),
            "rowPtr_CD": np.empty(self.n_rows + 1, np.int32), "colInd_CD": np.empty(s.nnzCD, np.int32),
            "val_CD": np.empty(s.nnzCD, vdt),
        }
        arr = _PartitionArrays(**{k: _ptr(v) for k, v in out.items()})
        self._ck(lib().mx_download_partition(self._h, C.byref(arr)))
        return out

    def spmv(self, x_dev, y_dev):
        """x_dev / y_dev: device pointers (ints) or torch CUDA tensors; asynchronous on ``self.stream``."""
        self._ck(lib().mx_spmv(self._h, _ptr(x_dev), _ptr(y_dev)))

    def spmv_peers(self, x_dev, peer_ptrs, row_offset: int):
        """Rows of this slab are stored into every GPU's full-length y (peer_ptrs: device addresses as ints)."""
        key = tuple(peer_ptrs)
        arr = self._peer_arrays.get(key)
        if arr is None:
            arr = self._peer_arrays[key] = (C.c_void_p * len(peer_ptrs))(*[C.c_void_p(int(p)) for p in peer_ptrs])
        self._ck(lib().mx_spmv_peers(self._h, _ptr(x_dev), arr, len(peer_ptrs), int(row_offset)))

    def spmv_multicast(self, x_dev, peer_ptrs, multicast_ptr: int, row_offset: int):
        """As spmv_peers, with the rows leaving through the buffers' NVLink multicast address (one store per row or
        row pair, replicated by the switch)."""
        key = tuple(peer_ptrs)
        arr = self._peer_arrays.get(key)
        if arr is None:
            arr = self._peer_arrays[key] = (C.c_void_p * len(peer_ptrs))(*[C.c_void_p(int(p)) for p in peer_ptrs])
        self._ck(lib().mx_spmv_multicast(self._h, _ptr(x_dev), arr, len(peer_ptrs), C.c_void_p(int(multicast_ptr)),
                                         int(row_offset)))

    def peer_push(self, peer_ptrs, self_rank: int, row_offset: int, n_rows: int, table_dev):
        """Copies this GPU's rows of y (already in its own full-length buffer) to every other GPU's buffer."""
        key = tuple(peer_ptrs)
        arr = self._peer_arrays.get(key)
        if arr is None:
            arr = self._peer_arrays[key] = (C.c_void_p * len(peer_ptrs))(*[C.c_void_p(int(p)) for p in peer_ptrs])
        _raise(lib().mx_peer_push(self.dtype, arr, len(peer_ptrs), self_rank, int(row_offset), int(n_rows),
                                  _ptr(table_dev), C.c_void_p(self.stream)))

    def spmv_host(self, x, y=None):
        """y = A x with HOST buffers (numpy arrays, or pinned torch CPU tensors of the handle's value type): copies x
        in, multiplies, copies y out, synchronises."""
        if isinstance(x, np.ndarray):
            x = _c(x, np_dtype(self.dtype))
        if y is None:
            y = np.empty(self.n_rows, np_dtype(self.dtype))
        self._ck(lib().mx_spmv_host(self._h, _ptr(x), _ptr(y)))
        return y

    def spmv_host_async(self, x, y):
        """Enqueues y = A x with HOST buffers and returns; consecutive calls overlap their copies with each other's
        kernels.  x and y (numpy arrays or torch CPU tensors of the handle's value type, page-locked for the overlap)
        must stay alive and untouched until host_sync()."""
        self._ck(lib().mx_spmv_host_async(self._h, _ptr(x), _ptr(y)))

    def host_sync(self):
        self._ck(lib().mx_host_sync(self._h))

    def spmv_timed(self, x_dev, y_dev, warm=20, iters=200):
        t, r, a = C.c_float(), C.c_float(), C.c_float()
        self._ck(lib().mx_spmv_timed(self._h, _ptr(x_dev), _ptr(y_dev), warm, iters, C.byref(t), C.byref(r), C.byref(a)))
        return {"ms_tile": t.value, "ms_resid": r.value, "ms_total": a.value}

    def features(self) -> MatrixFeatures:
        """Row / column distribution statistics of the uploaded matrix (the reference's ML feature vector)."""
        f = MatrixFeatures()
        self._ck(lib().mx_features(self._h, C.byref(f)))
        return f

    @property
    def csr_prefetch(self):
        """(residual half, core-dense block) L2 prefetch distance of the CSR kernel in tiles; 0 = off."""
        a, b = C.c_int(), C.c_int()
        self._ck(lib().mx_csr_prefetch(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def stream_gather_floor(self, x_dev, warm=5, iters=50) -> float:
        """ms of a pass that streams the uploaded CSR's indices and values and gathers x, with no row logic: the floor
        the matrix's index pattern sets for a CSR-ordered kernel on this GPU."""
        t = C.c_float()
        self._ck(lib().mx_stream_gather_floor(self._h, _ptr(x_dev), warm, iters, C.byref(t)))
        return t.value

    def set_dd_executor(self, mode: int):
        """0 = auto (by fill ratio), 1 = tensor-core tile kernel, 2 = CSR kernel on the core-dense block."""
        self._ck(lib().mx_set_dd_executor(self._h, mode))

    def set_column_space(self, mode: int):
        """0 = auto (timed at partition time), 1 = the partition's permuted numbering, 2 = original column ids."""
        self._ck(lib().mx_set_column_space(self._h, mode))

    @property
    def column_space(self):
        """(mode in use, ms per product permuted, ms per product original) of the last automatic choice."""
        a, b = C.c_float(), C.c_float()
        m = lib().mx_column_space(self._h, C.byref(a), C.byref(b))
        return m, a.value, b.value

    def set_row_offset(self, first_global_row: int):
        """Where this handle's row slab sits in the whole square matrix (before partition; places the band)."""
        self._ck(lib().mx_set_row_offset(self._h, int(first_global_row)))

    def set_column_slabs(self, count: int):
        """-1 = automatic (when x exceeds L2, timed), 0 = off, k >= 2 = k column slabs (tau = (0,0), FP64)."""
        self._ck(lib().mx_set_column_slabs(self._h, count))

    @property
    def column_slabs(self):
        """(slabs in use, 0 = plain kernel; ms per product plain; ms per product slabbed) of the last choice."""
        n, a, b = C.c_int(), C.c_float(), C.c_float()
        self._ck(lib().mx_column_slabs(self._h, C.byref(n), C.byref(a), C.byref(b)))
        return n.value, a.value, b.value

    def set_hot_prefix(self, mode: int):
        """0 = auto (timed at partition time), 1 = off, 2 = on: hot-column prefix of x in shared memory."""
        self._ck(lib().mx_set_hot_prefix(self._h, mode))

    @property
    def hot_prefix(self):
        """(columns of x held in shared memory, 0 = off; ms per product with; ms per product without)."""
        n, a, b = C.c_int(), C.c_float(), C.c_float()
        self._ck(lib().mx_hot_prefix(self._h, C.byref(n), C.byref(a), C.byref(b)))
        return n.value, a.value, b.value

    @property
    def dd_executor(self) -> int:
        return lib().mx_dd_executor(self._h)

    @property
    def dd_executor_times(self):
        """ms of the core-dense block alone through (tile, csr, sparse-encode) at the last automatic choice."""
        a, b, c = C.c_float(), C.c_float(), C.c_float()
        self._ck(lib().mx_dd_executor_times(self._h, C.byref(a), C.byref(b), C.byref(c)))
        return a.value, b.value, c.value

    @property
    def stream(self) -> int:
        return lib().mx_stream(self._h) or 0

    @property
    def launches_per_spmv(self) -> int:
        return lib().mx_spmv_launches(self._h)

    def sync(self):
        self._ck(lib().mx_sync(self._h))

    def device_error(self) -> int:
        e = C.c_int()
        self._ck(lib().mx_device_error(self._h, C.byref(e)))
        return e.value


MG_EXCHANGE_PEER, MG_EXCHANGE_NCCL = 0, 1


def mg_partition_rows(row_ptr, n_parts: int) -> np.ndarray:
    """nnz-balanced row boundaries (host code): bounds[g] = lower_bound(row_ptr, g * nnz / n_parts)."""
    row_ptr = _c(row_ptr, np.int32)
    bounds = np.empty(n_parts + 1, np.int32)
    _raise(lib().mx_mg_partition_rows(_ptr(row_ptr), len(row_ptr) - 1, n_parts, _ptr(bounds)))
    return bounds


class MultiGpu:
    """One matrix over several GPUs of one box, driven by this process (mx_mg_* of the C ABI)."""

    def __init__(self, dtype: int, n_devices: int, devices=None):
        self._h = C.c_void_p()
        self.dtype, self.n = dtype, n_devices
        devs = None if devices is None else (C.c_int * n_devices)(*devices)
        st = lib().mx_mg_create(C.byref(self._h), n_devices, devs, dtype)
        if st != 0:
            raise MxError(st, lib().mx_status_string(st).decode())
        self.n_rows = self.n_cols = 0

    def _ck(self, st):
        if st != 0:
            raise MxError(st, lib().mx_mg_last_error_string(self._h).decode())

    def upload_csr(self, n_rows, n_cols, row_ptr, col_ind, val):
        row_ptr, col_ind, val = _c(row_ptr, np.int32), _c(col_ind, np.int32), _c(val, np_dtype(self.dtype))
        self._ck(lib().mx_mg_upload_csr(self._h, n_rows, n_cols, len(col_ind), _ptr(row_ptr), _ptr(col_ind), _ptr(val)))
        self.n_rows, self.n_cols = n_rows, n_cols

    def partition(self, tau_c, tau_r):
        stats = (PartitionStats * self.n)()
        self._ck(lib().mx_mg_partition(self._h, float(tau_c), float(tau_r), stats))
        return list(stats)

    def set_exchange(self, mode: int):
        self._ck(lib().mx_mg_set_exchange(self._h, mode))

    def set_local_ranking(self, on: bool):
        self._ck(lib().mx_mg_set_local_ranking(self._h, int(on)))

    def handle(self, g: int) -> "MatXtract":
        """A view of slab g's handle (owned by the MultiGpu object: do not close it)."""
        v = MatXtract.__new__(MatXtract)
        v._h = C.c_void_p(lib().mx_mg_handle(self._h, g))
        v.dtype, v.device = self.dtype, g
        r, c, z = C.c_int(), C.c_int(), C.c_int()
        lib().mx_dims(v._h, C.byref(r), C.byref(c), C.byref(z))
        v.n_rows, v.n_cols, v.nnz = r.value, c.value, z.value
        v.stats = PartitionStats()
        lib().mx_partition_stats_get(v._h, C.byref(v.stats))
        v._peer_arrays = {}
        v.close = lambda: None
        return v

    @property
    def bounds(self) -> np.ndarray:
        b = np.empty(self.n + 1, np.int32)
        self._ck(lib().mx_mg_bounds(self._h, _ptr(b)))
        return b

    def spmv(self, x: np.ndarray) -> np.ndarray:
        x = _c(x, np_dtype(self.dtype))
        y = np.empty(self.n_rows, np_dtype(self.dtype))
        self._ck(lib().mx_mg_spmv(self._h, _ptr(x), _ptr(y)))
        return y

    def y_of(self, g: int) -> np.ndarray:
        y = np.empty(self.n_rows, np_dtype(self.dtype))
        self._ck(lib().mx_mg_download_y(self._h, g, _ptr(y)))
        return y

    def spmv_timed(self, x: np.ndarray, warm=5, iters=20) -> float:
        x = _c(x, np_dtype(self.dtype))
        ms = C.c_float()
        self._ck(lib().mx_mg_spmv_timed(self._h, _ptr(x), warm, iters, C.byref(ms)))
        return ms.value

    def close(self):
        if self._h:
            lib().mx_mg_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _raise(st):
    if st != 0:
        raise MxError(st, lib().mx_status_string(st).decode())


def check_partition_file(path, dtype: int) -> str:
    """'' when the stored partition at `path` passes the loader's host-side check, else what is wrong.  No GPU."""
    msg = C.create_string_buffer(256)
    lib().mx_check_partition_file(str(path).encode(), dtype, msg, 256)
    return msg.value.decode()


def read_matrix_market(path, dtype: int, threads: int = 0):
    """Matrix Market coordinate file -> (rows, cols, row_ptr, col_ind, val, is_symmetric), host arrays, parsed by
    `threads` host threads (0 = all).  Same CSR as the reference's ``mmio_allinone``.  Needs no GPU."""
    m, n, nnz, sym = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    rp, ci, va = C.POINTER(C.c_int)(), C.POINTER(C.c_int)(), C.c_void_p()
    st = lib().mx_read_matrix_market(str(path).encode(), dtype, threads, C.byref(m), C.byref(n), C.byref(nnz),
                                     C.byref(sym), C.byref(rp), C.byref(ci), C.byref(va))
    if st != 0:
        raise MxError(st, f"mx_read_matrix_market({path}) failed with the reference reader's code {st}")
    try:
        row_ptr = np.ctypeslib.as_array(rp, (m.value + 1,)).copy()
        col_ind = np.ctypeslib.as_array(ci, (max(nnz.value, 1),))[: nnz.value].copy()
        vdt = np_dtype(dtype)
        raw = (C.c_char * (max(nnz.value, 1) * np.dtype(vdt).itemsize)).from_address(va.value)
        val = np.frombuffer(raw, dtype=vdt)[: nnz.value].copy()
    finally:
        lib().mx_host_free(C.cast(rp, C.c_void_p))
        lib().mx_host_free(C.cast(ci, C.c_void_p))
        lib().mx_host_free(va)
    return m.value, n.value, row_ptr, col_ind, val, bool(sym.value)


def cdspmv(dtype, val, row_ptr, col_ind, x, y, warm=0, iters=0):
    """y += A x (host arrays).  Mirror of the reference's cdspmv (include/MatXtract.h:3-5)."""
    vdt = np_dtype(dtype)
    val, row_ptr, col_ind, x = _c(val, vdt), _c(row_ptr, np.int32), _c(col_ind, np.int32), _c(x, vdt)
    y = np.array(y, dtype=vdt, copy=True)
    ms, pre = C.c_double(), C.c_double()
    _raise(lib().mx_cdspmv(dtype, _ptr(val), _ptr(row_ptr), _ptr(col_ind), _ptr(x), _ptr(y), len(row_ptr) - 1, len(x),
                           len(col_ind), warm, iters, C.byref(ms), C.byref(pre)))
    return y, ms.value, pre.value


def du_tcspmv(dtype, chunkPtr, fragPtr, fragBit, tcVal, AToX, x_d, y, dRows, warm=0, iters=0):
    """Fragment-format SpMV (host arrays).  Mirror of du_tcspmv_fp64 / du_tcspmv_fp16_v2."""
    vdt = np_dtype(dtype)
    bdt = np.uint32 if dtype == FP64 else np.uint64
    chunkPtr, fragPtr, AToX = _c(chunkPtr, np.int32), _c(fragPtr, np.int32), _c(AToX, np.int32)
    fragBit, tcVal, x_d = _c(fragBit, bdt), _c(tcVal, vdt), _c(x_d, vdt)
    y = np.array(y, dtype=vdt, copy=True)
    ms = C.c_double()
    _raise(lib().mx_du_tcspmv(dtype, _ptr(chunkPtr), _ptr(fragPtr), _ptr(fragBit), _ptr(tcVal), len(tcVal), _ptr(AToX),
                              _ptr(x_d), _ptr(y), dRows, len(x_d), warm, iters, C.byref(ms)))
    return y, ms.value


def se_tcspmv(dtype, val, row_ptr, col_ind, x_d, warm=0, iters=0, num=4, threshold=0.75, block_longest=256):
    """SpMV of a core-dense block given as CSR (host arrays) through the sparse-encode layout.  Mirror of
    se_tcspmv_fp64 / se_tcspmv_fp16: returns (y, order, ms) with y[i] the result of input row order[i]."""
    vdt = np_dtype(dtype)
    val, row_ptr, col_ind, x_d = _c(val, vdt), _c(row_ptr, np.int32), _c(col_ind, np.int32), _c(x_d, vdt)
    rows = len(row_ptr) - 1
    y = np.zeros(rows, vdt)
    order = np.empty(rows, np.int32)
    ms = C.c_double()
    _raise(lib().mx_se_tcspmv(dtype, _ptr(val), _ptr(row_ptr), _ptr(col_ind), _ptr(x_d), _ptr(y), _ptr(order), rows,
                              len(x_d), len(col_ind), num, threshold, block_longest, warm, iters, C.byref(ms)))
    return y, order, ms.value


def csr_spmv_static(dtype, n_rows, n_cols, nnz, row_ptr_dev, col_ind_dev, val_dev, x_dev, y_dev, stream=0):
    """y = A x through the allocation-free entry point: all arrays are device pointers (ints) or CUDA tensors."""
    st = lib().mx_csr_spmv_static(dtype, n_rows, n_cols, nnz, _ptr(row_ptr_dev), _ptr(col_ind_dev), _ptr(val_dev),
                                  _ptr(x_dev), _ptr(y_dev), C.c_void_p(stream))
    _raise(st)
