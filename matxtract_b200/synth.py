"""Seeded synthetic matrices with the shape statistics of the five benchmark configurations.

The reference measures on SuiteSparse files, which are not available offline; these generators stand in for them.
Each configuration is a parameter set for the host generator in ``csrc/synth.cpp``; ``n`` can be overridden to get
a small matrix with the same per-row statistics for tests.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from pathlib import Path

from . import capi

_SYNTH_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libmx_synth.so"
_synth_lib = None


class SynthParams(C.Structure):
    _fields_ = [("kind", C.c_int), ("n", C.c_int64), ("seed", C.c_uint64), ("mean_len", C.c_double),
                ("zipf_s", C.c_double), ("alpha", C.c_double), ("max_len", C.c_int64), ("local_frac", C.c_double),
                ("local_halfwidth", C.c_int64), ("blocks_per_row", C.c_int), ("hot_col_frac", C.c_double),
                ("hot_nnz_frac", C.c_double), ("normal_values", C.c_int)]


def synth_lib() -> C.CDLL:
    """Loads libmx_synth.so: host code only, separate from the GPU library (``include/mx_synth.h``)."""
    global _synth_lib
    if _synth_lib is None:
        if not _SYNTH_LIB_PATH.exists():
            raise ImportError(f"{_SYNTH_LIB_PATH} is missing: run `python -m matxtract_b200.build`")
        L = C.CDLL(str(_SYNTH_LIB_PATH))
        vp = C.c_void_p
        L.mx_synth_row_lengths.restype = C.c_int
        L.mx_synth_row_lengths.argtypes = [C.POINTER(SynthParams), C.c_int64, C.c_int64, vp]
        L.mx_synth_fill.restype = C.c_int
        L.mx_synth_fill.argtypes = [C.POINTER(SynthParams), C.c_int, C.c_int64, C.c_int64, vp, vp, vp]
        L.mx_synth_vector.restype = C.c_int
        L.mx_synth_vector.argtypes = [C.c_uint64, C.c_int, C.c_int64, C.c_int64, vp]
        _synth_lib = L
    return _synth_lib


UNIFORM, POWERLAW, BLOCK, HOTCOL = 0, 1, 2, 3
BASE_SEED = 0x4D585452


@dataclass(frozen=True)
class Config:
    name: str
    kind: int
    n: int
    dtype: int
    tau: tuple
    mean_len: float = 0.0
    zipf_s: float = 0.0
    max_len: int = 0
    local_frac: float = 0.0
    local_halfwidth: int = 0
    blocks_per_row: int = 0
    hot_col_frac: float = 0.0
    hot_nnz_frac: float = 0.0
    normal_values: bool = False
    seed: int = BASE_SEED


CONFIGS = {
    # n=10,000, Poisson(10) rows, uniform columns, FP64, default tau
    "c1": Config("c1", UNIFORM, 10_000, capi.FP64, (0.0, 0.0), mean_len=10.0, seed=BASE_SEED + 1),
    # power-law graph, n=2e6, Zipf 2.1 clipped to [1,20000], mean 14, 60% within +-256, FP16
    "c2": Config("c2", POWERLAW, 2_000_000, capi.FP16, (0.46, 0.33), mean_len=14.0, zipf_s=2.1, max_len=20_000,
                 local_frac=0.6, local_halfwidth=256, seed=BASE_SEED + 2),
    # FEM-like dense 8x8 blocks, 8 block columns per block row within +-512 block columns, FP64
    "c3": Config("c3", BLOCK, 1_572_864, capi.FP64, (0.5, 0.5), local_halfwidth=512, blocks_per_row=8,
                 normal_values=True, seed=BASE_SEED + 3),
    # hot columns: 2% of columns receive 40% of nnz, mean 12 nnz/row geometric, FP16, tau sweep
    "c4": Config("c4", HOTCOL, 4_000_000, capi.FP16, (0.5, 0.25), mean_len=12.0, hot_col_frac=0.02, hot_nnz_frac=0.4,
                 seed=BASE_SEED + 4),
    # large power-law, n=64e6, Zipf 2.3 clipped to 1e5, mean 16, 50% within +-1024, FP64
    "c5": Config("c5", POWERLAW, 64_000_000, capi.FP64, (0.0, 0.0), mean_len=16.0, zipf_s=2.3, max_len=100_000,
                 local_frac=0.5, local_halfwidth=1024, seed=BASE_SEED + 5),
}
C4_TAUS = (0.0, 0.25, 0.5, 0.75)


def powerlaw_alpha(zipf_s: float, max_len: int, mean: float) -> float:
    """alpha such that E[clip(ceil(alpha*K), 1, max_len)] = mean for P(K >= k) = k^-(s-1) (bisection, deterministic)."""
    kmax = 1 << 20
    k = np.arange(1, kmax + 1, dtype=np.float64)
    tail = k ** (-(zipf_s - 1.0))
    pmf = tail - np.append(tail[1:], 0.0)  # last bin holds the remaining tail mass

    def expect(alpha):
        return float(np.sum(pmf * np.clip(np.ceil(alpha * k), 1, max_len)))

    lo, hi = 1e-3, 1e3
    for _ in range(80):
        mid = (lo * hi) ** 0.5
        if expect(mid) < mean:
            lo = mid
        else:
            hi = mid
    return (lo * hi) ** 0.5


_ALPHA_CACHE: dict = {}


def params(cfg: Config, n: int | None = None) -> SynthParams:
    n = cfg.n if n is None else int(n)
    alpha = 0.0
    if cfg.kind == POWERLAW:
        key = (cfg.zipf_s, cfg.max_len, cfg.mean_len)
        if key not in _ALPHA_CACHE:
            _ALPHA_CACHE[key] = powerlaw_alpha(*key)
        alpha = _ALPHA_CACHE[key]
    if cfg.kind == BLOCK and n % 8:
        raise ValueError("block-structured matrices need n % 8 == 0")
    return SynthParams(cfg.kind, n, cfg.seed, cfg.mean_len, cfg.zipf_s, alpha, cfg.max_len, cfg.local_frac,
                            cfg.local_halfwidth, cfg.blocks_per_row, cfg.hot_col_frac, cfg.hot_nnz_frac,
                            int(cfg.normal_values))


def generate(cfg: Config | str, n: int | None = None, rows: tuple | None = None, dtype: int | None = None,
             with_x: bool = True) -> dict:
    """Rows [rows[0], rows[1]) (default: all) of the n x n matrix of `cfg`, plus (with_x) the full x.

    Returns dict(n, row_begin, row_ptr (relative), col_ind, val, x, nnz, dtype).
    """
    if isinstance(cfg, str):
        cfg = CONFIGS[cfg]
    dtype = cfg.dtype if dtype is None else dtype
    p = params(cfg, n)
    n = int(p.n)
    r0, r1 = (0, n) if rows is None else rows
    L = synth_lib()
    row_ptr = np.empty(r1 - r0 + 1, np.int32)
    st = L.mx_synth_row_lengths(C.byref(p), r0, r1, capi._ptr(row_ptr))
    if st != 0:
        raise capi.MxError(st, "mx_synth_row_lengths")
    nnz = int(row_ptr[-1])
    col_ind = np.empty(nnz, np.int32)
    val = np.empty(nnz, capi.np_dtype(dtype))
    st = L.mx_synth_fill(C.byref(p), dtype, r0, r1, capi._ptr(row_ptr), capi._ptr(col_ind), capi._ptr(val))
    if st != 0:
        raise capi.MxError(st, "mx_synth_fill")
    x = None
    if with_x:
        x = np.empty(n, capi.np_dtype(dtype))
        st = L.mx_synth_vector(cfg.seed, dtype, 0, n, capi._ptr(x))
        if st != 0:
            raise capi.MxError(st, "mx_synth_vector")
    return dict(n=n, row_begin=r0, row_ptr=row_ptr, col_ind=col_ind, val=val, x=x, nnz=nnz, dtype=dtype, name=cfg.name)


def row_pointers(cfg: Config | str, n: int | None = None) -> np.ndarray:
    """Row pointers (int32, n+1) of the whole n x n matrix of `cfg`, without its entries: what a rank needs to find
    the nnz-balanced row range it owns before it generates that range."""
    if isinstance(cfg, str):
        cfg = CONFIGS[cfg]
    p = params(cfg, n)
    row_ptr = np.empty(int(p.n) + 1, np.int32)
    st = synth_lib().mx_synth_row_lengths(C.byref(p), 0, int(p.n), capi._ptr(row_ptr))
    if st != 0:
        raise capi.MxError(st, "mx_synth_row_lengths")
    return row_ptr


def algorithmic_bytes(n_rows: int, n_cols: int, nnz: int, dtype: int) -> int:
    """Original CSR + x + y, the reference's ``data_origin1`` (test/test_cdspmv.cpp:214)."""
    vb = 8 if dtype == capi.FP64 else 2
    return nnz * (vb + 4) + (n_rows + 1) * 4 + n_cols * vb + n_rows * vb
