"""B200-native MatXtract SpMV: cascaded compute-density extraction + split tile / CSR execution.

The package is a thin Python view of ``libmatxtract_b200.so`` (hand-written CUDA for sm_100a behind a C ABI,
``include/mx_capi.h``).  There is no CPU implementation: importing works anywhere (so the C ABI can be
inspected), but creating a handle without a CUDA device raises.
"""
from .capi import (  # noqa: F401
    COLSPACE_AUTO,
    COLSPACE_ORIGINAL,
    COLSPACE_PERMUTED,
    DD_AUTO,
    DD_CSR,
    DD_SE,
    DD_TILE,
    FP16,
    HOT_AUTO,
    HOT_OFF,
    HOT_ON,
    FP64,
    MatXtract,
    MultiGpu,
    mg_partition_rows,
    MxError,
    PartitionStats,
    cdspmv,
    du_tcspmv,
    lib,
    read_matrix_market,
    se_tcspmv,
)
from . import synth  # noqa: F401

__all__ = ["FP16", "FP64", "MatXtract", "MxError", "PartitionStats", "cdspmv", "du_tcspmv", "se_tcspmv", "lib", "read_matrix_market", "synth"]
