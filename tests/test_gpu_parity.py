"""Parity of the CUDA path (through the C ABI) with the CPU oracle.  Bit-exact for every array of the partition;
y within max|y - y_ref| / max_i(sum_j |a_ij||x_j|) <= 1e-12 (FP64) / 2e-3 (FP16)."""
from pathlib import Path

import numpy as np
import pytest

import matxtract_b200 as mx
import oracle
from matxtract_b200 import FP16, FP64, synth

from cases import TAUS, random_csr, small_cases, values

pytestmark = pytest.mark.gpu

TOL = {FP64: 1e-12, FP16: 2e-3}
CASES = small_cases()
PART_KEYS = ("xperm", "rId", "rowPtr_dd", "colInd_dd", "val_dd", "chunkPtr", "AToX", "fragPtr", "fragBit", "tcVal",
             "rowPtr_CD", "colInd_CD", "val_CD")
STAT_KEYS = ("dCols", "nnzColD", "sCols", "nnzColS", "dRows", "nnzRowD", "sRows", "nnzRowS", "chunkNum", "totalFrags",
             "nnzCD")


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint8)


def check_y(dtype, y, rp, ci, val, x):
    """Against the reference's serial valT-arithmetic result with the task's tolerance, and against an exactly
    accumulated product (the CUDA path accumulates FP16 in FP32, so it must be at least as close to that)."""
    y_ref = oracle.spmv_serial(dtype, rp, ci, val, x)
    err = oracle.y_error(dtype, y, y_ref, rp, ci, val, x)
    assert err <= TOL[dtype], f"error vs reference arithmetic {err}"
    exact = oracle.exact_spmv(rp, ci, val, x)
    err_exact = oracle.y_error(dtype, y, exact, rp, ci, val, x)
    assert err_exact <= (1e-13 if dtype == FP64 else 6e-4), f"error vs exact {err_exact}"
    assert oracle.eqcheck(dtype, y_ref, y) == -1 or dtype == FP16  # the reference's own 1e-8 relative check (FP64)
    return err


def assert_partition_equal(dtype, h, o):
    s = h.stats
    for k in STAT_KEYS:
        assert getattr(s, k) == o["stats"][k], k
    assert s.tc_nnz_ratio == pytest.approx(o["stats"]["tc_nnz_ratio"], rel=0, abs=0) or s.totalFrags == 0
    d = h.download_partition()
    for k in PART_KEYS:
        np.testing.assert_array_equal(_bits(d[k]), _bits(o[k]), err_msg=k)


@pytest.mark.parametrize("dtype", [FP64, FP16])
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_residual_only_tau_zero(dtype, case):
    name, n, rp, ci = case
    val, x = values(dtype, len(ci), 1), values(dtype, n, 2)
    h = mx.MatXtract(dtype)
    h.upload_csr(n, n, rp, ci, val)
    st = h.partition(0.0, 0.0)
    assert st.active == 0 and st.nnzCD == len(ci)
    y = h.spmv_host(x)
    check_y(dtype, y, rp, ci, val, x)
    y2 = h.spmv_host(x)
    np.testing.assert_array_equal(_bits(y), _bits(y2))  # no float atomics: bit-reproducible
    assert h.device_error() == 0
    h.close()


@pytest.mark.parametrize("dtype", [FP64, FP16])
@pytest.mark.parametrize("tau", TAUS)
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_partition_bit_exact_and_split_spmv(dtype, tau, case):
    name, n, rp, ci = case
    val, x = values(dtype, len(ci), 3), values(dtype, n, 4)
    try:
        o = oracle.partition(dtype, n, n, rp, ci, val, *tau)
    except oracle.OracleError as e:
        h = mx.MatXtract(dtype)
        h.upload_csr(n, n, rp, ci, val)
        with pytest.raises(mx.MxError) as ge:
            h.partition(*tau)
        assert ge.value.status == e.status
        return
    h = mx.MatXtract(dtype)
    h.upload_csr(n, n, rp, ci, val)
    h.partition(*tau)
    assert_partition_equal(dtype, h, o)
    for space in (mx.COLSPACE_PERMUTED, mx.COLSPACE_ORIGINAL, mx.COLSPACE_AUTO):  # both execution numberings
        h.set_column_space(space)
        assert space == mx.COLSPACE_AUTO or h.column_space[0] == space
        for mode in (mx.DD_TILE, mx.DD_CSR, mx.DD_AUTO):  # both executors of the core-dense block
            h.set_dd_executor(mode)
            assert mode == mx.DD_AUTO or h.dd_executor == mode
            y = h.spmv_host(x)
            check_y(dtype, y, rp, ci, val, x)
            np.testing.assert_array_equal(_bits(y), _bits(h.spmv_host(x)))
    assert_partition_equal(dtype, h, o)  # the execution numbering never changes the partition arrays
    assert h.device_error() == 0
    h.close()


GOLDEN = sorted((Path(__file__).parent / "golden").glob("*.npz"))


@pytest.mark.parametrize("path", GOLDEN, ids=[f.stem for f in GOLDEN])
def test_gpu_partition_reproduces_reference_golden(path):
    """Directly against the arrays the reference's own host code produced (no oracle in between)."""
    g = np.load(path)
    dtype, n = int(g["dtype"]), int(g["n"])
    val, x = oracle.init_vec(dtype, len(g["col_ind"])), oracle.init_vec(dtype, n)
    h = mx.MatXtract(dtype)
    h.upload_csr(n, n, g["row_ptr"], g["col_ind"], val)
    s = h.partition(*tuple(g["tau"]))
    assert [s.dRows, s.dCols, s.nnzRowD] == list(g["ref_se_dims"])
    d = h.download_partition()
    for k in ("rowPtr_CD", "colInd_CD", "val_CD", "rowPtr_dd", "colInd_dd", "val_dd", "chunkPtr", "AToX", "fragPtr",
              "fragBit", "tcVal"):
        np.testing.assert_array_equal(_bits(g["ref_" + k]), _bits(d[k]), err_msg=k)
    np.testing.assert_array_equal(_bits(g["ref_x_CD"]), _bits(x[d["xperm"]]))
    y = h.spmv_host(x)
    # values are small integers: FP64 sums are exact whatever the order, so y must equal the reference's bit for bit
    if dtype == FP64:
        np.testing.assert_array_equal(g["ref_y_final"], y)
    else:
        assert oracle.eqcheck(dtype, g["ref_y_final"], y) == -1
    h.close()


@pytest.mark.parametrize("dtype", [FP64, FP16])
def test_tau_c_below_tau_r_is_rejected(dtype):
    name, n, rp, ci = CASES[0]
    h = mx.MatXtract(dtype)
    h.upload_csr(n, n, rp, ci, values(dtype, len(ci), 1))
    for tc in (0.0, 0.25, 0.5):
        for tr in (0.25, 0.5, 0.75):
            if tc < tr:
                with pytest.raises(mx.MxError) as e:
                    h.partition(tc, tr)
                assert e.value.status == 3
    with pytest.raises(mx.MxError) as e:  # no plan after a rejected call
        h.spmv_host(values(dtype, n, 2))
    assert e.value.status == 4
    h.close()


@pytest.mark.parametrize("dtype", [FP64, FP16])
def test_edge_shapes(dtype):
    vdt = np.float64 if dtype == FP64 else np.float16
    # empty matrix, all-empty rows, a single dense row, one row longer than several tiles
    h = mx.MatXtract(dtype)
    n = 50
    h.upload_csr(n, n, np.zeros(n + 1, np.int32), np.zeros(0, np.int32), np.zeros(0, vdt))
    h.partition(0, 0)
    np.testing.assert_array_equal(h.spmv_host(np.ones(n, vdt)), np.zeros(n, vdt))
    n = 20000
    rp = np.zeros(n + 1, np.int32)
    rp[7:] = n  # row 6 holds every column, all other rows empty
    ci = np.arange(n, dtype=np.int32)
    val, x = values(dtype, n, 5), values(dtype, n, 6)
    h.upload_csr(n, n, rp, ci, val)
    h.partition(0, 0)
    check_y(dtype, h.spmv_host(x), rp, ci, val, x)
    h.partition(0.5, 0.5)
    check_y(dtype, h.spmv_host(x), rp, ci, val, x)
    h.close()


@pytest.mark.parametrize("dtype", [FP64, FP16])
def test_stateless_mirrors_of_the_reference_api(dtype):
    name, n, rp, ci = CASES[2]
    val, x = values(dtype, len(ci), 7), values(dtype, n, 8)
    y0 = values(dtype, n, 9)
    # cdspmv: y is in/out
    y, ms, pre = mx.cdspmv(dtype, val, rp, ci, x, y0, warm=2, iters=3)
    y_ref = oracle.spmv_serial(dtype, rp, ci, val, x, y0)
    denom = oracle.abs_rowsum_max(dtype, rp, ci, val, x) + float(np.abs(y0.astype(np.float64)).max())
    assert np.abs(y.astype(np.float64) - y_ref.astype(np.float64)).max() / denom <= TOL[dtype]
    assert ms > 0
    # du / se on the oracle's core-dense block
    o = oracle.partition(dtype, n, n, rp, ci, val, 0.75, 0.5)
    st = o["stats"]
    x_d = x[o["xperm"][: st["dCols"]]]
    want = oracle.exact_spmv(o["rowPtr_dd"], o["colInd_dd"], o["val_dd"], x_d)
    scale = oracle.abs_rowsum_max(dtype, o["rowPtr_dd"], o["colInd_dd"], o["val_dd"], x_d)
    y_du, _ = mx.du_tcspmv(dtype, o["chunkPtr"], o["fragPtr"], o["fragBit"], o["tcVal"], o["AToX"], x_d,
                           np.zeros(st["dRows"]), st["dRows"], warm=1, iters=2)
    assert np.abs(y_du.astype(np.float64) - want).max() / scale <= (1e-13 if dtype == FP64 else 6e-4)
    y_se, order, _ = mx.se_tcspmv(dtype, o["val_dd"], o["rowPtr_dd"], o["colInd_dd"], x_d, warm=1, iters=2)
    got = np.empty_like(y_se)
    got[order] = y_se
    assert np.abs(got.astype(np.float64) - want).max() / scale <= (1e-13 if dtype == FP64 else 6e-4)
    if dtype == FP64:  # du adds into y (the reference preloads it)
        y_du2, _ = mx.du_tcspmv(dtype, o["chunkPtr"], o["fragPtr"], o["fragBit"], o["tcVal"], o["AToX"], x_d,
                                np.ones(st["dRows"]), st["dRows"])
        np.testing.assert_allclose(y_du2, y_du + 1.0, rtol=0, atol=1e-12 * max(scale, 1))


MEDIUM = [("c1", 10_000, (0.0, 0.0)), ("c2", 200_000, (0.46, 0.33)), ("c3", 8 * 30_000, (0.5, 0.5)),
          ("c4", 300_000, (0.5, 0.25)), ("c4", 300_000, (0.75, 0.75)), ("c5", 400_000, (0.0, 0.0)),
          ("c5", 400_000, (0.7, 0.5))]


@pytest.mark.parametrize("name,n,tau", MEDIUM, ids=[f"{a}-{b}-{c}" for a, b, c in MEDIUM])
def test_benchmark_shapes_at_reduced_size(name, n, tau):
    m = synth.generate(name, n=n)
    dtype, rp, ci, val, x = m["dtype"], m["row_ptr"], m["col_ind"], m["val"], m["x"]
    h = mx.MatXtract(dtype)
    h.upload_csr(n, n, rp, ci, val)
    h.partition(*tau)
    if tau != (0.0, 0.0):
        assert_partition_equal(dtype, h, oracle.partition(dtype, n, n, rp, ci, val, *tau))
    for space in ((mx.COLSPACE_PERMUTED, mx.COLSPACE_ORIGINAL) if tau != (0.0, 0.0) else (mx.COLSPACE_AUTO,)):
        h.set_column_space(space)
        for mode in (mx.DD_TILE, mx.DD_CSR):
            h.set_dd_executor(mode)
            y = h.spmv_host(x)
            check_y(dtype, y, rp, ci, val, x)
            np.testing.assert_array_equal(_bits(y), _bits(h.spmv_host(x)))
    assert h.device_error() == 0
    h.close()


def test_c4_tau_sweep_valid_and_rejected_points():
    m = synth.generate("c4", n=100_000)
    n, rp, ci, val, x = m["n"], m["row_ptr"], m["col_ind"], m["val"], m["x"]
    h = mx.MatXtract(FP16)
    h.upload_csr(n, n, rp, ci, val)
    valid = rejected = 0
    for tc in synth.C4_TAUS:
        for tr in synth.C4_TAUS:
            if tc < tr:
                with pytest.raises(mx.MxError):
                    h.partition(tc, tr)
                rejected += 1
                continue
            h.partition(tc, tr)
            if (tc, tr) != (0.0, 0.0):
                assert_partition_equal(FP16, h, oracle.partition(FP16, n, n, rp, ci, val, tc, tr))
            check_y(FP16, h.spmv_host(x), rp, ci, val, x)
            valid += 1
    assert (valid, rejected) == (10, 6)
    h.close()


@pytest.mark.parametrize("dtype", [FP64, FP16])
def test_stored_partition_round_trip(dtype, tmp_path):
    """save -> load into a fresh handle: same arrays, same product bits, no matrix needed."""
    m = synth.generate("c4", n=50_000, dtype=dtype)
    n, rp, ci, val, x = m["n"], m["row_ptr"], m["col_ind"], m["val"], m["x"]
    a = mx.MatXtract(dtype)
    a.upload_csr(n, n, rp, ci, val)
    a.partition(0.5, 0.25)
    a.set_column_space(mx.COLSPACE_PERMUTED)
    ya = a.spmv_host(x)
    path = tmp_path / "part.mxp"
    a.save_partition(path)
    da = a.download_partition()
    b = mx.MatXtract(dtype)
    st = b.load_partition(path)
    assert (b.n_rows, b.n_cols, b.nnz) == (n, n, m["nnz"]) and st.active == 1
    db = b.download_partition()
    for k in PART_KEYS:
        np.testing.assert_array_equal(_bits(da[k]), _bits(db[k]), err_msg=k)
    b.set_column_space(mx.COLSPACE_PERMUTED)
    np.testing.assert_array_equal(_bits(ya), _bits(b.spmv_host(x)))
    b.set_column_space(mx.COLSPACE_ORIGINAL)
    check_y(dtype, b.spmv_host(x), rp, ci, val, x)
    with pytest.raises(mx.MxError) as e:  # the original CSR is not in the file
        b.partition(0.25, 0.25)
    assert e.value.status == 4
    other = mx.MatXtract(FP16 if dtype == FP64 else FP64)
    with pytest.raises(mx.MxError):
        other.load_partition(path)
    (tmp_path / "junk").write_bytes(b"not a partition")
    with pytest.raises(mx.MxError):
        b.load_partition(tmp_path / "junk")
    for h in (a, b, other):
        h.close()


def test_tau_search_on_the_device():
    m = synth.generate("c3", n=8 * 20_000)
    n, rp, ci, val, x = m["n"], m["row_ptr"], m["col_ind"], m["val"], m["x"]
    h = mx.MatXtract(FP64)
    h.upload_csr(n, n, rp, ci, val)
    tc, tr, ms_best, ms_plain = h.autotune_tau(grid=4)
    assert 0.0 <= tr <= tc <= 1.0 and ms_best > 0 and ms_best <= ms_plain * 1.0001
    # the winner is left installed
    check_y(FP64, h.spmv_host(x), rp, ci, val, x)
    if (tc, tr) != (0.0, 0.0):
        assert_partition_equal(FP64, h, oracle.partition(FP64, n, n, rp, ci, val, tc, tr))
    h.close()


@pytest.mark.parametrize("dtype", [FP64, FP16])
def test_l2_prefetch_distance_does_not_change_the_product(dtype, monkeypatch):
    """The CSR kernel's L2 prefetch of a later tile's streams is a hint: any distance, including one that points at
    the last full tile, leaves y bit-identical."""
    m = synth.generate("c2", n=120_000)
    n, rp, ci, x = m["n"], m["row_ptr"], m["col_ind"], m["x"].astype(np.float64 if dtype == FP64 else np.float16)
    val = values(dtype, len(ci), 5)
    ys = []
    for dist in ("0", "1", "3", "100000"):
        monkeypatch.setenv("MX_RESID_PREFETCH", dist)
        h = mx.MatXtract(dtype)
        h.upload_csr(n, n, rp, ci, val)
        h.partition(0.3, 0.2)
        ys.append(h.spmv_host(x))
        assert h.device_error() == 0
        h.close()
    check_y(dtype, ys[0], rp, ci, val, x)
    for y in ys[1:]:
        np.testing.assert_array_equal(_bits(y), _bits(ys[0]))


def test_stream_gather_floor_is_measured_below_the_product():
    import torch
    m = synth.generate("c2", n=400_000)
    n, rp, ci, val, x = m["n"], m["row_ptr"], m["col_ind"], m["val"], m["x"]
    h = mx.MatXtract(FP16)
    h.upload_csr(n, n, rp, ci, val)
    h.partition(0.0, 0.0)
    x_dev = torch.from_numpy(x.view(np.int16)).cuda().view(torch.float16)
    y_dev = torch.empty(n, dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    floor = h.stream_gather_floor(x_dev.data_ptr(), warm=2, iters=10)
    t = h.spmv_timed(x_dev.data_ptr(), y_dev.data_ptr(), warm=2, iters=10)["ms_total"]
    assert 0 < floor < t * 1.5   # no row logic, nothing written: cannot be much slower than the real product
    torch.cuda.synchronize()
    del x_dev, y_dev
    h.close()


@pytest.mark.parametrize("dtype", [FP64, FP16])
@pytest.mark.parametrize("dd", [mx.DD_CSR, mx.DD_TILE])
def test_hot_column_prefix_in_shared_memory_gives_the_same_bits(dtype, dd):
    """The persistent CSR kernel that serves the hot-column prefix of x from shared memory does the same arithmetic in
    the same order as the one-tile-per-CTA kernel: identical y bits, partition arrays untouched."""
    m = synth.generate("c4", n=60_000, dtype=dtype)
    n, rp, ci, val, x = m["n"], m["row_ptr"], m["col_ind"], m["val"], m["x"]
    h = mx.MatXtract(dtype)
    h.upload_csr(n, n, rp, ci, val)
    for tau in ((0.5, 0.25), (0.4, 0.0), (0.9, 0.9)):
        st = h.partition(*tau)
        h.set_dd_executor(dd)
        h.set_column_space(mx.COLSPACE_PERMUTED)
        h.set_hot_prefix(mx.HOT_OFF)
        assert h.hot_prefix[0] == 0
        y_off = h.spmv_host(x)
        before = h.download_partition()
        h.set_hot_prefix(mx.HOT_ON)
        cols = h.hot_prefix[0]
        assert 0 < cols <= st.dCols and (cols * (8 if dtype == FP64 else 2)) % 16 == 0
        y_on = h.spmv_host(x)
        np.testing.assert_array_equal(_bits(y_on), _bits(y_off))
        check_y(dtype, y_on, rp, ci, val, x)
        after = h.download_partition()
        for k in PART_KEYS:
            np.testing.assert_array_equal(_bits(before[k]), _bits(after[k]), err_msg=k)
        assert h.device_error() == 0
        h.set_hot_prefix(mx.HOT_AUTO)
    h.close()


@pytest.mark.parametrize("dtype", [FP64, FP16])
def test_sparse_encode_entry_point_honours_its_knobs(dtype):
    """mx_se_tcspmv builds the sparse-encode layout on the device: any NUM / threshold / block_longest gives the same
    product (within tolerance), returned in length-sorted row order with the permutation in order_rid."""
    rp, ci = random_csr(700, 9, 21, empty_rows=0.15, skew=True)   # empty rows, rows of 1-4, a few very long rows
    val = values(dtype, len(ci), 21)
    x = values(dtype, 700, 22)
    want = oracle.exact_spmv(rp, ci, val, x)
    scale = oracle.abs_rowsum_max(dtype, rp, ci, val, x)
    lens = np.diff(rp)
    for num, thr, longest in ((4, 0.75, 256), (1, 0.0, 8), (8, 1.0, 16), (3, 0.5, 40), (0, -1.0, 0)):
        y_se, order, _ = mx.se_tcspmv(dtype, val, rp, ci, x, warm=0, iters=1, num=num, threshold=thr,
                                      block_longest=longest)
        assert sorted(order.tolist()) == list(range(700))
        assert (np.diff(lens[order]) <= 0).all()  # longest rows first
        got = np.empty_like(y_se)
        got[order] = y_se
        err = np.abs(got.astype(np.float64) - want).max() / scale
        assert err <= (1e-13 if dtype == FP64 else 6e-4), (num, thr, longest, err)


@pytest.mark.parametrize("name,n,tau", [("c2", 200_000, (0.46, 0.33)), ("c4", 300_000, (0.5, 0.25)),
                                        ("c3", 8 * 30_000, (0.5, 0.5)), ("c5", 400_000, (0.7, 0.5))])
def test_core_dense_block_through_each_executor(name, n, tau):
    """tile / csr / sparse-encode executors of the core-dense block give the same y within tolerance, leave the
    partition arrays alone, and the automatic choice reports a time for each."""
    m = synth.generate(name, n=n)
    dtype, rp, ci, val, x = m["dtype"], m["row_ptr"], m["col_ind"], m["val"], m["x"]
    h = mx.MatXtract(dtype)
    h.upload_csr(n, n, rp, ci, val)
    h.partition(*tau)
    t_tile, t_csr, t_se = h.dd_executor_times
    assert min(t_tile, t_csr, t_se) > 0
    fastest = min(((t_tile, mx.DD_TILE), (t_csr, mx.DD_CSR), (t_se, mx.DD_SE)))[0]
    assert {mx.DD_TILE: t_tile, mx.DD_CSR: t_csr, mx.DD_SE: t_se}[h.dd_executor] == fastest
    before = h.download_partition()
    for ex in (mx.DD_TILE, mx.DD_CSR, mx.DD_SE):
        h.set_dd_executor(ex)
        assert h.dd_executor == ex
        for space in (mx.COLSPACE_PERMUTED, mx.COLSPACE_ORIGINAL):
            h.set_column_space(space)
            check_y(dtype, h.spmv_host(x), rp, ci, val, x)
    after = h.download_partition()
    for k in PART_KEYS:
        np.testing.assert_array_equal(_bits(before[k]), _bits(after[k]), err_msg=k)
    assert h.device_error() == 0
    h.close()


def test_column_slab_execution_matches_the_plain_kernel():
    """tau = (0,0), FP64: the product cut into column slabs (one pass per slab writing partial sums, combined in slab
    order by blocks of 2048 rows; the row count leaves a ragged last block) equals the reference within tolerance, is
    reproducible bit for bit, and is refused (plain kernel kept) when rows are not sorted by column."""
    m = synth.generate("c5", n=300_011)
    n, rp, ci, val, x = m["n"], m["row_ptr"], m["col_ind"], m["val"], m["x"]
    h = mx.MatXtract(FP64)
    h.upload_csr(n, n, rp, ci, val)
    h.partition(0.0, 0.0)
    assert h.column_slabs[0] == 0          # x (2.4 MB) fits L2: the automatic rule leaves the plain kernel
    y_plain = h.spmv_host(x)
    launches_plain = h.launches_per_spmv
    for count in (2, 7, 16):
        h.set_column_slabs(count)
        assert h.column_slabs[0] == count and h.launches_per_spmv > launches_plain
        y1 = h.spmv_host(x)
        y2 = h.spmv_host(x)
        np.testing.assert_array_equal(_bits(y1), _bits(y2))
        check_y(FP64, y1, rp, ci, val, x)
        assert np.abs(y1 - y_plain).max() <= 1e-13 * max(1.0, np.abs(y_plain).max())
    h.set_column_slabs(0)
    assert h.column_slabs[0] == 0
    np.testing.assert_array_equal(_bits(h.spmv_host(x)), _bits(y_plain))
    # rows with unsorted columns: the slabs cannot be cut, the plain kernel stays and the result is still right
    rp_u, ci_u = random_csr(2000, 8, 5, sort_rows=False)
    val_u, x_u = values(FP64, len(ci_u), 5), values(FP64, 2000, 6)
    h.upload_csr(2000, 2000, rp_u, ci_u, val_u)
    h.set_column_slabs(4)
    h.partition(0.0, 0.0)
    assert h.column_slabs[0] == 0
    check_y(FP64, h.spmv_host(x_u), rp_u, ci_u, val_u, x_u)
    # FP16 handles refuse a forced slab count
    g = mx.MatXtract(FP16)
    with pytest.raises(mx.MxError):
        g.set_column_slabs(4)
    g.close()
    h.close()


@pytest.mark.parametrize("name,n,tau,parts", [("c4", 60_000, (0.5, 0.25), 3), ("c2", 80_000, (0.46, 0.33), 2),
                                              ("c3", 8 * 3000, (0.5, 0.5), 4), ("c5", 90_000, (0.7, 0.5), 5)])
def test_slabs_extracted_with_global_rankings_reproduce_the_whole_partition(name, n, tau, parts):
    """A matrix cut into row slabs (one handle per slab, as on several GPUs) and extracted with the WHOLE matrix's
    column and row rankings: every slab has the whole matrix's hot columns in the same order (same dCols, same xperm),
    the slabs' hot rows together are exactly the whole matrix's hot rows, and the slabs' products concatenate to y."""
    import torch
    from matxtract_b200.distributed import nnz_balanced_bounds, slab

    m = synth.generate(name, n=n)
    dtype, rp, ci, val, x = m["dtype"], m["row_ptr"], m["col_ind"], m["val"], m["x"]
    nnz = m["nnz"]
    whole = mx.MatXtract(dtype)
    whole.upload_csr(n, n, rp, ci, val)
    sw = whole.partition(*tau)
    dw = whole.download_partition()
    bounds = nnz_balanced_bounds(rp, parts)
    hs = []
    total = torch.zeros(n, dtype=torch.int32, device="cuda")
    for g in range(parts):
        r0, r1 = bounds[g], bounds[g + 1]
        h = mx.MatXtract(dtype)
        h.upload_csr(r1 - r0, n, *slab(rp, ci, val, r0, r1))
        c = torch.zeros(n, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        h.col_counts(c)
        total += c
        hs.append(h)
    torch.cuda.synchronize()
    rows = torch.zeros(n, dtype=torch.int32, device="cuda")
    for g, h in enumerate(hs):
        part = torch.zeros(max(h.n_rows, 1), dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        h.row_counts_in_hot_columns(tau[0], total, nnz, part)
        rows[bounds[g]:bounds[g + 1]] = part[: h.n_rows]
    torch.cuda.synchronize()
    k, s, cut_count, cut_row = hs[0].rank_cut(rows, n, int(np.float32(np.int32(nnz)) * np.float32(tau[1])))
    assert (k, s) == (sw.dRows, sw.nnzRowD)
    hot, y = [], []
    for g, h in enumerate(hs):
        st = h.partition_global(tau[0], tau[1], total, nnz, cut_count, cut_row, bounds[g])
        d = h.download_partition()
        assert st.dCols == sw.dCols
        np.testing.assert_array_equal(d["xperm"], dw["xperm"])
        hot.append(d["rId"].astype(np.int64) + bounds[g])
        assert st.nnzRowD + st.nnzCD == h.nnz
        y.append(h.spmv_host(x))
        assert h.device_error() == 0
    hot = np.concatenate(hot)
    owners_without_hot_rows = sum(1 for g in range(parts)
                                  if not ((dw["rId"] >= bounds[g]) & (dw["rId"] < bounds[g + 1])).any())
    # a slab that owns none of the hot rows still extracts one row (the reference's cut is never empty)
    assert len(hot) == sw.dRows + owners_without_hot_rows
    assert set(dw["rId"].tolist()) <= set(hot.tolist())
    check_y(dtype, np.concatenate(y), rp, ci, val, x)
    for h in hs + [whole]:
        h.close()


def test_column_slabs_of_a_row_slab_with_its_band():
    """One GPU's share of a row-partitioned matrix (rows [r0, r1) x all columns): the entries near the diagonal form a
    band pass of their own, the far entries go through slab passes whose partial sums are combined first; the band
    pass runs last and adds to them - through mx_spmv into y, through mx_spmv_peers (here with this GPU's buffer as
    the only peer) into every GPU's buffer."""
    import torch

    n = 400_000
    m = synth.generate("c5", n=n)
    rp, ci, val, x = m["row_ptr"], m["col_ind"], m["val"], m["x"]
    want = oracle.exact_spmv(rp, ci, val, x)
    scale = oracle.abs_rowsum_max(FP64, rp, ci, val, x)
    from matxtract_b200.distributed import slab

    for r0, r1 in ((0, 150_001), (150_001, 333_333), (333_333, n)):
        h = mx.MatXtract(FP64)
        h.upload_csr(r1 - r0, n, *slab(rp, ci, val, r0, r1))
        h.set_row_offset(r0)
        h.partition(0.0, 0.0)
        y_plain = h.spmv_host(x)
        h.set_column_slabs(5)
        assert h.column_slabs[0] == 5
        y_slab = h.spmv_host(x)
        assert np.abs(y_slab - want[r0:r1]).max() / scale <= TOL[FP64]
        assert np.abs(y_slab - y_plain).max() <= 1e-13 * max(1.0, np.abs(y_plain).max())
        np.testing.assert_array_equal(_bits(y_slab), _bits(h.spmv_host(x)))
        # the fused-exchange order (far passes, band last) into a full-length buffer
        stream = torch.cuda.ExternalStream(h.stream)
        with torch.cuda.stream(stream):
            x_dev = torch.from_numpy(x).cuda()
            y_full = torch.full((n,), float("nan"), dtype=torch.float64, device="cuda")
        stream.synchronize()
        for _ in range(2):
            h.spmv_peers(x_dev, [y_full.data_ptr()], r0)
        h.sync()
        got = y_full.cpu().numpy()
        assert np.isnan(got[:r0]).all() and np.isnan(got[r1:]).all()  # only this slab's rows are written
        assert np.abs(got[r0:r1] - want[r0:r1]).max() / scale <= TOL[FP64]
        assert h.device_error() == 0
        del x_dev, y_full
        h.close()


@pytest.mark.parametrize("dtype", [FP64, FP16])
def test_pipelined_host_products_equal_the_synchronous_call(dtype):
    """mx_spmv_host_async: five products with different x enqueued back to back over the two staging slots (pinned
    buffers), one mx_host_sync; every y equals, bit for bit, what mx_spmv_host returns for the same x - before and
    after a new matrix is uploaded into the same handle, with and without an active partition."""
    import torch

    tdt = torch.float64 if dtype == FP64 else torch.float16
    h = mx.MatXtract(dtype)
    for n, per_row, tau in ((30_000, 9, (0.0, 0.0)), (12_345, 14, (0.5, 0.3))):
        rp, ci = random_csr(n, per_row, 21 + n)
        val = values(dtype, len(ci), 22)
        h.upload_csr(n, n, rp, ci, val)
        h.partition(*tau)
        xs = [values(dtype, n, 100 + i) for i in range(5)]
        want = [h.spmv_host(x).copy() for x in xs]
        check_y(dtype, want[0], rp, ci, val, xs[0])
        as_t = lambda a: torch.from_numpy(a.view(np.int16) if dtype == FP16 else a).view(tdt)
        x_pin = [as_t(x).pin_memory() for x in xs]
        y_pin = [torch.full((n,), float("nan"), dtype=tdt).pin_memory() for _ in xs]
        for rounds in range(2):
            for xp, yp in zip(x_pin, y_pin):
                h.spmv_host_async(xp, yp)
            h.host_sync()
            for yp, w in zip(y_pin, want):
                got = yp.numpy() if dtype == FP64 else yp.view(torch.int16).numpy().view(np.float16)
                np.testing.assert_array_equal(_bits(got), _bits(w))
                yp.fill_(float("nan"))
        # pageable memory is accepted too (no overlap, same result)
        y_np = np.empty(n, mx.capi.np_dtype(dtype))
        h.spmv_host_async(xs[1], y_np)
        h.host_sync()
        np.testing.assert_array_equal(_bits(y_np), _bits(want[1]))
    assert h.device_error() == 0
    h.close()
