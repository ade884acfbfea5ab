"""Host-side logic of the row-partitioned multi-GPU path, exercised with world_size = 2 (and 3) gloo ranks on the CPU:
slab boundaries, slab extraction, and the all-gather that assembles y (equal and unequal slab sizes).  The local
multiply is injected (an exactly accumulated numpy product), so no GPU is involved."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from matxtract_b200 import distributed as D
from matxtract_b200 import synth

import oracle


def test_nnz_balanced_bounds_properties():
    m = synth.generate("c2", n=5000)
    for world in (1, 2, 3, 8):
        b = D.nnz_balanced_bounds(m["row_ptr"], world)
        assert b[0] == 0 and b[-1] == m["n"] and all(b[i] <= b[i + 1] for i in range(world))
        per = [int(m["row_ptr"][b[g + 1]] - m["row_ptr"][b[g]]) for g in range(world)]
        assert sum(per) == m["nnz"]
        # no slab exceeds its share by more than the longest row
        longest = int(np.diff(m["row_ptr"]).max())
        assert max(per) <= m["nnz"] / world + longest
    assert D.equal_row_bounds(10, 3) == [0, 3, 6, 10]


def test_slabs_tile_the_matrix():
    m = synth.generate("c4", n=3000)
    b = D.nnz_balanced_bounds(m["row_ptr"], 4)
    cols = np.concatenate([D.slab(m["row_ptr"], m["col_ind"], m["val"], b[g], b[g + 1])[1] for g in range(4)])
    np.testing.assert_array_equal(cols, m["col_ind"])
    rp = D.slab(m["row_ptr"], m["col_ind"], m["val"], b[1], b[2])[0]
    assert rp[0] == 0 and rp[-1] == m["row_ptr"][b[2]] - m["row_ptr"][b[1]]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, balance, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m = synth.generate("c2", n=4000, dtype=0)

        def local(slab, x):
            rp, ci, v = slab
            return torch.from_numpy(oracle.exact_spmv(rp, ci, v, x.numpy()))

        d = D.DistributedSpMV(0, m["n"], m["row_ptr"], m["col_ind"], m["val"], rank, world, balance=balance,
                              local_spmv=local)
        y = d.spmv(torch.from_numpy(m["x"].astype(np.float64)))
        want = oracle.exact_spmv(m["row_ptr"], m["col_ind"], m["val"], m["x"])
        ok = bool(np.array_equal(y.numpy(), want))
        sizes = [d.bounds[g + 1] - d.bounds[g] for g in range(world)]
        q.put((rank, ok, sizes, d.local_nnz))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,balance", [(2, "nnz"), (2, "rows"), (3, "nnz")])
def test_all_gather_assembles_y_on_gloo(world, balance):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, balance, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _, _ in res)
    if balance == "nnz":
        assert len({tuple(s) for _, _, s, _ in res}) == 1  # every rank computed the same boundaries


def test_c_abi_row_partitioner_matches_the_python_one():
    """mx_mg_partition_rows (host code of the multi-GPU entry) = lower_bound(row_ptr, g * nnz / G), monotone."""
    import matxtract_b200 as mx
    from matxtract_b200.distributed import nnz_balanced_bounds

    rng = np.random.default_rng(3)
    for n, world in ((1, 1), (7, 3), (1000, 8), (1000, 1), (50, 8)):
        lens = rng.integers(0, 40, n)
        lens[rng.random(n) < 0.3] = 0
        rp = np.zeros(n + 1, np.int32)
        np.cumsum(lens, out=rp[1:])
        b = mx.mg_partition_rows(rp, world)
        assert b.tolist() == nnz_balanced_bounds(rp, world)
        assert b[0] == 0 and b[-1] == n and (np.diff(b) >= 0).all()
    # all non-zeros in one row: every boundary but the last collapses onto it
    rp = np.zeros(11, np.int32)
    rp[6:] = 100
    assert mx.mg_partition_rows(rp, 4).tolist() == nnz_balanced_bounds(rp, 4)
