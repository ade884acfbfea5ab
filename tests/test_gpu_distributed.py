"""Row-partitioned SpMV on 2 GPUs (one process per GPU, NCCL all-gather of y).  Skipped on a single-GPU box."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
import matxtract_b200 as mx
from matxtract_b200 import synth, distributed as D
import oracle
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
for name, n, tau in (("c2", 60000, (0.46, 0.33)), ("c3", 8 * 4000, (0.5, 0.5)), ("c5", 50000, (0.0, 0.0)),
                     ("c4", 60000, (0.5, 0.25))):
    m = synth.generate(name, n=n)
    dtype = m["dtype"]
    d = D.DistributedSpMV(dtype, n, m["row_ptr"], m["col_ind"], m["val"], rank, world, tau=tau)
    x = torch.from_numpy(m["x"].view(np.int16 if dtype == mx.FP16 else np.float64)).cuda()
    x = x.view(torch.float16) if dtype == mx.FP16 else x
    d.stream.wait_stream(torch.cuda.current_stream())
    y = d.spmv(x)
    d.stream.synchronize()
    y = y.cpu().numpy()
    y_ref = oracle.spmv_serial(dtype, m["row_ptr"], m["col_ind"], m["val"], m["x"])
    err = oracle.y_error(dtype, y, y_ref, m["row_ptr"], m["col_ind"], m["val"], m["x"])
    assert err <= (1e-12 if dtype == mx.FP64 else 2e-3), (name, err)
    assert sum(d.bounds[g + 1] - d.bounds[g] for g in range(world)) == n
    # the same product with the all-gather fused into the kernels (peer stores + one barrier): identical bits
    for how in ("epilogue", "push", "multicast"):
        # same executor of the core-dense block as the first handle (the automatic choice is a timing and may differ
        # between two handles; the executors sum in different orders)
        f = D.DistributedSpMV(dtype, n, m["row_ptr"], m["col_ind"], m["val"], rank, world, tau=tau, fused=how,
                              dd_executor=d.handle.dd_executor if d.stats.active else None)
        if how == "multicast" and not f.peer_y.multicast_ptr:
            print(f"rank {rank} {name}: no multicast address on this box, multicast stores not exercised", flush=True)
            f.close()
            continue
        f.stream.wait_stream(torch.cuda.current_stream())
        for _ in range(3):
            yf = f.spmv(x)
        f.stream.synchronize()
        assert np.array_equal(yf.cpu().numpy().view(np.uint8), y.view(np.uint8)), (name, how)
        print(f"rank {rank} {name} {how} identical", flush=True)
        del yf
        f.close()
    del y, x
    d.close()
    print(f"rank {rank} {name} ok err={err:.2e} rows={d.rows} nnz={d.local_nnz}", flush=True)
# column slabs on a row slab: far passes, combined sums, then the band in row ranges whose finished rows a second
# stream sends to the other GPU while the next range is computed; the same through slab passes + one copy
m = synth.generate("c5", n=1_200_000)
n = m["n"]
x = torch.from_numpy(m["x"]).cuda()
want = oracle.exact_spmv(m["row_ptr"], m["col_ind"], m["val"], m["x"])
scale = oracle.abs_rowsum_max(mx.FP64, m["row_ptr"], m["col_ind"], m["val"], m["x"])
got = {}
for how in ("epilogue", "push"):
    f = D.DistributedSpMV(mx.FP64, n, m["row_ptr"], m["col_ind"], m["val"], rank, world, tau=(0.0, 0.0), fused=how)
    f.handle.set_column_slabs(6)
    assert f.handle.column_slabs[0] == 6
    f.stream.wait_stream(torch.cuda.current_stream())
    for _ in range(3):
        yf = f.spmv(x)
    f.stream.synchronize()
    got[how] = yf.cpu().numpy()
    assert np.abs(got[how] - want).max() / scale <= 1e-12, how
    ck = torch.from_numpy(got[how].view(np.int64)).sum().reshape(1).cuda()
    cks = [torch.zeros_like(ck) for _ in range(world)]
    dist.all_gather(cks, ck)
    assert all(int(c) == int(cks[0]) for c in cks), how  # both GPUs hold the same bits
    del yf
    f.close()
# (the two cut the band into tiles at different places, so rows that span tiles are summed in a different order)
assert np.abs(got["epilogue"] - got["push"]).max() <= 1e-13 * scale
print(f"rank {rank} c5-slabs ok", flush=True)
dist.destroy_process_group()
'''


def test_two_rank_row_partition_matches_the_oracle(tmp_path):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), str(ROOT)],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count(" ok ") == 8
    assert r.stdout.count("c5-slabs ok") == 2
