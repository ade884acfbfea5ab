"""Row-partitioned SpMV over several GPUs of one box: one process per GPU, x replicated, y all-gathered.

The reference is single-GPU; the partition follows the usual 1-D scheme: contiguous row slabs with boundaries at
``lower_bound(row_ptr, g * nnz / G)`` so that every rank streams the same number of non-zeros.  Each rank extracts and
multiplies its own slab (``rows_g x all columns``) with its own (tau_c, tau_r) partition; parity across ranks is on y.
"""
from __future__ import annotations

import numpy as np


def nnz_balanced_bounds(row_ptr: np.ndarray, world: int) -> list[int]:
    """Row boundaries b[0]=0 <= ... <= b[world]=n with ~nnz/world non-zeros per slab."""
    row_ptr = np.asarray(row_ptr)
    n, nnz = len(row_ptr) - 1, int(row_ptr[-1])
    b = [int(np.searchsorted(row_ptr, (g * nnz) // world, side="left")) for g in range(world)] + [n]
    b[0] = 0
    for g in range(1, world + 1):  # monotone even with empty leading rows
        b[g] = max(b[g], b[g - 1])
    return b


def equal_row_bounds(n: int, world: int) -> list[int]:
    return [(g * n) // world for g in range(world)] + [n]


def slab(row_ptr, col_ind, val, r0: int, r1: int):
    """CSR of rows [r0, r1) with row pointers rebased to 0."""
    lo, hi = int(row_ptr[r0]), int(row_ptr[r1])
    return (np.asarray(row_ptr[r0:r1 + 1], np.int32) - lo).astype(np.int32), col_ind[lo:hi], val[lo:hi]


def all_gather_rows(y_local, bounds, group=None):
    """Assembles the full y from every rank's slice (unequal sizes allowed).  Works on NCCL and gloo tensors."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    sizes = [bounds[g + 1] - bounds[g] for g in range(world)]
    if len(set(sizes)) == 1:
        out = torch.empty(sum(sizes), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(out, y_local.contiguous(), group=group)
        return out
    # unequal slabs: pad every slice to the longest one, gather once, cut the padding out (same code on NCCL and gloo)
    longest = max(sizes)
    padded = torch.zeros(longest, dtype=y_local.dtype, device=y_local.device)
    padded[: y_local.numel()] = y_local
    out = torch.empty(world * longest, dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(out, padded, group=group)
    return torch.cat([out[g * longest: g * longest + sizes[g]] for g in range(world)])


def partition_with_global_rankings(handle, tau, bounds, rank, nnz_total, device, group=None):
    """Extracts this rank's slab with the rankings of the WHOLE matrix (one process per GPU): the slabs' column counts
    are summed (all-reduce), the per-row counts inside the hot columns are gathered in row order, every rank takes the
    same row cut, and ``mx_partition_global`` keeps the hot rows this rank owns.  Returns the slab's PartitionStats."""
    import torch
    import torch.distributed as dist

    tau_c, tau_r = float(tau[0]), float(tau[1])
    stream = torch.cuda.ExternalStream(handle.stream, device=device)
    with torch.cuda.stream(stream):
        counts = torch.zeros(handle.n_cols, dtype=torch.int32, device=device)
        stream.synchronize()
        handle.col_counts(counts)
        dist.all_reduce(counts, group=group)
        rows = torch.zeros(max(handle.n_rows, 1), dtype=torch.int32, device=device)[: handle.n_rows]
        stream.synchronize()
        handle.row_counts_in_hot_columns(tau_c, counts, nnz_total, rows)
        all_rows = all_gather_rows(rows, bounds, group).contiguous()
        stream.synchronize()
    threshold = int(np.float32(np.int32(nnz_total)) * np.float32(tau_r))  # the reference's int * float, truncated
    k, _, cut_count, cut_row = handle.rank_cut(all_rows, int(all_rows.numel()), threshold)
    if k == 0:
        from .capi import MxError

        raise MxError(3, "tau_r threshold never reached by the ranking prefix")
    return handle.partition_global(tau_c, tau_r, counts, nnz_total, cut_count, cut_row, bounds[rank])


class PeerY:
    """Full-length y of every GPU, mapped into every other GPU (torch symmetric memory over NVLink), double-buffered.

    ``mx_spmv_peers`` stores this rank's rows into all of them from inside the SpMV kernels; ``finish()`` is the one
    barrier after which every rank's y is complete.  Two buffers alternate so that a rank that is still reading the
    previous product (in stream order) is never overwritten by a faster peer's next product.
    """

    def __init__(self, n_total, torch_dtype, device, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        group = dist.group.WORLD if group is None else group
        self.bufs, self.hdls = [], []
        for _ in range(2):
            t = symm_mem.empty(n_total, dtype=torch_dtype, device=device)
            self.bufs.append(t)
            self.hdls.append(symm_mem.rendezvous(t, group))
        self.ptrs = [list(h.buffer_ptrs) for h in self.hdls]
        # NVLink multicast address of each buffer (0 when the box has no multicast support)
        self.mc_ptrs = [int(getattr(h, "multicast_ptr", 0) or 0) for h in self.hdls]
        self.k = 0

    def next(self):
        """(tensor that will hold the next product, device addresses of that buffer on every GPU)."""
        self.k ^= 1
        return self.bufs[self.k], self.ptrs[self.k]

    @property
    def multicast_ptr(self) -> int:
        """Multicast address of the buffer next() returned last (0: not available)."""
        return self.mc_ptrs[self.k]

    def finish(self):
        """Barrier across the GPUs on the current stream: afterwards the buffer returned by next() is complete."""
        self.hdls[self.k].barrier(channel=0)


class DistributedSpMV:
    """This rank's slab on its GPU plus the collective that assembles y.

    ``local_spmv`` (x_full -> y_slab tensor) can be injected to exercise the host-side logic without a GPU; by default
    the slab runs through a :class:`matxtract_b200.MatXtract` handle on ``device``.
    """

    def __init__(self, dtype, n_cols, row_ptr, col_ind, val, rank, world, tau=(0.0, 0.0), device=None, balance="nnz",
                 local_spmv=None, group=None, fused=False, dd_executor=None, ranking="global"):
        self.rank, self.world, self.group = rank, world, group
        n = len(row_ptr) - 1
        self.bounds = nnz_balanced_bounds(row_ptr, world) if balance == "nnz" else equal_row_bounds(n, world)
        r0, r1 = self.bounds[rank], self.bounds[rank + 1]
        self.rows = r1 - r0
        rp, ci, v = slab(row_ptr, col_ind, val, r0, r1)
        self.local_nnz = int(rp[-1])
        self._local = local_spmv
        self.handle = None
        if local_spmv is None:
            import torch

            from . import MatXtract

            self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)
            self.handle = MatXtract(dtype, device=self.device.index)
            self.handle.upload_csr(self.rows, n_cols, rp, ci, v)
            self.handle.set_row_offset(r0)
            if dd_executor is not None:  # fix the executor of the core-dense block instead of timing the three
                self.handle.set_dd_executor(dd_executor)
            if world > 1 and ranking == "global" and tuple(float(t) for t in tau) != (0.0, 0.0):
                self.stats = partition_with_global_rankings(self.handle, tau, self.bounds, rank, int(row_ptr[-1]),
                                                            self.device, group)
            else:
                self.stats = self.handle.partition(*tau)
            self.stream = torch.cuda.ExternalStream(self.handle.stream, device=self.device)
            tdt = torch.float64 if dtype == 0 else torch.float16
            self._y = torch.zeros(max(self.rows, 1), dtype=tdt, device=self.device)[: self.rows]
            # fused: the kernels store y rows straight into every GPU's y (peer-mapped), one barrier afterwards
            self.peer_y = PeerY(n, tdt, self.device, group) if fused else None
            # False (NCCL all-gather), True / "epilogue" (kernels store to all peers), "multicast", "push"
            self.fused = fused
            self._table = torch.zeros(8, dtype=torch.int64, device=self.device)
        else:
            self._slab = (rp, ci, v)

    def spmv(self, x_full):
        """y = A x for the whole matrix (every rank returns the full y)."""
        import torch

        if self._local is not None:
            y_local = self._local(self._slab, x_full)
            return all_gather_rows(y_local, self.bounds, self.group)
        if self.peer_y is not None:
            y, ptrs = self.peer_y.next()
            r0 = self.bounds[self.rank]
            if self.fused == "push":  # product into this GPU's own y, then 16-byte peer stores of the slab
                self.handle.spmv(x_full, y[r0: r0 + self.rows])
                self.handle.peer_push(ptrs, self.rank, r0, self.rows, self._table)
            elif self.fused == "multicast":  # rows leave through the NVLink multicast address of the buffers
                if not self.peer_y.multicast_ptr:
                    raise RuntimeError("symmetric memory has no multicast address on this box")
                self.handle.spmv_multicast(x_full, ptrs, self.peer_y.multicast_ptr, r0)
            else:
                self.handle.spmv_peers(x_full, ptrs, r0)
            with torch.cuda.stream(self.stream):
                self.peer_y.finish()
            return y
        self.handle.spmv(x_full, self._y)
        with torch.cuda.stream(self.stream):
            return all_gather_rows(self._y, self.bounds, self.group)

    def close(self):
        if self.handle is not None:
            import torch

            self.stream.synchronize()
            self._y = None
            self.peer_y = None
            self._table = None
            torch.cuda.synchronize()
            self.handle.close()
            self.handle = None
