"""Benchmark of the MatXtract SpMV path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c5|c1|c2|c3|c4] [--n ROWS]

One "step" is one SpMV y = A x of the workload matrix through the library (x permutation, core-dense block, residual
CSR kernel; with N > 1 also the exchange that leaves the whole y on every GPU).  The default workload is the largest
single-GPU configuration, the 1e9-non-zero power-law matrix (n = 64,000,000, FP64, tau = (0,0)), generated from shape
statistics (the reference's SuiteSparse inputs are not available offline).  With N > 1 (launched by torchrun, one rank
per GPU) the SAME matrix is cut into N contiguous row slabs of equal non-zero count (boundaries at
lower_bound(row_ptr, g*nnz/N)), x is replicated and every GPU ends the step with the whole y: strong scaling.
`--scaling weak` multiplies the row count by N instead.  Rank 0 prints one JSON line.

Keys beside the contract's: "cpu_baseline.parity" (at every N: rows sampled from the head and the tail of every slab of
the gathered y against the reference's serial SpMV, and whether all GPUs hold identical copies of y); at N = 1 two
comparators measured in the same run, "library_baseline" (cuSPARSE's CSR SpMV through torch.mv) and
"roofline.stream_gather_floor_ms" (a pass over the same CSR that streams indices and values and gathers x but has no
row logic and writes nothing); at N > 1 "exchange": per rank, the mean time of its own launches of a step and the mean
time it then waits for the other ranks' rows.

--impl reference times the reference's serial CPU SpMV (its spmv_serial, from oracle/_ref when that was built from the
reference sources, else the oracle port) on all host cores over row slabs of a bounded sample (the first rows) of the
same matrix, on rank 0 only.  That arm loads the input generator and the oracle, nothing of the GPU library.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import re
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "spmv_gflops"
UNIT = "GFLOP/s"
NOMINAL_HBM_GBS = 8000.0
KINDS = ["uniform", "power-law", "block 8x8", "hot-column"]


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed regions run."""

    def __init__(self, cuda_index: int, period_s: float = 0.005):
        super().__init__(daemon=True)
        self.period, self.samples, self.reasons, self.max_mhz = period_s, [], set(), None
        self.active = threading.Event()
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.dev = self._handle(pynvml, cuda_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.dev, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    @staticmethod
    def _handle(nv, cuda_index):
        # NVML numbers the GPUs of the machine, CUDA the visible ones: match by UUID
        try:
            import torch

            uuid = "GPU-" + str(torch.cuda.get_device_properties(cuda_index).uuid)
            try:
                return nv.nvmlDeviceGetHandleByUUID(uuid)
            except TypeError:
                return nv.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            return nv.nvmlDeviceGetHandleByIndex(cuda_index)

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._halt.is_set():
            if self.active.is_set():
                try:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(self.dev, nv.NVML_CLOCK_SM))
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.dev)
                    for bit, name in names.items():
                        if r & bit:
                            self.reasons.add(name)
                except Exception:
                    pass
            time.sleep(self.period)

    def stop(self):
        self._halt.set()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------------------------
# workload: shape, slabs, the `config` both arms print
# ---------------------------------------------------------------------------------------------------------------
def workload_shape(args, world):
    from matxtract_b200 import synth

    cfg = synth.CONFIGS[args.workload]
    if getattr(args, "dtype", None):  # the same shape in the other value type
        import dataclasses

        cfg = dataclasses.replace(cfg, dtype={"f64": 0, "f16": 1}[args.dtype])
    n_total = (args.n or cfg.n) * (world if args.scaling == "weak" else 1)
    if cfg.kind == synth.BLOCK:
        n_total -= n_total % 8
    tau = tuple(args.tau) if args.tau else cfg.tau
    return cfg, n_total, tau


def nnz_balanced_bounds(row_ptr, world):
    """Row boundaries with ~nnz/world non-zeros per slab: b[g] = lower_bound(row_ptr, g*nnz/world)."""
    from matxtract_b200.distributed import nnz_balanced_bounds as f

    return f(row_ptr, world)


def config_of(cfg, n_total, nnz_total, world, tau, scaling):
    """The `config` object: the same in the GPU arm and in the reference arm of one (workload, N)."""
    dt = "FP64" if cfg.dtype == 0 else "FP16"
    b_alg = nnz_total * ((8 if cfg.dtype == 0 else 2) + 4)
    return {
        "workload": f"{cfg.name}: synthetic {KINDS[cfg.kind]} square CSR, n={n_total}, {dt} "
                    f"(stand-in for the reference's SuiteSparse inputs)",
        "tau": list(tau), "n": n_total, "nnz": nnz_total, "scaling": scaling if world > 1 else "n/a (1 GPU)",
        "l2": "no flush: the matrix streamed per step is larger than the 126 MB L2" if b_alg / world > 126e6
        else "matrix smaller than L2: latency figure, not a bandwidth figure",
        "parallelism": (f"{world} contiguous row slabs of equal nnz (lower_bound(row_ptr, g*nnz/{world})), x replicated, "
                        f"y all-gathered") if world > 1 else "1 GPU",
    }


def native_libs():
    """The repository's own shared objects mapped into this process (evidence of which code ran)."""
    out = set()
    try:
        for ln in open("/proc/self/maps"):
            path = ln.split(None, 5)[-1].strip() if ln.count("/") else ""
            if path.startswith(str(ROOT)) and ".so" in path:
                out.add(str(Path(path).relative_to(ROOT)))
    except OSError:
        pass
    return sorted(out)


def cpu_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


# ---------------------------------------------------------------------------------------------------------------
# the reference's serial SpMV on the host (checker, CPU baseline, reference arm)
# ---------------------------------------------------------------------------------------------------------------
def reference_spmv_callable(dtype):
    """(fn(val, row_ptr_ptr, col, x, y, rows, cols, nnz) as a ctypes callable, kind)."""
    import oracle

    if oracle.ref_available():
        return oracle.rlib(dtype).ref_spmv_serial, "reference"
    L = oracle.olib()

    def port(val, ptr, ind, x, y, rows, cols, nnz):
        L.mxo_spmv_serial(dtype, val, ptr, ind, x, y, rows)

    return port, "port"


def cpu_spmv_time(dtype, m, x, rows, threads, repeats):
    """Best-of-`repeats` seconds of the reference's serial SpMV over the first `rows` rows of m, split into `threads`
    contiguous slabs of equal nnz (each slab is one call of the unmodified serial routine)."""
    fn, kind = reference_spmv_callable(dtype)
    rp = m["row_ptr"]
    nnz = int(rp[rows])
    bounds = [int(np.searchsorted(rp[: rows + 1], nnz * t // threads, side="left")) for t in range(threads)] + [rows]
    bounds[0] = 0
    vdt = np.float64 if dtype == 0 else np.float16
    y = np.zeros(rows, vdt)
    vp = ctypes.c_void_p
    isz = 4

    def slab(t):
        a, b = bounds[t], bounds[t + 1]
        if b <= a:
            return
        # the routine indexes val/col with the absolute row pointers, so only row_ptr and y are offset
        fn(vp(m["val"].ctypes.data), vp(rp.ctypes.data + a * isz), vp(m["col_ind"].ctypes.data), vp(x.ctypes.data),
           vp(y.ctypes.data + a * y.itemsize), b - a, m["n"], nnz)

    best = float("inf")
    for _ in range(repeats):
        y[:] = 0
        ts = [threading.Thread(target=slab, args=(t,)) for t in range(threads)]
        t0 = time.perf_counter()
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        best = min(best, time.perf_counter() - t0)
    return best, nnz, kind, y


def parity_sample_ranges(bounds, total_rows=200_000):
    """Row ranges to check: the head and the tail of every slab (where slabs meet), ~total_rows rows in all."""
    world = len(bounds) - 1
    k = max(1, total_rows // (2 * world))
    out = []
    for g in range(world):
        a, b = bounds[g], bounds[g + 1]
        if b - a <= 2 * k:
            if b > a:
                out.append((a, b))
        else:
            out += [(a, a + k), (b - k, b)]
    return out


def parity_against_reference(cfg, n_total, dtype, x, ranges, y_rows_of):
    """max |y - y_ref| over the sampled rows / max_i sum_j |a_ij||x_j| over the same rows; y_ref = the reference's
    serial SpMV on rows regenerated on the host.  y_rows_of(a, b) returns the product's rows [a, b) as numpy."""
    import oracle
    from matxtract_b200 import synth

    num = den = 0.0
    rows = 0
    for a, b in ranges:
        mm = synth.generate(cfg, n=n_total, rows=(a, b), with_x=False)
        mm["n"] = n_total
        _, _, _, y_ref = cpu_spmv_time(dtype, mm, x, b - a, 1, 1)
        y = y_rows_of(a, b)
        num = max(num, float(np.max(np.abs(y.astype(np.float64) - y_ref.astype(np.float64)))) if b > a else 0.0)
        den = max(den, oracle.abs_rowsum_max(dtype, mm["row_ptr"], mm["col_ind"], mm["val"], x))
        rows += b - a
    return (num / den if den > 0 else num), rows


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from matxtract_b200 import synth

    world = max(1, args.gpus)
    cfg, n_total, tau = workload_shape(args, world)
    dtype = cfg.dtype
    threads = cpu_threads()
    row_ptr_all = synth.row_pointers(cfg, n_total)  # the whole matrix's row lengths: its nnz, and where a sample ends
    nnz_total = int(row_ptr_all[-1])
    x = np.empty(n_total, np.float64 if dtype == 0 else np.float16)
    synth.synth_lib().mx_synth_vector(cfg.seed, dtype, 0, n_total, ctypes.c_void_p(x.ctypes.data))
    # bounded sample: calibrate on 50k rows, then size the sample so that all steps fit in ~100 s

    def sample(rows):
        m = synth.generate(cfg, n=n_total, rows=(0, rows), with_x=False)
        m["n"] = n_total
        return m

    probe_rows = min(n_total, 50_000)
    t_probe, nnz_probe, kind, _ = cpu_spmv_time(dtype, sample(probe_rows), x, probe_rows, threads, 1)
    rate = nnz_probe / max(t_probe, 1e-9)
    want_nnz = rate * 100.0 / max(1, args.steps + args.warmup)
    rows = int(min(n_total, max(probe_rows, np.searchsorted(row_ptr_all, want_nnz))))
    m = sample(rows)
    for _ in range(args.warmup):
        cpu_spmv_time(dtype, m, x, rows, threads, 1)
    times = []
    nnz = 0
    for _ in range(args.steps):
        t, nnz, kind, _ = cpu_spmv_time(dtype, m, x, rows, threads, 1)
        times.append(t)
    ms = 1e3 * float(np.mean(times))
    value = 2.0 * nnz / (ms * 1e-3) / 1e9
    what = f"first {rows} of {n_total} rows ({nnz} of {nnz_total} nnz), {threads} row slabs of the serial routine in parallel"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": "f64" if dtype == 0 else "f16", "data": "synthetic",
        "config": config_of(cfg, n_total, nnz_total, world, tau, args.scaling),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": what},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "native_libs": native_libs(),
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
# DRAM traffic of the dominant kernel, from the tracked ncu summary table (never typed into this file)
# ---------------------------------------------------------------------------------------------------------------
def profiled_traffic(workload, kernel, tau, n_total):
    """(bytes per launch or None, note).  Reads profiles/dram_traffic.md: one table row per captured (workload, tau,
    kernel) with the rows captured, the DRAM read+write bytes of one launch and the hash of the kernel sources the
    capture was taken on.  A capture of fewer rows is scaled by the row count and flagged."""
    table = ROOT / "profiles" / "dram_traffic.md"
    if not table.exists():
        return None, "no ncu capture on record"
    try:
        from matxtract_b200.build import source_hash

        cur = source_hash()
    except Exception:
        cur = None
    key_tau = f"{tau[0]:g},{tau[1]:g}"
    for ln in table.read_text().splitlines():
        cells = [c.strip() for c in ln.strip().strip("|").split("|")]
        if len(cells) < 6 or cells[0] != workload or cells[1] != key_tau or cells[2] != kernel:
            continue
        try:
            rows, nbytes, h = int(cells[3]), float(cells[4]), cells[5]
        except ValueError:
            continue
        note = f"ncu dram__bytes_read.sum+dram__bytes_write.sum per launch, captured on {rows} rows"
        if rows != n_total:
            nbytes *= n_total / rows
            note += f", scaled to {n_total} rows"
        note += "; kernel sources unchanged since the capture" if h == cur else "; kernel sources CHANGED since the capture"
        return nbytes, note
    return None, "no ncu capture on record for this workload"


def run_ours(args):
    import torch

    import matxtract_b200 as mx
    from matxtract_b200 import synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist_mod.init_process_group("nccl", device_id=dev)
        dist = dist_mod

    # ---- this rank's slab of the one matrix ----
    cfg, n_total, tau = workload_shape(args, world)
    dtype = cfg.dtype
    if world > 1:
        row_ptr_all = synth.row_pointers(cfg, n_total)
        bounds = nnz_balanced_bounds(row_ptr_all, world)
        nnz_total = int(row_ptr_all[-1])
        del row_ptr_all
    else:
        bounds = [0, n_total]
    r0, r1 = bounds[rank], bounds[rank + 1]
    n_local = r1 - r0
    m = synth.generate(cfg, n=n_total, rows=(r0, r1))
    if world == 1:
        nnz_total = m["nnz"]
    tdt = torch.float64 if dtype == mx.FP64 else torch.float16
    vb = 8 if dtype == mx.FP64 else 2

    h = mx.MatXtract(dtype, device=local)
    # rows [r0, r1) x all n_total columns, extracted on its own
    h.upload_csr(n_local, n_total, m["row_ptr"], m["col_ind"], m["val"])
    h.set_row_offset(r0)
    global_ranking = world > 1 and tuple(float(t) for t in tau) != (0.0, 0.0) and args.ranking == "global"

    def extract():
        if global_ranking:  # the whole matrix's column and row rankings: counts summed / gathered over the ranks
            from matxtract_b200.distributed import partition_with_global_rankings

            return partition_with_global_rankings(h, tau, bounds, rank, nnz_total, dev)
        return h.partition(*tau)

    if args.colslabs != -1:  # a forced slab count: mx_partition then builds that layout and times no alternative
        h.set_column_slabs(args.colslabs)
    st = extract()
    preprocess_ms_cold = st.preprocess_ms  # first call: includes CUDA module loading and memory-pool growth
    st = extract()                         # steady-state cost of the same extraction
    dd_times = h.dd_executor_times
    if args.dd != "auto":
        h.set_dd_executor({"tile": mx.DD_TILE, "csr": mx.DD_CSR, "se": mx.DD_SE}[args.dd])
    if args.colspace != "auto":
        h.set_column_space({"permuted": mx.COLSPACE_PERMUTED, "original": mx.COLSPACE_ORIGINAL}[args.colspace])
    slabs = h.column_slabs
    if args.hotx != "auto":
        h.set_hot_prefix({"off": mx.HOT_OFF, "on": mx.HOT_ON}[args.hotx])
    colspace = h.column_space
    hot = h.hot_prefix
    stream = torch.cuda.ExternalStream(h.stream, device=dev)

    x_host = torch.from_numpy(m["x"].view(np.int16 if dtype == mx.FP16 else np.float64)).view(tdt).pin_memory()
    y_host = torch.empty(n_local, dtype=tdt).pin_memory()  # what this rank's caller owns: its slab of y
    # end-to-end legs alternate between two pairs of pinned host buffers (consecutive products of a caller)
    x_host2 = (x_host.clone() if world == 1 else x_host[r0:r1].clone()).pin_memory()
    y_host2 = torch.empty(n_local, dtype=tdt).pin_memory()
    with torch.cuda.stream(stream):
        x_dev = x_host.to(dev, non_blocking=True)
        y_full = torch.zeros(n_total, dtype=tdt, device=dev)
        y_work = y_full if world == 1 else torch.zeros(n_local, dtype=tdt, device=dev)
    stream.synchronize()

    # N > 1: y is assembled either by the kernels themselves (rows stored into every GPU's peer-mapped y over NVLink,
    # one barrier afterwards) or by NCCL after the kernels
    peer_y = None
    method = ["nccl" if world > 1 else "none"]
    if world > 1 and args.gather != "nccl":
        try:
            from matxtract_b200.distributed import PeerY

            with torch.cuda.stream(stream):
                peer_y = PeerY(n_total, tdt, dev)
            method[0] = "epilogue" if args.gather == "auto" else args.gather
        except Exception as e:  # symmetric memory unavailable: keep the NCCL path
            if args.gather != "auto":
                raise
            peer_y = None
            method[0] = "nccl"
            print(f"[bench] symmetric memory unavailable ({type(e).__name__}): y is assembled by NCCL", file=sys.stderr)
    last_y = [y_full]
    push_table = torch.zeros(8, dtype=torch.int64, device=dev) if world > 1 else None
    sizes = [bounds[g + 1] - bounds[g] for g in range(world)]
    longest = max(sizes)
    if world > 1:  # NCCL path with unequal slabs: one padded all-gather, then the slabs are copied into place
        pad_in = torch.zeros(longest, dtype=tdt, device=dev)
        pad_out = torch.empty(world * longest, dtype=tdt, device=dev)

    def enqueue_product(x=None):
        """This rank's launches of one step (no barrier / collective)."""
        x = x_dev if x is None else x
        if world == 1:
            h.spmv(x, y_full)
        elif method[0] == "epilogue":
            buf, ptrs = peer_y.next()
            h.spmv_peers(x, ptrs, r0)
            last_y[0] = buf
        elif method[0] == "multicast":
            buf, ptrs = peer_y.next()
            h.spmv_multicast(x, ptrs, peer_y.multicast_ptr, r0)
            last_y[0] = buf
        elif method[0] == "push":
            buf, ptrs = peer_y.next()
            h.spmv(x, buf[r0:r1])
            h.peer_push(ptrs, rank, r0, n_local, push_table)
            last_y[0] = buf
        else:
            h.spmv(x, y_work)

    def enqueue_exchange():
        if world == 1:
            return
        with torch.cuda.stream(stream):
            if method[0] == "nccl":
                if len(set(sizes)) == 1:
                    dist.all_gather_into_tensor(y_full, y_work)
                else:
                    pad_in[:n_local].copy_(y_work)
                    dist.all_gather_into_tensor(pad_out, pad_in)
                    for g in range(world):
                        y_full[bounds[g]:bounds[g + 1]].copy_(pad_out[g * longest: g * longest + sizes[g]])
                last_y[0] = y_full
            else:
                peer_y.finish()

    def step_device():
        enqueue_product()
        enqueue_exchange()

    e2e_k = [0]
    peer_x = [None]

    def step_e2e():
        """One product from and to HOST memory.  1 GPU: the pipelined C-ABI call (x in, product, y out on three
        streams; the timed region ends with mx_host_sync).  N GPUs: every rank copies in its own share of x (the rows
        it owns of y), the shares are exchanged over NVLink (peer stores + one barrier), then product + y exchange,
        then the rank's slab of y goes back to its host."""
        e2e_k[0] ^= 1
        xh, yh = (x_host, y_host) if e2e_k[0] else (x_host2, y_host2)
        if world == 1:
            h.spmv_host_async(xh, yh)
            return
        if peer_x[0] is None:  # without symmetric memory: the whole x from this rank's host
            with torch.cuda.stream(stream):
                x_dev.copy_(x_host, non_blocking=True)
            step_device()
        else:
            xbuf, xptrs = peer_x[0].next()
            with torch.cuda.stream(stream):
                xbuf[r0:r1].copy_(x_host2, non_blocking=True)  # this rank's share of x
            h.peer_push(xptrs, rank, r0, n_local, push_table)
            with torch.cuda.stream(stream):
                peer_x[0].finish()
            enqueue_product(xbuf)
            enqueue_exchange()
        with torch.cuda.stream(stream):
            yh.copy_(last_y[0][r0:r1], non_blocking=True)

    def step_e2e_single_call():  # the synchronous C-ABI call: one product's latency with host buffers
        h.spmv_host(x_host, y_host)

    def barrier():
        stream.synchronize()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if dist is None:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, steps, warmup, min_total_ms=200.0, max_repeats=20, finish=None):
        """ms per step: EXACTLY `steps` steps between two events on the handle's stream, barrier + synchronise on both
        sides, max over ranks; the region is repeated until the repeats cover min_total_ms (so that the clock sampler
        sees the load) and the median repeat is returned.  finish (optional) runs after the last step, before the
        closing event: the pipelined host call ends its work on a copy stream, which finish waits for."""
        for _ in range(warmup):
            fn()
        if finish:
            finish()
        reps = []
        total = 0.0
        while True:
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            sampler.active.set()
            e0.record(stream)
            for _ in range(steps):
                fn()
            if finish:
                finish()
            e1.record(stream)
            barrier()
            sampler.active.clear()
            ms = max_over_ranks(e0.elapsed_time(e1))
            reps.append(ms / steps)
            total += ms
            if total >= min_total_ms or len(reps) >= max_repeats:
                break
        return float(np.median(reps)), len(reps)

    sampler = ClockSampler(local)
    sampler.start()

    trial = None
    if world > 1 and peer_y is not None and args.gather == "auto":
        # pick the fastest way of assembling y for this workload (all ranks agree: the times are max-reduced)
        trial = {}
        for mth in ("epilogue", "push", "nccl"):
            method[0] = mth
            trial[mth], _ = timed(step_device, 10, 3, min_total_ms=0.0)
        if slabs[0] > 0:
            # with column slabs the finished rows leave by a push after the last pass; the plain kernel can store them
            # from its epilogue while it is still computing: time that too (all ranks take the same decision)
            h.set_column_slabs(0)
            method[0] = "epilogue"
            trial["epilogue, plain kernel"], _ = timed(step_device, 10, 3, min_total_ms=0.0)
            if min(trial, key=trial.get) == "epilogue, plain kernel":
                slabs = h.column_slabs  # slabs stay off
            else:
                h.set_column_slabs(slabs[0])
        method[0] = min(trial, key=trial.get).split(",")[0]
    ms_step, repeats = timed(step_device, args.steps, max(3, args.warmup))
    value = 2.0 * nnz_total / (ms_step * 1e-3) / 1e9
    if world > 1 and peer_y is not None:
        try:
            with torch.cuda.stream(stream):
                peer_x[0] = PeerY(n_total, tdt, dev)
        except Exception:
            peer_x[0] = None
    ms_e2e, _ = timed(step_e2e, max(10, args.steps // 10), 3, min_total_ms=0.0,
                      finish=h.host_sync if world == 1 else None)
    e2e_value = 2.0 * nnz_total / (ms_e2e * 1e-3) / 1e9
    ms_e2e_single = timed(step_e2e_single_call, 5, 2, min_total_ms=0.0)[0] if world == 1 else None

    # ---- parity of the product that was just timed (every N): sampled rows of the gathered y on rank 0 against the
    #      reference's serial SpMV, and all GPUs' copies of y compared with each other ----
    step_device()
    barrier()
    y_final = last_y[0]
    # the host-buffer leg must have produced the same bits as the device-resident product (same x)
    y_e2e = y_host if e2e_k[0] else y_host2
    e2e_same = bool(torch.equal(y_e2e.view(torch.int16 if dtype == mx.FP16 else torch.int64),
                                y_final[r0:r1].cpu().view(torch.int16 if dtype == mx.FP16 else torch.int64)))
    del y_e2e  # a pinned buffer: no reference may outlive shutdown()
    replicas_identical = None
    if dist is not None:
        t = torch.tensor([1.0 if e2e_same else 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        e2e_same = bool(t.item() == 1.0)
    if dist is not None:
        ck = y_final.view(torch.int64 if dtype == mx.FP64 else torch.int16).to(torch.int64).sum().reshape(1)
        allck = [torch.zeros_like(ck) for _ in range(world)]
        dist.all_gather(allck, ck)
        replicas_identical = bool(all(int(c.item()) == int(allck[0].item()) for c in allck))

    # N > 1: where a step's time goes on every rank - this rank's kernels, then the wait for the others (barrier or
    # collective) - from events recorded inside a separate, untimed run of the same steps
    exchange = None
    if world > 1:
        k = min(100, max(10, args.steps // 2))
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(k)]
        barrier()
        for i in range(k):
            ev[i][0].record(stream)
            enqueue_product()
            ev[i][1].record(stream)
            enqueue_exchange()
            ev[i][2].record(stream)
        barrier()
        own = sum(e[0].elapsed_time(e[1]) for e in ev) / k
        wait = sum(e[1].elapsed_time(e[2]) for e in ev) / k
        t = torch.tensor([own, wait], device=dev, dtype=torch.float64)
        allt = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allt, t)
        exchange = {"steps": k, "own_kernels_ms_per_rank": [round(float(a[0]), 4) for a in allt],
                    "wait_for_others_ms_per_rank": [round(float(a[1]), 4) for a in allt],
                    "note": "own = this rank's launches of one step (rows stored to the peers included when fused); "
                            "wait = barrier or collective until every rank's rows have arrived"}

    # per-kernel timing (each half alone, CUDA events on the handle's stream) for the roofline of the dominant kernel
    sampler.active.set()
    halves = h.spmv_timed(x_dev, y_work, warm=3, iters=int(min(args.steps, max(10, 400.0 / max(ms_step, 1e-3)))))
    sampler.active.clear()
    stream.synchronize()
    sampler.stop()
    # library comparator on the same GPU and matrix: cuSPARSE CSR SpMV (through torch.mv on a sparse-CSR tensor)
    cusparse = None
    if world == 1 and not args.no_library_baseline and nnz_total <= 300_000_000:  # a second copy of the CSR
        try:
            with torch.cuda.stream(stream):
                y_ours = y_full.clone()
                A = torch.sparse_csr_tensor(
                    torch.from_numpy(m["row_ptr"].astype(np.int32)).to(dev),
                    torch.from_numpy(m["col_ind"].astype(np.int32)).to(dev),
                    torch.from_numpy(m["val"].view(np.int16 if dtype == mx.FP16 else np.float64)).view(tdt).to(dev),
                    size=(n_local, n_total))
                y_lib = torch.mv(A, x_dev)
                k = max(10, args.steps // 5)
                for _ in range(3):
                    torch.mv(A, x_dev, out=y_lib)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(k):
                    torch.mv(A, x_dev, out=y_lib)
                e1.record(stream)
            stream.synchronize()
            ms_lib = e0.elapsed_time(e1) / k
            err_lib = float((y_lib.double() - y_ours.double()).abs().max() / y_ours.double().abs().max().clamp_min(1e-30))
            cusparse = {"kind": "cuSPARSE CSR SpMV via torch.mv, same GPU, same matrix and x", "ms": ms_lib,
                        "gflops": 2.0 * nnz_total / (ms_lib * 1e-3) / 1e9, "max_rel_diff_to_ours": err_lib}
            del A, y_lib, y_ours
        except Exception as e:  # comparator only: never fails the run
            cusparse = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    # the product without its row logic (stream indices + values, gather x): what this matrix's index pattern allows
    gather_floor_ms = h.stream_gather_floor(x_dev, warm=3, iters=int(min(50, max(5, 200.0 / max(ms_step, 1e-3)))))

    b_alg_total = synth.algorithmic_bytes(n_total, n_total, nnz_total, dtype)
    # residual kernel: its own CSR + x + y; core-dense block: the original CSR bytes of the entries it covers + x_d + y_hot
    b_resid = st.nnzCD * (vb + 4) + (n_local + 1) * 4 + n_total * vb + n_local * vb
    b_dd = st.nnzRowD * (vb + 4) + (st.dRows + 1) * 4 + st.dCols * vb + st.dRows * vb
    peak, peak_kind = measured_peaks()
    dd_names = {1: "tile_kernel", 2: "resid_kernel on dd", 3: "se_kernel"}
    if st.active and halves["ms_tile"] > halves["ms_resid"]:
        dom, dom_ms, dom_bytes = dd_names.get(h.dd_executor, "dd"), halves["ms_tile"], b_dd
    else:
        dom, dom_ms, dom_bytes = "resid_kernel(+fixup)", halves["ms_resid"], b_resid
        if slabs[0] > 0:
            dom = f"resid_kernel(+fixup) x {slabs[0]} column-slab passes + k_combine" + (" + band" if world > 1 else "")
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
    # the table is keyed without the slab count (the tuner may settle on a neighbouring count from run to run)
    dom_key = "resid_kernel(+fixup) column-slab passes + k_combine" if slabs[0] > 0 else dom
    traffic, traffic_note = (profiled_traffic(cfg.name, dom_key, tau, n_total) if world == 1 else (None, "N > 1: not captured"))
    if slabs[0] > 0 and traffic is not None:
        traffic_note += " (sum over the launches of one product, captured with 12 slabs)"
    eff_gbs = b_alg_total / (ms_step * 1e-3) / 1e9

    y_np_of = None
    if rank == 0:
        def y_np_of(a, b):
            t = y_final[a:b].cpu()
            return t.numpy() if dtype == mx.FP64 else t.view(torch.int16).numpy().view(np.float16)

    def shutdown():
        # torch tensors that lived on the handle's stream must go before the stream does
        nonlocal x_dev, y_full, y_work, x_host, y_host, x_host2, y_host2, peer_y, push_table, y_final
        stream.synchronize()
        last_y[0] = None
        peer_y = None
        peer_x[0] = None
        push_table = None
        y_final = None
        del x_dev, y_full, y_work, x_host, y_host, x_host2, y_host2  # pinned buffers record events on the stream when freed
        import gc

        gc.collect()
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        h.close()
        if dist is not None:
            dist.destroy_process_group()

    if rank != 0:
        shutdown()
        return

    import oracle  # the checker: CPU restatement + the reference's own host code

    tol = 1e-12 if dtype == mx.FP64 else 2e-3
    ranges = parity_sample_ranges(bounds)
    err, rows_checked = parity_against_reference(cfg, n_total, dtype, m["x"], ranges, y_np_of)
    parity = {"rows_checked": rows_checked, "row_ranges": len(ranges), "slabs_covered": world,
              "max_err_over_max_abs_rowsum": float(err), "tolerance": tol, "ok": bool(err <= tol),
              "checker": "the reference's spmv_serial on rows regenerated on the host"}
    if replicas_identical is not None:
        parity["all_gpus_hold_identical_y"] = replicas_identical
        parity["ok"] = bool(parity["ok"] and replicas_identical)

    # CPU baseline: the reference's serial CSR SpMV on one core, bounded sample (timed at N = 1 only)
    cpu = {"parity": parity}
    if world == 1 and not args.no_cpu_baseline:
        probe = min(n_local, 100_000)
        t_probe, nnz_probe, kind, _ = cpu_spmv_time(dtype, m, m["x"], probe, 1, 1)
        rows = int(min(n_local, max(probe, np.searchsorted(m["row_ptr"], nnz_probe / max(t_probe, 1e-9) * 5.0))))
        t_cpu, nnz_cpu, kind, _ = cpu_spmv_time(dtype, m, m["x"], rows, 1, 3)
        cpu.update({"value": 2.0 * nnz_cpu / t_cpu / 1e9, "unit": UNIT, "cores": 1, "kind": kind,
                    "sample": f"first {rows} of {n_local} rows ({nnz_cpu} nnz), serial, best of 3",
                    "host_threads_available": cpu_threads()})
        if st.active and m["nnz"] <= 60_000_000:
            # the host extraction the device pipeline replaces, restated on the CPU (oracle), one run
            t0 = time.perf_counter()
            oracle.partition(dtype, n_local, n_total, m["row_ptr"], m["col_ind"], m["val"], *tau)
            cpu["preprocess_ms_cpu_port"] = 1e3 * (time.perf_counter() - t0)

    gather_names = {"none": "1 GPU", "epilogue": "fused into the SpMV epilogue (peer stores over NVLink + barrier)",
                    "multicast": "fused into the SpMV epilogue (multimem stores through NVSwitch multicast + barrier)",
                    "push": "peer push kernel (16-byte stores over NVLink + barrier)", "nccl": "NCCL all-gather"}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms_step, "timed_regions": repeats, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None,
        "dtype": "f64" if dtype == mx.FP64 else "f16", "data": "synthetic",
        "config": config_of(cfg, n_total, nnz_total, world, tau, args.scaling),
        "y_exchange": gather_names[method[0]] + (
            " [auto: " + ", ".join(f"{k} {v * 1e3:.0f} us" for k, v in trial.items()) + "]" if trial else ""),
        "rows_per_gpu": sizes,
        "effective_gbs": eff_gbs, "pct_of_8tbs": 100.0 * eff_gbs / NOMINAL_HBM_GBS / world,
        "pct_of_measured_hbm": 100.0 * eff_gbs / peak / world,
        "algorithmic_bytes_per_step": b_alg_total,
        "partition": {**{k: getattr(st, k) for k in ("active", "dCols", "dRows", "nnzRowD", "nnzCD", "totalFrags", "fragK")},
                      "ranking": "whole matrix (counts exchanged between the GPUs)" if global_ranking else
                      ("per slab" if world > 1 and st.active else "single matrix")},
        "dd_executor": {1: "tile (tensor cores)", 2: "csr (CUDA cores)", 3: "sparse-encode (tensor cores)"}.get(
            h.dd_executor, "none"),
        "dd_executor_tuned_ms": {"tile": dd_times[0], "csr": dd_times[1], "sparse_encode": dd_times[2]},
        "column_space": {"in_use": {1: "permuted", 2: "original"}.get(colspace[0], "n/a"),
                         "tuned_ms_permuted": colspace[1], "tuned_ms_original": colspace[2]},
        "column_slabs": {"in_use": slabs[0], "tuned_ms_plain": slabs[1], "tuned_ms_slabbed": slabs[2]},
        "hot_x_prefix": {"columns_in_shared_memory": hot[0], "tuned_ms_with": hot[1], "tuned_ms_without": hot[2]},
        "csr_l2_prefetch_tiles": {"resid": h.csr_prefetch[0], "dd": h.csr_prefetch[1]},
        "tc_nnz_ratio": st.tc_nnz_ratio, "preprocess_ms": st.preprocess_ms, "preprocess_ms_first_call": preprocess_ms_cold,
        "plan_tuning_ms": st.tuning_ms,
        "ms_dd_alone": halves["ms_tile"], "ms_resid_alone": halves["ms_resid"], "ms_sequence": halves["ms_total"],
        "launches_per_spmv": h.launches_per_spmv,
        "roofline": {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "peak_kind": peak_kind,
                     "unit": "GB/s", "frac": achieved / peak, "traffic": traffic, "traffic_note": traffic_note,
                     "algorithmic_bytes_per_launch": dom_bytes, "ms_per_launch": dom_ms,
                     "stream_gather_floor_ms": gather_floor_ms,
                     "floor_over_step": gather_floor_ms / (ms_step if world == 1 else halves["ms_total"])},
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": n_total * vb if (world == 1 or peer_x[0] is not None) else world * n_total * vb,
                "d2h_bytes_per_step": n_total * vb,  # whole job: every rank its own share
                "path": "mx_spmv_host_async x steps + mx_host_sync (C ABI; pinned host x in, product, host y out, the "
                        "copies of consecutive products overlapping the kernels)" if world == 1 else
                ("per rank: its share of x from pinned host memory, shares exchanged over NVLink (peer stores + "
                 "barrier), product + y exchange, this rank's slab of y -> pinned host" if peer_x[0] is not None else
                 "per rank: pinned x -> device, product + exchange, this rank's slab of y -> pinned host"),
                "ms_per_step_single_synchronous_call": ms_e2e_single,
                "same_bits_as_the_device_resident_product": e2e_same},
        "gpu_launches": (h.launches_per_spmv + (1 if method[0] == "push" else 0)) * args.steps * repeats,
        "clocks": sampler.summary(),
        "cpu_baseline": cpu,
        "native_libs": native_libs(),
    }
    if exchange is not None:
        line["exchange"] = exchange
    if cusparse is not None:
        line["library_baseline"] = cusparse
    print(json.dumps(line), flush=True)
    shutdown()


def main():
    ap = argparse.ArgumentParser(allow_abbrev=False)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-library-baseline", action="store_true", help="skip the cuSPARSE comparator")
    ap.add_argument("--workload", default="c5", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--n", "--rows", dest="n", type=int, default=0,
                    help="rows of the matrix (default: the configuration's size); spell it --rows under torchrun")
    ap.add_argument("--tau", type=float, nargs=2, default=None)
    ap.add_argument("--dtype", default=None, choices=["f64", "f16"],
                    help="value type (default: the configuration's own)")
    ap.add_argument("--gather", default="auto", choices=["auto", "epilogue", "multicast", "push", "nccl"],
                    help="N > 1: how y is assembled (auto = the fastest of epilogue / push / nccl, timed at set-up)")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: strong = the one matrix cut into N slabs (default), weak = N times the rows")
    ap.add_argument("--ranking", default="global", choices=["global", "local"],
                    help="N > 1, tau != (0,0): rank columns and rows over the whole matrix (default) or per slab")
    ap.add_argument("--dd", default="auto", choices=["auto", "tile", "csr", "se"],
                    help="executor of the core-dense block (auto = the fastest of the three, timed at partition time)")
    ap.add_argument("--colspace", default="auto", choices=["auto", "permuted", "original"],
                    help="column numbering used for execution")
    ap.add_argument("--colslabs", type=int, default=-1,
                    help="column slabs of the plain CSR product: -1 auto (when x exceeds L2), 0 off, k >= 2 forced")
    ap.add_argument("--hotx", default="auto", choices=["auto", "on", "off"],
                    help="hot-column prefix of x in shared memory (permuted numbering only)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the timed CPU baseline leg (profiling runs)")
    args = ap.parse_args()
    # torchrun pins every rank to one OpenMP thread; the input generator is host code that scales with threads, so give
    # every rank its share of the cores (set before anything loads the OpenMP runtime)
    world = max(1, int(os.environ.get("WORLD_SIZE", "1")))
    if world > 1 or "OMP_NUM_THREADS" not in os.environ:
        share = 1 if args.impl == "reference" else world  # the reference arm works on rank 0 only
        os.environ["OMP_NUM_THREADS"] = str(max(1, cpu_threads() // share))
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
