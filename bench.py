"""Benchmark of the MatXtract SpMV path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c4|c5|c1] [--n ROWS]

One "step" is one SpMV y = A x of the workload matrix through the extraction's split execution (x permutation, tile
kernel, residual CSR kernel).  The default workload is the power-law graph configuration (n = 2,000,000,
FP16, tau = (0.46, 0.33)) generated from shape statistics (the reference's SuiteSparse inputs are not available
offline).  With N > 1 (launched by torchrun, one rank per GPU) every rank owns an equal slab of rows of an
(N*n) x (N*n) matrix of the same shape, x is replicated and y is all-gathered over NCCL inside the timed step: weak
scaling.  Prints one JSON line (rank 0).  Beside the contract's keys it carries, at N = 1, two comparators measured in
the same run: "library_baseline" (cuSPARSE's CSR SpMV on the same matrix and x, through torch.mv) and
"roofline.stream_gather_floor_ms" (a pass over the same CSR that streams indices and values and gathers x but has no
row logic and writes nothing: what the matrix's index pattern allows a CSR-ordered kernel on this GPU), and
"csr_l2_prefetch_tiles" (what the plan-time tuner chose for the CSR kernels).  At N > 1 it carries "exchange": for every
rank, the mean time of its own launches of a step and the mean time it then waits for the other ranks' rows.

--impl reference times the reference's serial CPU SpMV (its spmv_serial, from oracle/_ref when that was built from the
reference sources, else the oracle port) on all host cores over row slabs of a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
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

    def __init__(self, index: int, period_s: float = 0.005):
        super().__init__(daemon=True)
        self.index, self.period, self.samples, self.reasons, self.max_mhz = index, period_s, [], set(), None
        self.active = threading.Event()
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.dev = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.dev, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

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


def workload_matrix(args, rank, world):
    """This rank's slab of the (world*n) x (world*n) matrix, the full x, and the shape description."""
    from matxtract_b200 import synth

    cfg = synth.CONFIGS[args.workload]
    if args.scaling == "strong":  # the whole matrix is fixed, every rank owns n/world rows
        n_total = args.n or cfg.n
        n_local = n_total // world
        n_total = n_local * world
    else:  # weak: every rank owns a slab of the configuration's size
        n_local = args.n or cfg.n
        n_total = n_local * world
    m = synth.generate(cfg, n=n_total, rows=(rank * n_local, (rank + 1) * n_local))
    return cfg, n_local, n_total, m


def cpu_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def reference_spmv_callable(dtype):
    """(fn(val, row_ptr_ptr, col, x, y, rows, cols, nnz) as a ctypes callable, kind)."""
    import oracle

    if oracle.ref_available():
        return oracle.rlib(dtype).ref_spmv_serial, "reference"
    L = oracle.olib()

    def port(val, ptr, ind, x, y, rows, cols, nnz):
        L.mxo_spmv_serial(dtype, val, ptr, ind, x, y, rows)

    return port, "port"


def cpu_spmv_time(dtype, m, rows, threads, repeats):
    """Best-of-`repeats` seconds of the reference's serial SpMV over the first `rows` rows, split into `threads`
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
        fn(vp(m["val"].ctypes.data), vp(rp.ctypes.data + a * isz), vp(m["col_ind"].ctypes.data), vp(m["x"].ctypes.data),
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


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg, n_local, n_total, m = workload_matrix(args, 0, 1)
    dtype = m["dtype"]
    threads = cpu_threads()
    # bounded sample: calibrate on 50k rows, then size the sample so that all steps fit in ~100 s
    probe_rows = min(n_local, 50_000)
    t_probe, nnz_probe, kind, _ = cpu_spmv_time(dtype, m, probe_rows, threads, 1)
    rate = nnz_probe / max(t_probe, 1e-9)
    budget_s = 100.0
    want_nnz = rate * budget_s / max(1, args.steps + args.warmup)
    rows = int(min(n_local, max(probe_rows, np.searchsorted(m["row_ptr"], want_nnz))))
    for _ in range(args.warmup):
        cpu_spmv_time(dtype, m, rows, threads, 1)
    times = []
    nnz = 0
    for _ in range(args.steps):
        t, nnz, kind, _ = cpu_spmv_time(dtype, m, rows, threads, 1)
        times.append(t)
    ms = 1e3 * float(np.mean(times))
    value = 2.0 * nnz / (ms * 1e-3) / 1e9
    sample = f"first {rows} of {n_local} rows ({nnz} nnz), {threads} row slabs of the serial routine in parallel"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64" if dtype == 0 else "f16", "data": "synthetic",
        "config": {"workload": describe(cfg, n_local, 1), "tau": list(cfg.tau)},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def describe(cfg, n_local, world):
    return (f"{cfg.name}: synthetic {['uniform', 'power-law', 'block 8x8', 'hot-column'][cfg.kind]} square CSR, "
            f"{n_local} rows per GPU x {world} GPU(s), {'FP64' if cfg.dtype == 0 else 'FP16'}")


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
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod

    cfg, n_local, n_total, m = workload_matrix(args, rank, world)
    dtype = m["dtype"]
    tdt = torch.float64 if dtype == mx.FP64 else torch.float16
    tau = tuple(args.tau) if args.tau else cfg.tau

    h = mx.MatXtract(dtype, device=local)
    # this rank's slab: rows [rank*n_local, (rank+1)*n_local) x all n_total columns, extracted on its own
    h.upload_csr(n_local, n_total, m["row_ptr"], m["col_ind"], m["val"])
    st = h.partition(*tau)
    preprocess_ms_cold = st.preprocess_ms  # first call: includes CUDA module loading and memory-pool growth
    st = h.partition(*tau)                 # steady-state cost of the same extraction
    if args.dd != "auto":
        h.set_dd_executor({"tile": mx.DD_TILE, "csr": mx.DD_CSR}[args.dd])
    if args.colspace != "auto":
        h.set_column_space({"permuted": mx.COLSPACE_PERMUTED, "original": mx.COLSPACE_ORIGINAL}[args.colspace])
    colspace = h.column_space
    stream = torch.cuda.ExternalStream(h.stream, device=torch.device("cuda", local))

    x_host = torch.from_numpy(m["x"].view(np.int16 if dtype == mx.FP16 else np.float64)).view(tdt).pin_memory()
    y_host = torch.empty(n_total, dtype=tdt).pin_memory()
    with torch.cuda.stream(stream):
        x_dev = x_host.to(f"cuda:{local}", non_blocking=True)
        y_full = torch.zeros(n_total, dtype=tdt, device=f"cuda:{local}")
        y_work = torch.zeros(n_local, dtype=tdt, device=f"cuda:{local}")
    stream.synchronize()

    # N > 1: y is assembled either by the kernels themselves (rows stored into every GPU's peer-mapped y over NVLink,
    # one barrier afterwards) or by an NCCL all-gather after the kernels
    peer_y = None
    gather = "none"
    if world > 1:
        gather = "nccl all-gather"
        if args.gather in ("auto", "fused"):
            try:
                from matxtract_b200.distributed import PeerY

                with torch.cuda.stream(stream):
                    peer_y = PeerY(n_total, tdt, torch.device("cuda", local))
                gather = "fused into the SpMV epilogue (peer stores over NVLink + barrier)"
            except Exception as e:  # symmetric memory unavailable: keep the NCCL path
                if args.gather == "fused":
                    raise
                peer_y = None
                gather = f"nccl all-gather (symmetric memory unavailable: {type(e).__name__})"
    last_y = [y_full]
    method = ["epilogue"]  # with peer buffers: "epilogue" (rows stored to all peers by the kernels) or "push"
    push_table = torch.zeros(8, dtype=torch.int64, device=f"cuda:{local}") if world > 1 else None

    def step_device():
        if world == 1:
            h.spmv(x_dev, y_full)
        elif peer_y is not None and method[0] == "epilogue":
            buf, ptrs = peer_y.next()
            h.spmv_peers(x_dev, ptrs, rank * n_local)
            with torch.cuda.stream(stream):
                peer_y.finish()
            last_y[0] = buf
        elif peer_y is not None and method[0] == "multicast":
            buf, ptrs = peer_y.next()
            h.spmv_multicast(x_dev, ptrs, peer_y.multicast_ptr, rank * n_local)
            with torch.cuda.stream(stream):
                peer_y.finish()
            last_y[0] = buf
        elif peer_y is not None and method[0] == "push":
            buf, ptrs = peer_y.next()
            h.spmv(x_dev, buf[rank * n_local: (rank + 1) * n_local])
            h.peer_push(ptrs, rank, rank * n_local, n_local, push_table)
            with torch.cuda.stream(stream):
                peer_y.finish()
            last_y[0] = buf
        else:
            h.spmv(x_dev, y_work)
            with torch.cuda.stream(stream):
                dist.all_gather_into_tensor(y_full, y_work)

    def step_e2e():
        with torch.cuda.stream(stream):
            x_dev.copy_(x_host, non_blocking=True)
        step_device()
        with torch.cuda.stream(stream):
            y_host.copy_(last_y[0], non_blocking=True)
        stream.synchronize()

    def barrier():
        stream.synchronize()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler.active.set()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        sampler.active.clear()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device=f"cuda:{local}", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    sampler = ClockSampler(local)
    sampler.start()
    nnz_local = m["nnz"]
    nnz_total = nnz_local
    if dist is not None:
        t = torch.tensor([nnz_local], device=f"cuda:{local}", dtype=torch.int64)
        dist.all_reduce(t)
        nnz_total = int(t.item())

    if world > 1 and peer_y is not None and args.gather == "auto":
        # pick the fastest way of assembling y for this workload (all ranks agree: the times are max-reduced)
        trial = {}
        # multicast stores measured slower than the plain peer stores (2-byte rows, 8 GPUs): timed only on request
        want_mc = peer_y.mc_ptrs[0] and os.environ.get("MX_BENCH_MULTICAST", "0") == "1"
        for mth in ("epilogue", "multicast", "push", "nccl") if want_mc else ("epilogue", "push", "nccl"):
            saved = peer_y
            if mth == "nccl":
                peer_y = None
            else:
                method[0] = mth
            trial[mth] = timed(step_device, 30, 5)
            peer_y = saved
        best = min(trial, key=trial.get)
        if best == "nccl":
            peer_y = None
            gather = "nccl all-gather"
        else:
            method[0] = best
            gather = {"epilogue": "fused into the SpMV epilogue (peer stores over NVLink + barrier)",
                      "multicast": "fused into the SpMV epilogue (multimem stores through NVSwitch multicast + barrier)",
                      "push": "peer push kernel (16-byte stores over NVLink + barrier)"}[best]
        gather += " [auto: " + ", ".join(f"{k} {v * 1e3:.0f} us" for k, v in trial.items()) + "]"
    ms_step = timed(step_device, args.steps, max(3, args.warmup))
    value = 2.0 * nnz_total / (ms_step * 1e-3) / 1e9
    ms_e2e = timed(step_e2e, max(10, args.steps // 10), 3)
    e2e_value = 2.0 * nnz_total / (ms_e2e * 1e-3) / 1e9

    # N > 1: where a step's time goes on every rank - this rank's kernels, then the wait for the others (barrier or
    # collective) - from events recorded inside a separate, untimed run of the same steps
    exchange = None
    if world > 1:
        k = min(200, max(20, args.steps // 2))
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(k)]
        barrier()
        for i in range(k):
            ev[i][0].record(stream)
            if peer_y is not None:
                buf, ptrs = peer_y.next()
                if method[0] == "push":
                    h.spmv(x_dev, buf[rank * n_local: (rank + 1) * n_local])
                    h.peer_push(ptrs, rank, rank * n_local, n_local, push_table)
                elif method[0] == "multicast":
                    h.spmv_multicast(x_dev, ptrs, peer_y.multicast_ptr, rank * n_local)
                else:
                    h.spmv_peers(x_dev, ptrs, rank * n_local)
                ev[i][1].record(stream)
                with torch.cuda.stream(stream):
                    peer_y.finish()
            else:
                h.spmv(x_dev, y_work)
                ev[i][1].record(stream)
                with torch.cuda.stream(stream):
                    dist.all_gather_into_tensor(y_full, y_work)
            ev[i][2].record(stream)
        barrier()
        own = sum(e[0].elapsed_time(e[1]) for e in ev) / k
        wait = sum(e[1].elapsed_time(e[2]) for e in ev) / k
        t = torch.tensor([own, wait], device=f"cuda:{local}", dtype=torch.float64)
        allt = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allt, t)
        exchange = {"steps": k, "own_kernels_ms_per_rank": [round(float(a[0]), 4) for a in allt],
                    "wait_for_others_ms_per_rank": [round(float(a[1]), 4) for a in allt],
                    "note": "own = this rank's launches of one step (rows stored to the peers included when fused); "
                            "wait = barrier or collective until every rank's rows have arrived"}

    # per-kernel timing (each half alone, CUDA events on the handle's stream) for the roofline of the dominant kernel
    sampler.active.set()
    halves = h.spmv_timed(x_dev, y_work, warm=max(3, args.warmup), iters=args.steps)
    sampler.active.clear()
    stream.synchronize()
    sampler.stop()
    # library comparator on the same GPU and matrix: cuSPARSE CSR SpMV (through torch.mv on a sparse-CSR tensor)
    cusparse = None
    if world == 1 and not args.no_library_baseline and nnz_total <= 300_000_000:  # a second copy of the CSR
        try:
            with torch.cuda.stream(stream):
                A = torch.sparse_csr_tensor(
                    torch.from_numpy(m["row_ptr"].astype(np.int32)).to(f"cuda:{local}"),
                    torch.from_numpy(m["col_ind"].astype(np.int32)).to(f"cuda:{local}"),
                    torch.from_numpy(m["val"].view(np.int16 if dtype == mx.FP16 else np.float64)).view(tdt).to(f"cuda:{local}"),
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
            err_lib = float((y_lib.double() - y_full.double()).abs().max() / y_full.double().abs().max().clamp_min(1e-30))
            cusparse = {"kind": "cuSPARSE CSR SpMV via torch.mv, same GPU, same matrix and x", "ms": ms_lib,
                        "gflops": 2.0 * nnz_total / (ms_lib * 1e-3) / 1e9, "max_rel_diff_to_ours": err_lib}
            del A, y_lib
        except Exception as e:  # comparator only: never fails the run
            cusparse = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    # the product without its row logic (stream indices + values, gather x): what this matrix's index pattern allows
    gather_floor_ms = h.stream_gather_floor(x_dev, warm=3, iters=max(10, args.steps // 10))

    vb = 8 if dtype == mx.FP64 else 2
    n_rows_h = n_local
    b_alg_total = synth.algorithmic_bytes(n_total, n_total, nnz_total, dtype)
    # residual kernel: its own CSR + x + y; tile kernel: the original CSR bytes of the entries it covers + x_d + y_hot
    b_resid = st.nnzCD * (vb + 4) + (n_rows_h + 1) * 4 + n_total * vb + n_rows_h * vb
    b_tile = st.nnzRowD * (vb + 4) + (st.dRows + 1) * 4 + st.dCols * vb + st.dRows * vb
    peak, peak_kind = measured_peaks()
    if st.active and halves["ms_tile"] > halves["ms_resid"]:
        dom, dom_ms, dom_bytes = ("tile_kernel" if h.dd_executor == 1 else "resid_kernel on dd"), halves["ms_tile"], b_tile
    else:
        dom, dom_ms, dom_bytes = "resid_kernel(+fixup)", halves["ms_resid"], b_resid
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
    # DRAM read + write bytes of the dominant kernel per launch, from the ncu captures summarised under profiles/
    # (resid_kernel_c2_fp16.md, tile_and_resid_kernels_c3_fp64.md); null for workloads that were not captured
    traffic = None
    if world == 1 and not args.n:
        tau_key = "default" if not args.tau else ("tau0" if tuple(args.tau) == (0.0, 0.0) else None)
        traffic = {("c2", "resid_kernel(+fixup)", "default"): 136.5e6, ("c3", "resid_kernel(+fixup)", "default"): 645.7e6,
                   ("c3", "tile_kernel", "default"): 489.1e6,
                   ("c3", "resid_kernel(+fixup)", "tau0"): 1240.9e6}.get((cfg.name, dom, tau_key))
    eff_gbs = b_alg_total / (ms_step * 1e-3) / 1e9

    def shutdown():
        # torch tensors that lived on the handle's stream must go before the stream does
        nonlocal x_dev, y_full, y_work, x_host, y_host, peer_y, push_table
        stream.synchronize()
        last_y[0] = None
        peer_y = None
        push_table = None
        del x_dev, y_full, y_work, x_host, y_host  # pinned buffers record events on the stream when freed
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        h.close()
        if dist is not None:
            dist.destroy_process_group()

    if rank != 0:
        shutdown()
        return

    # CPU baseline (rank 0, N = 1 only): the reference's serial CSR SpMV on one core, bounded sample
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        probe = min(n_local, 100_000)
        t_probe, nnz_probe, kind, _ = cpu_spmv_time(dtype, m, probe, 1, 1)
        rows = int(min(n_local, max(probe, np.searchsorted(m["row_ptr"], nnz_probe / max(t_probe, 1e-9) * 4.0))))
        t_cpu, nnz_cpu, kind, y_cpu = cpu_spmv_time(dtype, m, rows, 1, 3)
        cpu = {"value": 2.0 * nnz_cpu / t_cpu / 1e9, "unit": UNIT, "cores": 1, "kind": kind,
               "sample": f"first {rows} of {n_local} rows ({nnz_cpu} nnz), serial, best of 3",
               "host_threads_available": cpu_threads()}
        # the serial result doubles as the checker of the product that was just timed (same rows, same x)
        import oracle

        y_dev_rows = y_full[:rows].cpu().numpy() if dtype == mx.FP64 else y_full[:rows].cpu().view(torch.int16).numpy().view(np.float16)
        rp_s = m["row_ptr"][: rows + 1]
        err = oracle.y_error(dtype, y_dev_rows, y_cpu, rp_s, m["col_ind"], m["val"], m["x"])
        tol = 1e-12 if dtype == mx.FP64 else 2e-3
        cpu["parity"] = {"rows_checked": rows, "max_err_over_max_abs_rowsum": float(err), "tolerance": tol,
                         "ok": bool(err <= tol)}
        if st.active and m["nnz"] <= 60_000_000:
            # the host extraction the device pipeline replaces, restated on the CPU (oracle), one run
            import oracle

            t0 = time.perf_counter()
            oracle.partition(dtype, n_local, n_total, m["row_ptr"], m["col_ind"], m["val"], *tau)
            cpu["preprocess_ms_cpu_port"] = 1e3 * (time.perf_counter() - t0)

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": "f64" if dtype == mx.FP64 else "f16", "data": "synthetic",
        "config": {"workload": describe(cfg, n_local, world), "tau": list(tau), "n": n_total, "nnz": nnz_total,
                   "l2": "no flush: the matrix streamed per step is larger than the 126 MB L2"
                   if b_alg_total / world > 126e6 else "matrix smaller than L2: latency figure, not a bandwidth figure",
                   "parallelism": f"rows x{world}, x replicated, y: {gather}" if world > 1 else "1 GPU"},
        "effective_gbs": eff_gbs, "pct_of_8tbs": 100.0 * eff_gbs / NOMINAL_HBM_GBS / world,
        "pct_of_measured_hbm": 100.0 * eff_gbs / peak / world,
        "algorithmic_bytes_per_step": b_alg_total,
        "partition": {k: getattr(st, k) for k in ("active", "dCols", "dRows", "nnzRowD", "nnzCD", "totalFrags", "fragK")},
        "dd_executor": {1: "tile (tensor cores)", 2: "csr (CUDA cores)"}.get(h.dd_executor, "none"),
        "column_space": {"in_use": {1: "permuted", 2: "original"}.get(colspace[0], "n/a"),
                         "tuned_ms_permuted": colspace[1], "tuned_ms_original": colspace[2]},
        "csr_l2_prefetch_tiles": {"resid": h.csr_prefetch[0], "dd": h.csr_prefetch[1]},
        "tc_nnz_ratio": st.tc_nnz_ratio, "preprocess_ms": st.preprocess_ms, "preprocess_ms_first_call": preprocess_ms_cold,
        "ms_tile_alone": halves["ms_tile"], "ms_resid_alone": halves["ms_resid"], "ms_sequence": halves["ms_total"],
        "roofline": {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "peak_kind": peak_kind,
                     "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                     "algorithmic_bytes_per_launch": dom_bytes, "ms_per_launch": dom_ms,
                     "stream_gather_floor_ms": gather_floor_ms,
                     "floor_over_step": gather_floor_ms / (ms_step if world == 1 else halves["ms_total"])},
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": n_total * vb,
                "d2h_bytes_per_step": n_total * vb},
        "gpu_launches": h.launches_per_spmv * args.steps,
        "clocks": sampler.summary(),
    }
    if exchange is not None:
        line["exchange"] = exchange
    if cusparse is not None:
        line["library_baseline"] = cusparse
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)
    shutdown()


def main():
    ap = argparse.ArgumentParser(allow_abbrev=False)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-library-baseline", action="store_true", help="skip the cuSPARSE comparator")
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--n", "--rows", dest="n", type=int, default=0,
                    help="rows per GPU (default: the configuration's size); spell it --rows under torchrun")
    ap.add_argument("--tau", type=float, nargs=2, default=None)
    ap.add_argument("--gather", default="auto", choices=["auto", "fused", "nccl"],
                    help="N > 1: how y is assembled (auto = fused peer stores when symmetric memory is available)")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="N > 1: weak = --n rows per GPU (default), strong = --n rows in total, split over the GPUs")
    ap.add_argument("--dd", default="auto", choices=["auto", "tile", "csr"], help="executor of the core-dense block")
    ap.add_argument("--colspace", default="auto", choices=["auto", "permuted", "original"],
                    help="column numbering used for execution")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
