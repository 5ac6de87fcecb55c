#!/usr/bin/env python
"""Benchmark of the CSR SpMV / SpMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl ours|reference]

One "step" is one product over one batch of synthetic input: y = alpha*A*x + beta*y (or the SpMM
equivalent) with A resident on the device(s).  The headline workload is c2, the 27-point stencil on a
160^3 grid (4 096 000 rows, 109 215 352 non-zeros), the configuration the headline metric is quoted
on.  The same run then measures the other configurations of ops_sparse_b200/workloads.py (c1, c3, c4,
c5 at one GPU; c3 and c4 at several) the same way and reports them under "configs" in the same line;
--configs picks another list, --configs none skips them.  At one GPU "configs" also holds the headline
workload with its values and x stored as fp16 (fp32 result), "<workload>_fp16".

At N GPUs (launched by torchrun, one rank per GPU) the same matrix is row-block sharded by nnz, x / B
is replicated and every step ends with the reassembly of y / C on every rank, so total work is fixed
("strong" scaling).  Timing: W warm-up steps, then K steps between barriers and device
synchronisations, each step bracketed by CUDA events on the launching stream; the reported time is
the maximum over ranks.  The matrix alone (0.9 - 5.7 GB) is far larger than the 126 MB L2, so every
step streams it from HBM again (c1, 2 MB, is L2-resident by nature and is reported as such).

Every rank compares the WHOLE result it holds (all rows of the reassembled y / C) with the oracle's
fp64 truth, once before the timed steps and once after the last of them; the line reports the rows
checked, the number of ranks that checked and the largest violation count over ranks and checks.

Rank 0 prints one JSON line.  Keys beyond the usual ones:
  roofline      the product kernels of one step: algorithmic bytes (the CSR arrays, x or B, y or C,
                each once) / event-timed duration, against the measured HBM copy bandwidth.  At one
                GPU the step is exactly those kernels (one graph replay); at several GPUs they are
                timed as their own graph replay with the reassembly switched off
  e2e           the same product driven from HOST buffers: each rank copies its share of x (or B) from
                pinned host memory, the shares are all-gathered into the replicas over NVLink, the
                sharded product step runs, and each rank copies its own row block of y (or C) back to
                pinned host memory, all inside the timed region; at one GPU that is the plain
                aclsparseSpMV / aclsparseSpMM call between two copies
  cpu_baseline  the test oracle's restatement of the reference's host golden, timed on one host core
                (the way the reference's tests time it) on the same inputs
  --impl reference times that CPU golden with all host threads instead of the GPU path.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from ops_sparse_b200 import workloads  # noqa: E402

FALLBACK_HBM_GBS = 6650.0

# DRAM read + write bytes per algorithmic byte, from ncu captures of the kernels named (profiles/):
# SpMV traffic is proportional to the algorithmic bytes, so a 1 M-row capture scales; the SpMM figures
# are from one full-size launch each.
TRAFFIC_RATIO = {
    "c2": 224.06 / 223.71,   # SpmvRowBlockKernel, 1 M-row stencil
    "c3": 286.29 / 285.02,   # SpmvTileKernel, 1 M-row power-law case
    "c4": 7.972 / 1.2122,    # SpmmTileKernel, one full-size launch
}


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.out = None

    def start(self):
        try:
            self.out = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.gpu)], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.flush()
        self.out.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.out.read().splitlines():
            f = [s.strip() for s in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        self.out.close()
        os.unlink(self.out.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no_samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


def host_threads() -> int:
    """Every core this process may run on: torchrun exports OMP_NUM_THREADS=1, which must not shrink a CPU leg."""
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def cpu_golden_seconds(cfg: dict, threads: int, repeats: int) -> float:
    """Average seconds of one product by the oracle's restatement of the reference's host golden."""
    from oracle import oracle as O
    best = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        if cfg["kind"] == "spmv":
            O.spmv_f64(cfg["row_ptr"], cfg["col_ind"], cfg["values"], cfg["x"], cfg["y"], cfg["alpha"], cfg["beta"],
                       threads=threads)
        else:
            n = cfg["n"]
            O.spmm_f32(cfg["row_ptr"], cfg["col_ind"], cfg["values"], cfg["b"], n, cfg["c"], n, n, cfg["alpha"],
                       cfg["beta"], threads=threads)
        best.append(time.perf_counter() - t0)
    return float(np.mean(best))


def cpu_sample(cfg: dict, max_rows: int) -> dict:
    """The leading row block of the workload, so that a CPU pass stays within seconds."""
    if cfg["rows"] <= max_rows:
        return cfg
    r = max_rows
    p = int(cfg["row_ptr"][r])
    out = dict(cfg)
    out.update(rows=r, row_ptr=cfg["row_ptr"][: r + 1], col_ind=cfg["col_ind"][:p], values=cfg["values"][:p], nnz=p)
    if cfg["kind"] == "spmv":
        out.update(y=cfg["y"][:r])
    else:
        out.update(c=cfg["c"][:r])
    return out


def metric_name(cfg: dict) -> str:
    return "spmv_gflops" if cfg["kind"] == "spmv" else "spmm_gflops"


def describe(cfg: dict) -> str:
    text = {
        "c1": "c1: CSR SpMV fp32 16384^2, Poisson(16) rows clamped to [1,64], alpha=1 beta=0",
        "c2": "c2: CSR SpMV fp32, 27-point stencil on a 160^3 grid, alpha=1 beta=0",
        "c3": "c3: CSR SpMV fp32 power-law 4194304^2, Zipf(2.0) rows mean 32 cap 200000, alpha=1.5 beta=0.5",
        "c4": "c4: CSR SpMM fp32 1048576^2 Poisson(16) rows, B 1048576x128 row-major, alpha=1 beta=0",
        "c5": "c5: CSR SpMM fp32 power-law 8388608^2, Zipf(2.1) rows mean 20 cap 500000, B 8388608x64",
    }[cfg["name"]]
    return f"{text} ({cfg['rows']} rows, {cfg['nnz']} nnz)"


def run_reference(args, cfg):
    """The reference's CPU golden path on the host cores (all threads), same workload and metric."""
    threads = host_threads()
    sample = cpu_sample(cfg, args.cpu_rows)
    for _ in range(max(args.warmup, 1)):
        cpu_golden_seconds(sample, threads, 1)
    secs = cpu_golden_seconds(sample, threads, args.steps)
    gflops = workloads.flops(sample) / secs / 1e9
    what = (f"{sample['rows']} of {cfg['rows']} rows ({sample['nnz']} non-zeros) of {cfg['name']}, "
            f"fp64-accumulated SpmvCpu restatement" if cfg["kind"] == "spmv" else
            f"{sample['rows']} of {cfg['rows']} rows ({sample['nnz']} non-zeros) of {cfg['name']}, "
            f"fp32 SpmmCpuFp32 restatement")
    line = {
        "impl": "reference", "metric": metric_name(cfg), "value": gflops, "unit": "GFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": describe(cfg), "device": "host CPU", "threads": threads},
        "cpu_baseline": {"value": gflops, "unit": "GFLOP/s", "cores": threads, "kind": "port", "sample": what},
        "e2e": {"value": gflops, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


class Context:
    """Process group, device and the small collectives the measurement needs."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        from ops_sparse_b200 import _lib as L
        from ops_sparse_b200 import sharded

        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the operators have no CPU implementation")
        L.lib()  # fails loudly when libops_sparse.so is missing
        self.torch, self.dist, self.sharded = torch, dist, sharded
        self.rank, self.world, self.device = sharded.init_process_group_from_env()
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}: launch with torchrun --nproc-per-node N")

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())


def shared_dir(ctx: Context) -> str:
    """Scratch directory in shared memory that the ranks of this run exchange host arrays through."""
    return os.path.join("/dev/shm", f"aclsp_bench_{os.environ.get('MASTER_PORT', '0')}_{os.getuid()}")


def make_workload(ctx: Context, name: str, rows) -> dict:
    """The configuration's host arrays: generated once (rank 0) and mapped by the other ranks, so that N ranks do
    not spend N times the generation time and memory."""
    if ctx.world == 1:
        return workloads.make(name, rows=rows)
    base = os.path.join(shared_dir(ctx), f"cfg_{name}")
    if ctx.rank == 0:
        cfg = workloads.make(name, rows=rows)
        os.makedirs(base, exist_ok=True)
        scalars = {}
        for key, value in cfg.items():
            if isinstance(value, np.ndarray):
                np.save(os.path.join(base, key + ".npy"), value)
            else:
                scalars[key] = value
        with open(os.path.join(base, "scalars.json"), "w") as f:
            json.dump(scalars, f)
    ctx.barrier()
    if ctx.rank != 0:
        with open(os.path.join(base, "scalars.json")) as f:
            cfg = json.load(f)
        for fname in os.listdir(base):
            if fname.endswith(".npy"):
                cfg[fname[:-4]] = np.asarray(np.load(os.path.join(base, fname), mmap_mode="r"))
    ctx.barrier()
    return cfg


def cleanup_shared(ctx: Context) -> None:
    if ctx.world > 1:
        ctx.barrier()
        if ctx.rank == 0:
            import shutil
            shutil.rmtree(shared_dir(ctx), ignore_errors=True)


_truth_serial = [0]


def check_whole_result(ctx: Context, cfg: dict, full, alpha: float, beta: float) -> dict:
    """This rank's whole reassembled y / C against the oracle's fp64 truth; reduced over ranks.  The truth is
    computed once per check: every rank computes an equal share of the rows with its share of the host threads
    and the shares are exchanged through shared memory; the comparison covers all rows on every rank."""
    from oracle import oracle as O
    threads = max(1, host_threads() // ctx.world)
    rows = cfg["rows"]
    spmv = cfg["kind"] == "spmv"
    n = 1 if spmv else cfg["n"]

    def truth_of(r0, r1):
        if spmv:
            sub_ptr = np.ascontiguousarray(cfg["row_ptr"][r0:r1 + 1])
            p0, p1 = int(sub_ptr[0]), int(sub_ptr[-1])
            return O.spmv_f64(sub_ptr - p0, cfg["col_ind"][p0:p1], cfg["values"][p0:p1], cfg["x"], cfg["y"][r0:r1],
                              alpha, beta, threads=threads)
        return O.spmm_f64(cfg["row_ptr"], cfg["col_ind"], cfg["values"], cfg["b"], n, cfg["c"], n, n, cfg["cols"],
                          alpha, beta, row_begin=r0, row_end=r1, threads=threads)

    bad, max_abs, max_rel = 0, 0.0, 0.0
    chunk = max(1, (1 << 27) // n)  # a GiB of fp64 truth at a time
    if ctx.world == 1:
        for r0 in range(0, rows, chunk):
            r1 = min(rows, r0 + chunk)
            b, a, r = O.check_tolerance(full[r0:r1].cpu().numpy(), truth_of(r0, r1))
            bad, max_abs, max_rel = bad + b, max(max_abs, a), max(max_rel, r)
    else:
        _truth_serial[0] += 1
        base = os.path.join(shared_dir(ctx), f"truth_{cfg['name']}_{_truth_serial[0]}")
        share = (rows + ctx.world - 1) // ctx.world
        lo, hi = min(ctx.rank * share, rows), min((ctx.rank + 1) * share, rows)
        if ctx.rank == 0:
            os.makedirs(base, exist_ok=True)
        ctx.barrier()
        np.save(os.path.join(base, f"{ctx.rank}.npy"), truth_of(lo, hi) if hi > lo else np.empty((0,) + (() if spmv else (n,))))
        ctx.barrier()
        for g in range(ctx.world):
            g0, g1 = min(g * share, rows), min((g + 1) * share, rows)
            if g1 <= g0:
                continue
            truth = np.load(os.path.join(base, f"{g}.npy"), mmap_mode="r")
            for r0 in range(g0, g1, chunk):
                r1 = min(g1, r0 + chunk)
                b, a, r = O.check_tolerance(full[r0:r1].cpu().numpy(), np.asarray(truth[r0 - g0:r1 - g0]))
                bad, max_abs, max_rel = bad + b, max(max_abs, a), max(max_rel, r)
        ctx.barrier()
        if ctx.rank == 0:
            import shutil
            shutil.rmtree(base, ignore_errors=True)
    return {"rows_checked": rows, "violations": int(ctx.max_over_ranks(float(bad))),
            "ranks_checked": int(ctx.sum_over_ranks(1.0)), "max_abs_err": ctx.max_over_ranks(max_abs),
            "max_rel_err": ctx.max_over_ranks(max_rel), "rtol": 1e-5, "atol": 1e-6}


def merge_checks(a: dict, b: dict) -> dict:
    out = dict(a)
    out["violations"] = max(a["violations"], b["violations"])
    out["max_abs_err"] = max(a["max_abs_err"], b["max_abs_err"])
    out["max_rel_err"] = max(a["max_rel_err"], b["max_rel_err"])
    out["ranks_checked"] = min(a["ranks_checked"], b["ranks_checked"])
    out["checks"] = "whole result on every rank, before the timed steps and after the last of them"
    return out


def measure(ctx: Context, args, cfg: dict, steps: int, warmup: int, min_warm_seconds: float) -> dict:
    """Everything that is reported about one configuration (see the module docstring)."""
    torch, dist, sharded = ctx.torch, ctx.dist, ctx.sharded
    rank, world, device = ctx.rank, ctx.world, ctx.device
    spmv = cfg["kind"] == "spmv"
    op = (sharded.ShardedSpMV if spmv else sharded.ShardedSpMM)(cfg, rank, world, device, gather=args.gather)
    alpha, beta = cfg["alpha"], cfg["beta"]
    out0 = torch.from_numpy(cfg["y"] if spmv else cfg["c"])
    local0 = out0[op.r0:op.r1].to(device)
    local = op.y_local if spmv else op.c_local

    def reset_output():
        if beta != 0.0:
            local.copy_(local0)  # outside the event pairs: keeps the input of every step identical

    # ---- correctness of the very data that is timed: the whole result, on every rank
    reset_output()
    full = op.step(alpha, beta)
    torch.cuda.synchronize()
    check = None if args.no_check else check_whole_result(ctx, cfg, full, alpha, beta)
    del full
    ctx.barrier()  # the next step overwrites the buffers the ranks have just read
    graphed = (not args.no_graph) and op.capture(alpha, beta)

    # ---- device-resident steps
    # nvidia-smi needs about a second to deliver its first sample: warm-up keeps the GPU under the same
    # load at least that long where a clock sample is wanted for this configuration.
    warm_until = time.perf_counter() + min_warm_seconds
    done = 0
    while done < warmup or (rank == 0 and world == 1 and time.perf_counter() < warm_until):
        reset_output()
        op.step(alpha, beta)
        done += 1
        if done % 16 == 0:
            torch.cuda.synchronize()
    ctx.barrier()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        reset_output()
        starts[i].record()
        op.step(alpha, beta)
        ends[i].record()
    ctx.barrier()
    per_step = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    ms_step = ctx.max_over_ranks(float(sum(per_step))) / steps

    # ---- the whole result once more, after the last timed (graph-replayed) step
    if check is not None:
        reset_output()
        full = op.step(alpha, beta)
        torch.cuda.synchronize()
        check = merge_checks(check, check_whole_result(ctx, cfg, full, alpha, beta))
        del full
        ctx.barrier()

    # ---- the product kernels alone, for the roofline.  At one GPU the step is exactly them; at several
    # GPUs they are replayed as a graph of their own with the reassembly (output mirrors) switched off.
    k_ms = ms_step
    if world > 1:
        k_ms = 0.0
        op.reassemble_in_kernel(False)
        if op.r1 > op.r0:
            replay = op.capture_product(alpha, beta) if not args.no_graph else None
            run = replay if replay is not None else (lambda: op.op(alpha, beta))
            for _ in range(3):
                run()
            ks = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
            ke = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
            for i in range(steps):
                reset_output()
                ks[i].record()
                run()
                ke[i].record()
            torch.cuda.synchronize()
            k_ms = float(np.mean([s.elapsed_time(e) for s, e in zip(ks, ke)]))
        k_ms = ctx.max_over_ranks(k_ms)
        op.reassemble_in_kernel(True)

    # ---- end to end from host buffers through the public API
    e2e = None
    try:
        host_in = op.pinned_input_share(cfg)
        host_out = torch.empty_like(out0[op.r0:op.r1]).pin_memory()
        e_steps = max(1, min(steps, 3 if not spmv else steps))
        # The result goes back on a copy stream of its own, so that the download of step i and the upload of
        # step i + 1 share the (full-duplex) host link; events keep the order: a download starts after its
        # product, and the next product, which overwrites y / C, starts after the download.
        main = torch.cuda.current_stream()
        copy_stream = torch.cuda.Stream(device=device)
        downloaded = None
        ctx.barrier()
        for it in range(1 + e_steps):
            if it == 1:
                main.wait_stream(copy_stream)
                ctx.barrier()
                t0 = torch.cuda.Event(enable_timing=True)
                t1 = torch.cuda.Event(enable_timing=True)
                t0.record()
            op.load_input_share(host_in)
            if downloaded is not None:
                main.wait_event(downloaded)
            reset_output()
            result = op.step(alpha, beta)
            computed = torch.cuda.Event()
            computed.record(main)
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(computed)
                host_out.copy_(result[op.r0:op.r1].view(host_out.shape), non_blocking=True)
                downloaded = torch.cuda.Event()
                downloaded.record(copy_stream)
        main.wait_stream(copy_stream)  # the last download is inside the timed region
        t1.record()
        ctx.barrier()
        e_ms = ctx.max_over_ranks(t0.elapsed_time(t1)) / e_steps
        h2d = int(ctx.sum_over_ranks(float(host_in.numel() * 4)))
        d2h = int(ctx.sum_over_ranks(float(host_out.numel() * 4)))
        e2e = {"value": workloads.flops(cfg) / (e_ms * 1e-3) / 1e9, "unit": "GFLOP/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": e_ms, "steps": e_steps,
               "what": "per rank and step: its share of x (or B) pinned host -> device, all-gather of the shares "
                       "into the replicas, the sharded product step, its own row block of y (or C) -> pinned host "
                       "on a copy stream, so that one step's download overlaps the next step's upload; every "
                       "copy of every step is inside the timed region; A resident; bytes are summed over ranks"}
        del host_in, host_out
    except (RuntimeError, ValueError, TypeError) as err:  # the same on every rank: none is left waiting
        e2e = None
        print(f"[bench] end-to-end leg of {cfg['name']} failed: {err!r}", file=sys.stderr)

    peak, peak_kind = measured_peak()
    flop = workloads.flops(cfg)
    abytes = workloads.algorithmic_bytes(cfg)
    achieved = abytes / (k_ms * 1e-3) / 1e9 if k_ms else None
    ratio = TRAFFIC_RATIO.get(cfg["name"])
    traffic = int(abytes * ratio) if ratio and args.rows is None else None
    launches = op.launches_per_step(alpha, beta)
    result = {
        "metric": metric_name(cfg), "value": flop / (ms_step * 1e-3) / 1e9, "unit": "GFLOP/s",
        "ms_per_step": ms_step, "steps": steps, "warmup": done,
        "dtype": "f32 data, f64 accumulate",
        "algorithm": op.algorithm,
        "config": {"workload": describe(cfg), "sharding": f"row blocks by nnz over {world} GPU(s), x/B replicated, "
                   f"reassembly of y/C inside the step ({op.gather_mode if world > 1 else 'none at 1 GPU'})",
                   "launch": "one CUDA graph replay per step" if graphed else "kernel by kernel",
                   "l2": ("the whole problem fits L2: no flush, reported as L2-resident" if abytes < 100e6 else
                          "inputs larger than L2 (matrix streamed from HBM every step); no flush"),
                   "per_step_ms_min_median_max": [float(np.min(per_step)), float(np.median(per_step)),
                                                  float(np.max(per_step))]},
        "gpu_launches": launches * steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak * world, "peak_per_gpu": peak, "unit": "GB/s",
                     "frac": achieved / (peak * world) if achieved else None, "traffic": traffic,
                     "peak_kind": peak_kind, "algorithmic_bytes_per_launch": abytes, "kernel_ms": k_ms,
                     "frac_of_nominal_8000": achieved / (8000.0 * world) if achieved else None,
                     "kernels": op.kernel_names,
                     "hbm_gbs_at_step_time": abytes / (ms_step * 1e-3) / 1e9},
        "check": check,
    }
    if not spmv:
        result["roofline"]["gather_bytes"] = 4 * cfg["nnz"] * cfg["n"]
    if e2e is not None:
        result["e2e"] = e2e
    op.close()
    del op, local0, out0
    gc.collect()
    torch.cuda.empty_cache()
    return result


def measure_narrow(ctx: Context, args, cfg: dict, kind: str, steps: int, warmup: int) -> dict:
    """SpMV of `cfg` with its values and x stored as fp16 or bf16 and an fp32 result, one GPU, through the C ABI:
    device-resident steps timed with CUDA events, the whole result checked against the fp64 truth of the rounded
    data.  Algorithmic bytes: 6 per non-zero instead of 8, 2 per element of x."""
    from oracle import oracle as O
    from ops_sparse_b200 import api
    torch = ctx.torch
    dev = ctx.device
    dtype = torch.float16 if kind == "fp16" else torch.bfloat16
    alpha, beta = cfg["alpha"], cfg["beta"]
    va = torch.from_numpy(cfg["values"]).to(dev).to(dtype)
    x = torch.from_numpy(cfg["x"]).to(dev).to(dtype)
    rp = torch.from_numpy(cfg["row_ptr"]).to(dev)
    ci = torch.from_numpy(cfg["col_ind"]).to(dev)
    y0 = torch.from_numpy(cfg["y"]).to(dev)
    y = y0.clone()
    handle = api.Handle()
    mat = api.CsrMatrix(cfg["rows"], cfg["cols"], rp, ci, va)
    op = api.SpMV(handle, mat, api.DnVec(x), api.DnVec(y))
    op.preprocess(alpha, beta)
    op(alpha, beta)
    torch.cuda.synchronize()
    threads = host_threads()
    truth = O.spmv_f64(cfg["row_ptr"], cfg["col_ind"], va.float().cpu().numpy(), x.float().cpu().numpy(), cfg["y"],
                       alpha, beta, threads=threads)
    bad, max_abs, max_rel = O.check_tolerance(y.cpu().numpy(), truth)
    for _ in range(warmup):
        y.copy_(y0)
        op(alpha, beta)
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    launches0 = api.kernel_launches()
    for i in range(steps):
        y.copy_(y0)
        starts[i].record()
        op(alpha, beta)
        ends[i].record()
    torch.cuda.synchronize()
    launches = api.kernel_launches() - launches0
    ms = float(np.mean([s.elapsed_time(e) for s, e in zip(starts, ends)]))
    m, nnz = cfg["rows"], cfg["nnz"]
    abytes = nnz * 6 + (m + 1) * 4 + cfg["cols"] * 2 + m * 4 * (2 if beta != 0.0 else 1)
    peak, peak_kind = measured_peak()
    achieved = abytes / (ms * 1e-3) / 1e9
    return {"metric": "spmv_gflops", "value": workloads.flops(cfg) / (ms * 1e-3) / 1e9, "unit": "GFLOP/s",
            "ms_per_step": ms, "steps": steps, "warmup": warmup, "dtype": f"{kind} data, f64 accumulate, f32 result",
            "config": {"workload": describe(cfg) + f", values and x rounded to {kind}", "launch": "kernel by kernel"},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_kind": peak_kind, "algorithmic_bytes_per_launch": abytes,
                         "kernel_ms": ms, "kernels": ["SpmvTileKernel<vector, narrow>", "SpmvCarryFixupKernel"]},
            "check": {"rows_checked": m, "violations": int(bad), "ranks_checked": 1, "max_abs_err": max_abs,
                      "max_rel_err": max_rel, "rtol": 1e-5, "atol": 1e-6}}


def measure_col_slabs(ctx: Context, args, cfg: dict, width: int, steps: int, warmup: int) -> dict:
    """The SpMM of `cfg` computed as n / width library calls, one per slab of `width` columns of B and C (dense
    descriptors over the slab with the full leading dimension, so nothing is copied), one GPU.  A is streamed once
    per slab; the point is whether a slab of B stays in L2 between the non-zeros that gather from it."""
    from ops_sparse_b200 import api
    torch = ctx.torch
    dev = ctx.device
    n, k, m = cfg["n"], cfg["cols"], cfg["rows"]
    alpha, beta = cfg["alpha"], cfg["beta"]
    rp = torch.from_numpy(cfg["row_ptr"]).to(dev)
    ci = torch.from_numpy(cfg["col_ind"]).to(dev)
    va = torch.from_numpy(cfg["values"]).to(dev)
    b = torch.from_numpy(cfg["b"]).to(dev).view(k, n)
    c0 = torch.from_numpy(cfg["c"]).to(dev).view(m, n)
    c = c0.clone()
    handle = api.Handle()
    mat = api.CsrMatrix(m, k, rp, ci, va)
    ops = []
    for j in range(0, n, width):
        w = min(width, n - j)
        ops.append(api.SpMM(handle, mat, api.DnMat(k, w, n, b[:, j:j + w]), api.DnMat(m, w, n, c[:, j:j + w])))
        ops[-1].preprocess(alpha, beta)

    def step():
        for op in ops:
            op(alpha, beta)

    step()
    torch.cuda.synchronize()
    check = None if args.no_check else check_whole_result(ctx, cfg, c, alpha, beta)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        if beta != 0.0:
            c.copy_(c0)
        starts[i].record()
        step()
        ends[i].record()
    torch.cuda.synchronize()
    ms = float(np.mean([s.elapsed_time(e) for s, e in zip(starts, ends)]))
    peak, peak_kind = measured_peak()
    abytes = workloads.algorithmic_bytes(cfg)
    return {"metric": metric_name(cfg), "value": workloads.flops(cfg) / (ms * 1e-3) / 1e9, "unit": "GFLOP/s",
            "ms_per_step": ms, "steps": steps, "warmup": warmup, "col_slab_width": width, "calls_per_step": len(ops),
            "config": {"workload": describe(cfg) + f", as {len(ops)} calls on column slabs of {width}"},
            "roofline": {"bound": "hbm", "achieved": abytes / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": abytes / (ms * 1e-3) / 1e9 / peak, "peak_kind": peak_kind,
                         "algorithmic_bytes_per_launch": abytes},
            "check": check}


def run_ours(args):
    ctx = Context(args)
    rank, world = ctx.rank, ctx.world
    sampler = ClockSampler(ctx.device.index or 0)
    if rank == 0:
        sampler.start()
    cfg = make_workload(ctx, args.workload, args.rows)
    if args.col_slabs:
        if world != 1 or cfg["kind"] != "spmm":
            raise SystemExit("--col-slabs: one GPU, an SpMM workload")
        print(json.dumps(measure_col_slabs(ctx, args, cfg, args.col_slabs, max(3, min(args.steps, 10)), 3)))
        cleanup_shared(ctx)
        return
    head = measure(ctx, args, cfg, args.steps, args.warmup, 1.5)
    clocks = sampler.stop() if rank == 0 else None
    narrow = None
    if world == 1 and cfg["kind"] == "spmv" and not args.no_narrow:
        narrow = measure_narrow(ctx, args, cfg, "fp16", args.steps, max(3, args.warmup))

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        sample = cpu_sample(cfg, args.cpu_rows)
        secs = cpu_golden_seconds(sample, 1, args.cpu_repeats)
        cpu = {"value": workloads.flops(sample) / secs / 1e9, "unit": "GFLOP/s", "cores": 1, "kind": "port",
               "sample": f"{sample['rows']} of {cfg['rows']} rows ({sample['nnz']} non-zeros) x {args.cpu_repeats} "
                         "passes, single thread, the reference's host golden restated in oracle/oracle.c",
               "host_cores_available": os.cpu_count()}
    del cfg
    gc.collect()

    names = args.configs
    if names is None:
        names = ["c1", "c3", "c4", "c5"] if world == 1 else ["c3", "c4"]
    configs = {}
    for name in names:
        if name == args.workload and args.rows is None:
            continue
        other = make_workload(ctx, name, args.rows if args.rows is not None and name != "c1" else None)
        steps = args.steps if other["kind"] == "spmv" else max(3, min(args.steps, 10))
        configs[name] = measure(ctx, args, other, steps, max(3, args.warmup), 0.25)
        del other
        gc.collect()

    if narrow is not None:
        configs[f"{args.workload}_fp16"] = narrow
    cleanup_shared(ctx)
    if world > 1:
        ctx.dist.barrier()  # last collective: every rank reaches it before any rank leaves
    if rank != 0:
        return
    line = {"metric": head["metric"], "value": head["value"], "unit": head["unit"], "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic",
            "algorithm": head["algorithm"], "config": head["config"], "clocks": clocks,
            "gpu_launches": head["gpu_launches"], "roofline": head["roofline"], "check": head["check"]}
    if "e2e" in head:
        line["e2e"] = head["e2e"]
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if configs:
        line["configs"] = configs
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--configs", default=None,
                    help="comma-separated further configurations measured in the same run and reported under "
                    "'configs' (default: c1,c3,c4,c5 at one GPU, c3,c4 at several); 'none' for none")
    ap.add_argument("--rows", type=int, default=None, help="row count override (smaller case of the same shape)")
    ap.add_argument("--cpu-rows", type=int, default=1 << 22, help="row block the CPU baseline runs on")
    ap.add_argument("--cpu-repeats", type=int, default=3)
    ap.add_argument("--gather", default="multicast", choices=["multicast", "fused", "push", "nccl"],
                    help="reassembly of y/C at N > 1: multimem.st to the NVLink multicast address inside the "
                    "product kernels (default), per-peer mirror stores inside them, a separate peer-store "
                    "kernel, or the NCCL all-gather")
    ap.add_argument("--no-graph", action="store_true", help="launch every step kernel by kernel instead of "
                    "replaying the step as one CUDA graph")
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--col-slabs", type=int, default=0, help="experiment: compute the SpMM workload as one call per "
                    "slab of this many columns of B and C, print that measurement alone")
    ap.add_argument("--no-narrow", action="store_true", help="skip the fp16-storage variant of the headline workload")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.configs is not None:
        args.configs = [] if args.configs.lower() in ("none", "") else [c.strip() for c in args.configs.split(",")]

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return  # the CPU arm runs on rank 0 only
        run_reference(args, workloads.make(args.workload, rows=args.rows))
        return
    run_ours(args)
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
