#!/usr/bin/env python
"""Benchmark of the CSR SpMV / SpMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl ours|reference]

One "step" is one product over one batch of synthetic input: y = alpha*A*x + beta*y (or the SpMM
equivalent) with A resident on the device(s).  The default workload is c2, the 27-point stencil on a
160^3 grid (4 096 000 rows, 109 215 352 non-zeros), the configuration the headline metric is quoted
on; c1/c3/c4/c5 select the other configurations of ops_sparse_b200/workloads.py.

At N GPUs (launched by torchrun, one rank per GPU) the same matrix is row-block sharded by nnz, x / B
is replicated and every step ends with the all-gather that reassembles y / C on every rank, so total
work is fixed ("strong" scaling).  Timing: W warm-up steps, then K steps between barriers and device
synchronisations, each step bracketed by CUDA events on the launching stream; the reported time is
the maximum over ranks.  The matrix alone (0.9 - 5.7 GB) is far larger than the 126 MB L2, so every
step streams it from HBM again.

Rank 0 prints one JSON line.  Keys beyond the usual ones:
  roofline      SpMV/SpMM kernels of one product: algorithmic bytes (the CSR arrays, x or B, y or C,
                each once) / event-timed duration, against the measured HBM copy bandwidth
  e2e           the same product driven from HOST vectors through the C API: pinned x (or B) is copied
                to the device, the product runs, y (or C) is copied back, all inside the timed region
  cpu_baseline  the test oracle's restatement of the reference's host golden, timed on one host core
                (the way the reference's tests time it) on the same inputs
  --impl reference times that CPU golden with all host threads instead of the GPU path.
"""
from __future__ import annotations

import argparse
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


def run_reference(args, cfg):
    """The reference's CPU golden path on the host cores (all threads), same workload and metric."""
    # Every core this process may run on: torchrun exports OMP_NUM_THREADS=1, which must not shrink the baseline.
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
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


def describe(cfg: dict) -> str:
    text = {
        "c1": "c1: CSR SpMV fp32 16384^2, Poisson(16) rows clamped to [1,64], alpha=1 beta=0",
        "c2": "c2: CSR SpMV fp32, 27-point stencil on a 160^3 grid, alpha=1 beta=0",
        "c3": "c3: CSR SpMV fp32 power-law 4194304^2, Zipf(2.0) rows mean 32 cap 200000, alpha=1.5 beta=0.5",
        "c4": "c4: CSR SpMM fp32 1048576^2 Poisson(16) rows, B 1048576x128 row-major, alpha=1 beta=0",
        "c5": "c5: CSR SpMM fp32 power-law 8388608^2, Zipf(2.1) rows mean 20 cap 500000, B 8388608x64",
    }[cfg["name"]]
    return f"{text} ({cfg['rows']} rows, {cfg['nnz']} nnz)"


def run_ours(args, cfg):
    import torch
    import torch.distributed as dist

    from ops_sparse_b200 import _lib as L
    from ops_sparse_b200 import sharded

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU implementation")
    L.lib()  # fails loudly when libops_sparse.so is missing
    rank, world, device = sharded.init_process_group_from_env()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node N")
    spmv = cfg["kind"] == "spmv"
    op = (sharded.ShardedSpMV if spmv else sharded.ShardedSpMM)(cfg, rank, world, device, gather=args.gather)
    alpha, beta = cfg["alpha"], cfg["beta"]
    out0 = torch.from_numpy(cfg["y"] if spmv else cfg["c"])
    local0 = out0[op.r0:op.r1].to(device)
    local = op.y_local if spmv else op.c_local

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- correctness of the very data that is timed: one step against the oracle (rank 0's rows)
    full = op.step(alpha, beta)
    torch.cuda.synchronize()
    check = None
    if rank == 0 and not args.no_check:
        from oracle import oracle as O
        rows = min(cfg["rows"], args.check_rows)
        if spmv:
            sub = cpu_sample(cfg, rows)
            truth = O.spmv_f64(sub["row_ptr"], sub["col_ind"], sub["values"], cfg["x"], sub["y"], alpha, beta,
                               threads=O.max_threads())
            bad, max_abs, max_rel = O.check_tolerance(full[:rows].cpu().numpy(), truth)
        else:
            n = cfg["n"]
            truth = O.spmm_f64(cfg["row_ptr"], cfg["col_ind"], cfg["values"], cfg["b"], n, cfg["c"], n, n,
                               cfg["cols"], alpha, beta, row_begin=0, row_end=rows, threads=O.max_threads())
            bad, max_abs, max_rel = O.check_tolerance(full[:rows].cpu().numpy(), truth)
        check = {"rows_checked": rows, "violations": bad, "max_abs_err": max_abs, "max_rel_err": max_rel,
                 "rtol": 1e-5, "atol": 1e-6}
    del full
    barrier()  # the next step overwrites the buffers rank 0 has just read
    graphed = (not args.no_graph) and op.capture(alpha, beta)

    # ---- device-resident steps
    # nvidia-smi needs about a second to deliver its first sample, far longer than a few steps take:
    # sampling starts here, warm-up keeps the GPU under the same load until samples arrive, and
    # the sampler runs on through the timed steps and the kernel-only and host-buffer loops.
    sampler = ClockSampler(device.index or 0)
    if rank == 0:
        sampler.start()
    warm_until = time.perf_counter() + 1.5
    done = 0
    while done < args.warmup or (rank == 0 and world == 1 and time.perf_counter() < warm_until):
        if beta != 0.0:
            local.copy_(local0)
        op.step(alpha, beta)
        done += 1
        if done % 16 == 0:
            torch.cuda.synchronize()
    barrier()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    for i in range(args.steps):
        if beta != 0.0:
            local.copy_(local0)  # outside the event pair: keeps the input of every step identical
        starts[i].record()
        op.step(alpha, beta)
        ends[i].record()
    barrier()
    per_step = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    ms_total = max_over_ranks(float(sum(per_step)))
    ms_step = ms_total / args.steps

    # ---- the product kernels alone (no reassembly: mirrors of the output cleared), for the roofline
    k_ms = None
    op.reassemble_in_kernel(False)
    if hasattr(op, "op") and op.r1 > op.r0:
        ks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        ke = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        for i in range(args.steps):
            if beta != 0.0:
                local.copy_(local0)
            ks[i].record()
            op.op(alpha, beta)
            ke[i].record()
        torch.cuda.synchronize()
        k_ms = float(np.mean([s.elapsed_time(e) for s, e in zip(ks, ke)]))
    k_ms = max_over_ranks(k_ms if k_ms is not None else 0.0)
    op.reassemble_in_kernel(True)

    # ---- end to end from host buffers through the public API
    # Every rank copies x (or B) from pinned host memory, takes part in the step and copies the whole
    # reassembled y (or C) back; at one GPU the step is the plain aclsparseSpMV / SpMM call.
    e2e = None
    try:
        inp = torch.from_numpy(cfg["x"] if spmv else cfg["b"]).pin_memory()
        host_out = torch.empty_like(out0).pin_memory()
        dev_in = op.x if spmv else op.b
        e_steps = max(1, min(args.steps, 5 if not spmv else args.steps))
        barrier()
        for it in range(1 + e_steps):
            if it == 1:
                barrier()
                t0 = torch.cuda.Event(enable_timing=True)
                t1 = torch.cuda.Event(enable_timing=True)
                t0.record()
            dev_in.copy_(inp, non_blocking=True)
            if beta != 0.0:
                local.copy_(local0)
            result = op.step(alpha, beta)
            host_out.copy_(result.view(host_out.shape), non_blocking=True)
        t1.record()
        barrier()
        e_ms = max_over_ranks(t0.elapsed_time(t1)) / e_steps
        e2e = {"value": workloads.flops(cfg) / (e_ms * 1e-3) / 1e9, "unit": "GFLOP/s",
               "h2d_bytes_per_step": int(inp.numel() * 4) * world, "d2h_bytes_per_step": int(host_out.numel() * 4) * world,
               "ms_per_step": e_ms, "steps": e_steps,
               "what": "per rank: pinned host x (or B) -> device, the sharded product step, whole y (or C) -> pinned host; "
                       "A resident; bytes are summed over ranks"}
    except (RuntimeError, ValueError, TypeError) as err:  # the same on every rank: none is left waiting
        e2e = None
        print(f"[bench] end-to-end leg failed: {err!r}", file=sys.stderr)

    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        dist.barrier()  # last collective: every rank reaches it before any rank leaves
    if rank != 0:
        return
    peak, peak_kind = measured_peak()
    flop = workloads.flops(cfg)
    abytes = workloads.algorithmic_bytes(cfg)
    achieved = abytes / (k_ms * 1e-3) / 1e9 if k_ms else None
    # DRAM read + write bytes per launch, from the ncu captures of the 1 M-row cases of the same kernel
    # (stencil: 225.04 MB for 223.71 MB algorithmic; power-law: 273.9 MB for 272.2 MB), scaled by the algorithmic
    # bytes: SpMV traffic is proportional to them.  The SpMM traffic depends on the ratio of B to L2 and no
    # small capture scales to the full sizes, so it stays null.
    ratio = {"c2": 225.04 / 223.71, "c3": 273.9 / 272.24}.get(cfg["name"])
    traffic = int(abytes * ratio) if ratio and args.rows is None and world == 1 else None
    line = {
        "metric": metric_name(cfg), "value": flop / (ms_step * 1e-3) / 1e9, "unit": "GFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32 data, f64 accumulate" if spmv else "f32",
        "data": "synthetic",
        "config": {"workload": describe(cfg), "sharding": f"row blocks by nnz over {world} GPU(s), x/B replicated, "
                   f"reassembly of y/C inside the step ({op.gather_mode if world > 1 else 'none at 1 GPU'})",
                   "launch": "one CUDA graph replay per step" if graphed else "kernel by kernel", "l2": "inputs larger than L2 (matrix streamed from HBM every "
                   "step); no flush", "per_step_ms_min_median_max": [float(np.min(per_step)),
                                                                     float(np.median(per_step)),
                                                                     float(np.max(per_step))]},
        "clocks": clocks,
        # tile kernel + carry fix-up kernel (+ the push kernel at N > 1) per timed step and rank
        "gpu_launches": (3 if world > 1 and op.gather_mode == "push" else 2) * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak * world, "peak_per_gpu": peak, "unit": "GB/s",
                     "frac": achieved / (peak * world) if achieved else None, "traffic": traffic, "peak_kind": peak_kind,
                     "algorithmic_bytes_per_launch": abytes, "kernel_ms": k_ms,
                     "frac_of_nominal_8000": achieved / (8000.0 * world) if achieved else None,
                     "kernels": "SpmvTileKernel + SpmvCarryFixupKernel" if spmv else
                                "SpmmTileKernel + SpmmCarryFixupKernel",
                     "hbm_gbs_at_step_time": abytes / (ms_step * 1e-3) / 1e9},
        "check": check,
    }
    if e2e is not None:
        line["e2e"] = e2e
    if world == 1 and not args.no_cpu:
        sample = cpu_sample(cfg, args.cpu_rows)
        secs = cpu_golden_seconds(sample, 1, args.cpu_repeats)
        line["cpu_baseline"] = {
            "value": workloads.flops(sample) / secs / 1e9, "unit": "GFLOP/s", "cores": 1, "kind": "port",
            "sample": f"{sample['rows']} of {cfg['rows']} rows ({sample['nnz']} non-zeros) x {args.cpu_repeats} "
                      "passes, single thread, the reference's host golden restated in oracle/oracle.c",
            "host_cores_available": os.cpu_count()}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--rows", type=int, default=None, help="row count override (smaller case of the same shape)")
    ap.add_argument("--check-rows", type=int, default=1 << 20, help="rows compared with the oracle before timing")
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
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference" and int(os.environ.get("RANK", "0")) != 0:
        return  # the CPU arm runs on rank 0 only
    cfg = workloads.make(args.workload, rows=args.rows)
    if args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_ours(args, cfg)
    if args.impl == "ours":
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
