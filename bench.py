#!/usr/bin/env python
"""Benchmark of the sparse-kernel hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one pass of the operator over one batch of seeded synthetic operands. The
default workload is the largest CSR add of the benchmark configurations (2^20 x 2^20, 64 M
entries per operand, uniform rows). Rank 0 prints one JSON line:

  value      effective GB/s = algorithmic bytes (operands + result) / time, operands resident in
             HBM when the timed region starts, whole job over all ranks
  e2e        the same metric through the public operator with HOST operands: pinned host ->
             device copies of the operands and a device -> host copy of the result are inside
             the timed region
  roofline   dominant kernel: algorithmic bytes per launch / its mean launch time (CUDA events
             on the launching stream), against the measured HBM copy peak
  cpu_baseline  the reference's own CPU kernels (or the C oracle port when they are not built)
             timed on the host cores on a bounded row block of the same workload

With N > 1 (launched by torch.distributed.run) every rank holds its own row block of the same
size (weak scaling); the only exchange is the all-gather of (rows, nnz) per block that stitches
the global row offsets, and it is inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


# ------------------------------------------------------------------------------ workloads ----

WORKLOADS = {
    # name: (operator, generator description)
    "c3_csr_add_sigma0": dict(op="csr_add", sigma=0),
    "c3_csr_add_sigma1": dict(op="csr_add", sigma=1),
    "c3_csr_add_sigma2": dict(op="csr_add", sigma=2),
    "c3_csr_add_sigma3": dict(op="csr_add", sigma=3),
    "c2_csr_mul": dict(op="csr_mul"),
    "c1_csr_add": dict(op="csr_add"),
}


def make_operands(name: str, rank: int, device, rows_scale: float = 1.0):
    """Synthetic operands (tuples from nacho_b200.synth) of workload `name` for one rank."""
    from nacho_b200 import synth
    seed_shift = 7919 * rank
    if name.startswith("c3_csr_add"):
        sigma = WORKLOADS[name]["sigma"]
        rows = int((1 << 20) * rows_scale)
        nnz = int((1 << 26) * rows_scale)
        return [synth.c3_csr(k, sigma, rows=rows, cols=1 << 20, nnz=nnz, seed=3000 + seed_shift, device=device)
                for k in range(2)]
    if name == "c2_csr_mul":
        return list(synth.c2_pair(rows=int((1 << 20) * rows_scale), seed=2000 + seed_shift, device=device))
    if name == "c1_csr_add":
        return [synth.c1_csr(k, seed=1000 + seed_shift, device=device) for k in range(2)]
    raise SystemExit(f"unknown workload {name}")


def algorithmic_bytes(rows: int, nnz_in: int, nnz_out: int, n_ops: int) -> int:
    """Operand + result bytes of a CSR element-wise operator: 4-byte row offsets of every
    operand and of the result, 8 bytes (column + value) per stored entry read or written."""
    return 4 * (rows + 1) * (n_ops + 1) + 8 * nnz_in + 8 * nnz_out


# --------------------------------------------------------------------------------- clocks ----

class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.samples = []
        self.proc = None
        self.gpu_index = gpu_index
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for p in self.samples:
            try:
                sm.append(float(p[0]))
                mx.append(float(p[1]))
            except ValueError:
                continue
            for name, flag in zip(names, p[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- CPU baseline ----

def cpu_baseline(name: str, operands_np, steps: int = 3, warmup: int = 1):
    """Times the reference's emitted CPU kernels (all host threads) -- or, when they are not
    built on this machine, the C oracle port -- on `operands_np` (oracle-style CSR tuples)."""
    from oracle.cpu_oracle import Oracle, Reference, default_threads
    op = WORKLOADS[name]["op"]
    if Reference.available():
        impl, kind = Reference(), "reference"
        cores = impl.threads()
        run = {"csr_add": lambda: impl.csr_add(*operands_np), "csr_mul": lambda: impl.csr_mul(*operands_np)}[op]
    else:
        impl, kind = Oracle(), "port"
        cores = default_threads()
        run = {"csr_add": lambda: impl.csr_add(*operands_np, cores), "csr_mul": lambda: impl.csr_mul(*operands_np, cores)}[op]
    out = None
    for _ in range(warmup):
        out = run()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        out = run()
        times.append(time.perf_counter() - t0)
    a = operands_np[0]
    nnz_in = sum(len(m.col) for m in operands_np)
    nbytes = algorithmic_bytes(a.rows, nnz_in, len(out.col), len(operands_np))
    t = statistics.mean(times)
    return {"value": nbytes / t / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
            "nnz_per_s": nnz_in / t, "ms": t * 1e3}, nbytes


def row_block(t, rows_keep: int):
    """First `rows_keep` rows of a synth CSR tuple, as an oracle-style numpy CSR."""
    import numpy as np
    from oracle.cpu_oracle import CSR
    rows, cols, rp, col, val = t
    rows_keep = min(rows_keep, rows)
    rp_np = rp[: rows_keep + 1].cpu().numpy()
    n = int(rp_np[-1])
    return CSR(rows_keep, cols, np.ascontiguousarray(rp_np), col[:n].cpu().numpy(), val[:n].cpu().numpy())


# ----------------------------------------------------------------------------------- main ----

def run_reference(args):
    """`--impl reference`: the reference's CPU implementation of the path on the host cores,
    each step one bounded row block of the workload. Rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    ops = make_operands(args.workload, 0, dev, rows_scale=args.cpu_rows_scale)
    ops_np = [row_block(t, ops[0][0]) for t in ops]
    base, nbytes = cpu_baseline(args.workload, ops_np, steps=args.steps, warmup=args.warmup)
    sample = f"first {ops_np[0].rows} rows of {args.workload} ({sum(len(m.col) for m in ops_np)} operand entries)"
    line = {
        "impl": "reference", "metric": f"{WORKLOADS[args.workload]['op']} effective HBM GB/s (operand + result bytes)",
        "value": base["value"], "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": base["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": args.workload, "sample": sample},
        "cpu_baseline": {"value": base["value"], "unit": "GB/s", "cores": base["cores"], "kind": base["kind"],
                         "sample": sample},
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "nnz_per_s": base["nnz_per_s"],
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c3_csr_add_sigma0", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-rows-scale", type=float, default=0.125,
                    help="fraction of the workload's rows in the CPU-baseline sample")
    ap.add_argument("--rows-scale", type=float, default=1.0,
                    help="shrink the workload's rows and entries by this factor (profiling captures only; "
                         "a line printed with a factor other than 1 is not a benchmark result)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    from nacho_b200 import _capi, nacho

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    spec = WORKLOADS[args.workload]
    op_fn = {"csr_add": nacho.gpu_csr_add_f32, "csr_mul": nacho.gpu_csr_mul_f32}[spec["op"]]
    ops = make_operands(args.workload, rank, dev, rows_scale=args.rows_scale)
    tensors = [nacho.CSR_gpu(rp, col, val, torch.tensor([rows, cols], dtype=torch.int32))
               for rows, cols, rp, col, val in ops]
    rows = ops[0][0]
    nnz_in = sum(t.values.numel() for t in tensors)
    stitch_in = torch.zeros(2, dtype=torch.int64, device=dev)
    stitch_out = torch.zeros(2 * world, dtype=torch.int64, device=dev)

    def step():
        z = op_fn(*tensors)
        if world > 1:  # stitch: every block's (rows, nnz) -> global row-offset bases
            stitch_in[0] = rows
            stitch_in[1] = z.values.numel()
            dist.all_gather_into_tensor(stitch_out, stitch_in)
        return z

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    z = None
    for _ in range(args.warmup):
        z = step()
    nnz_out = z.values.numel()
    nbytes = algorithmic_bytes(rows, nnz_in, nnz_out, len(tensors))

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    stream = torch.cuda.current_stream()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches0 = _capi.launch_count()
    start.record(stream)
    for _ in range(args.steps):
        z = step()
    stop.record(stream)
    barrier()
    launches = _capi.launch_count() - launches0
    elapsed_ms = start.elapsed_time(stop)
    clocks = sampler.stop() if rank == 0 else None

    # ---- per-kernel timing of the dominant kernel, same workload, events on the launching stream
    fill_name = spec["op"] + "_fused"
    _capi.profile_reset()
    _capi.profile_enable(True)
    for _ in range(max(3, min(args.steps, 10))):
        step()
    torch.cuda.synchronize()
    _capi.profile_enable(False)
    kernels = {}
    for kname in _capi.profile_names():
        n, ms = _capi.profile_read(kname)
        if n:
            kernels[kname] = {"launches": n, "avg_ms": ms / n}

    # ---- end to end with host operands
    e2e = None
    if not args.no_e2e:
        host = [[x.cpu().pin_memory() for x in (t.dim_j_offsets, t.dim_j_indices, t.values)] for t in tensors]
        shapes = [t.shape for t in tensors]

        def e2e_step():
            dev_ops = [nacho.CSR_gpu(*[x.to(dev, non_blocking=True) for x in h], s) for h, s in zip(host, shapes)]
            zz = op_fn(*dev_ops)
            out = [x.cpu() for x in (zz.dim_j_offsets, zz.dim_j_indices, zz.values)]
            return out

        for _ in range(2):
            e2e_step()
        barrier()
        k = max(2, min(args.steps, 5))
        t0 = time.perf_counter()
        for _ in range(k):
            e2e_step()
        barrier()
        e2e_s = (time.perf_counter() - t0) / k
        h2d = sum(x.numel() * x.element_size() for h in host for x in h)
        d2h = 4 * (rows + 1) + 8 * nnz_out
        e2e = {"seconds": e2e_s, "h2d": h2d, "d2h": d2h}

    # ---- reduce over ranks: max time, summed bytes
    if world > 1:
        t = torch.tensor([elapsed_ms, e2e["seconds"] if e2e else 0.0], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_s_max = float(t[0]), float(t[1])
        b = torch.tensor([nbytes, nnz_in, launches], dtype=torch.int64, device=dev)
        dist.all_reduce(b, op=dist.ReduceOp.SUM)
        total_bytes, total_nnz_in, launches = int(b[0]), int(b[1]), int(b[2])
    else:
        e2e_s_max = e2e["seconds"] if e2e else 0.0
        total_bytes, total_nnz_in = nbytes, nnz_in

    if rank == 0:
        ms_per_step = elapsed_ms / args.steps
        value = total_bytes / (ms_per_step * 1e-3) / 1e9
        peak, peak_kind = measured_peaks()
        roof = None
        if fill_name in kernels:
            achieved = nbytes / (kernels[fill_name]["avg_ms"] * 1e-3) / 1e9
            roof = {"bound": "hbm", "kernel": fill_name, "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "peak_kind": peak_kind, "traffic": None,
                    "avg_launch_ms": kernels[fill_name]["avg_ms"]}
        base = None
        if not args.no_cpu_baseline:
            keep = max(1, int(rows * args.cpu_rows_scale))
            ops_np = [row_block(t, keep) for t in ops]
            base, _ = cpu_baseline(args.workload, ops_np)
            base["sample"] = (f"first {keep} rows of {args.workload} "
                              f"({sum(len(m.col) for m in ops_np)} operand entries), mean of 3 runs")
        line = {
            "metric": f"{spec['op']} effective HBM GB/s (operand + result bytes)",
            "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "rows_scale": args.rows_scale, "rows_per_gpu": rows, "operand_nnz_per_gpu": nnz_in,
                       "result_nnz_per_gpu": nnz_out, "algorithmic_bytes_per_gpu": nbytes,
                       "l2_policy": "inputs_larger_than_L2" if nbytes > 2 * 126e6 else "inputs fit L2 (latency-bound case)",
                       "parallelism": f"row blocks x{world}, all-gather of (rows, nnz) per step"},
            "nnz_per_s": total_nnz_in / (ms_per_step * 1e-3),
            "roofline": roof, "kernels": kernels, "cpu_baseline": base,
            "e2e": ({"value": total_bytes / e2e_s_max / 1e9, "unit": "GB/s", "h2d_bytes_per_step": e2e["h2d"],
                     "d2h_bytes_per_step": e2e["d2h"], "ms_per_step": e2e_s_max * 1e3} if e2e else None),
            "gpu_launches": launches, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
