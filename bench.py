#!/usr/bin/env python
"""Benchmark of the sparse-kernel hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one pass of the operator over one batch of seeded synthetic operands. The
default workload is the largest CSR add of the benchmark configurations (2^20 x 2^20, 64 M
entries per operand, uniform rows). Rank 0 prints one JSON line:

  value      effective GB/s = algorithmic bytes (operands + result) / time, operands resident in
             HBM when the timed region starts, whole job over all ranks
  e2e        the same metric through the public operator with HOST operands: pinned host ->
             device copies of the operands and a device -> pinned host copy of the result are
             inside the timed region
  roofline   dominant kernel: algorithmic bytes per step / the time the step spends in that
             kernel (CUDA events on the launching stream), against the measured HBM copy peak
  cpu_baseline  the reference's own CPU kernels (the C oracle port where the reference has
             none, i.e. SpGEMM) timed on the host cores on a bounded sample of the workload
  ref_gpu_baseline  at N = 1: the reference's own GPU kernels (emitted by its compiler, recompiled
             unchanged for sm_100a) on the same device operands, whole driver call, default grid;
             null where that library was not built, "unavailable" where the input exceeds the
             reference's int32 product counters

CSR add / multiply run through the row-block operator of nacho_b200.shard at every N: the operator
is queued without a wait on the host (result length and status stay on the device) and, with
N > 1 (launched by torch.distributed.run), the all-gather of (rows, nnz) per block that stitches
the global row offsets is an asynchronous collective inside the timed region. With N > 1 the
default is STRONG scaling: one fixed operand pair (the N = 1 workload, same seed on every rank)
cut into N row blocks of equal stored entries by shard.row_block_cuts_device; every rank's block
result is checked, outside the timed region, against the unsharded result. `--scaling weak` gives
every rank its own operand pair of the N = 1 size instead, as do the other operators (SpGEMM's B
is replicated by a broadcast before the timed region).

Timing: W >= 3 warm-up steps, then windows of exactly K steps each (barrier + synchronize on both
sides, CUDA events on the launching stream, maximum over ranks) repeated until at least half a
second has been timed; the reported ms_per_step is the median window's. Workloads smaller than
twice the L2 are timed step by step with the L2 flushed (a 256 MiB fill) before every step.
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

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per algorithmic byte of one launch
# of a kernel, from one ncu capture of a reduced case each (profiles/*.md give the commands);
# traffic grows in proportion to the entries, so the ratio is applied to the full launch.
TRAFFIC_PER_ALGORITHMIC_BYTE = {"csr_add_fused": 0.816, "coo3_add_fused": 0.92}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


# ------------------------------------------------------------------------------ workloads ----

# name -> operator, tensor format, generator parameters
WORKLOADS = {
    "c1_csr_add": dict(op="csr_add", fmt="csr"),
    "c2_csr_mul": dict(op="csr_mul", fmt="csr"),
    "c3_csr_add_sigma0": dict(op="csr_add", fmt="csr", sigma=0),
    "c3_csr_add_sigma1": dict(op="csr_add", fmt="csr", sigma=1),
    "c3_csr_add_sigma2": dict(op="csr_add", fmt="csr", sigma=2),
    "c3_csr_add_sigma3": dict(op="csr_add", fmt="csr", sigma=3),
    "c3_csr_add_3_sigma0": dict(op="csr_add_3", fmt="csr", sigma=0),
    "c3_csr_add_3_sigma2": dict(op="csr_add_3", fmt="csr", sigma=2),
    "c4a_spgemm_rmat": dict(op="spgemm", fmt="csr"),
    "c4b_spgemm_laplacian": dict(op="spgemm", fmt="csr"),
    "c5_coo3d_add": dict(op="coo3d_add", fmt="coo3"),
    "c5_csf_add": dict(op="csf_add", fmt="csf3"),
    "n1_sssmm_rmat": dict(op="sssmm", fmt="csr"),
}
RMAT_WORKLOADS = ("c4a_spgemm_rmat", "n1_sssmm_rmat")


def make_operands(name: str, rank: int, device, scale: float = 1.0, rmat_scale: int = 16):
    """Synthetic operands (tuples from nacho_b200.synth) of workload `name` for one rank.
    `scale` shrinks rows and entries together (CPU samples, profiling captures)."""
    from nacho_b200 import synth
    shift = 7919 * rank
    spec = WORKLOADS[name]
    if name.startswith("c3_"):
        rows, nnz = max(1, int((1 << 20) * scale)), max(1, int((1 << 26) * scale))
        n_ops = 3 if spec["op"] == "csr_add_3" else 2
        return [synth.c3_csr(k, spec["sigma"], rows=rows, cols=1 << 20, nnz=nnz, seed=3000 + shift, device=device)
                for k in range(n_ops)]
    if name == "c2_csr_mul":
        return list(synth.c2_pair(rows=max(1, int((1 << 20) * scale)), seed=2000 + shift, device=device))
    if name == "c1_csr_add":
        return [synth.c1_csr(k, seed=1000 + shift, device=device) for k in range(2)]
    if name == "c4a_spgemm_rmat":
        a = synth.rmat_csr(scale=rmat_scale, seed=4000 + shift, device=device)
        return [a, synth.transpose_csr(a)]
    if name == "c4b_spgemm_laplacian":
        a = synth.laplacian_csr(max(8, int(512 * scale ** 0.5)), device=device)
        return [a, a]
    if name == "n1_sssmm_rmat":  # the product A, A masked by A, as the reference's sssmm benchmark runs square matrices
        a = synth.rmat_csr(scale=rmat_scale, seed=4000 + shift, device=device)
        return [a, a, a]
    if name in ("c5_coo3d_add", "c5_csf_add"):
        return list(synth.c5_pair(nnz=max(1000, int(100_000_000 * scale)), seed=5000 + shift, device=device))
    raise SystemExit(f"unknown workload {name}")


def csf3_arrays(t, device):
    """COO3 synth tuple -> the six CSF3 level arrays as torch tensors on `device`, built on the
    device by the package's own converter (100 M entries take seconds)."""
    from nacho_b200.nacho.convert import csf3_levels_device
    dims, i, j, k, v = t
    levels = csf3_levels_device(i.to(device), j.to(device), k.to(device))
    return dims, tuple(levels) + (v.to(device=device).contiguous(),)


def bytes_csr(rows: int, nnz: int) -> int:
    return 4 * (rows + 1) + 8 * nnz


def algorithmic_bytes(spec, operands_meta, result_meta) -> int:
    """Operand + result bytes of one step. CSR: 4-byte row offsets of every operand and of the
    result plus 8 bytes (column + value) per stored entry; COO3: 16 bytes per entry; CSF3: the
    level arrays as built."""
    if spec["fmt"] == "csr":
        return sum(bytes_csr(r, n) for r, n in operands_meta) + bytes_csr(*result_meta)
    if spec["fmt"] == "coo3":
        return 16 * (sum(operands_meta) + result_meta)
    return sum(operands_meta) + result_meta  # csf3: metas are byte counts already


# --------------------------------------------------------------------------------- clocks ----

class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi; `window` keeps the samples that
    arrived between two wall-clock instants (the timed region)."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.samples = []
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append((time.perf_counter(), parts))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        inside = [p for t, p in self.samples if t0 <= t <= t1 + 0.03]
        used = inside or [p for _, p in self.samples[-3:]]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for p in used:
            try:
                sm.append(float(p[0]))
                mx.append(float(p[1]))
            except ValueError:
                continue
            for name, flag in zip(names, p[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_in_timed_region": len(inside)}


# --------------------------------------------------------------------------- CPU baseline ----

def to_oracle(spec, t):
    """Synth tuple (torch) -> oracle-style numpy tuple of the workload's format."""
    import numpy as np
    from nacho_b200 import synth
    from oracle.cpu_oracle import COO3, CSF3, CSR
    if spec["fmt"] == "csr":
        return CSR(*synth.to_numpy(t))
    dims, i, j, k, v = synth.to_numpy(t)
    if spec["fmt"] == "coo3":
        return COO3(dims, i, j, k, v)
    from nacho_b200.nacho.convert import csf3_levels
    lv = [np.asarray(x, np.int32) for x in csf3_levels(np.stack([i, j, k], 1))]
    return CSF3(dims, *lv, v)


def cpu_baseline(name: str, operands, steps: int = 3, warmup: int = 1):
    """Times the reference's emitted CPU kernels with all host threads (kind "reference"), or
    the C oracle port where the reference has no CPU kernel (SpGEMM) or is not built here
    (kind "port"), on `operands` (oracle-style tuples). Returns the result dict and metas."""
    from oracle.cpu_oracle import Oracle, Reference, default_threads
    spec = WORKLOADS[name]
    op = spec["op"]
    cores = default_threads()
    use_ref = Reference.available() and op not in ("spgemm", "sssmm")
    if use_ref:
        impl = Reference()
        cores = impl.threads()
        run = {"csr_add": lambda: impl.csr_add(*operands), "csr_mul": lambda: impl.csr_mul(*operands),
               "csr_add_3": lambda: impl.csr_add_3(*operands), "coo3d_add": lambda: impl.coo3_add(*operands),
               "csf_add": lambda: impl.csf3_add(*operands)}[op]
    else:
        impl = Oracle()
        run = {"csr_add": lambda: impl.csr_add(*operands, cores), "csr_mul": lambda: impl.csr_mul(*operands, cores),
               "csr_add_3": lambda: impl.csr_add_3(*operands, cores), "coo3d_add": lambda: impl.coo3_add(*operands, cores),
               "csf_add": lambda: impl.csf3_add(*operands), "spgemm": lambda: impl.spgemm(*operands, cores),
               "sssmm": lambda: impl.csr_mul(impl.spgemm(operands[0], operands[1], cores), operands[2], cores)}[op]
        if op == "csf_add":
            cores = 1
    out = None
    for _ in range(warmup):
        out = run()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        out = run()
        times.append(time.perf_counter() - t0)
    if spec["fmt"] == "csr":
        metas = [(m.rows, len(m.col)) for m in operands]
        nbytes = algorithmic_bytes(spec, metas, (out.rows, len(out.col)))
        nnz_in = sum(n for _, n in metas)
    elif spec["fmt"] == "coo3":
        nbytes = algorithmic_bytes(spec, [len(m.val) for m in operands], len(out.val))
        nnz_in = sum(len(m.val) for m in operands)
    else:
        size = lambda m: sum(getattr(m, f).nbytes for f in ("i_idx", "j_ptr", "j_idx", "k_ptr", "k_idx", "val"))
        nbytes = algorithmic_bytes(spec, [size(m) for m in operands], size(out))
        nnz_in = sum(len(m.val) for m in operands)
    t = statistics.mean(times)
    rows = operands[0].rows if spec["fmt"] == "csr" else int(operands[0].dims[0])
    return {"value": nbytes / t / 1e9, "unit": "GB/s", "cores": cores, "kind": "reference" if use_ref else "port",
            "nnz_per_s": nnz_in / t, "ms": t * 1e3, "rows": rows, "nnz_in": nnz_in, "nnz_out": len(out.val), "bytes": nbytes}


def ref_gpu_baseline(spec, tensors, nbytes, products=None, runs: int = 3):
    """Times the reference's own GPU kernels (emitted by its compiler, recompiled unchanged for
    sm_100a into oracle/_ref/libnacho_ref_gpu.so) on the device operands of this run, default grid
    256 x 256, whole driver call (its allocations and its length read-back included). Returns None
    where that library was not built, and skips SpGEMM inputs whose product count would overflow
    the reference's int32 counters."""
    from oracle.gpu_reference import DEFAULT_GRID, ReferenceGpu
    if not ReferenceGpu.available():
        return None
    op = spec["op"]
    if op in ("spgemm", "sssmm") and (products is None or products >= (1 << 31) - (1 << 24)):
        return {"unavailable": f"{products} products do not fit the reference's int32 product counters"}
    ref = ReferenceGpu()
    if spec["fmt"] == "csr":
        tup = [(int(t.shape[0]), int(t.shape[1]), t.dim_j_offsets, t.dim_j_indices, t.values) for t in tensors]
    elif spec["fmt"] == "coo3":
        tup = [(tuple(int(x) for x in t.shape), t.dim_i_indices, t.dim_j_indices, t.dim_k_indices, t.values) for t in tensors]
    else:
        tup = [(tuple(int(x) for x in t.shape), t.dim_i_indices, t.dim_j_offsets, t.dim_j_indices, t.dim_k_offsets,
                t.dim_k_indices, t.values) for t in tensors]
    fn = {"csr_add": ref.csr_add, "csr_mul": ref.csr_mul, "csr_add_3": ref.csr_add_3, "spgemm": ref.spgemm,
          "coo3d_add": ref.coo3_add, "csf_add": ref.csf3_add,
          "sssmm": ref.sssmm if hasattr(ref.lib, "ref_gpu_sssmm") else None}.get(op)
    if fn is None:
        return {"unavailable": f"the reference's {op} GPU kernel is not among the ones built into oracle/_ref"}
    times = []
    for k in range(runs + 1):  # the first call is the warm-up
        fn(*tup, keep=False)
        if k:
            times.append(ref.last_ms)
    ms = statistics.mean(times)
    return {"value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms": ms, "grid": list(DEFAULT_GRID), "runs": runs,
            "kind": "reference GPU kernels as emitted by its compiler, recompiled for sm_100a; whole driver call"}


def cpu_sample_scale(name: str, requested: float | None) -> float:
    """Fraction of the workload's rows / entries the CPU legs run: the whole workload wherever a
    CPU step takes a second or two (configurations 1, 2, 3, 4b), one eighth for configuration 5
    (100 M entries per operand) unless --cpu-scale says otherwise."""
    if requested is not None:
        return requested
    return 0.125 if name.startswith("c5") else 1.0


def job_config(args, world: int, scaling: str, rows: int, nnz_in: int, nnz_out: int, nbytes: int, extra=None) -> dict:
    """The `config` object of a result line. Whole-job figures only (nothing per rank), so that the
    reference arm, which runs the same job on the host cores, prints the same object."""
    cfg = {"workload": args.workload, "rows_scale": args.rows_scale, "scaling": scaling, "rows": rows,
           "operand_nnz": nnz_in, "result_nnz": nnz_out, "algorithmic_bytes": nbytes,
           "l2_policy": ("inputs_larger_than_L2" if nbytes / max(world, 1) > 2 * 126e6
                         else "L2 flushed (256 MiB fill) before every timed step"),
           "parallelism": (f"{world} row blocks of equal stored entries, all-gather of (rows, nnz) per step" if scaling == "strong"
                           else f"one operand set per rank x{world}, all-gather of (rows, nnz) per step")}
    if args.workload in RMAT_WORKLOADS:
        cfg["rmat_scale"] = args.rmat_scale
    cfg.update(extra or {})
    return cfg


def default_scaling(args, spec) -> str:
    if args.gpus > 1 and spec["op"] in ("csr_add", "csr_mul"):
        return args.scaling or "strong"
    return "weak"


def run_reference(args):
    """`--impl reference`: the reference's CPU implementation of the path on the host cores, on
    the same workload as the other arm (the whole job: under strong scaling that is the one fixed
    operand pair whatever N is). Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    spec = WORKLOADS[args.workload]
    scale = cpu_sample_scale(args.workload, args.cpu_scale) * args.rows_scale
    cpu_rmat = min(args.rmat_scale, 14)  # the CPU port sorts every product; keep its sample bounded
    ops = make_operands(args.workload, 0, dev, scale=scale, rmat_scale=cpu_rmat)
    ops_np = [to_oracle(spec, t) for t in ops]
    del ops
    base = cpu_baseline(args.workload, ops_np, steps=args.steps, warmup=args.warmup)
    whole = scale == args.rows_scale and (args.workload not in RMAT_WORKLOADS or cpu_rmat == args.rmat_scale)
    sample = ("the whole workload" if whole else f"{args.workload} at scale {scale:g} of its rows/entries"
              + (f", R-MAT scale {cpu_rmat}" if args.workload in RMAT_WORKLOADS else ""))
    scaling = default_scaling(args, spec)
    config = job_config(args, args.gpus, scaling, base["rows"], base["nnz_in"], base["nnz_out"], base["bytes"])
    if not whole:
        config["sample"] = sample
    line = {
        "impl": "reference", "metric": f"{spec['op']} effective HBM GB/s (operand + result bytes)",
        "value": base["value"], "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": base["ms"], "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": base["value"], "unit": "GB/s", "cores": base["cores"], "kind": base["kind"],
                         "sample": sample},
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "nnz_per_s": base["nnz_per_s"],
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------- main ----

def build_device_operands(spec, ops, dev):
    """Synth tuples -> the mirror's tensor objects on `dev`, plus metas for the byte count."""
    import torch
    from nacho_b200 import nacho
    if spec["fmt"] == "csr":
        tensors = [nacho.CSR_gpu(rp.to(dev), col.to(dev), val.to(dev), torch.tensor([rows, cols], dtype=torch.int32))
                   for rows, cols, rp, col, val in ops]
        metas = [(t[0], t[3].numel()) for t in ops]
    elif spec["fmt"] == "coo3":
        tensors = [nacho.COO3_gpu(i.to(dev), j.to(dev), k.to(dev), v.to(dev), torch.tensor(list(dims), dtype=torch.int32))
                   for dims, i, j, k, v in ops]
        metas = [t[4].numel() for t in ops]
    else:
        tensors, metas = [], []
        for t in ops:
            dims, arrays = csf3_arrays(t, dev)
            tensors.append(nacho.CSF3_gpu(*arrays, torch.tensor(list(dims), dtype=torch.int32)))
            metas.append(sum(a.numel() * 4 for a in arrays))
    return tensors, metas


def buffers_of(t):
    """The device arrays of a mirror tensor, in constructor order."""
    names = {"CSR_gpu": ("dim_j_offsets", "dim_j_indices", "values"),
             "COO3_gpu": ("dim_i_indices", "dim_j_indices", "dim_k_indices", "values"),
             "CSF3_gpu": ("dim_i_indices", "dim_j_offsets", "dim_j_indices", "dim_k_offsets", "dim_k_indices", "values")}
    return [getattr(t, n) for n in names[type(t).__name__]]


def result_meta(spec, z):
    if spec["fmt"] == "csr":
        return (int(z.shape[0]), z.values.numel())
    if spec["fmt"] == "coo3":
        return z.values.numel()
    return sum(b.numel() * 4 for b in buffers_of(z))


def row_block(t, r0: int, r1: int):
    """Rows [r0, r1) of a CSR synth tuple on the device: row offsets rebased to 0 (a new array),
    columns and values as views."""
    rows, cols, rp, col, val = t
    lo, hi = int(rp[r0]), int(rp[r1])
    return r1 - r0, cols, (rp[r0:r1 + 1] - rp[r0]).contiguous(), col[lo:hi], val[lo:hi]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c3_csr_add_sigma0", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-scale", type=float, default=None,
                    help="fraction of the workload's rows/entries in the CPU legs (default: 1 = the same workload, "
                         "except configuration 5)")
    ap.add_argument("--scaling", choices=["strong", "weak"], default=None,
                    help="N > 1, CSR add / multiply: one fixed operand pair cut into N row blocks (strong, default) "
                         "or one pair of the N = 1 size per rank (weak)")
    ap.add_argument("--min-seconds", type=float, default=0.5, help="timed K-step windows are repeated until this much is timed")
    ap.add_argument("--rows-scale", type=float, default=1.0,
                    help="shrink the workload by this factor (profiling captures only; a line printed with a "
                         "factor other than 1 is not a benchmark result)")
    ap.add_argument("--rmat-scale", type=int, default=16,
                    help="log2 of the rows of the R-MAT SpGEMM operand (configuration 4a names 18)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip timing the reference's own GPU kernels beside ours")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    from nacho_b200 import _capi, nacho, shard

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    spec = WORKLOADS[args.workload]
    args.gpus = world
    scaling = default_scaling(args, spec)
    block_op = spec["op"] in ("csr_add", "csr_mul")
    op_fn = getattr(nacho, f"gpu_{spec['op']}_f32")
    full_ops = None
    cuts = None
    if scaling == "strong":
        # one fixed operand pair, the same on every rank (same seed, same device type), cut into
        # `world` row blocks of equal stored entries; each rank keeps its block resident
        full_ops = make_operands(args.workload, 0, dev, scale=args.rows_scale, rmat_scale=args.rmat_scale)
        cuts = shard.row_block_cuts_device([t[2] for t in full_ops], world)
        ops = [row_block(t, cuts[rank], cuts[rank + 1]) for t in full_ops]
    else:
        ops = make_operands(args.workload, rank, dev, scale=args.rows_scale, rmat_scale=args.rmat_scale)
    if spec["op"] == "spgemm" and world > 1:
        # B is replicated: rank 0's B goes to every rank (A stays a per-rank row block)
        rows_b, cols_b, rp_b, col_b, val_b = ops[1]
        rp_b, col_b, val_b, shape_b = shard.broadcast_csr(rp_b if rank == 0 else None, col_b if rank == 0 else None,
                                                          val_b if rank == 0 else None, (rows_b, cols_b), 0)
        ops[1] = (shape_b[0], shape_b[1], rp_b, col_b, val_b)
    tensors, metas = build_device_operands(spec, ops, dev)
    nnz_in = sum(t.values.numel() for t in tensors)
    rows_local = int(tensors[0].shape[0])
    oper = shard.CsrRowBlockOp("add" if spec["op"] == "csr_add" else "mul", tensors[0], tensors[1]) if block_op else None

    def step():
        if block_op:  # queued without a host wait; the stitch is an asynchronous collective
            oper.launch()
            return None
        z = op_fn(*tensors)
        if world > 1:  # stitch: every block's (rows, nnz) -> global row-offset bases, left on the device
            shard.stitch_on_device(rows_local, z.values.numel(), device=dev)
        return z

    def finish():
        if block_op:
            oper.drain()  # the launching stream waits for the collectives still in flight

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    z = None
    for _ in range(args.warmup):
        z = step()
    finish()
    if block_op:
        z, _, _ = oper.result()
    torch.cuda.synchronize()
    zmeta = result_meta(spec, z)
    nbytes = algorithmic_bytes(spec, metas, zmeta)
    nnz_out = z.values.numel()
    flush = nbytes < 2 * 126e6
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if flush else None

    # ---- timed windows of exactly K steps each, repeated until min-seconds are timed
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    stream = torch.cuda.current_stream()

    def window():
        """One window of K steps; returns its device time in ms (this rank)."""
        barrier()
        if flush:  # L2-resident workload: every step starts from a flushed L2, timed on its own
            total = 0.0
            for _ in range(args.steps):
                flush_buf.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                step()
                finish()
                e1.record(stream)
                e1.synchronize()
                total += e0.elapsed_time(e1)
            barrier()
            return total
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step()
        finish()
        e1.record(stream)
        barrier()
        return e0.elapsed_time(e1)

    launches0 = _capi.launch_count()
    t_wall0 = time.perf_counter()
    first = window()
    launches = _capi.launch_count() - launches0
    n_windows = max(1, min(500, int(args.min_seconds * 1e3 / max(first, 1e-3)) + 1))
    if world > 1:  # every rank runs the same number of windows
        nw = torch.tensor([n_windows], dtype=torch.int64, device=dev)
        dist.all_reduce(nw, op=dist.ReduceOp.MAX)
        n_windows = int(nw[0])
    window_ms = [first] + [window() for _ in range(n_windows - 1)]
    t_wall1 = time.perf_counter()
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    if world > 1:  # a window's time is the slowest rank's
        wm = torch.tensor(window_ms, dtype=torch.float64, device=dev)
        dist.all_reduce(wm, op=dist.ReduceOp.MAX)
        window_ms = wm.cpu().tolist()
    elapsed_ms = statistics.median(window_ms)

    # ---- strong scaling: the blocks of all ranks together must be the unsharded result
    verified = None
    if scaling == "strong":
        full_tensors, _ = build_device_operands(spec, full_ops, dev)
        whole = op_fn(*full_tensors)
        rows_base, nnz_base, counts = oper.bases()
        zb, n_blk, _ = oper.result()
        lo, r0, r1 = int(nnz_base), cuts[rank], cuts[rank + 1]
        ok = (int(rows_base) == r0 and int(counts[:, 1].sum()) == whole.values.numel()
              and torch.equal(whole.dim_j_offsets[r0:r1 + 1], zb.dim_j_offsets + lo)
              and torch.equal(whole.dim_j_indices[lo:lo + n_blk], zb.dim_j_indices)
              and torch.equal(whole.values[lo:lo + n_blk].view(torch.int32), zb.values.view(torch.int32)))
        flag = torch.tensor([1 if ok else 0], dtype=torch.int64, device=dev)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        verified = bool(int(flag[0]))
        del full_tensors, whole

    # ---- the drop-in operator (allocates its result, reads the length back) on the same operands
    dropin_ms = None
    if block_op:
        for _ in range(3):
            op_fn(*tensors)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k = max(3, min(args.steps, 20))
        e0.record(stream)
        for _ in range(k):
            op_fn(*tensors)
        e1.record(stream)
        barrier()
        dropin_ms = e0.elapsed_time(e1) / k

    # ---- masked product: the unfused route (whole product, then the intersection with the mask) beside it
    unfused_ms = None
    if spec["op"] == "sssmm":
        unfused = lambda: nacho.gpu_csr_mul_f32(nacho.gpu_spgemm_f32(tensors[0], tensors[1]), tensors[2])
        for _ in range(2):
            unfused()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(5):
            unfused()
        e1.record(stream)
        barrier()
        unfused_ms = e0.elapsed_time(e1) / 5

    # ---- per-kernel timing, same workload, events on the launching stream
    prof_steps = max(3, min(args.steps, 10))
    _capi.profile_reset()
    _capi.profile_enable(True)
    for _ in range(prof_steps):
        step()
    finish()
    torch.cuda.synchronize()
    _capi.profile_enable(False)
    kernels = {}
    for kname in _capi.profile_names():
        n, ms = _capi.profile_read(kname)
        if n:
            kernels[kname] = {"launches_per_step": n / prof_steps, "avg_ms": ms / n, "ms_per_step": ms / prof_steps}

    # ---- end to end with host operands (pinned), result back into pinned host buffers
    e2e = None
    if not args.no_e2e:
        host_in = [[b.cpu().pin_memory() for b in buffers_of(t)] for t in tensors]
        shapes = [t.shape for t in tensors]
        cls = type(tensors[0])
        host_out = [torch.empty(b.numel(), dtype=b.dtype).pin_memory() for b in buffers_of(z)]

        streamed = spec["op"] in ("csr_add", "csr_mul")
        if streamed:
            # host-buffer entry point: row blocks streamed through the GPU, copies overlap the merge
            from nacho_b200 import host as host_api
            host_fn = host_api.csr_add_host if spec["op"] == "csr_add" else host_api.csr_mul_host
            host_ops = [(int(s[0]), int(s[1]), *h) for h, s in zip(host_in, shapes)]
            cap = sum(h[1].numel() for h in host_in) if spec["op"] == "csr_add" else min(h[1].numel() for h in host_in)
            out_buf = host_api.result_buffers(rows_local, cap)

        def e2e_step():
            if streamed:
                host_fn(host_ops[0], host_ops[1], out=out_buf, device=dev)
                return
            dev_ops = [cls(*[b.to(dev, non_blocking=True) for b in h], s) for h, s in zip(host_in, shapes)]
            zz = op_fn(*dev_ops)
            for dst, src in zip(host_out, buffers_of(zz)):
                dst[: src.numel()].copy_(src, non_blocking=True)
            torch.cuda.synchronize()

        for _ in range(2):
            e2e_step()
        barrier()
        k = max(2, min(args.steps, 5))
        t0 = time.perf_counter()
        for _ in range(k):
            e2e_step()
        barrier()
        e2e = {"seconds": (time.perf_counter() - t0) / k,
               "h2d": sum(b.numel() * b.element_size() for h in host_in for b in h),
               "d2h": sum(b.numel() * b.element_size() for b in buffers_of(z))}

    # ---- reduce over ranks: max time, summed bytes
    if world > 1:
        t = torch.tensor([e2e["seconds"] if e2e else 0.0, dropin_ms or 0.0], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s, dropin_ms = float(t[0]), (float(t[1]) if dropin_ms is not None else None)
        b = torch.tensor([nbytes, nnz_in, launches, rows_local, nnz_out, e2e["h2d"] if e2e else 0, e2e["d2h"] if e2e else 0],
                         dtype=torch.int64, device=dev)
        dist.all_reduce(b, op=dist.ReduceOp.SUM)
        total_bytes, total_nnz_in, launches, total_rows, total_nnz_out, h2d, d2h = (int(x) for x in b)
    else:
        e2e_s = e2e["seconds"] if e2e else 0.0
        total_bytes, total_nnz_in, total_rows, total_nnz_out = nbytes, nnz_in, rows_local, nnz_out
        h2d, d2h = (e2e["h2d"], e2e["d2h"]) if e2e else (0, 0)

    if rank == 0:
        ms_per_step = elapsed_ms / args.steps
        peak, peak_kind = measured_peaks()
        roof, extra = None, {}
        if kernels:
            top = max(kernels, key=lambda k: kernels[k]["ms_per_step"])
            roof_bytes = nbytes
            if spec["op"] in ("spgemm", "sssmm"):
                # expand-sort-compress model: A once, 8 bytes of B per product, C once (sssmm: the mask once more)
                b_len = (ops[1][2][1:] - ops[1][2][:-1]).to(torch.int64)
                products = int(b_len[ops[0][3].to(torch.int64)].sum())
                roof_bytes = bytes_csr(*metas[0]) + 8 * products + bytes_csr(*zmeta)
                if spec["op"] == "sssmm":
                    roof_bytes += bytes_csr(*metas[2])
                extra = {"products": products, "esc_model_bytes": roof_bytes}
                if unfused_ms is not None:
                    extra["unfused_spgemm_then_csr_mul_ms"] = unfused_ms
            roof_ms, roof_kernel = kernels[top]["ms_per_step"], top
            if spec["op"] in ("spgemm", "sssmm", "csf_add", "csr_add_3"):
                # several kernels share the step's bytes (row bins; expand / merge / compress):
                # the fraction is taken over all of them, not over the longest one alone
                roof_ms = sum(k["ms_per_step"] for k in kernels.values())
                roof_kernel = f"all {len(kernels)} kernels of the step (longest: {top})"
            achieved = roof_bytes / (roof_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "kernel": roof_kernel, "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "peak_kind": f"{peak_kind} HBM copy bandwidth",
                    "traffic": (TRAFFIC_PER_ALGORITHMIC_BYTE[top] * roof_bytes / max(kernels[top]["launches_per_step"], 1)
                                if top in TRAFFIC_PER_ALGORITHMIC_BYTE else None),
                    "kernel_ms_per_step": roof_ms, "frac_of_nominal_8TBs": achieved / 8000.0,
                    "scope": "this rank's block" if world > 1 else "the whole workload"}
        base = None
        if not args.no_cpu_baseline and world == 1:
            scale = cpu_sample_scale(args.workload, args.cpu_scale) * args.rows_scale
            cpu_rmat = min(args.rmat_scale, 14)  # the CPU port sorts every product; keep its sample bounded
            same = scale == args.rows_scale and (args.workload not in RMAT_WORKLOADS or cpu_rmat == args.rmat_scale)
            cpu_ops = ops if same else make_operands(args.workload, 0, dev, scale=scale, rmat_scale=cpu_rmat)
            base = cpu_baseline(args.workload, [to_oracle(spec, t) for t in cpu_ops])
            base["sample"] = (("the whole workload" if same else f"{args.workload} at scale {scale:g} of its rows/entries")
                              + (f", R-MAT scale {cpu_rmat}" if args.workload in RMAT_WORKLOADS and not same else "")
                              + ", mean of 3 runs")
        ref_gpu = None
        if world == 1 and not args.no_ref_gpu:
            ref_gpu = ref_gpu_baseline(spec, tensors, nbytes, extra.get("products"))
        line = {
            "metric": f"{spec['op']} effective HBM GB/s (operand + result bytes)",
            "value": total_bytes / (ms_per_step * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": job_config(args, world, scaling, total_rows, total_nnz_in, total_nnz_out, total_bytes, extra),
            "nnz_per_s": total_nnz_in / (ms_per_step * 1e-3),
            "timing": {"windows": len(window_ms), "window_ms_median": elapsed_ms, "window_ms_min": min(window_ms),
                       "window_ms_max": max(window_ms), "timed_seconds": sum(window_ms) / 1e3,
                       "operator": ("shard.CsrRowBlockOp: nb200_csr_*_f32_async + asynchronous all-gather" if block_op
                                    else f"nacho.gpu_{spec['op']}_f32"),
                       "dropin_operator_ms_per_step": dropin_ms},
            "verified_against_unsharded": verified,
            "roofline": roof, "kernels": kernels, "cpu_baseline": base, "ref_gpu_baseline": ref_gpu,
            "e2e": ({"value": total_bytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                     "d2h_bytes_per_step": d2h, "ms_per_step": e2e_s * 1e3} if e2e else None),
            "gpu_launches": launches, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
