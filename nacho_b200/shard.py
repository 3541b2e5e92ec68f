"""Row-block sharding of the hot path across the GPUs of one node (one process per GPU,
``torch.distributed``; NCCL on GPUs, gloo in the CPU tests).

Every result row (CSR) and every coordinate range (COO3) depends on the matching rows / range
of the operands only, so the path shards with no data-path collective:

* CSR add / mul / add_3: contiguous row blocks cut where the summed row offsets of all
  operands cross k/G of the total, the same bisection the reference does per thread
  (src/backend/partition.cpp:628-811); each rank runs the single-GPU operator on its block.
* SpGEMM: A in row blocks of balanced product counts, B replicated with a broadcast.
* COO3 add: merge-path diagonal cuts of the flat merged coordinate sequence that never
  split an equal pair (src/backend/partition.cpp:964-983).

The one exchange is ``stitch``: an all-gather of (rows, nnz) per block, whose exclusive prefix
gives each block's global row base and the base to add to its row offsets.
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch
import torch.distributed as dist


def _np(x) -> np.ndarray:
    return x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else np.asarray(x)


def row_block_cuts(row_ptrs: Sequence, parts: int) -> list[int]:
    """Row indices c[0]=0 <= ... <= c[parts]=rows such that block g = rows [c[g], c[g+1]) holds
    about 1/parts of the stored entries of all operands together."""
    work = None
    for rp in row_ptrs:
        w = _np(rp).astype(np.int64)
        w = w - w[0]
        work = w if work is None else work + w
    rows = len(work) - 1
    total = int(work[-1])
    cuts = [0]
    for g in range(1, parts):
        target = (total * g) // parts
        # first row whose preceding work reaches the target
        cuts.append(int(np.searchsorted(work, target, side="left")))
    cuts.append(rows)
    for g in range(1, parts + 1):
        cuts[g] = min(max(cuts[g], cuts[g - 1]), rows)
    return cuts


def product_balanced_cuts(a_row_ptr, a_col, b_row_ptr, parts: int) -> list[int]:
    """Row cuts of A that balance the SpGEMM product counts sum_j nnz(B_j) over the blocks."""
    a_rp, b_rp = _np(a_row_ptr).astype(np.int64), _np(b_row_ptr).astype(np.int64)
    per_entry = np.diff(b_rp)[_np(a_col).astype(np.int64)]
    prefix = np.concatenate([[0], np.cumsum(per_entry)])
    work = prefix[a_rp - a_rp[0]]  # products in rows before i
    return row_block_cuts([work], parts)


def csr_row_block(row_ptr, col, val, r0: int, r1: int):
    """Rows [r0, r1) of a CSR matrix as (row_ptr, col, val): row_ptr is rebased to start at 0
    (a new rows+1 array), col / val are views, not copies."""
    lo, hi = int(row_ptr[r0]), int(row_ptr[r1])
    return row_ptr[r0:r1 + 1] - row_ptr[r0], col[lo:hi], val[lo:hi]


def coo3_cuts(a_keys, b_keys, parts: int) -> list[tuple[int, int]]:
    """Merge-path cuts (x, y) of two sorted unique key arrays into ``parts`` ranges of about
    equal merged length; equal keys stay on one side of a cut."""
    a, b = _np(a_keys), _np(b_keys)
    na, nb = len(a), len(b)
    total = na + nb
    cuts = [(0, 0)]
    for g in range(1, parts):
        d = (total * g) // parts
        lo, hi = max(0, d - nb), min(d, na)
        while lo < hi:  # ties take A first
            mid = (lo + hi) // 2
            if a[mid] <= b[d - 1 - mid]:
                lo = mid + 1
            else:
                hi = mid
        x, y = lo, d - lo
        if x > 0 and y < nb and a[x - 1] == b[y]:
            y += 1
        cuts.append((x, y))
    cuts.append((na, nb))
    return cuts


def stitch(rows_local: int, nnz_local: int, group=None, device=None):
    """All-gathers (rows, nnz) of every block. Returns (row_base, nnz_base, rows_all, nnz_all):
    this rank's global first row and the amount to add to its local row offsets, plus the
    per-rank lists."""
    if not dist.is_available() or not dist.is_initialized():
        return 0, 0, [rows_local], [nnz_local]
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else "cpu"
    mine = torch.tensor([rows_local, nnz_local], dtype=torch.int64, device=device)
    gathered = torch.empty(2 * world, dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(gathered, mine, group=group)
    pairs = gathered.view(world, 2).cpu()
    rows_all, nnz_all = pairs[:, 0].tolist(), pairs[:, 1].tolist()
    return sum(rows_all[:rank]), sum(nnz_all[:rank]), rows_all, nnz_all


def broadcast_csr(row_ptr, col, val, shape, src: int = 0, group=None, device=None):
    """Replicates a CSR operand from ``src`` on every rank (SpGEMM's B): the three array lengths
    go first, then the arrays, each with one broadcast."""
    rank = dist.get_rank(group)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else "cpu"
    meta = torch.zeros(4, dtype=torch.int64, device=device)
    if rank == src:
        meta = torch.tensor([row_ptr.numel(), col.numel(), int(shape[0]), int(shape[1])], dtype=torch.int64, device=device)
    dist.broadcast(meta, src, group=group)
    n_rp, n_nz, rows, cols = (int(x) for x in meta.cpu())
    if rank != src:
        row_ptr = torch.empty(n_rp, dtype=torch.int32, device=device)
        col = torch.empty(n_nz, dtype=torch.int32, device=device)
        val = torch.empty(n_nz, dtype=torch.float32, device=device)
    for t in (row_ptr, col, val):
        dist.broadcast(t, src, group=group)
    return row_ptr, col, val, (rows, cols)


def concat_csr_blocks(blocks):
    """Host-side reassembly of stitched row blocks [(row_ptr, col, val), ...] into one CSR
    triple (used by tests; the sharded result normally stays sharded)."""
    rps, cols, vals, base = [np.zeros(1, np.int64)], [], [], 0
    for rp, c, v in blocks:
        rp = _np(rp).astype(np.int64)
        rps.append(rp[1:] + base)
        base += int(rp[-1])
        cols.append(_np(c))
        vals.append(_np(v))
    return (np.concatenate(rps).astype(np.int32), np.concatenate(cols).astype(np.int32),
            np.concatenate(vals).astype(np.float32))
