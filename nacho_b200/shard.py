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
* CSF3 add: the same cuts on the innermost (k) level. A cut may fall inside a fibre, so a block
  can start or end with a partial ``i`` slice / ``(i, j)`` fibre; the same node then closes one
  result block and opens the next, and the stitch counts it once.

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


def row_block_cuts_device(row_ptrs: Sequence[torch.Tensor], parts: int) -> list[int]:
    """``row_block_cuts`` for row offsets that live on a GPU: the summed offsets and the ``parts - 1``
    searches run on the device (``torch.searchsorted``); only the cut rows come back to the host."""
    work = None
    for rp in row_ptrs:
        w = rp.to(torch.int64)
        w = w - w[0]
        work = w if work is None else work + w
    rows = work.numel() - 1
    total = int(work[-1])
    targets = torch.tensor([(total * g) // parts for g in range(1, parts)], dtype=torch.int64, device=work.device)
    inner = torch.searchsorted(work, targets, right=False).cpu().tolist() if parts > 1 else []
    cuts = [0] + [int(c) for c in inner] + [rows]
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


def csf3_keys(levels, dims) -> np.ndarray:
    """int64 key ``(i * dims[1] + j) * dims[2] + k`` of every stored entry of a CSF3 tensor given
    as (i_idx, j_ptr, j_idx, k_ptr, k_idx): the order the k level is stored in."""
    i_idx, j_ptr, j_idx, k_ptr, k_idx = (_np(x).astype(np.int64) for x in levels)
    i_of_j = np.repeat(i_idx, np.diff(j_ptr))
    fibre = i_of_j * int(dims[1]) + j_idx
    return np.repeat(fibre, np.diff(k_ptr)) * int(dims[2]) + k_idx


def csf3_block(levels, val, k0: int, k1: int):
    """The sub-tensor holding the k-level positions [k0, k1) of a CSF3 tensor, as
    (i_idx, j_ptr, j_idx, k_ptr, k_idx, val) with offsets rebased to 0. The first and last
    fibre (and slice) are clipped where the range cuts through them."""
    i_idx, j_ptr, j_idx, k_ptr, k_idx = (_np(x) for x in levels)
    val = _np(val)
    if k1 <= k0:
        z = np.zeros(0, np.int32)
        return z, np.zeros(1, np.int32), z, np.zeros(1, np.int32), z, np.zeros(0, np.float32)
    kp, jp = k_ptr.astype(np.int64), j_ptr.astype(np.int64)
    j0 = int(np.searchsorted(kp, k0, side="right")) - 1          # fibre holding position k0
    j1 = int(np.searchsorted(kp, k1 - 1, side="right"))           # one past the fibre holding k1 - 1
    i0 = int(np.searchsorted(jp, j0, side="right")) - 1
    i1 = int(np.searchsorted(jp, j1 - 1, side="right"))
    new_kp = (np.clip(kp[j0:j1 + 1], k0, k1) - k0).astype(np.int32)
    new_jp = (np.clip(jp[i0:i1 + 1], j0, j1) - j0).astype(np.int32)
    return (i_idx[i0:i1].astype(np.int32), new_jp, j_idx[j0:j1].astype(np.int32), new_kp,
            k_idx[k0:k1].astype(np.int32), val[k0:k1].astype(np.float32))


def csf3_cuts(a_levels, b_levels, dims, parts: int) -> list[tuple[int, int]]:
    """Cuts (x, y) of the k levels of two CSF3 tensors into ``parts`` ranges of about equal merged
    length; a coordinate stored in both stays on one side of a cut."""
    return coo3_cuts(csf3_keys(a_levels, dims), csf3_keys(b_levels, dims), parts)


def csf3_seam(prev_block, block) -> tuple[int, int]:
    """(shared_i, shared_j): 1 where ``block`` opens with the slice / fibre that ``prev_block``
    closed with (that node is one node of the whole tensor), else 0."""
    pi, _, pj = prev_block[0], prev_block[1], prev_block[2]
    bi, _, bj = block[0], block[1], block[2]
    if len(pi) == 0 or len(bi) == 0 or int(pi[-1]) != int(bi[0]):
        return 0, 0
    return 1, int(len(pj) > 0 and len(bj) > 0 and int(pj[-1]) == int(bj[0]))


def concat_csf3_blocks(blocks):
    """Host-side reassembly of the result blocks of a CSF3 add (each a tuple
    (i_idx, j_ptr, j_idx, k_ptr, k_idx, val) over consecutive coordinate ranges) into one CSF3
    tree: offsets are rebased and a slice / fibre cut by a block boundary is stored once."""
    blocks = [tuple(_np(x) for x in b) for b in blocks if len(b[4])]
    if not blocks:
        z = np.zeros(0, np.int32)
        return z, np.zeros(1, np.int32), z, np.zeros(1, np.int32), z, np.zeros(0, np.float32)
    i_idx = np.zeros(0, np.int64)
    j_cnt = np.zeros(0, np.int64)   # fibres per stitched slice
    j_idx = np.zeros(0, np.int64)
    k_cnt = np.zeros(0, np.int64)   # entries per stitched fibre
    for n, b in enumerate(blocks):
        bi, bj = b[0].astype(np.int64), b[2].astype(np.int64)
        jc, kc = np.diff(b[1].astype(np.int64)), np.diff(b[3].astype(np.int64))
        si, sj = csf3_seam(blocks[n - 1], b) if n else (0, 0)
        if sj:   # the first fibre continues the previous block's last one
            k_cnt[-1] += kc[0]
            kc, bj = kc[1:], bj[1:]
            jc[0] -= 1
        if si:   # the first slice continues the previous block's last one
            j_cnt[-1] += jc[0]
            jc, bi = jc[1:], bi[1:]
        i_idx, j_cnt = np.concatenate([i_idx, bi]), np.concatenate([j_cnt, jc])
        j_idx, k_cnt = np.concatenate([j_idx, bj]), np.concatenate([k_cnt, kc])
    ptr = lambda counts: np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    return (i_idx.astype(np.int32), ptr(j_cnt), j_idx.astype(np.int32), ptr(k_cnt),
            np.concatenate([b[4] for b in blocks]).astype(np.int32), np.concatenate([b[5] for b in blocks]).astype(np.float32))


def stitch_csf3(block, group=None, device=None):
    """All-gathers, per result block of a CSF3 add, its node counts and its first and last
    (i, j): returns (i_base, j_base, k_base, shared_i, shared_j) for this rank -- where its nodes
    start in the stitched tree and whether its first slice / fibre is the previous block's last
    one (then that node is not counted again) -- plus the stitched totals (n_i, n_j, n_k)."""
    i_idx, _, j_idx, _, k_idx = (_np(x) for x in block[:5])
    has = len(k_idx) > 0
    mine = [len(i_idx), len(j_idx), len(k_idx),
            int(i_idx[0]) if has else -1, int(j_idx[0]) if has else -1,
            int(i_idx[-1]) if has else -1, int(j_idx[-1]) if has else -1]
    if not dist.is_available() or not dist.is_initialized():
        return (0, 0, 0, 0, 0), tuple(mine[:3])
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor(mine, dtype=torch.int64, device=device)
    gathered = torch.empty(7 * world, dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(gathered, t, group=group)
    rows = gathered.view(world, 7).cpu().tolist()
    i_base = j_base = k_base = 0
    last = None   # (i, j) that closed the latest non-empty block
    out = None
    for r, (ni, nj, nk, fi, fj, li, lj) in enumerate(rows):
        si = int(nk > 0 and last is not None and last[0] == fi)
        sj = int(si and last[1] == fj)
        if r == rank:
            out = (i_base - si, j_base - sj, k_base, si, sj)
        i_base += ni - si
        j_base += nj - sj
        k_base += nk
        if nk > 0:
            last = (li, lj)
    return out, (i_base, j_base, k_base)


def stitch_on_device(rows_local: int, nnz_local: int, group=None, device=None):
    """The same exchange as ``stitch`` without a host read-back: returns (bases, counts), two
    int64 device tensors of shape (2,) and (world, 2): this rank's (row_base, nnz_base) and every
    block's (rows, nnz). A consumer that adds the bases to the block's row offsets on the device
    never has to wait for them on the host."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else "cpu"
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    mine = torch.tensor([rows_local, nnz_local], dtype=torch.int64, device=device)
    gathered = torch.empty(2 * world, dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(gathered, mine, group=group)
    counts = gathered.view(world, 2)
    return counts[:rank].sum(dim=0), counts


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


class CsrRowBlockOp:
    """CSR add or multiply of one rank's row block, run without any wait on the host: the operator
    is queued with ``nb200_csr_{add,mul}_f32_async`` (result length and status stay in device
    words) and the stitch -- the all-gather of every block's (rows, nnz) whose exclusive prefix is
    the block's global row base and the amount to add to its row offsets -- is issued as an
    asynchronous collective that reads those device words, so that it overlaps the next step's
    kernels. Result arrays are allocated once, at the worst-case length.

        op = CsrRowBlockOp("add", a_block, b_block)      # CSR_gpu row blocks of this rank
        op.launch()                                      # queue operator + stitch; returns at once
        rows_base, nnz_base, counts = op.bases()         # device tensors ((world, 2): rows, nnz); waits on the device only
        z, nnz, status = op.result()                     # host read-back (tests, end of a job)
    """

    def __init__(self, op: str, a, b, group=None, slots: int = 4):
        import ctypes as C
        from . import _capi
        from ._capi import CsrStruct, lib
        self._C, self._capi, self._CsrStruct = C, _capi, CsrStruct
        self._entry = {"add": lib.nb200_csr_add_f32_async, "mul": lib.nb200_csr_mul_f32_async}[op]
        self.a, self.b, self.group = a, b, group
        dev = a.values.device
        na, nb = a.values.numel(), b.values.numel()
        self.capacity = na + nb if op == "add" else min(na, nb)
        self.rows = int(a.shape[0])
        self.row_ptr = torch.empty(self.rows + 1, dtype=torch.int32, device=dev)
        self.col = torch.empty(max(self.capacity, 1), dtype=torch.int32, device=dev)
        self.val = torch.empty(max(self.capacity, 1), dtype=torch.float32, device=dev)
        self.distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        # per launch: [nnz, status, rows] written by the library -- a block's whole contribution to the
        # stitch, all-gathered as it is -- and every rank's three words
        self._result = [torch.zeros(3, dtype=torch.int64, device=dev) for _ in range(slots)]
        self._gathered = [torch.zeros(3 * self.world, dtype=torch.int64, device=dev) for _ in range(slots)]
        self._pending = [None] * slots
        self._n = 0

    def launch(self):
        C = self._C
        k = self._n % len(self._result)
        if self._pending[k] is not None:  # the slot's previous collective must be done before its buffers are reused
            self._pending[k].wait()
            self._pending[k] = None
        sa, sb = self.a._struct(), self.b._struct()
        sz = self._CsrStruct(self.rows, sa.cols, 0, self.row_ptr.data_ptr(), self.col.data_ptr(), self.val.data_ptr())
        stream = torch.cuda.current_stream(self.val.device).cuda_stream
        with torch.cuda.device(self.val.device):
            status = self._entry(C.byref(sa), C.byref(sb), C.byref(sz), self.capacity, self._result[k].data_ptr(), stream)
        self._capi.check(status, "CsrRowBlockOp.launch")
        if self.distributed:
            self._pending[k] = dist.all_gather_into_tensor(self._gathered[k], self._result[k], group=self.group, async_op=True)
        self._n += 1
        return k

    def bases(self, slot: int | None = None):
        """(row_base, nnz_base, counts) of the latest launch (or of ``slot``) as device tensors;
        the current stream waits for the collective, the host does not."""
        k = (self._n - 1) % len(self._result) if slot is None else slot
        if not self.distributed:
            z = torch.zeros(1, dtype=torch.int64, device=self.val.device)
            return z, z, torch.stack([self._result[k][2], self._result[k][0]]).view(1, 2)
        if self._pending[k] is not None:
            self._pending[k].wait()
            self._pending[k] = None
        words = self._gathered[k].view(self.world, 3)
        counts = torch.stack([words[:, 2], words[:, 0]], dim=1)  # (rows, nnz) of every block
        base = counts[: self.rank].sum(dim=0)
        return base[0:1], base[1:2], counts

    def drain(self):
        for k, w in enumerate(self._pending):
            if w is not None:
                w.wait()
                self._pending[k] = None

    def result(self):
        """Host read-back of the latest launch: (CSR_gpu of this block, nnz, status)."""
        from .nacho import nacho_ext
        k = (self._n - 1) % len(self._result)
        self.drain()
        nnz, status, _ = (int(x) for x in self._result[k].cpu())
        self._capi.check(status, "CsrRowBlockOp.result")
        z = nacho_ext.CSR_gpu(self.row_ptr, self.col[:nnz], self.val[:nnz], self.a.shape.clone())
        return z, nnz, status


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
