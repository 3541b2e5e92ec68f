"""CPU suite: the multi-GPU host logic -- nnz-balanced row cuts, product-balanced cuts,
merge-path coordinate cuts and the all-gather stitch -- with gloo ranks on CPU. Each rank
computes its block with the C oracle (the CUDA operator takes that place on GPUs); the
stitched blocks must equal the unsharded result bit-for-bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import assert_same, synth_csr
from nacho_b200 import shard, synth
from oracle.cpu_oracle import COO3, CSR, Oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_device_cuts_equal_host_cuts():
    """row_block_cuts_device (torch.searchsorted on the tensors' device) returns the host version's cuts."""
    for sigma, parts in ((0, 2), (2, 3), (3, 8), (3, 1)):
        ta = synth.c3_csr(0, sigma, rows=4096, cols=1 << 16, nnz=1 << 16)
        tb = synth.c3_csr(1, sigma, rows=4096, cols=1 << 16, nnz=1 << 16)
        host = shard.row_block_cuts([ta[2].numpy(), tb[2].numpy()], parts)
        assert shard.row_block_cuts_device([ta[2], tb[2]], parts) == host
    # a view that does not start at zero (a block of a larger matrix)
    rp = torch.arange(100, 1101, 10, dtype=torch.int32)
    assert shard.row_block_cuts_device([rp, rp], 4) == shard.row_block_cuts([rp.numpy(), rp.numpy()], 4)


def test_row_block_cuts_balance_and_edges():
    a = synth_csr(synth.c3_csr(0, 3, rows=4096, cols=1 << 16, nnz=1 << 16))
    b = synth_csr(synth.c3_csr(1, 3, rows=4096, cols=1 << 16, nnz=1 << 16))
    for parts in (1, 2, 4, 8):
        cuts = shard.row_block_cuts([a.row_ptr, b.row_ptr], parts)
        assert cuts[0] == 0 and cuts[-1] == a.rows and len(cuts) == parts + 1
        assert all(x <= y for x, y in zip(cuts, cuts[1:]))
        work = (a.row_ptr.astype(np.int64) + b.row_ptr)[cuts]
        per = np.diff(work)
        biggest_row = int((np.diff(a.row_ptr) + np.diff(b.row_ptr)).max())
        assert per.max() <= work[-1] / parts + biggest_row + 1  # off by at most one row's work
    empty = np.zeros(11, np.int32)
    assert shard.row_block_cuts([empty, empty], 4) == [0, 0, 0, 0, 10]


def test_product_balanced_cuts():
    a = synth_csr(synth.rmat_csr(scale=10, seed=4010))
    b = synth_csr(synth.transpose_csr(synth.rmat_csr(scale=10, seed=4010)))
    cuts = shard.product_balanced_cuts(a.row_ptr, a.col, b.row_ptr, 4)
    per_entry = np.diff(b.row_ptr)[a.col]
    prefix = np.concatenate([[0], np.cumsum(per_entry)])[a.row_ptr]
    per = np.diff(prefix[cuts])
    row_max = np.diff(prefix).max()
    assert per.sum() == prefix[-1] and per.max() <= prefix[-1] / 4 + row_max + 1


def test_coo3_cuts_never_split_a_pair():
    rng = np.random.default_rng(1)
    a = np.unique(rng.integers(0, 5000, 3000))
    b = np.unique(np.concatenate([a[rng.random(len(a)) < 0.5], rng.integers(0, 5000, 2000)]))
    for parts in (2, 3, 8):
        cuts = shard.coo3_cuts(a, b, parts)
        assert cuts[0] == (0, 0) and cuts[-1] == (len(a), len(b))
        merged = []
        for (x0, y0), (x1, y1) in zip(cuts, cuts[1:]):
            assert x0 <= x1 and y0 <= y1
            part = np.union1d(a[x0:x1], b[y0:y1])
            if merged and len(part):
                assert merged[-1] < part[0]  # ranges are disjoint and ordered: no key on both sides
            merged.extend(part.tolist())
        assert np.array_equal(np.array(merged), np.union1d(a, b))


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        oracle = Oracle()
        ta = synth.c3_csr(0, 2, rows=2048, cols=1 << 14, nnz=1 << 15)
        tb = synth.c3_csr(1, 2, rows=2048, cols=1 << 14, nnz=1 << 15)
        cuts = shard.row_block_cuts([ta[2], tb[2]], world)
        r0, r1 = cuts[rank], cuts[rank + 1]
        blocks = []
        for t in (ta, tb):
            rp, col, val = shard.csr_row_block(t[2], t[3], t[4], r0, r1)
            blocks.append(CSR(r1 - r0, t[1], rp.numpy(), col.numpy(), val.numpy()))
        z = oracle.csr_add(blocks[0], blocks[1], 2)
        row_base, nnz_base, rows_all, nnz_all = shard.stitch(z.rows, len(z.col))
        assert row_base == r0 and sum(rows_all) == 2048
        bases, counts = shard.stitch_on_device(z.rows, len(z.col))
        assert bases.tolist() == [row_base, nnz_base] and counts[:, 0].tolist() == rows_all and counts[:, 1].tolist() == nnz_all
        np.savez(os.path.join(out_dir, f"block{rank}.npz"), rp=z.row_ptr, col=z.col, val=z.val,
                 row_base=row_base, nnz_base=nnz_base)
        # SpGEMM's replication step: rank 0 owns B, everyone ends up with it
        if rank == 0:
            rp_b, col_b, val_b, shape = shard.broadcast_csr(tb[2], tb[3], tb[4], (tb[0], tb[1]), 0)
        else:
            rp_b, col_b, val_b, shape = shard.broadcast_csr(None, None, None, None, 0)
        assert shape == (tb[0], tb[1]) and torch.equal(col_b, tb[3]) and torch.equal(val_b, tb[4])
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_add_equals_unsharded(tmp_path, oracle, world):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    blocks, bases = [], []
    for r in range(world):
        f = np.load(tmp_path / f"block{r}.npz")
        blocks.append((f["rp"], f["col"], f["val"]))
        bases.append(int(f["nnz_base"]))
    rp, col, val = shard.concat_csr_blocks(blocks)
    a = synth_csr(synth.c3_csr(0, 2, rows=2048, cols=1 << 14, nnz=1 << 15))
    b = synth_csr(synth.c3_csr(1, 2, rows=2048, cols=1 << 14, nnz=1 << 15))
    want = oracle.csr_add(a, b, 4)
    assert_same(CSR(want.rows, want.cols, rp, col, val), want, "stitched blocks")
    assert bases == [int(x) for x in np.concatenate([[0], np.cumsum([b[0][-1] for b in blocks])])[:-1]]


# ---- CSF3: cuts on the k level, blocks with clipped first / last fibres, seam-aware stitch ----

def _csf3_pair(dims, n, seed):
    from nacho_b200.nacho.convert import csf3_levels
    rng = np.random.default_rng(seed)
    draw = lambda m: np.unique(np.stack([rng.integers(0, e, m) for e in dims], axis=1), axis=0)
    ca = draw(n)
    cb = np.unique(np.concatenate([ca[rng.random(len(ca)) < 0.3], draw(n)]), axis=0)
    out = []
    for c in (ca, cb):
        levels = [np.asarray(x, np.int32) for x in csf3_levels(c)]
        out.append((levels, rng.uniform(-1, 1, len(c)).astype(np.float32)))
    return out


def _csf3_result_blocks(oracle, dims, a, b, parts):
    from oracle.cpu_oracle import CSF3
    (la, va), (lb, vb) = a, b
    cuts = shard.csf3_cuts(la, lb, dims, parts)
    blocks = []
    for (x0, y0), (x1, y1) in zip(cuts, cuts[1:]):
        z = oracle.csf3_add(CSF3(dims, *shard.csf3_block(la, va, x0, x1)), CSF3(dims, *shard.csf3_block(lb, vb, y0, y1)))
        blocks.append((z.i_idx, z.j_ptr, z.j_idx, z.k_ptr, z.k_idx, z.val))
    return blocks


@pytest.mark.parametrize("dims,n", [((6, 5, 40), 300), ((50, 40, 30), 5000), ((3, 3, 2000), 3000), ((2000, 3, 3), 4000),
                                    ((1, 1, 5000), 900)])
def test_csf3_blocks_stitch_to_the_unsharded_tree(oracle, dims, n):
    """Cuts through the middle of slices and fibres (few slices, many entries each) and cuts
    that leave blocks empty (more parts than fibres) all reassemble to the unsharded result."""
    from oracle.cpu_oracle import CSF3
    a, b = _csf3_pair(dims, n, seed=sum(dims))
    want = oracle.csf3_add(CSF3(dims, *a[0], a[1]), CSF3(dims, *b[0], b[1]))
    for parts in (1, 2, 3, 8, 64):
        got = shard.concat_csf3_blocks(_csf3_result_blocks(oracle, dims, a, b, parts))
        for g, w, name in zip(got, (want.i_idx, want.j_ptr, want.j_idx, want.k_ptr, want.k_idx, want.val),
                              ("i_idx", "j_ptr", "j_idx", "k_ptr", "k_idx", "val")):
            assert np.array_equal(g, w), f"{dims} in {parts} parts: {name} differs"


def _csf3_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dims = (5, 7, 300)   # 5 slices over 3 ranks: every boundary cuts a slice, most cut a fibre
        a, b = _csf3_pair(dims, 4000, seed=77)
        block = _csf3_result_blocks(Oracle(), dims, a, b, world)[rank]
        (i_base, j_base, k_base, si, sj), totals = shard.stitch_csf3(block)
        np.savez(os.path.join(out_dir, f"csf{rank}.npz"), bases=[i_base, j_base, k_base, si, sj], totals=totals,
                 **{f"b{n}": x for n, x in enumerate(block)})
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_csf3_stitch_bases_over_gloo(tmp_path, oracle, world):
    mp.spawn(_csf3_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    files = [np.load(tmp_path / f"csf{r}.npz") for r in range(world)]
    blocks = [tuple(f[f"b{n}"] for n in range(6)) for f in files]
    whole = shard.concat_csf3_blocks(blocks)
    for f in files:
        assert tuple(int(x) for x in f["totals"]) == (len(whole[0]), len(whole[2]), len(whole[4]))
    for r, (f, blk) in enumerate(zip(files, blocks)):
        i_base, j_base, k_base, si, sj = (int(x) for x in f["bases"])
        # the block's nodes sit at their bases in the stitched tree (a shared first node sits at the base itself)
        assert np.array_equal(whole[0][i_base:i_base + len(blk[0])], blk[0])
        assert np.array_equal(whole[2][j_base:j_base + len(blk[2])], blk[2])
        assert np.array_equal(whole[4][k_base:k_base + len(blk[4])], blk[4])
        assert (si, sj) == (shard.csf3_seam(blocks[r - 1], blk) if r else (0, 0))
