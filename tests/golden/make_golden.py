"""Generates the golden fixtures in this folder from the reference's own CPU kernels.

Run where the reference checker library exists (``make -C oracle ref`` needs the reference
checkout): ``python tests/golden/make_golden.py``. Inputs are seeded; outputs are whatever
``<kernel>_cpu_i32_f32`` of the reference returns for them, stored bit-for-bit. The tests
compare the C oracle (CPU suite) and the CUDA path (GPU suite) against these files, so the
fixtures travel to machines that have no reference checkout.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle.cpu_oracle import COO3, CSF3, CSR, Reference  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def rand_csr(rng, rows, cols, density, lengths=None):
    if lengths is None:
        lengths = rng.binomial(cols, density, rows)
    rp = np.zeros(rows + 1, np.int32)
    rp[1:] = np.cumsum(lengths)
    col = np.concatenate([np.sort(rng.choice(cols, int(n), replace=False)) for n in lengths] + [np.zeros(0, np.int64)])
    val = rng.uniform(-1, 1, len(col)).astype(np.float32)
    return CSR(rows, cols, rp, col.astype(np.int32), val)


def csr_cases():
    rng = np.random.default_rng(20240)
    cases = {}
    # the reference's smoke-test shape (tests/smoke.py:20-31)
    cases["smoke"] = [rand_csr(rng, 200, 180, 0.05) for _ in range(3)]
    cases["tiny"] = [rand_csr(rng, 7, 5, 0.4) for _ in range(3)]
    cases["one_row"] = [rand_csr(rng, 1, 300, 0.5) for _ in range(3)]
    cases["all_empty"] = [rand_csr(rng, 64, 64, 0.0) for _ in range(3)]
    a = rand_csr(rng, 50, 40, 0.2)
    cases["one_empty"] = [a, rand_csr(rng, 50, 40, 0.0), rand_csr(rng, 50, 40, 0.1)]
    cases["identical"] = [a, a, a]
    cases["cancel"] = [a, CSR(a.rows, a.cols, a.row_ptr, a.col, -a.val), rand_csr(rng, 50, 40, 0.05)]
    lens = np.zeros(400, np.int64)
    lens[100:300] = rng.integers(0, 8, 200)
    cases["empty_ends"] = [rand_csr(rng, 400, 64, 0, lens), rand_csr(rng, 400, 64, 0, np.roll(lens, 37) * (np.arange(400) > 50)),
                           rand_csr(rng, 400, 64, 0, lens[::-1].copy())]
    giant = np.zeros(30, np.int64)
    giant[11] = 3500
    small = rng.integers(0, 3, 30)
    cases["giant_row"] = [rand_csr(rng, 30, 5000, 0, giant), rand_csr(rng, 30, 5000, 0, small + giant // 2),
                          rand_csr(rng, 30, 5000, 0, small)]
    # disjoint column sets: evens vs odds
    e = rand_csr(rng, 40, 50, 0.3)
    cases["disjoint"] = [CSR(40, 100, e.row_ptr, e.col * 2, e.val), CSR(40, 100, e.row_ptr, e.col * 2 + 1, e.val),
                         rand_csr(rng, 40, 100, 0.1)]
    # several thousand entries with wide rows: spans many tiles of the GPU kernels
    cases["medium"] = [rand_csr(rng, 300, 3000, 0.012) for _ in range(3)]
    return cases


def rand_coo3(rng, dims, n):
    c = np.unique(np.stack([rng.integers(0, e, n) for e in dims], axis=1), axis=0) if n else np.zeros((0, 3), np.int64)
    return c.astype(np.int32), rng.uniform(-1, 1, len(c)).astype(np.float32)


def csf3_levels(c):
    sys.path.insert(0, ROOT)
    n = c.shape[0]
    if n == 0:
        z = np.zeros(0, np.int32)
        return z, np.zeros(1, np.int32), z, np.zeros(1, np.int32), z
    new_ij = np.ones(n, bool)
    new_ij[1:] = (c[1:, 0] != c[:-1, 0]) | (c[1:, 1] != c[:-1, 1])
    ij = np.flatnonzero(new_ij)
    new_i = np.ones(len(ij), bool)
    new_i[1:] = c[ij[1:], 0] != c[ij[:-1], 0]
    i_st = np.flatnonzero(new_i)
    return (c[ij[i_st], 0].astype(np.int32), np.append(i_st, len(ij)).astype(np.int32), c[ij, 1].astype(np.int32),
            np.append(ij, n).astype(np.int32), c[:, 2].astype(np.int32))


def coo3_cases():
    rng = np.random.default_rng(20241)
    cases = {}
    for name, dims, n in (("smoke", (40, 30, 25), 900), ("tiny", (3, 2, 2), 10), ("line", (100, 1, 1), 60),
                          ("empty", (5, 5, 5), 0), ("medium", (64, 48, 40), 9000)):
        cases[name] = (dims, rand_coo3(rng, dims, n), rand_coo3(rng, dims, n))
    dims = (20, 20, 20)
    a = rand_coo3(rng, dims, 500)
    keep = rng.random(len(a[1])) < 0.3
    extra = rand_coo3(rng, dims, 300)
    cb = np.unique(np.concatenate([a[0][keep], extra[0]]), axis=0)
    cases["overlap"] = (dims, a, (cb.astype(np.int32), rng.uniform(-1, 1, len(cb)).astype(np.float32)))
    cases["one_empty"] = (dims, a, rand_coo3(rng, dims, 0))
    return cases


def main():
    ref = Reference()
    out = {}
    for name, (a, b, c) in csr_cases().items():
        for tag, m in (("a", a), ("b", b), ("c", c)):
            out[f"{name}.{tag}.shape"] = np.array([m.rows, m.cols], np.int32)
            out[f"{name}.{tag}.rp"], out[f"{name}.{tag}.col"], out[f"{name}.{tag}.val"] = m.row_ptr, m.col, m.val
        for op, z in (("add", ref.csr_add(a, b)), ("mul", ref.csr_mul(a, b)), ("add3", ref.csr_add_3(a, b, c))):
            out[f"{name}.{op}.rp"], out[f"{name}.{op}.col"], out[f"{name}.{op}.val"] = z.row_ptr, z.col, z.val
    np.savez_compressed(os.path.join(HERE, "csr_golden.npz"), **out)
    n_csr = len(out)

    out = {}
    for name, (dims, (ca, va), (cb, vb)) in coo3_cases().items():
        out[f"{name}.dims"] = np.array(dims, np.int32)
        out[f"{name}.a.coords"], out[f"{name}.a.val"] = ca, va
        out[f"{name}.b.coords"], out[f"{name}.b.val"] = cb, vb
        z = ref.coo3_add(COO3(dims, ca[:, 0], ca[:, 1], ca[:, 2], va), COO3(dims, cb[:, 0], cb[:, 1], cb[:, 2], vb))
        out[f"{name}.coo3.coords"] = np.stack([z.i, z.j, z.k], axis=1) if len(z.val) else np.zeros((0, 3), np.int32)
        out[f"{name}.coo3.val"] = z.val
        f = ref.csf3_add(CSF3(dims, *csf3_levels(ca), va), CSF3(dims, *csf3_levels(cb), vb))
        for fld in ("i_idx", "j_ptr", "j_idx", "k_ptr", "k_idx", "val"):
            out[f"{name}.csf3.{fld}"] = getattr(f, fld)
    np.savez_compressed(os.path.join(HERE, "tensor3_golden.npz"), **out)
    print(f"wrote csr_golden.npz ({n_csr} arrays) and tensor3_golden.npz ({len(out)} arrays), "
          f"reference threads = {ref.threads()}")


if __name__ == "__main__":
    main()
