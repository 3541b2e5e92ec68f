"""Shared helpers of the test-suite: fixture decoding, bit-exact comparison, and moving
operands between numpy (oracle side) and the GPU tensor classes (product side)."""
from __future__ import annotations

import numpy as np

from oracle.cpu_oracle import COO3, CSF3, CSR

CSR_CASES = ["smoke", "tiny", "one_row", "all_empty", "one_empty", "identical", "cancel", "empty_ends",
             "giant_row", "disjoint", "medium"]
T3_CASES = ["smoke", "tiny", "line", "empty", "medium", "overlap", "one_empty"]


def golden_csr(g, case, tag) -> CSR:
    rows, cols = (int(x) for x in g[f"{case}.{tag}.shape"]) if f"{case}.{tag}.shape" in g else (None, None)
    if rows is None:
        rows, cols = (int(x) for x in g[f"{case}.a.shape"])
    return CSR(rows, cols, g[f"{case}.{tag}.rp"], g[f"{case}.{tag}.col"], g[f"{case}.{tag}.val"])


def golden_coo3(g, case, tag) -> COO3:
    dims = tuple(int(x) for x in g[f"{case}.dims"])
    c = g[f"{case}.{tag}.coords"].reshape(-1, 3)
    return COO3(dims, c[:, 0].copy(), c[:, 1].copy(), c[:, 2].copy(), g[f"{case}.{tag}.val"])


def golden_csf3(g, case) -> CSF3:
    dims = tuple(int(x) for x in g[f"{case}.dims"])
    return CSF3(dims, *[g[f"{case}.csf3.{f}"] for f in ("i_idx", "j_ptr", "j_idx", "k_ptr", "k_idx", "val")])


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint32) if a.dtype == np.float32 else a


def assert_same(x, y, what=""):
    """Bit-exact equality of two oracle-style tuples (index arrays and float32 values)."""
    assert type(x).__name__ == type(y).__name__, what
    for f in x._fields:
        a, b = getattr(x, f), getattr(y, f)
        if isinstance(a, np.ndarray) or isinstance(b, np.ndarray):
            a, b = np.asarray(a), np.asarray(b)
            assert a.shape == b.shape, f"{what}: field {f} has shape {a.shape} vs {b.shape}"
            if a.dtype == np.float32 or b.dtype == np.float32:
                assert a.dtype == b.dtype == np.float32, f"{what}: field {f} dtype"
            same = np.array_equal(bits(a), bits(b))
            if not same:
                bad = np.flatnonzero(bits(a) != bits(b))
                raise AssertionError(f"{what}: field {f} differs at {len(bad)} places, first {bad[:5]}: "
                                     f"{a[bad[:5]]} vs {b[bad[:5]]}")
        else:
            assert tuple(np.atleast_1d(a)) == tuple(np.atleast_1d(b)), f"{what}: field {f}"


def csf3_levels(coords):
    from nacho_b200.nacho.convert import csf3_levels as lv
    return tuple(np.asarray(x, dtype=np.int32) for x in lv(coords))


# ---- product side (imports torch / the CUDA library lazily) ----

def csr_to_gpu(m: CSR, device="cuda"):
    import torch
    from nacho_b200 import nacho
    return nacho.CSR_gpu(torch.from_numpy(np.ascontiguousarray(m.row_ptr, np.int32)).to(device),
                         torch.from_numpy(np.ascontiguousarray(m.col, np.int32)).to(device),
                         torch.from_numpy(np.ascontiguousarray(m.val, np.float32)).to(device),
                         torch.tensor([m.rows, m.cols], dtype=torch.int32))


def csr_from_gpu(z) -> CSR:
    import torch
    torch.cuda.synchronize()
    return CSR(int(z.shape[0]), int(z.shape[1]), z.dim_j_offsets.cpu().numpy(), z.dim_j_indices.cpu().numpy(),
               z.values.cpu().numpy())


def synth_csr(t) -> CSR:
    """Tuple from nacho_b200.synth -> oracle CSR with numpy arrays."""
    from nacho_b200 import synth
    return CSR(*synth.to_numpy(t))


def synth_to_gpu(t, device="cuda"):
    import torch
    from nacho_b200 import nacho
    rows, cols, rp, col, val = t
    return nacho.CSR_gpu(rp.to(device), col.to(device), val.to(device), torch.tensor([rows, cols], dtype=torch.int32))
