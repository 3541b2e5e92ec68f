"""The step before the hot path: reading coordinate files and putting coordinates in the order the
kernels need, with the sort and the merge of duplicates done on the GPU.

* ``parse2D(path)`` / ``parse3D_i32_f32(path, N, M, K)`` read Matrix Market ``.mtx`` and FROSTT
  ``.tns`` files and return objects with the attribute names the reference's readers expose
  (``row``, ``col``[, ``dep``], ``data``, ``N``, ``M``[, ``K``, ``nnz``]; runtime/io/parse.h:21-263,
  registered at runtime/register_runtime.cpp:20-39): coordinates zero-based and in file order,
  int32 / float32 CPU tensors, symmetric and skew-symmetric matrices expanded to their full form.
  The file is tokenised by numpy in one pass instead of a stream extraction per number.
* ``coalesce_coo(…)`` / ``coalesce_coo3(…)`` sort coordinates lexicographically and add up the values
  of repeated coordinates **on the device** (one 64-bit key sort and a segmented sum), which is what
  the reference's dataset script does on the host with pandas before its benchmarks can run
  (benchmarks/datasets/sort_frostt.py). The result feeds ``to_coo`` / ``to_coo3`` / ``to_csf3``
  without leaving the GPU.
"""
from __future__ import annotations

import numpy as np
import torch

__all__ = ["COO2D", "COO3D_parsed", "parse2D", "parse3D_i32_f32", "coalesce_coo", "coalesce_coo3"]


class COO2D:
    """What ``parse2D`` returns: ``row``, ``col``, ``data`` (CPU tensors) and the extents ``N``, ``M``."""

    __slots__ = ("row", "col", "data", "N", "M")

    def __init__(self, row, col, data, N, M):
        self.row, self.col, self.data, self.N, self.M = row, col, data, int(N), int(M)


class COO3D_parsed:
    """What ``parse3D_i32_f32`` returns: ``row``, ``col``, ``dep``, ``data``, ``N``, ``M``, ``K``, ``nnz``."""

    __slots__ = ("row", "col", "dep", "data", "N", "M", "K", "nnz")

    def __init__(self, row, col, dep, data, N, M, K):
        self.row, self.col, self.dep, self.data = row, col, dep, data
        self.N, self.M, self.K, self.nnz = int(N), int(M), int(K), int(data.numel())


def _numbers(lines, columns: int) -> np.ndarray:
    """All whitespace-separated numbers of ``lines`` as a float64 array of shape (-1, columns)."""
    flat = np.array(" ".join(lines).split(), dtype=np.float64)
    if flat.size % columns:
        raise ValueError(f"expected {columns} numbers per entry, found {flat.size} numbers in all")
    return flat.reshape(-1, columns)


def parse2D(filename: str) -> COO2D:
    """Matrix Market coordinate file -> zero-based (row, col, data) in file order. Real fields only;
    ``symmetric`` and ``skew-symmetric`` files get their mirrored entries appended (negated for
    skew), as the reference's reader does (runtime/io/parse.h:28-168)."""
    with open(filename) as f:
        header = f.readline().split()
        if len(header) < 5 or header[0] != "%%MatrixMarket":
            raise ValueError(f"{filename}: not a Matrix Market file")
        _, kind, layout, field, symmetry = (h.lower() if n else h for n, h in enumerate(header[:5]))
        if kind not in ("matrix", "tensor") or layout != "coordinate":
            raise ValueError(f"{filename}: only coordinate matrices are read (found {kind} {layout})")
        if field != "real":
            raise ValueError(f"{filename}: field '{field}' is not read (real only)")
        if symmetry not in ("general", "symmetric", "skew-symmetric"):
            raise ValueError(f"{filename}: symmetry '{symmetry}' is not read")
        line = f.readline()
        while line.startswith("%"):
            line = f.readline()
        n_rows, n_cols, nnz = (int(x) for x in line.split()[:3])
        body = _numbers(f.readlines(), 3) if nnz else np.zeros((0, 3))
    if body.shape[0] != nnz:
        raise ValueError(f"{filename}: header promises {nnz} entries, file holds {body.shape[0]}")
    row, col, val = body[:, 0].astype(np.int64) - 1, body[:, 1].astype(np.int64) - 1, body[:, 2]
    if symmetry != "general":
        off = row != col
        sign = -1.0 if symmetry == "skew-symmetric" else 1.0
        row, col, val = (np.concatenate([row, col[off]]), np.concatenate([col, row[off]]),
                         np.concatenate([val, sign * val[off]]))
    return COO2D(torch.from_numpy(row.astype(np.int32)), torch.from_numpy(col.astype(np.int32)),
                 torch.from_numpy(val.astype(np.float32)), n_rows, n_cols)


def parse3D_i32_f32(filename: str, N: int, M: int, K: int) -> COO3D_parsed:
    """FROSTT ``.tns`` file (``i j k value`` per line, one-based) -> zero-based coordinates in file
    order (runtime/io/parse.h:179-263). The extents are the caller's, as in the reference."""
    with open(filename) as f:
        body = _numbers([ln for ln in f if ln.strip() and not ln.startswith("#")], 4)
    idx = body[:, :3].astype(np.int64)
    if idx.size and (idx.min() < 1 or (idx.max(axis=0) > np.array([N, M, K])).any()):
        raise ValueError(f"{filename}: a coordinate lies outside the stated extents ({N}, {M}, {K})")
    idx -= 1
    return COO3D_parsed(*[torch.from_numpy(idx[:, q].astype(np.int32)) for q in range(3)],
                        torch.from_numpy(body[:, 3].astype(np.float32)), N, M, K)


def _coalesce(keys: torch.Tensor, values: torch.Tensor):
    """Sorted unique keys and the float32 sum of the values of each key (summed in the order the sort
    leaves them, which is stable: file order within a coordinate)."""
    order = torch.argsort(keys, stable=True)
    keys, values = keys[order], values[order].to(torch.float32)
    uniq, counts = torch.unique_consecutive(keys, return_counts=True)
    if uniq.numel() == keys.numel():
        return uniq, values
    seg = torch.repeat_interleave(torch.arange(uniq.numel(), device=keys.device), counts)
    return uniq, torch.zeros(uniq.numel(), dtype=torch.float32, device=keys.device).index_add_(0, seg, values)


def coalesce_coo(row, col, data, shape, device="cuda"):
    """(row, col, data) in any order, repeats allowed -> sorted unique (row, col) and summed values,
    as int32 / float32 tensors on ``device`` ready for ``COO_gpu``. The work happens on ``device``."""
    rows, cols = int(shape[0]), int(shape[1])
    r, c = (torch.as_tensor(x).to(device=device, dtype=torch.int64) for x in (row, col))
    keys, vals = _coalesce(r * cols + c, torch.as_tensor(data).to(device))
    return (torch.div(keys, cols, rounding_mode="floor").to(torch.int32), (keys % cols).to(torch.int32), vals,
            torch.tensor([rows, cols], dtype=torch.int32))


def coalesce_coo3(row, col, dep, data, shape, device="cuda"):
    """(i, j, k, value) in any order, repeats allowed -> an (n, 3) int32 tensor of sorted unique
    coordinates and the summed float32 values, both on ``device`` (the arguments ``to_coo3`` and
    ``to_csf3`` take). The three extents together must fit 63 bits for the packed sort key."""
    d0, d1, d2 = (int(x) for x in shape)
    if d0 * d1 * d2 >= 1 << 63:
        raise ValueError("extents too wide for one 64-bit sort key")
    i, j, k = (torch.as_tensor(x).to(device=device, dtype=torch.int64) for x in (row, col, dep))
    keys, vals = _coalesce((i * d1 + j) * d2 + k, torch.as_tensor(data).to(device))
    jk = d1 * d2
    ci = torch.div(keys, jk, rounding_mode="floor")
    rem = keys - ci * jk
    cj = torch.div(rem, d2, rounding_mode="floor")
    coords = torch.stack([ci, cj, rem - cj * d2], dim=1).to(torch.int32).contiguous()
    return coords, vals
