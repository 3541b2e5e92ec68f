"""Seeded synthetic operands with the shapes and distributions of the benchmark configurations
(they stand in for the SuiteSparse / FROSTT files the reference's benchmarks read, which need
a network to fetch). Row / slice length vectors are drawn with numpy; the bulk index and value
arrays are drawn with torch on the requested device so that the large configurations can be
generated on the GPU in seconds. A given (config, seed, device type) always yields the same
tensors.

Every generator returns plain tuples of torch tensors:
  CSR  -> (rows, cols, row_ptr int32[rows+1], col int32[nnz], val float32[nnz])
  COO3 -> (dims, i int32[nnz], j int32[nnz], k int32[nnz], val float32[nnz])
Columns are sorted and unique within a row; COO3 coordinates are lexicographically sorted
and unique.
"""
from __future__ import annotations

import numpy as np
import torch


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def _values(n: int, g: torch.Generator, device) -> torch.Tensor:
    return (torch.rand(n, generator=g, device=device, dtype=torch.float32) * 2.0 - 1.0)


def _csr_from_keys(keys: torch.Tensor, rows: int, cols: int, g, device):
    """Sorted unique int64 keys row * cols + col -> CSR tuple with fresh U(-1, 1) values."""
    r = torch.div(keys, cols, rounding_mode="floor")
    col = (keys - r * cols).to(torch.int32)
    counts = torch.bincount(r, minlength=rows)
    row_ptr = torch.zeros(rows + 1, dtype=torch.int64, device=device)
    row_ptr[1:] = torch.cumsum(counts, 0)
    return rows, cols, row_ptr.to(torch.int32), col, _values(keys.numel(), g, device)


def csr_from_lengths(lengths, cols: int, seed: int, device="cpu", exact: bool = True):
    """CSR matrix whose row i holds ``lengths[i]`` distinct uniform columns, sorted.

    Columns are drawn with replacement and deduplicated; with ``exact`` the missing entries are
    topped up until every row has its full length (sampling without replacement). Rows longer
    than a quarter of the columns are drawn as a prefix of a random permutation instead.
    """
    lengths = np.minimum(np.asarray(lengths, dtype=np.int64), cols)
    rows = len(lengths)
    g = _gen(seed, device)
    dense = np.flatnonzero(lengths > cols // 4)
    sparse_len = lengths.copy()
    sparse_len[dense] = 0
    want = torch.from_numpy(sparse_len).to(device)
    row_ids = torch.arange(rows, device=device, dtype=torch.int64)
    keys = torch.empty(0, dtype=torch.int64, device=device)
    need = want.clone()
    for _ in range(12 if exact else 1):
        n_new = int(need.sum())
        if n_new == 0:
            break
        r = torch.repeat_interleave(row_ids, need)
        c = torch.randint(0, cols, (n_new,), generator=g, device=device, dtype=torch.int64)
        keys = torch.unique(torch.cat([keys, r * cols + c]))
        have = torch.bincount(torch.div(keys, cols, rounding_mode="floor"), minlength=rows)
        need = want - have
    parts = [keys]
    for i in dense:
        perm = torch.randperm(cols, generator=g, device=device)[: int(lengths[i])].to(torch.int64)
        parts.append(int(i) * cols + perm)
    if len(parts) > 1:
        keys = torch.sort(torch.cat(parts)).values
    return _csr_from_keys(keys, rows, cols, g, device)


# ---------------------------------------------------------------------------- configs ----

def c1_csr(operand: int, rows: int = 4096, cols: int = 4096, mean: float = 40.0, seed: int = 1000,
           device="cpu"):
    """Config 1 operand: Poisson(mean) columns per row, clipped to [0, cols]."""
    rng = np.random.default_rng(seed + operand)
    lengths = np.clip(rng.poisson(mean, rows), 0, cols)
    return csr_from_lengths(lengths, cols, seed + operand, device)


def zipf_lengths(rows: int, mean: float, cap: int, seed: int):
    """Zipf(2.0) row lengths clipped to [1, cap], rescaled until the mean is within 0.5 %."""
    rng = np.random.default_rng(seed)
    z = np.clip(rng.zipf(2.0, rows), 1, cap).astype(np.float64)
    scale = mean / z.mean()
    lengths = np.clip(np.round(z * scale), 1, cap)
    for _ in range(30):
        err = lengths.mean() / mean
        if abs(err - 1.0) < 0.005:
            break
        scale /= err
        lengths = np.clip(np.round(z * scale), 1, cap)
    return lengths.astype(np.int64)


def c2_pair(rows: int = 1 << 20, cols: int = 1 << 20, mean: float = 16.0, cap: int = 10000,
            seed: int = 2000, device="cpu"):
    """Config 2 operands (A, B): A has Zipf row lengths; B keeps a random half of A's positions
    and adds as many fresh uniform positions per row."""
    cap = min(cap, cols)
    a = csr_from_lengths(zipf_lengths(rows, mean, cap, seed), cols, seed, device, exact=False)
    g = _gen(seed + 1, device)
    _, _, a_rp, a_col, _ = a
    n = a_col.numel()
    a_rows = torch.repeat_interleave(torch.arange(rows, device=device, dtype=torch.int64),
                                     (a_rp[1:] - a_rp[:-1]).to(torch.int64))
    keep = torch.rand(n, generator=g, device=device) < 0.5
    kept_keys = a_rows[keep] * cols + a_col[keep].to(torch.int64)
    kept_per_row = torch.bincount(a_rows[keep], minlength=rows)
    fresh_r = torch.repeat_interleave(torch.arange(rows, device=device, dtype=torch.int64), kept_per_row)
    fresh_c = torch.randint(0, cols, (fresh_r.numel(),), generator=g, device=device, dtype=torch.int64)
    keys = torch.unique(torch.cat([kept_keys, fresh_r * cols + fresh_c]))
    b = _csr_from_keys(keys, rows, cols, g, device)
    return a, b


def lognormal_lengths(rows: int, cols: int, nnz: int, sigma: float, seed: int):
    """Row lengths proportional to lognormal(0, sigma) weights, normalised to ``nnz`` entries
    and clipped to the number of columns (sigma = 0 gives equal rows)."""
    rng = np.random.default_rng(seed)
    w = rng.lognormal(0.0, sigma, rows) if sigma > 0 else np.ones(rows)
    return np.clip(np.round(w / w.sum() * nnz), 0, cols).astype(np.int64)


def c3_csr(operand: int, sigma: float, rows: int = 1 << 20, cols: int = 1 << 20, nnz: int = 1 << 26,
           seed: int = 3000, device="cpu"):
    """Config 3 operand: 2^20 x 2^20 with ~64 M entries and lognormal row skew. Columns are
    drawn with replacement and deduplicated (counts end slightly under budget at high skew);
    the few near-dense rows are drawn without replacement."""
    lengths = lognormal_lengths(rows, cols, nnz, sigma, seed + 10 * operand + int(sigma))
    return csr_from_lengths(lengths, cols, seed + 100 * operand + int(sigma), device, exact=False)


def rmat_csr(scale: int = 18, edge_factor: int = 16, probs=(0.57, 0.19, 0.19, 0.05), seed: int = 4000,
             device="cpu"):
    """Config 4a operand A: R-MAT pattern, deduplicated, U(-1, 1) values."""
    g = _gen(seed, device)
    n = 1 << scale
    m = edge_factor * n
    a, b, c, _ = probs
    r = torch.zeros(m, dtype=torch.int64, device=device)
    cidx = torch.zeros(m, dtype=torch.int64, device=device)
    for bit in range(scale):
        u = torch.rand(m, generator=g, device=device)
        down = u >= a + b
        right = ((u >= a) & (u < a + b)) | (u >= a + b + c)
        r |= down.to(torch.int64) << bit
        cidx |= right.to(torch.int64) << bit
    keys = torch.unique(r * n + cidx)
    return _csr_from_keys(keys, n, n, g, device)


def transpose_csr(m, device=None):
    """CSR of the transpose (values carried)."""
    rows, cols, rp, col, val = m
    device = device or col.device
    r = torch.repeat_interleave(torch.arange(rows, device=device, dtype=torch.int64),
                                (rp[1:] - rp[:-1]).to(torch.int64))
    keys = col.to(torch.int64) * rows + r
    order = torch.argsort(keys)
    keys = keys[order]
    counts = torch.bincount(torch.div(keys, rows, rounding_mode="floor"), minlength=cols)
    t_rp = torch.zeros(cols + 1, dtype=torch.int64, device=device)
    t_rp[1:] = torch.cumsum(counts, 0)
    return cols, rows, t_rp.to(torch.int32), (keys % rows).to(torch.int32), val[order].contiguous()


def laplacian_csr(grid: int = 512, device="cpu"):
    """Config 4b operand: 5-point Laplacian on a grid x grid mesh (diagonal 4, neighbours -1)."""
    n = grid * grid
    idx = torch.arange(n, device=device, dtype=torch.int64)
    x, y = idx % grid, idx // grid
    rows_l, cols_l, vals_l = [idx], [idx], [torch.full((n,), 4.0, device=device)]
    for ok, off in ((y > 0, -grid), (x > 0, -1), (x < grid - 1, 1), (y < grid - 1, grid)):
        rows_l.append(idx[ok])
        cols_l.append(idx[ok] + off)
        vals_l.append(torch.full((int(ok.sum()),), -1.0, device=device))
    r, c, v = torch.cat(rows_l), torch.cat(cols_l), torch.cat(vals_l)
    order = torch.argsort(r * n + c)
    r, c, v = r[order], c[order], v[order]
    rp = torch.zeros(n + 1, dtype=torch.int64, device=device)
    rp[1:] = torch.cumsum(torch.bincount(r, minlength=n), 0)
    return n, n, rp.to(torch.int32), c.to(torch.int32), v.to(torch.float32)


def _coo3_from_keys(keys, dims, g, device):
    jk = dims[1] * dims[2]
    i = torch.div(keys, jk, rounding_mode="floor")
    rem = keys - i * jk
    j = torch.div(rem, dims[2], rounding_mode="floor")
    k = rem - j * dims[2]
    return tuple(dims), i.to(torch.int32), j.to(torch.int32), k.to(torch.int32), _values(keys.numel(), g, device)


def c5_pair(dims=(1 << 17, 1 << 16, 1 << 12), nnz: int = 100_000_000, overlap: float = 0.3,
            seed: int = 5000, device="cpu"):
    """Config 5 operands (A, B) in COO3: mode-0 slice sizes follow a power law (rank^-1.5 over a
    random permutation of i), (j, k) uniform, sorted and deduplicated; B shares a random
    ``overlap`` fraction of A's coordinates and is topped up with fresh draws."""
    d0, d1, d2 = dims
    rng = np.random.default_rng(seed)
    w = np.arange(1, d0 + 1, dtype=np.float64) ** -1.5
    w = w[rng.permutation(d0)]
    sizes = np.minimum(np.round(w / w.sum() * nnz), d1 * d2).astype(np.int64)
    jk = d1 * d2

    def draw(slice_sizes, g):
        s = torch.from_numpy(slice_sizes).to(device)
        i = torch.repeat_interleave(torch.arange(d0, device=device, dtype=torch.int64), s)
        r = torch.randint(0, jk, (i.numel(),), generator=g, device=device, dtype=torch.int64)
        return i * jk + r

    ga, gb = _gen(seed, device), _gen(seed + 1, device)
    a_keys = torch.unique(draw(sizes, ga))
    shared = a_keys[torch.rand(a_keys.numel(), generator=gb, device=device) < overlap]
    fresh_sizes = np.round(sizes * (1.0 - overlap)).astype(np.int64)
    b_keys = torch.unique(torch.cat([shared, draw(fresh_sizes, gb)]))
    return _coo3_from_keys(a_keys, dims, ga, device), _coo3_from_keys(b_keys, dims, gb, device)


def random_csr(rows: int, cols: int, density: float, seed: int, device="cpu"):
    """Small uniform-density CSR matrix (the shape of the reference's smoke-test inputs,
    tests/smoke.py:20-31)."""
    rng = np.random.default_rng(seed)
    lengths = rng.binomial(cols, density, rows)
    return csr_from_lengths(lengths, cols, seed, device)


def to_numpy(t):
    """Tuple of torch tensors / ints -> the same with numpy arrays."""
    return tuple(x.cpu().numpy() if isinstance(x, torch.Tensor) else x for x in t)
