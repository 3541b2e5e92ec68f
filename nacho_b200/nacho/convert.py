"""torch tensors -> nacho tensor classes: same names, arguments and buffer order as the
reference's converters (python/nacho/convert.py:23-118). Only CUDA targets exist here; asking
for ``device="cpu"`` raises, because this package has no CPU kernels.
"""
from __future__ import annotations

import numpy as np
import torch

from . import nacho_ext as _ext

__all__ = ["to_csr", "to_dcsr", "to_coo", "to_coo3", "to_csf3"]


def _gpu_only(device) -> torch.device:
    dev = torch.device(device)
    if dev.type != "cuda":
        raise ValueError("nacho_b200 provides the GPU tensor classes only (device must be CUDA)")
    return dev


def _shape(*sizes) -> torch.Tensor:
    return torch.tensor(list(sizes), dtype=torch.int32)


def to_csr(csr, device="cuda"):
    """torch CSR -> CSR_gpu (python/nacho/convert.py:23-31)."""
    dev = _gpu_only(device)
    return _ext.CSR_gpu(
        csr.crow_indices().to(dtype=torch.int32, device=dev),
        csr.col_indices().to(dtype=torch.int32, device=dev),
        csr.values().to(dtype=torch.float32, device=dev),
        _shape(csr.shape[0], csr.shape[1]),
    )


def to_dcsr(csr, device="cuda"):
    """torch CSR -> DCSR_gpu: empty rows are dropped and the surviving row numbers stored
    (python/nacho/convert.py:34-56). The row selection runs on the tensor's own device."""
    dev = _gpu_only(device)
    indptr = csr.crow_indices().to(dtype=torch.int64)
    per_row = indptr[1:] - indptr[:-1]
    present = torch.nonzero(per_row > 0).squeeze(-1)
    offsets = torch.zeros(present.numel() + 1, dtype=torch.int64, device=indptr.device)
    offsets[1:] = torch.cumsum(per_row[present], 0)
    return _ext.DCSR_gpu(
        present.to(dtype=torch.int32, device=dev),
        offsets.to(dtype=torch.int32, device=dev),
        csr.col_indices().to(dtype=torch.int32, device=dev),
        csr.values().to(dtype=torch.float32, device=dev),
        _shape(csr.shape[0], csr.shape[1]),
    )


def to_coo(coo, device="cuda"):
    """torch COO -> COO_gpu; coalesced first so that the coordinates are sorted and unique
    (python/nacho/convert.py:58-67)."""
    dev = _gpu_only(device)
    coo = coo.coalesce()
    indices = coo.indices()
    return _ext.COO_gpu(
        indices[0].to(dtype=torch.int32, device=dev).contiguous(),
        indices[1].to(dtype=torch.int32, device=dev).contiguous(),
        coo.values().to(dtype=torch.float32, device=dev),
        _shape(coo.shape[0], coo.shape[1]),
    )


def _tensor(array, dtype, dev):
    if isinstance(array, torch.Tensor):
        return array.to(dtype=dtype, device=dev).contiguous()
    return torch.from_numpy(np.ascontiguousarray(array)).to(dtype=dtype, device=dev)


def to_coo3(coordinates, values, shape, device="cuda"):
    """Sorted, deduplicated (i, j, k) rows -> COO3_gpu (python/nacho/convert.py:70-87)."""
    dev = _gpu_only(device)
    return _ext.COO3_gpu(
        _tensor(coordinates[:, 0], torch.int32, dev),
        _tensor(coordinates[:, 1], torch.int32, dev),
        _tensor(coordinates[:, 2], torch.int32, dev),
        _tensor(values, torch.float32, dev),
        torch.tensor(list(shape), dtype=torch.int32),
    )


def csf3_levels(coordinates):
    """Level arrays of the CSF3 tree over sorted unique (i, j, k) rows: (i_idx, j_ptr, j_idx,
    k_ptr, k_idx) as numpy arrays. Runs are found by comparing neighbours, which equals the
    reference's np.unique-based run detection (python/nacho/convert.py:97-108) on sorted input."""
    c = np.asarray(coordinates)
    n = c.shape[0]
    if n == 0:
        z = np.zeros(0, np.int64)
        return z, np.zeros(1, np.int64), z, np.zeros(1, np.int64), z
    new_ij = np.ones(n, bool)
    new_ij[1:] = (c[1:, 0] != c[:-1, 0]) | (c[1:, 1] != c[:-1, 1])
    ij_starts = np.flatnonzero(new_ij)
    ij_i = c[ij_starts, 0]
    new_i = np.ones(len(ij_starts), bool)
    new_i[1:] = ij_i[1:] != ij_i[:-1]
    i_starts = np.flatnonzero(new_i)
    return (ij_i[i_starts], np.append(i_starts, len(ij_starts)), c[ij_starts, 1],
            np.append(ij_starts, n), c[:, 2])


def csf3_levels_device(i, j, k):
    """The same level arrays built on the device from three CUDA coordinate tensors (sorted unique
    (i, j, k)): neighbour compares, ``nonzero`` and gathers, no host round trip. Returns int32 CUDA
    tensors (i_idx, j_ptr, j_idx, k_ptr, k_idx)."""
    n = i.numel()
    dev = i.device
    i32 = lambda t: t.to(torch.int32).contiguous()
    if n == 0:
        z = torch.zeros(0, dtype=torch.int32, device=dev)
        one = torch.zeros(1, dtype=torch.int32, device=dev)
        return z, one, z.clone(), one.clone(), z.clone()
    new_ij = torch.ones(n, dtype=torch.bool, device=dev)
    new_ij[1:] = (i[1:] != i[:-1]) | (j[1:] != j[:-1])
    ij_starts = torch.nonzero(new_ij).squeeze(1)
    ij_i = i[ij_starts]
    new_i = torch.ones(ij_starts.numel(), dtype=torch.bool, device=dev)
    new_i[1:] = ij_i[1:] != ij_i[:-1]
    i_starts = torch.nonzero(new_i).squeeze(1)
    end = lambda t, x: torch.cat([t, torch.tensor([x], dtype=t.dtype, device=dev)])
    return (i32(ij_i[i_starts]), i32(end(i_starts, ij_starts.numel())), i32(j[ij_starts]), i32(end(ij_starts, n)), i32(k))


def to_csf3(coordinates, values, shape, device="cuda"):
    """Sorted, deduplicated (i, j, k) rows -> CSF3_gpu (python/nacho/convert.py:90-118). Coordinates
    given as a CUDA tensor of shape (n, 3) are turned into level arrays on the device; numpy arrays
    and CPU tensors take the host path, like the reference."""
    dev = _gpu_only(device)
    if isinstance(coordinates, torch.Tensor) and coordinates.is_cuda:
        c = coordinates.to(dev)
        levels = csf3_levels_device(c[:, 0].contiguous(), c[:, 1].contiguous(), c[:, 2].contiguous())
        vals = values if isinstance(values, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(values))
        return _ext.CSF3_gpu(*levels, vals.to(dtype=torch.float32, device=dev).contiguous(), torch.tensor(list(shape), dtype=torch.int32))
    if isinstance(coordinates, torch.Tensor):
        coordinates = coordinates.numpy()
    i_idx, j_ptr, j_idx, k_ptr, k_idx = csf3_levels(coordinates)
    return _ext.CSF3_gpu(
        _tensor(i_idx, torch.int32, dev),
        _tensor(j_ptr, torch.int32, dev),
        _tensor(j_idx, torch.int32, dev),
        _tensor(k_ptr, torch.int32, dev),
        _tensor(k_idx, torch.int32, dev),
        _tensor(values, torch.float32, dev),
        torch.tensor(list(shape), dtype=torch.int32),
    )
