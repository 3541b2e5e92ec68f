"""Operators on HOST-resident CSR matrices: the operands are CPU torch tensors (pin them for
full PCIe speed), the result comes back in CPU tensors, and the library streams row blocks
through the GPU so that uploads, merges and downloads overlap (``nb200_csr_*_f32_host``).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _capi
from ._capi import CsrStruct, lib


def _host_array(t, dtype, name):
    if not isinstance(t, torch.Tensor) or t.is_cuda or t.dtype != dtype or t.dim() != 1 or not t.is_contiguous():
        raise TypeError(f"{name}: expected a 1-D contiguous CPU tensor of dtype {dtype}")
    return t


def _view(rows, cols, rp, col, val):
    _host_array(rp, torch.int32, "row_ptr"), _host_array(col, torch.int32, "col"), _host_array(val, torch.float32, "val")
    if rp.numel() != rows + 1 or col.numel() != val.numel():
        raise ValueError("row_ptr must hold rows + 1 entries and col / val must have equal lengths")
    return CsrStruct(rows, cols, val.numel(), rp.data_ptr(), col.data_ptr(), val.data_ptr())


def result_buffers(rows: int, capacity: int, pin: bool = True):
    """CPU tensors (row_ptr, col, val) for a result of up to ``capacity`` entries. Pinning takes
    milliseconds per hundred megabytes, so callers in a loop should allocate these once."""
    mk = lambda n, dt: torch.empty(max(n, 1), dtype=dt, pin_memory=pin)
    return mk(rows + 1, torch.int32), mk(capacity, torch.int32), mk(capacity, torch.float32)


def _run(entry, where, a, b, capacity, out, device):
    rows, cols = int(a[0]), int(a[1])
    if (rows, cols) != (int(b[0]), int(b[1])):
        raise ValueError("operands differ in shape")
    sa, sb = _view(rows, cols, *a[2:]), _view(rows, cols, *b[2:])
    rp, col, val = out if out is not None else result_buffers(rows, capacity)
    if rp.numel() < rows + 1 or min(col.numel(), val.numel()) < capacity:
        raise ValueError("result buffers are smaller than the stated capacity")
    sz = CsrStruct(rows, cols, 0, rp.data_ptr(), col.data_ptr(), val.data_ptr())
    with torch.cuda.device(device):
        status = entry(C.byref(sa), C.byref(sb), C.byref(sz), capacity)
    _capi.check(status, where)
    n = int(sz.nnz)
    return rows, cols, rp[: rows + 1], col[:n], val[:n]


def csr_add_host(a, b, out=None, device=None):
    """Z = A + B for host-resident operands ``(rows, cols, row_ptr, col, val)``; returns the same
    kind of tuple. ``out`` = ``result_buffers(rows, nnz(A) + nnz(B))`` avoids re-pinning."""
    return _run(lib.nb200_csr_add_f32_host, "csr_add_host", a, b, a[3].numel() + b[3].numel(), out, device)


def csr_mul_host(a, b, out=None, device=None):
    """Z = A .* B for host-resident operands."""
    return _run(lib.nb200_csr_mul_f32_host, "csr_mul_host", a, b, min(a[3].numel(), b[3].numel()), out, device)
