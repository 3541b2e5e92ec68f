"""Host-side mirror of the reference's generated extension module ``nacho_ext``: the GPU tensor
classes and the ``gpu_<kernel>_f32`` operators, with the names, argument order, defaults and
read-only attributes the reference's binding generator emits
(src/backend/generate_bindings.cpp:84-154 classes, :288-331 operators, :317-327 keyword names
and the 256 x 256 default grid). Every operator forwards to the C ABI in ``libnacho_b200.so``;
nothing is computed in Python or torch.

Tensors are 1-D contiguous CUDA torch tensors (int32 indices, float32 values) and ``shape`` is
a host int32 tensor, as in runtime/nacho_nb.h:22-31. Operands are borrowed; results are fresh
torch tensors owned by the returned object.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _capi
from .._capi import Coo3Struct, CooStruct, CsrStruct, Csf3Struct, DcsrStruct, lib

__all__ = ["CSR_gpu", "COO3_gpu", "CSF3_gpu", "COO_gpu", "DCSR_gpu", "Scalar_gpu", "gpu_csr_add_f32", "gpu_csr_add_3_f32",
           "gpu_csr_mul_f32", "gpu_spgemm_f32", "gpu_coo3d_add_f32", "gpu_csf_add_f32", "gpu_coo_add_f32", "gpu_coo_mul_f32",
           "gpu_coo_csr_add_f32", "gpu_dcsr_add_f32", "gpu_dcsr_mul_f32", "gpu_dcsr_mul_without_recursive_partitioning_f32",
           "gpu_inner_prod_f32", "gpu_inner_prod_coo_f32", "gpu_sssmm_f32"]


def _dev_array(t, dtype, name):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name}: expected a torch tensor")
    if not t.is_cuda or t.dtype != dtype or t.dim() != 1 or not t.is_contiguous():
        raise TypeError(f"{name}: expected a 1-D contiguous CUDA tensor of dtype {dtype}")
    return t


def _shape_array(t, rank, name="shape"):
    if not isinstance(t, torch.Tensor):
        t = torch.tensor(list(t), dtype=torch.int32)
    if t.is_cuda or t.dtype != torch.int32 or t.dim() != 1 or t.numel() != rank:
        raise TypeError(f"{name}: expected a host int32 tensor of {rank} entries")
    return t.contiguous()


def _stream_for(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


class CSR_gpu:
    """CSR matrix on the GPU: ``CSR_gpu(dim_j_offsets, dim_j_indices, values, shape)``
    (attribute names as emitted by src/backend/generate_bindings.cpp:84-154)."""

    __slots__ = ("_offsets", "_indices", "_values", "_shape", "_rows", "_cols")

    def __init__(self, dim_j_offsets, dim_j_indices, values, shape):
        self._offsets = _dev_array(dim_j_offsets, torch.int32, "dim_j_offsets")
        self._indices = _dev_array(dim_j_indices, torch.int32, "dim_j_indices")
        self._values = _dev_array(values, torch.float32, "values")
        self._shape = _shape_array(shape, 2)
        self._rows, self._cols = (int(x) for x in self._shape)
        if self._indices.numel() != self._values.numel():
            raise ValueError("dim_j_indices and values differ in length")
        if self._offsets.numel() != self._rows + 1:
            raise ValueError("dim_j_offsets must hold rows + 1 entries")
        if not (self._offsets.device == self._indices.device == self._values.device):
            raise ValueError("all buffers of a tensor must live on one device")

    dim_j_offsets = property(lambda self: self._offsets)
    dim_j_indices = property(lambda self: self._indices)
    values = property(lambda self: self._values)
    shape = property(lambda self: self._shape)

    @property
    def device(self):
        return self._values.device

    def _struct(self) -> CsrStruct:
        return CsrStruct(self._rows, self._cols, self._values.numel(),
                         self._offsets.data_ptr(), self._indices.data_ptr(), self._values.data_ptr())

    def __repr__(self):
        return f"CSR_gpu(shape=({self._rows}, {self._cols}), nnz={self._values.numel()})"


def _same_device(*tensors):
    dev = tensors[0].device
    for t in tensors[1:]:
        if t.device != dev:
            raise ValueError("operands live on different devices")
    return dev


def _csr_result(rows, cols, dev):
    return torch.empty(rows + 1, dtype=torch.int32, device=dev)


def _csr_binary(entry, where, a: CSR_gpu, b: CSR_gpu, capacity: int) -> CSR_gpu:
    if not isinstance(a, CSR_gpu) or not isinstance(b, CSR_gpu):
        raise TypeError(f"{where}: operands must be CSR_gpu")
    dev = _same_device(a, b)
    sa, sb = a._struct(), b._struct()
    with torch.cuda.device(dev):
        row_ptr = _csr_result(sa.rows, sa.cols, dev)
        col = torch.empty(max(capacity, 1), dtype=torch.int32, device=dev)
        val = torch.empty(max(capacity, 1), dtype=torch.float32, device=dev)
        sz = CsrStruct(sa.rows, sa.cols, 0, row_ptr.data_ptr(), col.data_ptr(), val.data_ptr())
        status = entry(C.byref(sa), C.byref(sb), C.byref(sz), capacity, _stream_for(row_ptr))
    _capi.check(status, where)
    n = int(sz.nnz)
    return CSR_gpu(row_ptr, col[:n], val[:n], torch.tensor([sz.rows, sz.cols], dtype=torch.int32))


def gpu_csr_add_f32(a: CSR_gpu, b: CSR_gpu, num_blocks: int = 256, threads_per_block: int = 256) -> CSR_gpu:
    """Z = A + B (sorted union per row; explicit zeros kept). ``num_blocks`` and
    ``threads_per_block`` are accepted for compatibility and ignored."""
    return _csr_binary(lib.nb200_csr_add_f32_into, "gpu_csr_add_f32", a, b,
                       a.values.numel() + b.values.numel())


def gpu_csr_mul_f32(a: CSR_gpu, b: CSR_gpu, num_blocks: int = 256, threads_per_block: int = 256) -> CSR_gpu:
    """Z = A .* B (sorted intersection per row)."""
    return _csr_binary(lib.nb200_csr_mul_f32_into, "gpu_csr_mul_f32", a, b,
                       min(a.values.numel(), b.values.numel()))


def gpu_csr_add_3_f32(a: CSR_gpu, b: CSR_gpu, c: CSR_gpu, num_blocks: int = 256,
                      threads_per_block: int = 256) -> CSR_gpu:
    """Z = (A + B) + C, the reference's association."""
    for t in (a, b, c):
        if not isinstance(t, CSR_gpu):
            raise TypeError("gpu_csr_add_3_f32: operands must be CSR_gpu")
    dev = _same_device(a, b, c)
    sa, sb, sc = a._struct(), b._struct(), c._struct()
    capacity = sa.nnz + sb.nnz + sc.nnz
    with torch.cuda.device(dev):
        row_ptr = _csr_result(sa.rows, sa.cols, dev)
        col = torch.empty(max(capacity, 1), dtype=torch.int32, device=dev)
        val = torch.empty(max(capacity, 1), dtype=torch.float32, device=dev)
        sz = CsrStruct(sa.rows, sa.cols, 0, row_ptr.data_ptr(), col.data_ptr(), val.data_ptr())
        status = lib.nb200_csr_add_3_f32_into(C.byref(sa), C.byref(sb), C.byref(sc), C.byref(sz), capacity,
                                              _stream_for(row_ptr))
    _capi.check(status, "gpu_csr_add_3_f32")
    n = int(sz.nnz)
    return CSR_gpu(row_ptr, col[:n], val[:n], torch.tensor([sz.rows, sz.cols], dtype=torch.int32))


def gpu_spgemm_f32(a: CSR_gpu, b: CSR_gpu, num_blocks: int = 256, threads_per_block: int = 256) -> CSR_gpu:
    """C = A @ B by expand-sort-compress; sorted columns per row, explicit zeros kept."""
    if not isinstance(a, CSR_gpu) or not isinstance(b, CSR_gpu):
        raise TypeError("gpu_spgemm_f32: operands must be CSR_gpu")
    dev = _same_device(a, b)
    sa, sb = a._struct(), b._struct()
    with torch.cuda.device(dev):
        row_ptr = torch.empty(sa.rows + 1, dtype=torch.int32, device=dev)
        sc = CsrStruct(sa.rows, sb.cols, 0, row_ptr.data_ptr(), None, None)
        stream = _stream_for(row_ptr)
        _capi.check(lib.nb200_spgemm_f32_symbolic(C.byref(sa), C.byref(sb), C.byref(sc), None, stream), "gpu_spgemm_f32")
        n = int(sc.nnz)
        col = torch.empty(n, dtype=torch.int32, device=dev)
        val = torch.empty(n, dtype=torch.float32, device=dev)
        sc.col, sc.val = col.data_ptr() if n else None, val.data_ptr() if n else None
        _capi.check(lib.nb200_spgemm_f32_numeric(C.byref(sa), C.byref(sb), C.byref(sc), stream), "gpu_spgemm_f32")
    return CSR_gpu(row_ptr, col, val, torch.tensor([sc.rows, sc.cols], dtype=torch.int32))


class COO3_gpu:
    """3-mode tensor as parallel coordinate arrays:
    ``COO3_gpu(dim_i_indices, dim_j_indices, dim_k_indices, values, shape)``."""

    __slots__ = ("_i", "_j", "_k", "_values", "_shape")

    def __init__(self, dim_i_indices, dim_j_indices, dim_k_indices, values, shape):
        self._i = _dev_array(dim_i_indices, torch.int32, "dim_i_indices")
        self._j = _dev_array(dim_j_indices, torch.int32, "dim_j_indices")
        self._k = _dev_array(dim_k_indices, torch.int32, "dim_k_indices")
        self._values = _dev_array(values, torch.float32, "values")
        self._shape = _shape_array(shape, 3)
        n = self._values.numel()
        if not (self._i.numel() == self._j.numel() == self._k.numel() == n):
            raise ValueError("coordinate arrays and values differ in length")

    dim_i_indices = property(lambda self: self._i)
    dim_j_indices = property(lambda self: self._j)
    dim_k_indices = property(lambda self: self._k)
    values = property(lambda self: self._values)
    shape = property(lambda self: self._shape)

    @property
    def device(self):
        return self._values.device

    def _struct(self) -> Coo3Struct:
        dims = (C.c_int32 * 3)(*[int(x) for x in self._shape])
        return Coo3Struct(dims, self._values.numel(), self._i.data_ptr(), self._j.data_ptr(), self._k.data_ptr(),
                          self._values.data_ptr())

    def __repr__(self):
        return f"COO3_gpu(shape={tuple(int(x) for x in self._shape)}, nnz={self._values.numel()})"


class CSF3_gpu:
    """3-mode tensor with three compressed levels: ``CSF3_gpu(dim_i_indices, dim_j_offsets,
    dim_j_indices, dim_k_offsets, dim_k_indices, values, shape)``; ``dim_j_offsets`` holds
    ``len(dim_i_indices) + 1`` entries and ``dim_k_offsets`` ``len(dim_j_indices) + 1``
    (src/backend/generate_bindings.cpp:119-143)."""

    __slots__ = ("_i", "_jp", "_j", "_kp", "_k", "_values", "_shape")

    def __init__(self, dim_i_indices, dim_j_offsets, dim_j_indices, dim_k_offsets, dim_k_indices, values, shape):
        self._i = _dev_array(dim_i_indices, torch.int32, "dim_i_indices")
        self._jp = _dev_array(dim_j_offsets, torch.int32, "dim_j_offsets")
        self._j = _dev_array(dim_j_indices, torch.int32, "dim_j_indices")
        self._kp = _dev_array(dim_k_offsets, torch.int32, "dim_k_offsets")
        self._k = _dev_array(dim_k_indices, torch.int32, "dim_k_indices")
        self._values = _dev_array(values, torch.float32, "values")
        self._shape = _shape_array(shape, 3)
        if self._jp.numel() != self._i.numel() + 1 or self._kp.numel() != self._j.numel() + 1:
            raise ValueError("offset arrays must hold one entry more than the level above has coordinates")
        if self._k.numel() != self._values.numel():
            raise ValueError("dim_k_indices and values differ in length")

    dim_i_indices = property(lambda self: self._i)
    dim_j_offsets = property(lambda self: self._jp)
    dim_j_indices = property(lambda self: self._j)
    dim_k_offsets = property(lambda self: self._kp)
    dim_k_indices = property(lambda self: self._k)
    values = property(lambda self: self._values)
    shape = property(lambda self: self._shape)

    @property
    def device(self):
        return self._values.device

    def _struct(self) -> Csf3Struct:
        dims = (C.c_int32 * 3)(*[int(x) for x in self._shape])
        return Csf3Struct(dims, self._i.numel(), self._j.numel(), self._k.numel(), self._i.data_ptr(),
                          self._jp.data_ptr(), self._j.data_ptr(), self._kp.data_ptr(), self._k.data_ptr(),
                          self._values.data_ptr())

    def __repr__(self):
        return (f"CSF3_gpu(shape={tuple(int(x) for x in self._shape)}, levels=({self._i.numel()}, "
                f"{self._j.numel()}, {self._k.numel()}))")


def gpu_coo3d_add_f32(a: COO3_gpu, b: COO3_gpu, num_blocks: int = 256, threads_per_block: int = 256) -> COO3_gpu:
    """Z = A + B over sorted unique (i, j, k) coordinates."""
    if not isinstance(a, COO3_gpu) or not isinstance(b, COO3_gpu):
        raise TypeError("gpu_coo3d_add_f32: operands must be COO3_gpu")
    dev = _same_device(a, b)
    sa, sb = a._struct(), b._struct()
    cap = sa.nnz + sb.nnz
    with torch.cuda.device(dev):
        zi, zj, zk = (torch.empty(max(cap, 1), dtype=torch.int32, device=dev) for _ in range(3))
        zv = torch.empty(max(cap, 1), dtype=torch.float32, device=dev)
        sz = Coo3Struct((C.c_int32 * 3)(), 0, zi.data_ptr(), zj.data_ptr(), zk.data_ptr(), zv.data_ptr())
        status = lib.nb200_coo3d_add_f32_into(C.byref(sa), C.byref(sb), C.byref(sz), cap, _stream_for(zv))
    _capi.check(status, "gpu_coo3d_add_f32")
    n = int(sz.nnz)
    return COO3_gpu(zi[:n], zj[:n], zk[:n], zv[:n], torch.tensor(list(sz.dims), dtype=torch.int32))


def gpu_csf_add_f32(a: CSF3_gpu, b: CSF3_gpu, num_blocks: int = 256, threads_per_block: int = 256) -> CSF3_gpu:
    """Z = A + B for CSF3 operands."""
    if not isinstance(a, CSF3_gpu) or not isinstance(b, CSF3_gpu):
        raise TypeError("gpu_csf_add_f32: operands must be CSF3_gpu")
    dev = _same_device(a, b)
    sa, sb = a._struct(), b._struct()
    cap_i, cap_j, cap_k = sa.n_i + sb.n_i, sa.n_j + sb.n_j, sa.n_k + sb.n_k
    with torch.cuda.device(dev):
        new = lambda n, dt=torch.int32: torch.empty(max(n, 1), dtype=dt, device=dev)
        zi, zjp, zj, zkp, zk, zv = new(cap_i), new(cap_i + 1), new(cap_j), new(cap_j + 1), new(cap_k), new(cap_k, torch.float32)
        sz = Csf3Struct((C.c_int32 * 3)(), 0, 0, 0, zi.data_ptr(), zjp.data_ptr(), zj.data_ptr(), zkp.data_ptr(),
                        zk.data_ptr(), zv.data_ptr())
        status = lib.nb200_csf_add_f32_into(C.byref(sa), C.byref(sb), C.byref(sz), cap_i, cap_j, cap_k, _stream_for(zv))
    _capi.check(status, "gpu_csf_add_f32")
    ni, nj, nk = int(sz.n_i), int(sz.n_j), int(sz.n_k)
    return CSF3_gpu(zi[:ni], zjp[:ni + 1], zj[:nj], zkp[:nj + 1], zk[:nk], zv[:nk],
                    torch.tensor(list(sz.dims), dtype=torch.int32))


# ---- the rest of the element-wise family: 2-D COO, DCSR, inner products, masked SpGEMM ----

class COO_gpu:
    """2-D coordinate list sorted by (i, j): ``COO_gpu(dim_i_indices, dim_j_indices, values, shape)``."""

    __slots__ = ("_i", "_j", "_values", "_shape")

    def __init__(self, dim_i_indices, dim_j_indices, values, shape):
        self._i = _dev_array(dim_i_indices, torch.int32, "dim_i_indices")
        self._j = _dev_array(dim_j_indices, torch.int32, "dim_j_indices")
        self._values = _dev_array(values, torch.float32, "values")
        self._shape = _shape_array(shape, 2)
        if not (self._i.numel() == self._j.numel() == self._values.numel()):
            raise ValueError("coordinate arrays and values differ in length")

    dim_i_indices = property(lambda self: self._i)
    dim_j_indices = property(lambda self: self._j)
    values = property(lambda self: self._values)
    shape = property(lambda self: self._shape)

    @property
    def device(self):
        return self._values.device

    def _struct(self) -> CooStruct:
        return CooStruct(int(self._shape[0]), int(self._shape[1]), self._values.numel(), self._i.data_ptr(),
                         self._j.data_ptr(), self._values.data_ptr())

    def __repr__(self):
        return f"COO_gpu(shape=({int(self._shape[0])}, {int(self._shape[1])}), nnz={self._values.numel()})"


class DCSR_gpu:
    """CSR with a compressed row level: ``DCSR_gpu(dim_i_indices, dim_j_offsets, dim_j_indices, values,
    shape)``; ``dim_i_indices`` lists the rows that hold entries, ``dim_j_offsets`` has one entry more."""

    __slots__ = ("_i", "_jp", "_j", "_values", "_shape")

    def __init__(self, dim_i_indices, dim_j_offsets, dim_j_indices, values, shape):
        self._i = _dev_array(dim_i_indices, torch.int32, "dim_i_indices")
        self._jp = _dev_array(dim_j_offsets, torch.int32, "dim_j_offsets")
        self._j = _dev_array(dim_j_indices, torch.int32, "dim_j_indices")
        self._values = _dev_array(values, torch.float32, "values")
        self._shape = _shape_array(shape, 2)
        if self._jp.numel() != self._i.numel() + 1:
            raise ValueError("dim_j_offsets must hold one entry more than dim_i_indices")
        if self._j.numel() != self._values.numel():
            raise ValueError("dim_j_indices and values differ in length")

    dim_i_indices = property(lambda self: self._i)
    dim_j_offsets = property(lambda self: self._jp)
    dim_j_indices = property(lambda self: self._j)
    values = property(lambda self: self._values)
    shape = property(lambda self: self._shape)

    @property
    def device(self):
        return self._values.device

    def _struct(self) -> DcsrStruct:
        return DcsrStruct(int(self._shape[0]), int(self._shape[1]), self._i.numel(), self._values.numel(),
                          self._i.data_ptr(), self._jp.data_ptr(), self._j.data_ptr(), self._values.data_ptr())

    def __repr__(self):
        return f"DCSR_gpu(shape=({int(self._shape[0])}, {int(self._shape[1])}), rows_stored={self._i.numel()}, nnz={self._values.numel()})"


class Scalar_gpu:
    """Result of a full reduction: ``values`` is a one-element float32 CUDA tensor."""

    __slots__ = ("_values",)

    def __init__(self, values):
        self._values = _dev_array(values, torch.float32, "values")

    values = property(lambda self: self._values)

    @property
    def device(self):
        return self._values.device


def _coo_binary(entry, where, a: COO_gpu, b: COO_gpu, capacity: int) -> COO_gpu:
    if not isinstance(a, COO_gpu) or not isinstance(b, COO_gpu):
        raise TypeError(f"{where}: operands must be COO_gpu")
    dev = _same_device(a, b)
    sa, sb = a._struct(), b._struct()
    with torch.cuda.device(dev):
        zi, zj = (torch.empty(max(capacity, 1), dtype=torch.int32, device=dev) for _ in range(2))
        zv = torch.empty(max(capacity, 1), dtype=torch.float32, device=dev)
        sz = CooStruct(sa.rows, sa.cols, 0, zi.data_ptr(), zj.data_ptr(), zv.data_ptr())
        status = entry(C.byref(sa), C.byref(sb), C.byref(sz), capacity, _stream_for(zv))
    _capi.check(status, where)
    n = int(sz.nnz)
    return COO_gpu(zi[:n], zj[:n], zv[:n], torch.tensor([sz.rows, sz.cols], dtype=torch.int32))


def gpu_coo_add_f32(a: COO_gpu, b: COO_gpu, num_blocks: int = 256, threads_per_block: int = 256) -> COO_gpu:
    """Z = A + B over sorted unique (i, j) lists."""
    return _coo_binary(lib.nb200_coo_add_f32_into, "gpu_coo_add_f32", a, b, a.values.numel() + b.values.numel())


def gpu_coo_mul_f32(a: COO_gpu, b: COO_gpu, num_blocks: int = 256, threads_per_block: int = 256) -> COO_gpu:
    """Z = A .* B over sorted unique (i, j) lists."""
    return _coo_binary(lib.nb200_coo_mul_f32_into, "gpu_coo_mul_f32", a, b, min(a.values.numel(), b.values.numel()))


def gpu_coo_csr_add_f32(a: CSR_gpu, b: COO_gpu, num_blocks: int = 256, threads_per_block: int = 256) -> CSR_gpu:
    """Z = A + B with A in CSR and B a coordinate list; the result is CSR."""
    if not isinstance(a, CSR_gpu) or not isinstance(b, COO_gpu):
        raise TypeError("gpu_coo_csr_add_f32: operands must be (CSR_gpu, COO_gpu)")
    dev = _same_device(a, b)
    sa, sb = a._struct(), b._struct()
    capacity = sa.nnz + sb.nnz
    with torch.cuda.device(dev):
        row_ptr = _csr_result(sa.rows, sa.cols, dev)
        col = torch.empty(max(capacity, 1), dtype=torch.int32, device=dev)
        val = torch.empty(max(capacity, 1), dtype=torch.float32, device=dev)
        sz = CsrStruct(sa.rows, sa.cols, 0, row_ptr.data_ptr(), col.data_ptr(), val.data_ptr())
        status = lib.nb200_coo_csr_add_f32_into(C.byref(sa), C.byref(sb), C.byref(sz), capacity, _stream_for(row_ptr))
    _capi.check(status, "gpu_coo_csr_add_f32")
    n = int(sz.nnz)
    return CSR_gpu(row_ptr, col[:n], val[:n], torch.tensor([sz.rows, sz.cols], dtype=torch.int32))


def _dcsr_binary(entry, where, a: DCSR_gpu, b: DCSR_gpu, cap_i: int, capacity: int) -> DCSR_gpu:
    if not isinstance(a, DCSR_gpu) or not isinstance(b, DCSR_gpu):
        raise TypeError(f"{where}: operands must be DCSR_gpu")
    dev = _same_device(a, b)
    sa, sb = a._struct(), b._struct()
    with torch.cuda.device(dev):
        zi = torch.empty(max(cap_i, 1), dtype=torch.int32, device=dev)
        zjp = torch.empty(cap_i + 1, dtype=torch.int32, device=dev)
        zj = torch.empty(max(capacity, 1), dtype=torch.int32, device=dev)
        zv = torch.empty(max(capacity, 1), dtype=torch.float32, device=dev)
        sz = DcsrStruct(sa.rows, sa.cols, 0, 0, zi.data_ptr(), zjp.data_ptr(), zj.data_ptr(), zv.data_ptr())
        status = entry(C.byref(sa), C.byref(sb), C.byref(sz), cap_i, capacity, _stream_for(zv))
    _capi.check(status, where)
    ni, n = int(sz.n_i), int(sz.nnz)
    return DCSR_gpu(zi[:ni], zjp[:ni + 1], zj[:n], zv[:n], torch.tensor([sz.rows, sz.cols], dtype=torch.int32))


def gpu_dcsr_add_f32(a: DCSR_gpu, b: DCSR_gpu, num_blocks: int = 256, threads_per_block: int = 256) -> DCSR_gpu:
    """Z = A + B for DCSR operands."""
    rows = int(a.shape[0])
    return _dcsr_binary(lib.nb200_dcsr_add_f32_into, "gpu_dcsr_add_f32", a, b,
                        min(a.dim_i_indices.numel() + b.dim_i_indices.numel(), rows), a.values.numel() + b.values.numel())


def gpu_dcsr_mul_f32(a: DCSR_gpu, b: DCSR_gpu, num_blocks: int = 256, threads_per_block: int = 256) -> DCSR_gpu:
    """Z = A .* B for DCSR operands; a row both operands store stays, even with no common column."""
    return _dcsr_binary(lib.nb200_dcsr_mul_f32_into, "gpu_dcsr_mul_f32", a, b,
                        min(a.dim_i_indices.numel(), b.dim_i_indices.numel()), min(a.values.numel(), b.values.numel()))


def gpu_dcsr_mul_without_recursive_partitioning_f32(a: DCSR_gpu, b: DCSR_gpu, num_blocks: int = 256,
                                                    threads_per_block: int = 256) -> DCSR_gpu:
    """The reference emits the DCSR product twice to compare two partitioning strategies of its code
    generator (compiler.cpp:128-133); both compute the same tensor, and so does this alias."""
    return gpu_dcsr_mul_f32(a, b, num_blocks, threads_per_block)


def _inner(entry, where, a, b, cls) -> Scalar_gpu:
    if not isinstance(a, cls) or not isinstance(b, cls):
        raise TypeError(f"{where}: operands must be {cls.__name__}")
    dev = _same_device(a, b)
    sa, sb = a._struct(), b._struct()
    with torch.cuda.device(dev):
        z = torch.empty(1, dtype=torch.float32, device=dev)
        status = entry(C.byref(sa), C.byref(sb), z.data_ptr(), _stream_for(z))
    _capi.check(status, where)
    return Scalar_gpu(z)


def gpu_inner_prod_f32(a: CSF3_gpu, b: CSF3_gpu, num_blocks: int = 256, threads_per_block: int = 256) -> Scalar_gpu:
    """sum_ijk a_ijk * b_ijk for CSF3 operands."""
    return _inner(lib.nb200_inner_prod_f32, "gpu_inner_prod_f32", a, b, CSF3_gpu)


def gpu_inner_prod_coo_f32(a: COO3_gpu, b: COO3_gpu, num_blocks: int = 256, threads_per_block: int = 256) -> Scalar_gpu:
    """sum_ijk a_ijk * b_ijk for COO3 operands."""
    return _inner(lib.nb200_inner_prod_coo_f32, "gpu_inner_prod_coo_f32", a, b, COO3_gpu)


def gpu_sssmm_f32(a: CSR_gpu, b: CSR_gpu, c: CSR_gpu, num_blocks: int = 256, threads_per_block: int = 256) -> CSR_gpu:
    """Z_ik = sum_j a_ij * b_jk * c_ik on the positions C stores and a product reaches (masked SpGEMM,
    compiler.cpp:150-153): one fused pass in which the mask drives the accumulation."""
    for t in (a, b, c):
        if not isinstance(t, CSR_gpu):
            raise TypeError("gpu_sssmm_f32: operands must be CSR_gpu")
    dev = _same_device(a, b, c)
    sa, sb, sc = a._struct(), b._struct(), c._struct()
    capacity = sc.nnz
    with torch.cuda.device(dev):
        row_ptr = torch.empty(sa.rows + 1, dtype=torch.int32, device=dev)
        col = torch.empty(max(capacity, 1), dtype=torch.int32, device=dev)
        val = torch.empty(max(capacity, 1), dtype=torch.float32, device=dev)
        sz = CsrStruct(sa.rows, sb.cols, 0, row_ptr.data_ptr(), col.data_ptr(), val.data_ptr())
        status = lib.nb200_sssmm_f32_into(C.byref(sa), C.byref(sb), C.byref(sc), C.byref(sz), capacity, _stream_for(row_ptr))
    _capi.check(status, "gpu_sssmm_f32")
    n = int(sz.nnz)
    return CSR_gpu(row_ptr, col[:n], val[:n], torch.tensor([sz.rows, sz.cols], dtype=torch.int32))
