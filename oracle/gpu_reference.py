"""ctypes front-end of the reference-GPU checker (test infrastructure only).

``ReferenceGpu`` -> ``_ref/libnacho_ref_gpu.so``: the GPU drivers emitted by the reference's own
compiler (``<kernel>_gpu_i32_f32``), compiled unchanged for sm_100a by ``make ref_gpu``. It is the
only reference implementation of SpGEMM, and the on-device referee for the other kernels.

Only the GPU tests and the baseline leg of the benchmark may import this module; product code
never does. Operands and results are tuples of torch CUDA tensors in the layouts of
``cpu_oracle`` (CSR = (rows, cols, row_ptr, col, val), COO3 = (dims, i, j, k, val),
CSF3 = (dims, i_idx, j_ptr, j_idx, k_ptr, k_idx, val)).

The emitted SpGEMM counts products in int32: keep the product count of a call below 2^31.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_GPU_SO = os.path.join(HERE, "_ref", "libnacho_ref_gpu.so")
DEFAULT_GRID = (256, 256)  # num_blocks, threads_per_block (src/backend/generate_bindings.cpp:317-327)

_I32P = C.POINTER(C.c_int32)
_F32P = C.POINTER(C.c_float)


def build() -> None:
    """Compile ``_ref/libnacho_ref_gpu.so`` (needs the reference checkout and nvcc)."""
    from .cpu_oracle import reference_root
    ref_root = reference_root()
    if ref_root is None:
        raise FileNotFoundError("the reference checkout was not found: set NACHO_REF_ROOT")
    subprocess.run(["make", "-s", "-j8", "-C", HERE, "ref_gpu", f"REF={ref_root}"], check=True)


class _CSR(C.Structure):
    _fields_ = [("rows", C.c_int32), ("cols", C.c_int32), ("nnz", C.c_int32),
                ("row_ptr", C.c_void_p), ("col", C.c_void_p), ("val", C.c_void_p)]


class _COO3(C.Structure):
    _fields_ = [("dims", C.c_int32 * 3), ("nnz", C.c_int32),
                ("i", C.c_void_p), ("j", C.c_void_p), ("k", C.c_void_p), ("val", C.c_void_p)]


class _CSF3(C.Structure):
    _fields_ = [("dims", C.c_int32 * 3), ("n_i", C.c_int32), ("n_j", C.c_int32), ("n_k", C.c_int32),
                ("i_idx", C.c_void_p), ("j_ptr", C.c_void_p), ("j_idx", C.c_void_p), ("k_ptr", C.c_void_p),
                ("k_idx", C.c_void_p), ("val", C.c_void_p)]


class ReferenceGpu:
    """The reference's own emitted GPU kernels (``ref_shim/ref_gpu_abi.h``)."""

    def __init__(self, path: str = REF_GPU_SO):
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} missing: run `make -C oracle ref_gpu` where the reference checkout is present")
        self.lib = C.CDLL(path)
        L = self.lib
        P = C.POINTER
        L.ref_gpu_free.argtypes = [C.c_void_p]
        L.ref_gpu_copy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        for name, n, t in (("csr_add", 3, _CSR), ("csr_mul", 3, _CSR), ("csr_add_3", 4, _CSR), ("spgemm", 3, _CSR), ("sssmm", 4, _CSR),
                           ("coo3d_add", 3, _COO3), ("csf_add", 3, _CSF3)):
            getattr(L, "ref_gpu_" + name).argtypes = [P(t)] * n + [C.c_int, C.c_int]
        self.last_ms = 0.0  # wall-clock of the last driver call, device synchronised on both sides

    @staticmethod
    def available(path: str = REF_GPU_SO) -> bool:
        return os.path.exists(path)

    # ---- helpers ------------------------------------------------------------------------
    def _call(self, fn, *args):
        import torch
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        err = fn(*args)
        self.last_ms = (time.perf_counter() - t0) * 1e3
        if err:
            raise RuntimeError(f"reference GPU driver reported CUDA error {err}")

    def _adopt(self, ptr, n, dtype, keep):
        """Copies a driver-allocated device array into a torch tensor and frees the original."""
        import torch
        out = None
        if keep:
            out = torch.empty(max(int(n), 0), dtype=dtype, device="cuda")
            if n > 0 and ptr:
                err = self.lib.ref_gpu_copy(out.data_ptr(), ptr, int(n) * out.element_size())
                if err:
                    raise RuntimeError(f"device copy failed with CUDA error {err}")
        if ptr:
            self.lib.ref_gpu_free(ptr)
        return out

    @staticmethod
    def _csr_in(m):
        rows, cols, rp, col, val = m
        keep = (rp.contiguous(), col.contiguous(), val.contiguous())
        return _CSR(int(rows), int(cols), keep[1].numel(), keep[0].data_ptr(), keep[1].data_ptr(), keep[2].data_ptr()), keep

    def _csr_out(self, z, keep):
        import torch
        rp = self._adopt(z.row_ptr, z.rows + 1, torch.int32, keep)
        col = self._adopt(z.col, z.nnz, torch.int32, keep)
        val = self._adopt(z.val, z.nnz, torch.float32, keep)
        return (z.rows, z.cols, rp, col, val) if keep else None

    def _csr_op(self, name, operands, grid, keep):
        structs, alive = zip(*[self._csr_in(m) for m in operands])
        z = _CSR()
        self._call(getattr(self.lib, "ref_gpu_" + name), *[C.byref(s) for s in structs], C.byref(z), int(grid[0]), int(grid[1]))
        return self._csr_out(z, keep)

    # ---- kernels ------------------------------------------------------------------------
    def csr_add(self, a, b, grid=DEFAULT_GRID, keep=True):
        return self._csr_op("csr_add", (a, b), grid, keep)

    def csr_mul(self, a, b, grid=DEFAULT_GRID, keep=True):
        return self._csr_op("csr_mul", (a, b), grid, keep)

    def csr_add_3(self, a, b, c, grid=DEFAULT_GRID, keep=True):
        return self._csr_op("csr_add_3", (a, b, c), grid, keep)

    def spgemm(self, a, b, grid=DEFAULT_GRID, keep=True):
        return self._csr_op("spgemm", (a, b), grid, keep)

    def sssmm(self, a, b, c, grid=DEFAULT_GRID, keep=True):
        """Masked product sum_j a_ij b_jk c_ik (compiler.cpp:150-153)."""
        return self._csr_op("sssmm", (a, b, c), grid, keep)

    def coo3_add(self, a, b, grid=DEFAULT_GRID, keep=True):
        import torch

        def mk(t):
            dims, i, j, k, val = t
            alive = (i.contiguous(), j.contiguous(), k.contiguous(), val.contiguous())
            return _COO3((C.c_int32 * 3)(*[int(d) for d in dims]), alive[3].numel(), *[x.data_ptr() for x in alive]), alive

        sa, ka = mk(a)
        sb, kb = mk(b)
        z = _COO3()
        self._call(self.lib.ref_gpu_coo3d_add, C.byref(sa), C.byref(sb), C.byref(z), int(grid[0]), int(grid[1]))
        out = [self._adopt(p, z.nnz, torch.int32, keep) for p in (z.i, z.j, z.k)]
        val = self._adopt(z.val, z.nnz, torch.float32, keep)
        return (tuple(z.dims), *out, val) if keep else None

    def csf3_add(self, a, b, grid=DEFAULT_GRID, keep=True):
        import torch

        def mk(t):
            dims, i_idx, j_ptr, j_idx, k_ptr, k_idx, val = t
            alive = tuple(x.contiguous() for x in (i_idx, j_ptr, j_idx, k_ptr, k_idx, val))
            return _CSF3((C.c_int32 * 3)(*[int(d) for d in dims]), alive[0].numel(), alive[2].numel(), alive[4].numel(),
                         *[x.data_ptr() for x in alive]), alive

        sa, ka = mk(a)
        sb, kb = mk(b)
        z = _CSF3()
        self._call(self.lib.ref_gpu_csf_add, C.byref(sa), C.byref(sb), C.byref(z), int(grid[0]), int(grid[1]))
        i_idx = self._adopt(z.i_idx, z.n_i, torch.int32, keep)
        j_ptr = self._adopt(z.j_ptr, z.n_i + 1, torch.int32, keep)
        j_idx = self._adopt(z.j_idx, z.n_j, torch.int32, keep)
        k_ptr = self._adopt(z.k_ptr, z.n_j + 1, torch.int32, keep)
        k_idx = self._adopt(z.k_idx, z.n_k, torch.int32, keep)
        val = self._adopt(z.val, z.n_k, torch.float32, keep)
        return (tuple(z.dims), i_idx, j_ptr, j_idx, k_ptr, k_idx, val) if keep else None
