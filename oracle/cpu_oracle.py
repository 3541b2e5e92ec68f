"""ctypes front-end of the two CPU checkers (test infrastructure only).

* ``Oracle``  -> ``liboracle.so``: the plain-C restatement in ``oracle.c``.
* ``Reference`` -> ``_ref/libnacho_ref_cpu.so``: the reference's own emitted CPU kernels
  (``<kernel>_cpu_i32_f32``), built by ``make ref`` from the reference checkout.

Only the tests, the smoke check and the CPU-baseline leg of the benchmark may import this
module; product code never does. Operands and results are plain tuples of numpy arrays:

* CSR  = (rows, cols, row_ptr[int32 rows+1], col[int32 nnz], val[float32 nnz])
* COO3 = (dims(3), i, j, k, val)
* CSF3 = (dims(3), i_idx, j_ptr, j_idx, k_ptr, k_idx, val)
* COO  = (rows, cols, i, j, val);  DCSR = (rows, cols, i_idx, j_ptr[len(i_idx)+1], j_idx, val)
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from collections import namedtuple

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libnacho_ref_cpu.so")

CSR = namedtuple("CSR", "rows cols row_ptr col val")
COO3 = namedtuple("COO3", "dims i j k val")
CSF3 = namedtuple("CSF3", "dims i_idx j_ptr j_idx k_ptr k_idx val")
COO = namedtuple("COO", "rows cols i j val")                    # 2-D coordinate list, sorted by (i, j)
DCSR = namedtuple("DCSR", "rows cols i_idx j_ptr j_idx val")    # CSR whose row level is compressed too

_I32P = C.POINTER(C.c_int32)
_F32P = C.POINTER(C.c_float)
_F64P = C.POINTER(C.c_double)


def reference_root() -> str | None:
    """Where the reference checkout lies: ``$NACHO_REF_ROOT``, else a folder ``reference`` beside
    this repository. None if neither holds the reference's sources."""
    for cand in (os.environ.get("NACHO_REF_ROOT"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "src")) and os.path.exists(os.path.join(cand, "compiler.cpp")):
            return cand
    return None


def build(ref: bool | None = None) -> None:
    """Compile ``liboracle.so`` and, if the reference checkout is present (or ``ref`` is
    true), ``_ref/libnacho_ref_cpu.so``."""
    subprocess.run(["make", "-s", "-C", HERE, "oracle"], check=True)
    ref_root = reference_root()
    if ref is None:
        ref = ref_root is not None
    if ref:
        if ref_root is None:
            raise FileNotFoundError("the reference checkout was not found: set NACHO_REF_ROOT")
        subprocess.run(["make", "-s", "-j8", "-C", HERE, "ref", f"REF={ref_root}"], check=True)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a, t):
    return a.ctypes.data_as(t)


def default_threads() -> int:
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


class Oracle:
    """The plain-C restatement (``oracle.h``)."""

    def __init__(self, path: str = ORACLE_SO):
        if not os.path.exists(path):
            build(ref=False)
        self.lib = C.CDLL(path)
        L = self.lib
        csr2 = [C.c_int32, _I32P, _I32P, _F32P, _I32P, _I32P, _F32P, _I32P, _I32P, _F32P, C.c_int]
        for name in ("orc_csr_add", "orc_csr_mul"):
            getattr(L, name).argtypes = csr2
            getattr(L, name).restype = C.c_int64
        L.orc_csr_add3.argtypes = [C.c_int32] + [_I32P, _I32P, _F32P] * 3 + [_I32P, _I32P, _F32P, C.c_int]
        L.orc_csr_add3.restype = C.c_int64
        L.orc_coo3_add.argtypes = ([C.c_int32, _I32P, _I32P, _I32P, _F32P] * 2
                                   + [_I32P, _I32P, _I32P, _F32P, C.c_int])
        L.orc_coo3_add.restype = C.c_int64
        L.orc_csf3_add.argtypes = ([C.c_int32, _I32P, _I32P, _I32P, _I32P, _I32P, _F32P] * 2
                                   + [_I32P, _I32P, _I32P, _I32P, _I32P, _F32P, _I32P])
        L.orc_csf3_add.restype = C.c_int64
        L.orc_spgemm_symbolic.argtypes = [C.c_int32, C.c_int32, _I32P, _I32P, _I32P, _I32P, _I32P,
                                          C.POINTER(C.c_int64), C.c_int]
        L.orc_spgemm_symbolic.restype = C.c_int64
        L.orc_spgemm_numeric.argtypes = [C.c_int32, C.c_int32, _I32P, _I32P, _F32P, _I32P, _I32P,
                                         _F32P, _I32P, _I32P, _F32P, _F64P, _F64P, C.c_int]
        L.orc_spgemm_numeric.restype = C.c_int64

    @staticmethod
    def _csr_args(m: CSR):
        rp, col, val = _i32(m.row_ptr), _i32(m.col), _f32(m.val)
        return (rp, col, val), [_p(rp, _I32P), _p(col, _I32P), _p(val, _F32P)]

    def _csr_binary(self, fn, a: CSR, b: CSR, cap: int, threads: int) -> CSR:
        assert a.rows == b.rows
        ka, pa = self._csr_args(a)
        kb, pb = self._csr_args(b)
        rp = np.empty(a.rows + 1, np.int32)
        col = np.empty(max(cap, 1), np.int32)
        val = np.empty(max(cap, 1), np.float32)
        n = fn(a.rows, *pa, *pb, _p(rp, _I32P), _p(col, _I32P), _p(val, _F32P), threads)
        assert n >= 0
        del ka, kb
        return CSR(a.rows, a.cols, rp, col[:n].copy(), val[:n].copy())

    def csr_add(self, a: CSR, b: CSR, threads: int = 1) -> CSR:
        return self._csr_binary(self.lib.orc_csr_add, a, b, len(a.col) + len(b.col), threads)

    def csr_mul(self, a: CSR, b: CSR, threads: int = 1) -> CSR:
        return self._csr_binary(self.lib.orc_csr_mul, a, b, min(len(a.col), len(b.col)), threads)

    def csr_add_3(self, a: CSR, b: CSR, c: CSR, threads: int = 1) -> CSR:
        ka, pa = self._csr_args(a)
        kb, pb = self._csr_args(b)
        kc, pc = self._csr_args(c)
        cap = max(len(a.col) + len(b.col) + len(c.col), 1)
        rp = np.empty(a.rows + 1, np.int32)
        col = np.empty(cap, np.int32)
        val = np.empty(cap, np.float32)
        n = self.lib.orc_csr_add3(a.rows, *pa, *pb, *pc, _p(rp, _I32P), _p(col, _I32P),
                                  _p(val, _F32P), threads)
        del ka, kb, kc
        return CSR(a.rows, a.cols, rp, col[:n].copy(), val[:n].copy())

    def coo3_add(self, a: COO3, b: COO3, threads: int = 1) -> COO3:
        arrs_a = [_i32(a.i), _i32(a.j), _i32(a.k), _f32(a.val)]
        arrs_b = [_i32(b.i), _i32(b.j), _i32(b.k), _f32(b.val)]
        cap = max(len(a.val) + len(b.val), 1)
        zi, zj, zk = (np.empty(cap, np.int32) for _ in range(3))
        zv = np.empty(cap, np.float32)

        def ptrs(arrs):
            return [_p(arrs[0], _I32P), _p(arrs[1], _I32P), _p(arrs[2], _I32P), _p(arrs[3], _F32P)]

        n = self.lib.orc_coo3_add(len(a.val), *ptrs(arrs_a), len(b.val), *ptrs(arrs_b),
                                  _p(zi, _I32P), _p(zj, _I32P), _p(zk, _I32P), _p(zv, _F32P), threads)
        return COO3(tuple(a.dims), zi[:n].copy(), zj[:n].copy(), zk[:n].copy(), zv[:n].copy())

    def csf3_add(self, a: CSF3, b: CSF3) -> CSF3:
        def prep(t):
            arrs = [_i32(t.i_idx), _i32(t.j_ptr), _i32(t.j_idx), _i32(t.k_ptr), _i32(t.k_idx), _f32(t.val)]
            return arrs, [_p(x, _I32P) for x in arrs[:5]] + [_p(arrs[5], _F32P)]

        ka, pa = prep(a)
        kb, pb = prep(b)
        ni, nj, nk = (len(a.i_idx) + len(b.i_idx), len(a.j_idx) + len(b.j_idx), len(a.k_idx) + len(b.k_idx))
        zi = np.empty(max(ni, 1), np.int32)
        zjp = np.empty(ni + 1, np.int32)
        zj = np.empty(max(nj, 1), np.int32)
        zkp = np.empty(nj + 1, np.int32)
        zk = np.empty(max(nk, 1), np.int32)
        zv = np.empty(max(nk, 1), np.float32)
        counts = np.zeros(3, np.int32)
        self.lib.orc_csf3_add(len(a.i_idx), *pa, len(b.i_idx), *pb, _p(zi, _I32P), _p(zjp, _I32P),
                              _p(zj, _I32P), _p(zkp, _I32P), _p(zk, _I32P), _p(zv, _F32P),
                              _p(counts, _I32P))
        ci, cj, ck = (int(x) for x in counts)
        del ka, kb
        return CSF3(tuple(a.dims), zi[:ci].copy(), zjp[:ci + 1].copy(), zj[:cj].copy(),
                    zkp[:cj + 1].copy(), zk[:ck].copy(), zv[:ck].copy())

    def spgemm(self, a: CSR, b: CSR, threads: int = 1, extras: bool = False):
        """C = A @ B. Returns CSR, or (CSR, val64, abs64, products) when ``extras``."""
        assert a.cols == b.rows
        ka, pa = self._csr_args(a)
        kb, pb = self._csr_args(b)
        rp = np.empty(a.rows + 1, np.int32)
        products = C.c_int64(0)
        n = self.lib.orc_spgemm_symbolic(a.rows, b.cols, pa[0], pa[1], pb[0], pb[1], _p(rp, _I32P),
                                         C.byref(products), threads)
        col = np.empty(max(n, 1), np.int32)
        val = np.empty(max(n, 1), np.float32)
        v64 = np.empty(max(n, 1), np.float64) if extras else None
        a64 = np.empty(max(n, 1), np.float64) if extras else None
        self.lib.orc_spgemm_numeric(a.rows, b.cols, *pa, *pb, _p(rp, _I32P), _p(col, _I32P),
                                    _p(val, _F32P), _p(v64, _F64P) if extras else None,
                                    _p(a64, _F64P) if extras else None, threads)
        del ka, kb
        out = CSR(a.rows, b.cols, rp, col[:n].copy(), val[:n].copy())
        if extras:
            return out, v64[:n].copy(), a64[:n].copy(), int(products.value)
        return out


class _RefCSR(C.Structure):
    _fields_ = [("rows", C.c_int32), ("cols", C.c_int32), ("nnz", C.c_int32),
                ("row_ptr", _I32P), ("col", _I32P), ("val", _F32P)]


class _RefCOO3(C.Structure):
    _fields_ = [("dims", C.c_int32 * 3), ("nnz", C.c_int32),
                ("i", _I32P), ("j", _I32P), ("k", _I32P), ("val", _F32P)]


class _RefCSF3(C.Structure):
    _fields_ = [("dims", C.c_int32 * 3), ("n_i", C.c_int32), ("n_j", C.c_int32), ("n_k", C.c_int32),
                ("i_idx", _I32P), ("j_ptr", _I32P), ("j_idx", _I32P), ("k_ptr", _I32P),
                ("k_idx", _I32P), ("val", _F32P)]


class _RefCOO(C.Structure):
    _fields_ = [("rows", C.c_int32), ("cols", C.c_int32), ("nnz", C.c_int32),
                ("i", _I32P), ("j", _I32P), ("val", _F32P)]


class _RefDCSR(C.Structure):
    _fields_ = [("rows", C.c_int32), ("cols", C.c_int32), ("n_i", C.c_int32), ("nnz", C.c_int32),
                ("i_idx", _I32P), ("j_ptr", _I32P), ("j_idx", _I32P), ("val", _F32P)]


def _take(ptr, n, dtype):
    if n <= 0 or not ptr:
        return np.empty(0, dtype)
    return np.ctypeslib.as_array(ptr, shape=(n,)).astype(dtype, copy=True)


class Reference:
    """The reference's own emitted CPU kernels (``ref_shim/ref_abi.h``)."""

    def __init__(self, path: str = REF_SO):
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} missing: run `make -C oracle ref` where the reference checkout is present")
        self.lib = C.CDLL(path)
        L = self.lib
        L.ref_threads.restype = C.c_int
        L.ref_free.argtypes = [C.c_void_p]
        P = C.POINTER
        L.ref_csr_add.argtypes = [P(_RefCSR)] * 3
        L.ref_csr_mul.argtypes = [P(_RefCSR)] * 3
        L.ref_csr_add_3.argtypes = [P(_RefCSR)] * 4
        L.ref_coo3d_add.argtypes = [P(_RefCOO3)] * 3
        L.ref_csf_add.argtypes = [P(_RefCSF3)] * 3
        if hasattr(L, "ref_coo_add"):  # the element-wise family beyond the five benchmarked kernels
            L.ref_coo_add.argtypes = [P(_RefCOO)] * 3
            L.ref_coo_mul.argtypes = [P(_RefCOO)] * 3
            L.ref_coo_csr_add.argtypes = [P(_RefCSR), P(_RefCOO), P(_RefCSR)]
            L.ref_dcsr_add.argtypes = [P(_RefDCSR)] * 3
            L.ref_dcsr_mul.argtypes = [P(_RefDCSR)] * 3
            L.ref_inner_prod.argtypes = [P(_RefCSF3)] * 2
            L.ref_inner_prod.restype = C.c_float
            L.ref_inner_prod_coo.argtypes = [P(_RefCOO3)] * 2
            L.ref_inner_prod_coo.restype = C.c_float

    @staticmethod
    def available(path: str = REF_SO) -> bool:
        return os.path.exists(path)

    def threads(self) -> int:
        return int(self.lib.ref_threads())

    def _free(self, *ptrs):
        for p in ptrs:
            if p:
                self.lib.ref_free(C.cast(p, C.c_void_p))

    @staticmethod
    def _csr_in(m: CSR):
        rp, col, val = _i32(m.row_ptr), _i32(m.col), _f32(m.val)
        s = _RefCSR(m.rows, m.cols, len(col), _p(rp, _I32P), _p(col, _I32P), _p(val, _F32P))
        return s, (rp, col, val)

    def _csr_out(self, z: _RefCSR, keep: bool = True) -> CSR:
        out = CSR(z.rows, z.cols, _take(z.row_ptr, z.rows + 1, np.int32), _take(z.col, z.nnz, np.int32),
                  _take(z.val, z.nnz, np.float32)) if keep else None
        self._free(z.row_ptr, z.col, z.val)
        return out

    def csr_add(self, a: CSR, b: CSR, keep: bool = True) -> CSR:
        sa, ka = self._csr_in(a)
        sb, kb = self._csr_in(b)
        z = _RefCSR()
        self.lib.ref_csr_add(C.byref(sa), C.byref(sb), C.byref(z))
        return self._csr_out(z, keep)

    def csr_mul(self, a: CSR, b: CSR, keep: bool = True) -> CSR:
        sa, ka = self._csr_in(a)
        sb, kb = self._csr_in(b)
        z = _RefCSR()
        self.lib.ref_csr_mul(C.byref(sa), C.byref(sb), C.byref(z))
        return self._csr_out(z, keep)

    def csr_add_3(self, a: CSR, b: CSR, c: CSR, keep: bool = True) -> CSR:
        sa, ka = self._csr_in(a)
        sb, kb = self._csr_in(b)
        sc, kc = self._csr_in(c)
        z = _RefCSR()
        self.lib.ref_csr_add_3(C.byref(sa), C.byref(sb), C.byref(sc), C.byref(z))
        return self._csr_out(z, keep)

    def coo3_add(self, a: COO3, b: COO3, keep: bool = True) -> COO3:
        def mk(t):
            arrs = (_i32(t.i), _i32(t.j), _i32(t.k), _f32(t.val))
            s = _RefCOO3((C.c_int32 * 3)(*t.dims), len(arrs[3]), _p(arrs[0], _I32P), _p(arrs[1], _I32P),
                         _p(arrs[2], _I32P), _p(arrs[3], _F32P))
            return s, arrs

        sa, ka = mk(a)
        sb, kb = mk(b)
        z = _RefCOO3()
        self.lib.ref_coo3d_add(C.byref(sa), C.byref(sb), C.byref(z))
        out = COO3(tuple(z.dims), _take(z.i, z.nnz, np.int32), _take(z.j, z.nnz, np.int32),
                   _take(z.k, z.nnz, np.int32), _take(z.val, z.nnz, np.float32)) if keep else None
        self._free(z.i, z.j, z.k, z.val)
        return out

    def csf3_add(self, a: CSF3, b: CSF3, keep: bool = True) -> CSF3:
        def mk(t):
            arrs = (_i32(t.i_idx), _i32(t.j_ptr), _i32(t.j_idx), _i32(t.k_ptr), _i32(t.k_idx), _f32(t.val))
            s = _RefCSF3((C.c_int32 * 3)(*t.dims), len(arrs[0]), len(arrs[2]), len(arrs[4]),
                         *[_p(x, _I32P) for x in arrs[:5]], _p(arrs[5], _F32P))
            return s, arrs

        sa, ka = mk(a)
        sb, kb = mk(b)
        z = _RefCSF3()
        self.lib.ref_csf_add(C.byref(sa), C.byref(sb), C.byref(z))
        out = CSF3(tuple(z.dims), _take(z.i_idx, z.n_i, np.int32), _take(z.j_ptr, z.n_i + 1, np.int32),
                   _take(z.j_idx, z.n_j, np.int32), _take(z.k_ptr, z.n_j + 1, np.int32),
                   _take(z.k_idx, z.n_k, np.int32), _take(z.val, z.n_k, np.float32)) if keep else None
        self._free(z.i_idx, z.j_ptr, z.j_idx, z.k_ptr, z.k_idx, z.val)
        return out

    # ---- the rest of the element-wise family (2-D COO, DCSR, inner products) ----

    @staticmethod
    def _coo_in(m: COO):
        arrs = (_i32(m.i), _i32(m.j), _f32(m.val))
        return _RefCOO(m.rows, m.cols, len(arrs[2]), _p(arrs[0], _I32P), _p(arrs[1], _I32P), _p(arrs[2], _F32P)), arrs

    def _coo_binary(self, fn, a: COO, b: COO) -> COO:
        sa, ka = self._coo_in(a)
        sb, kb = self._coo_in(b)
        z = _RefCOO()
        fn(C.byref(sa), C.byref(sb), C.byref(z))
        out = COO(z.rows, z.cols, _take(z.i, z.nnz, np.int32), _take(z.j, z.nnz, np.int32), _take(z.val, z.nnz, np.float32))
        self._free(z.i, z.j, z.val)
        return out

    def coo_add(self, a: COO, b: COO) -> COO:
        return self._coo_binary(self.lib.ref_coo_add, a, b)

    def coo_mul(self, a: COO, b: COO) -> COO:
        return self._coo_binary(self.lib.ref_coo_mul, a, b)

    def coo_csr_add(self, a: CSR, b: COO) -> CSR:
        sa, ka = self._csr_in(a)
        sb, kb = self._coo_in(b)
        z = _RefCSR()
        self.lib.ref_coo_csr_add(C.byref(sa), C.byref(sb), C.byref(z))
        return self._csr_out(z)

    @staticmethod
    def _dcsr_in(m: DCSR):
        arrs = (_i32(m.i_idx), _i32(m.j_ptr), _i32(m.j_idx), _f32(m.val))
        s = _RefDCSR(m.rows, m.cols, len(arrs[0]), len(arrs[3]), _p(arrs[0], _I32P), _p(arrs[1], _I32P),
                     _p(arrs[2], _I32P), _p(arrs[3], _F32P))
        return s, arrs

    def _dcsr_binary(self, fn, a: DCSR, b: DCSR) -> DCSR:
        sa, ka = self._dcsr_in(a)
        sb, kb = self._dcsr_in(b)
        z = _RefDCSR()
        fn(C.byref(sa), C.byref(sb), C.byref(z))
        out = DCSR(z.rows, z.cols, _take(z.i_idx, z.n_i, np.int32), _take(z.j_ptr, z.n_i + 1, np.int32),
                   _take(z.j_idx, z.nnz, np.int32), _take(z.val, z.nnz, np.float32))
        self._free(z.i_idx, z.j_ptr, z.j_idx, z.val)
        return out

    def dcsr_add(self, a: DCSR, b: DCSR) -> DCSR:
        return self._dcsr_binary(self.lib.ref_dcsr_add, a, b)

    def dcsr_mul(self, a: DCSR, b: DCSR) -> DCSR:
        return self._dcsr_binary(self.lib.ref_dcsr_mul, a, b)

    def inner_prod(self, a: CSF3, b: CSF3) -> float:
        def mk(t):
            arrs = (_i32(t.i_idx), _i32(t.j_ptr), _i32(t.j_idx), _i32(t.k_ptr), _i32(t.k_idx), _f32(t.val))
            s = _RefCSF3((C.c_int32 * 3)(*t.dims), len(arrs[0]), len(arrs[2]), len(arrs[4]),
                         *[_p(x, _I32P) for x in arrs[:5]], _p(arrs[5], _F32P))
            return s, arrs
        sa, ka = mk(a)
        sb, kb = mk(b)
        return float(self.lib.ref_inner_prod(C.byref(sa), C.byref(sb)))

    def inner_prod_coo(self, a: COO3, b: COO3) -> float:
        def mk(t):
            arrs = (_i32(t.i), _i32(t.j), _i32(t.k), _f32(t.val))
            s = _RefCOO3((C.c_int32 * 3)(*t.dims), len(arrs[3]), _p(arrs[0], _I32P), _p(arrs[1], _I32P),
                         _p(arrs[2], _I32P), _p(arrs[3], _F32P))
            return s, arrs
        sa, ka = mk(a)
        sb, kb = mk(b)
        return float(self.lib.ref_inner_prod_coo(C.byref(sa), C.byref(sb)))


def csr_to_dcsr(m: CSR) -> DCSR:
    """Drops the empty rows of a CSR matrix (what the reference's to_dcsr does,
    python/nacho/convert.py:34-56)."""
    lens = np.diff(np.asarray(m.row_ptr, np.int64))
    present = np.flatnonzero(lens > 0)
    ptr = np.zeros(len(present) + 1, np.int32)
    ptr[1:] = np.cumsum(lens[present])
    return DCSR(m.rows, m.cols, present.astype(np.int32), ptr, np.asarray(m.col, np.int32), np.asarray(m.val, np.float32))


def csr_to_coo(m: CSR) -> COO:
    lens = np.diff(np.asarray(m.row_ptr, np.int64))
    return COO(m.rows, m.cols, np.repeat(np.arange(m.rows, dtype=np.int32), lens), np.asarray(m.col, np.int32),
               np.asarray(m.val, np.float32))
