"""ctypes binding of ``libnacho_b200.so`` (the C ABI declared in ``include/nacho_b200.h``).

The library is the product's only compute path: if it is missing or fails to load, importing
this module raises. There is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# NACHO_B200_LIB selects another build of the same library (e.g. a tuning variant).
LIB_PATH = os.environ.get("NACHO_B200_LIB") or os.path.join(HERE, "libnacho_b200.so")

_I32P = C.POINTER(C.c_int32)
_F32P = C.POINTER(C.c_float)


class CsrStruct(C.Structure):
    """``nb200_csr``."""
    _fields_ = [("rows", C.c_int32), ("cols", C.c_int32), ("nnz", C.c_int32),
                ("row_ptr", C.c_void_p), ("col", C.c_void_p), ("val", C.c_void_p)]


class Coo3Struct(C.Structure):
    """``nb200_coo3``."""
    _fields_ = [("dims", C.c_int32 * 3), ("nnz", C.c_int32),
                ("i", C.c_void_p), ("j", C.c_void_p), ("k", C.c_void_p), ("val", C.c_void_p)]


class Csf3Struct(C.Structure):
    """``nb200_csf3``."""
    _fields_ = [("dims", C.c_int32 * 3), ("n_i", C.c_int32), ("n_j", C.c_int32), ("n_k", C.c_int32),
                ("i_idx", C.c_void_p), ("j_ptr", C.c_void_p), ("j_idx", C.c_void_p),
                ("k_ptr", C.c_void_p), ("k_idx", C.c_void_p), ("val", C.c_void_p)]


class CooStruct(C.Structure):
    """``nb200_coo``."""
    _fields_ = [("rows", C.c_int32), ("cols", C.c_int32), ("nnz", C.c_int32),
                ("i", C.c_void_p), ("j", C.c_void_p), ("val", C.c_void_p)]


class DcsrStruct(C.Structure):
    """``nb200_dcsr``."""
    _fields_ = [("rows", C.c_int32), ("cols", C.c_int32), ("n_i", C.c_int32), ("nnz", C.c_int32),
                ("i_idx", C.c_void_p), ("j_ptr", C.c_void_p), ("j_idx", C.c_void_p), ("val", C.c_void_p)]


OK, E_BADARG, E_CUDA, E_OVERFLOW, E_CAPACITY, E_TIMEOUT, E_NOMEM, E_UNSUPPORTED = range(8)

# name -> (restype, argtypes); every symbol include/nacho_b200.h declares.
_P = C.POINTER
PROTOTYPES = {
    "nb200_version": (C.c_int, []),
    "nb200_strerror": (C.c_char_p, [C.c_int]),
    "nb200_last_cuda_error": (C.c_char_p, []),
    "nb200_free_async": (C.c_int, [C.c_void_p, C.c_void_p]),
    "nb200_release_workspaces": (C.c_int, []),
    "nb200_launch_count": (C.c_uint64, []),
    "nb200_profile_enable": (C.c_int, [C.c_int]),
    "nb200_profile_reset": (C.c_int, []),
    "nb200_profile_read": (C.c_int, [C.c_char_p, _P(C.c_int64), _P(C.c_double)]),
    "nb200_profile_names": (C.c_int, [C.c_char_p, C.c_size_t]),
    "nb200_csr_add_f32": (C.c_int, [_P(CsrStruct)] * 3 + [C.c_int32, C.c_int32, C.c_void_p]),
    "nb200_csr_add_f32_into": (C.c_int, [_P(CsrStruct)] * 3 + [C.c_int64, C.c_void_p]),
    "nb200_csr_add_f32_noalloc": (C.c_int, [_P(CsrStruct)] * 3 + [C.c_int64, C.c_void_p]),
    "nb200_csr_add_f32_async": (C.c_int, [_P(CsrStruct)] * 3 + [C.c_int64, C.c_void_p, C.c_void_p]),
    "nb200_csr_mul_f32_async": (C.c_int, [_P(CsrStruct)] * 3 + [C.c_int64, C.c_void_p, C.c_void_p]),
    "nb200_selftest_lookback_timeout": (C.c_int, [_P(CsrStruct)] * 3 + [C.c_int64, C.c_int32, C.c_void_p]),
    "nb200_csr_mul_f32": (C.c_int, [_P(CsrStruct)] * 3 + [C.c_int32, C.c_int32, C.c_void_p]),
    "nb200_csr_mul_f32_into": (C.c_int, [_P(CsrStruct)] * 3 + [C.c_int64, C.c_void_p]),
    "nb200_csr_add_f32_host": (C.c_int, [_P(CsrStruct)] * 3 + [C.c_int64]),
    "nb200_csr_mul_f32_host": (C.c_int, [_P(CsrStruct)] * 3 + [C.c_int64]),
    "nb200_csr_add_3_f32": (C.c_int, [_P(CsrStruct)] * 4 + [C.c_int32, C.c_int32, C.c_void_p]),
    "nb200_csr_add_3_f32_into": (C.c_int, [_P(CsrStruct)] * 4 + [C.c_int64, C.c_void_p]),
    "nb200_spgemm_f32": (C.c_int, [_P(CsrStruct)] * 3 + [C.c_int32, C.c_int32, C.c_void_p]),
    "nb200_sssmm_f32_into": (C.c_int, [_P(CsrStruct)] * 4 + [C.c_int64, C.c_void_p]),
    "nb200_spgemm_f32_symbolic": (C.c_int, [_P(CsrStruct)] * 3 + [_P(C.c_int64), C.c_void_p]),
    "nb200_spgemm_f32_numeric": (C.c_int, [_P(CsrStruct)] * 3 + [C.c_void_p]),
    "nb200_coo3d_add_f32": (C.c_int, [_P(Coo3Struct)] * 3 + [C.c_int32, C.c_int32, C.c_void_p]),
    "nb200_coo3d_add_f32_into": (C.c_int, [_P(Coo3Struct)] * 3 + [C.c_int64, C.c_void_p]),
    "nb200_csf_add_f32": (C.c_int, [_P(Csf3Struct)] * 3 + [C.c_int32, C.c_int32, C.c_void_p]),
    "nb200_csf_add_f32_into": (C.c_int, [_P(Csf3Struct)] * 3 + [C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "nb200_coo_add_f32_into": (C.c_int, [_P(CooStruct)] * 3 + [C.c_int64, C.c_void_p]),
    "nb200_coo_mul_f32_into": (C.c_int, [_P(CooStruct)] * 3 + [C.c_int64, C.c_void_p]),
    "nb200_coo_csr_add_f32_into": (C.c_int, [_P(CsrStruct), _P(CooStruct), _P(CsrStruct), C.c_int64, C.c_void_p]),
    "nb200_dcsr_add_f32_into": (C.c_int, [_P(DcsrStruct)] * 3 + [C.c_int64, C.c_int64, C.c_void_p]),
    "nb200_dcsr_mul_f32_into": (C.c_int, [_P(DcsrStruct)] * 3 + [C.c_int64, C.c_int64, C.c_void_p]),
    "nb200_inner_prod_f32": (C.c_int, [_P(Csf3Struct)] * 2 + [C.c_void_p, C.c_void_p]),
    "nb200_inner_prod_coo_f32": (C.c_int, [_P(Coo3Struct)] * 2 + [C.c_void_p, C.c_void_p]),
}


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m nacho_b200.build` (needs nvcc). "
            "nacho_b200 has no fallback path.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class NachoB200Error(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        text = lib.nb200_strerror(status).decode()
        if status in (E_CUDA, E_TIMEOUT):
            text += " (" + lib.nb200_last_cuda_error().decode() + ")"
        super().__init__(f"{where}: {text} [status {status}]")


def check(status: int, where: str) -> None:
    """Raises on a non-zero status: MemoryError for allocation failures, RuntimeError otherwise
    (the two exception types the reference's benchmarks catch, benchmarks/spgemm.py:31-34)."""
    if status == OK:
        return
    if status == E_NOMEM:
        raise MemoryError(f"{where}: device allocation failed")
    raise NachoB200Error(status, where)


def launch_count() -> int:
    return int(lib.nb200_launch_count())


def profile_enable(on: bool) -> None:
    check(lib.nb200_profile_enable(1 if on else 0), "nb200_profile_enable")


def profile_reset() -> None:
    check(lib.nb200_profile_reset(), "nb200_profile_reset")


def profile_names() -> list[str]:
    buf = C.create_string_buffer(4096)
    check(lib.nb200_profile_names(buf, 4096), "nb200_profile_names")
    return [s for s in buf.value.decode().split(",") if s]


def profile_read(name: str) -> tuple[int, float]:
    n = C.c_int64(0)
    ms = C.c_double(0.0)
    check(lib.nb200_profile_read(name.encode(), C.byref(n), C.byref(ms)), "nb200_profile_read")
    return int(n.value), float(ms.value)
