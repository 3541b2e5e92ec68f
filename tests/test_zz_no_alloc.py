"""GPU suite, collected last: the entry point that allocates nothing.

nb200_csr_add_f32_noalloc serves callers that cannot allocate while they run (allocator
callbacks, fixed-budget plug-ins, latency-critical loops); its kernel scratch is a fixed array
inside the library. Called through the C ABI twice in a row -- the second call reuses the
array the first one dirtied -- and compared bit-for-bit with nb200_csr_add_f32_into.
"""
import ctypes as C

import numpy as np
import pytest

from helpers import assert_same, golden_csr, csr_to_gpu, synth_to_gpu
from oracle.cpu_oracle import CSR

pytestmark = pytest.mark.gpu


def _run(fn, ga, gb, capacity):
    import torch
    from nacho_b200._capi import CsrStruct
    sa, sb = ga._struct(), gb._struct()
    rp = torch.empty(sa.rows + 1, dtype=torch.int32, device="cuda")
    col = torch.full((max(capacity, 1),), -7, dtype=torch.int32, device="cuda")
    val = torch.full((max(capacity, 1),), float("nan"), dtype=torch.float32, device="cuda")
    z = CsrStruct(sa.rows, sa.cols, 0, rp.data_ptr(), col.data_ptr(), val.data_ptr())
    status = fn(C.byref(sa), C.byref(sb), C.byref(z), capacity, None)
    torch.cuda.synchronize()
    n = int(z.nnz)
    return status, CSR(sa.rows, sa.cols, rp.cpu().numpy(), col[:n].cpu().numpy(), val[:n].cpu().numpy())


def test_noalloc_matches_existing_entry_point_twice(csr_golden):
    import torch
    assert torch.cuda.is_available()
    from nacho_b200 import synth
    from nacho_b200._capi import OK, lib
    # a multi-tile seeded pair first, then a small golden case: the second call runs on scratch
    # the first call left behind, with fewer tiles than before
    ta, tb = synth.random_csr(3000, 20000, 0.004, 31), synth.random_csr(3000, 20000, 0.004, 32)
    big = (synth_to_gpu(ta), synth_to_gpu(tb))
    small = (csr_to_gpu(golden_csr(csr_golden, "medium", "a")), csr_to_gpu(golden_csr(csr_golden, "medium", "b")))
    for round_no in range(2):
        for ga, gb in (big, small):
            cap = ga.values.numel() + gb.values.numel()
            st_ref, want = _run(lib.nb200_csr_add_f32_into, ga, gb, cap)
            st_new, got = _run(lib.nb200_csr_add_f32_noalloc, ga, gb, cap)
            assert st_ref == OK and st_new == OK
            assert_same(got, want, f"noalloc vs into (round {round_no})")
    assert_same(_run(lib.nb200_csr_add_f32_noalloc, *small, small[0].values.numel() + small[1].values.numel())[1],
                golden_csr(csr_golden, "medium", "add"), "noalloc vs golden")


def test_noalloc_limits(csr_golden):
    import torch
    from nacho_b200 import _capi
    from nacho_b200._capi import CsrStruct, lib
    ga = csr_to_gpu(golden_csr(csr_golden, "smoke", "a"))
    gb = csr_to_gpu(golden_csr(csr_golden, "smoke", "b"))
    status, _ = _run(lib.nb200_csr_add_f32_noalloc, ga, gb, 10)  # below nnz(A) + nnz(B)
    assert status == _capi.E_CAPACITY
    # an operand pair beyond the fixed scratch is refused before anything is launched
    sa, sb = ga._struct(), gb._struct()
    sa.nnz = 2_000_000_000
    z = CsrStruct(sa.rows, sa.cols, 0, ga.dim_j_offsets.data_ptr(), ga.dim_j_indices.data_ptr(), ga.values.data_ptr())
    assert lib.nb200_csr_add_f32_noalloc(C.byref(sa), C.byref(sb), C.byref(z), 1 << 40, None) == _capi.E_UNSUPPORTED
    empty = csr_to_gpu(golden_csr(csr_golden, "all_empty", "a"))
    status, got = _run(lib.nb200_csr_add_f32_noalloc, empty, empty, 0)
    assert status == _capi.OK and len(got.col) == 0 and not got.row_ptr.any()
