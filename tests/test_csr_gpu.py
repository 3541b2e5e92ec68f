"""GPU suite: the CUDA CSR add / multiply paths, called through the C ABI, against the golden
vectors made by the reference's CPU kernels, against the C oracle on seeded inputs, and -- at
the benchmark's full sizes -- through properties that need no CPU run."""
import ctypes as C

import numpy as np
import pytest

from helpers import (CSR_CASES, assert_same, csr_from_gpu, csr_to_gpu, golden_csr, synth_csr, synth_to_gpu)
from oracle.cpu_oracle import CSR

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nacho():
    import torch
    assert torch.cuda.is_available(), "GPU suite needs a CUDA device"
    from nacho_b200 import nacho as mod
    return mod


@pytest.mark.parametrize("case", CSR_CASES)
def test_golden_add_mul(nacho, csr_golden, case):
    a, b = golden_csr(csr_golden, case, "a"), golden_csr(csr_golden, case, "b")
    ga, gb = csr_to_gpu(a), csr_to_gpu(b)
    assert_same(csr_from_gpu(nacho.gpu_csr_add_f32(ga, gb)), golden_csr(csr_golden, case, "add"), f"{case} add")
    assert_same(csr_from_gpu(nacho.gpu_csr_mul_f32(ga, gb)), golden_csr(csr_golden, case, "mul"), f"{case} mul")
    gc = csr_to_gpu(golden_csr(csr_golden, case, "c"))
    assert_same(csr_from_gpu(nacho.gpu_csr_add_3_f32(ga, gb, gc)), golden_csr(csr_golden, case, "add3"), f"{case} add3")
    # the two launch-shape arguments of the reference signature are accepted
    z = nacho.gpu_csr_add_f32(ga, gb, num_blocks=64, threads_per_block=128)
    assert_same(csr_from_gpu(z), golden_csr(csr_golden, case, "add"), f"{case} add (grid args)")


SEEDED = [
    # rows, cols, density, seed
    (200, 180, 0.05, 11), (1, 4000, 0.6, 12), (5000, 64, 0.2, 13), (3000, 100000, 0.0005, 14),
    (100000, 50, 0.01, 15), (257, 2815, 0.5, 16), (40, 1 << 22, 0.0005, 17),
]


@pytest.mark.parametrize("rows,cols,density,seed", SEEDED)
def test_seeded_vs_oracle(nacho, oracle, rows, cols, density, seed):
    from nacho_b200 import synth
    ta, tb = synth.random_csr(rows, cols, density, seed), synth.random_csr(rows, cols, density, seed + 500)
    a, b = synth_csr(ta), synth_csr(tb)
    ga, gb = synth_to_gpu(ta), synth_to_gpu(tb)
    assert_same(csr_from_gpu(nacho.gpu_csr_add_f32(ga, gb)), oracle.csr_add(a, b, 8), "add")
    assert_same(csr_from_gpu(nacho.gpu_csr_mul_f32(ga, gb)), oracle.csr_mul(a, b, 8), "mul")
    tc = synth.random_csr(rows, cols, density, seed + 900)
    assert_same(csr_from_gpu(nacho.gpu_csr_add_3_f32(ga, gb, synth_to_gpu(tc))), oracle.csr_add_3(a, b, synth_csr(tc), 8), "add3")


def test_config1_vs_oracle(nacho, oracle):
    from nacho_b200 import synth
    ta, tb = synth.c1_csr(0), synth.c1_csr(1)
    assert_same(csr_from_gpu(nacho.gpu_csr_add_f32(synth_to_gpu(ta), synth_to_gpu(tb))),
                oracle.csr_add(synth_csr(ta), synth_csr(tb), 8), "config 1")


def test_config2_small_vs_oracle(nacho, oracle):
    from nacho_b200 import synth
    ta, tb = synth.c2_pair(rows=1 << 15, cols=1 << 20, seed=2100)
    assert_same(csr_from_gpu(nacho.gpu_csr_mul_f32(synth_to_gpu(ta), synth_to_gpu(tb))),
                oracle.csr_mul(synth_csr(ta), synth_csr(tb), 8), "config 2 (2^15 rows)")


@pytest.mark.parametrize("sigma", [0, 2, 3])
def test_config3_small_vs_oracle(nacho, oracle, sigma):
    from nacho_b200 import synth
    ta = synth.c3_csr(0, sigma, rows=1 << 14, cols=1 << 20, nnz=1 << 20)
    tb = synth.c3_csr(1, sigma, rows=1 << 14, cols=1 << 20, nnz=1 << 20)
    assert_same(csr_from_gpu(nacho.gpu_csr_add_f32(synth_to_gpu(ta), synth_to_gpu(tb))),
                oracle.csr_add(synth_csr(ta), synth_csr(tb), 8), f"config 3 sigma={sigma}")
    tc = synth.c3_csr(2, sigma, rows=1 << 14, cols=1 << 20, nnz=1 << 20)
    assert_same(csr_from_gpu(nacho.gpu_csr_add_3_f32(synth_to_gpu(ta), synth_to_gpu(tb), synth_to_gpu(tc))),
                oracle.csr_add_3(synth_csr(ta), synth_csr(tb), synth_csr(tc), 8), f"config 3 add3 sigma={sigma}")


def test_long_runs_of_empty_rows(nacho, oracle):
    """Tiles spanning far more rows than a 32-bit composite key can number (wide-key path)."""
    rng = np.random.default_rng(5)
    rows, cols = 3_000_000, 1 << 20
    def make(seed):
        r = np.random.default_rng(seed)
        lengths = np.zeros(rows, np.int64)
        hot = r.choice(rows, 3000, replace=False)
        lengths[hot] = r.integers(1, 6, 3000)
        rp = np.zeros(rows + 1, np.int32)
        rp[1:] = np.cumsum(lengths)
        n = int(rp[-1])
        col = np.concatenate([np.sort(r.choice(cols, int(k), replace=False)) for k in lengths[np.sort(hot)]]).astype(np.int32)
        return CSR(rows, cols, rp, col, r.uniform(-1, 1, n).astype(np.float32))
    a, b = make(1), make(2)
    b = CSR(rows, cols, b.row_ptr, b.col, b.val)
    ga, gb = csr_to_gpu(a), csr_to_gpu(b)
    assert_same(csr_from_gpu(nacho.gpu_csr_add_f32(ga, gb)), oracle.csr_add(a, b, 8), "empty runs add")
    assert_same(csr_from_gpu(nacho.gpu_csr_mul_f32(ga, ga)), oracle.csr_mul(a, a, 8), "empty runs mul")
    # the fused three-operand kernel has no wide-key body: it reports the tile and the call reruns
    # on the chained two-operand route
    c = make(3)
    assert_same(csr_from_gpu(nacho.gpu_csr_add_3_f32(ga, gb, csr_to_gpu(c))), oracle.csr_add_3(a, b, c, 8), "empty runs add3")


def test_full_size_properties(nacho):
    """Config 3 at full size (2^20 rows, 64 M entries per operand): properties of a sorted
    union / intersection that hold for any input, checked on the device."""
    import torch
    from nacho_b200 import synth
    ta = synth.c3_csr(0, 1, device="cuda")
    tb = synth.c3_csr(1, 1, device="cuda")
    a, b = synth_to_gpu(ta), synth_to_gpu(tb)
    z = nacho.gpu_csr_add_f32(a, b)
    m = nacho.gpu_csr_mul_f32(a, b)
    torch.cuda.synchronize()
    rows, cols = ta[0], ta[1]
    na, nb, nz, nm = a.values.numel(), b.values.numel(), z.values.numel(), m.values.numel()
    # inclusion-exclusion on the structure
    assert nz + nm == na + nb
    for t in (z, m):
        rp = t.dim_j_offsets.to(torch.int64)
        assert int(rp[0]) == 0 and int(rp[-1]) == t.values.numel()
        assert bool((rp[1:] >= rp[:-1]).all())
        row = torch.repeat_interleave(torch.arange(rows, device="cuda"), rp[1:] - rp[:-1])
        key = row * cols + t.dim_j_indices.to(torch.int64)
        assert bool((key[1:] > key[:-1]).all()), "columns not strictly increasing within rows"
        del row, key
    # per-row lengths: |A_i u B_i| + |A_i n B_i| = |A_i| + |B_i|
    d = lambda t: (t.dim_j_offsets[1:] - t.dim_j_offsets[:-1]).to(torch.int64)
    assert bool((d(z) + d(m) == d(a) + d(b)).all())
    # linearity of the value sum (float64 accumulation): sum(Z) = sum(A) + sum(B)
    s = lambda t: float(t.values.to(torch.float64).sum())
    assert abs(s(z) - (s(a) + s(b))) <= 1e-6 * (na + nb) ** 0.5 + 1e-3
    # idempotence of the structure: (A + B) + B keeps Z's pattern; A .* A keeps A's pattern
    z2 = nacho.gpu_csr_add_f32(z, b)
    assert torch.equal(z2.dim_j_offsets, z.dim_j_offsets) and torch.equal(z2.dim_j_indices, z.dim_j_indices)
    sq = nacho.gpu_csr_mul_f32(a, a)
    assert torch.equal(sq.dim_j_offsets, a.dim_j_offsets) and torch.equal(sq.dim_j_indices, a.dim_j_indices)
    assert torch.equal(sq.values, a.values * a.values)


def _d2h(ptr, count, dtype):
    import torch
    out = np.empty(count, dtype)
    if count:
        rt = C.CDLL("libcudart.so.12")
        rt.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
        assert rt.cudaMemcpy(out.ctypes.data, ptr, out.nbytes, 2) == 0
    return out


def test_allocating_entry_points(nacho, csr_golden):
    """nb200_csr_add_f32 / nb200_csr_mul_f32 allocate their own result arrays, which are then
    released one by one with nb200_free_async, as an adopting binding would."""
    import torch
    from nacho_b200._capi import CsrStruct, check, lib
    for case in ("smoke", "medium", "all_empty"):
        a, b = golden_csr(csr_golden, case, "a"), golden_csr(csr_golden, case, "b")
        ga, gb = csr_to_gpu(a), csr_to_gpu(b)
        for fn, tag in ((lib.nb200_csr_add_f32, "add"), (lib.nb200_csr_mul_f32, "mul")):
            z = CsrStruct()
            sa, sb = ga._struct(), gb._struct()
            check(fn(C.byref(sa), C.byref(sb), C.byref(z), 256, 256, None), tag)
            torch.cuda.synchronize()
            got = CSR(z.rows, z.cols, _d2h(z.row_ptr, z.rows + 1, np.int32), _d2h(z.col, z.nnz, np.int32),
                      _d2h(z.val, z.nnz, np.float32))
            assert_same(got, golden_csr(csr_golden, case, tag), f"{case} {tag} (allocating)")
            if z.nnz == 0:
                assert not z.col and not z.val
            for p in (z.row_ptr, z.col, z.val):
                check(lib.nb200_free_async(p, None), "free")


def test_allocating_add_3_entry_point(nacho, csr_golden):
    """nb200_csr_add_3_f32 allocates its own result arrays (freed one by one afterwards)."""
    import torch
    from nacho_b200._capi import CsrStruct, check, lib
    for case in ("smoke", "medium", "all_empty", "cancel"):
        ops = [csr_to_gpu(golden_csr(csr_golden, case, tag)) for tag in ("a", "b", "c")]
        structs = [g._struct() for g in ops]
        z = CsrStruct()
        check(lib.nb200_csr_add_3_f32(*[C.byref(x) for x in structs], C.byref(z), 256, 256, None), "add3")
        torch.cuda.synchronize()
        got = CSR(z.rows, z.cols, _d2h(z.row_ptr, z.rows + 1, np.int32), _d2h(z.col, z.nnz, np.int32),
                  _d2h(z.val, z.nnz, np.float32))
        assert_same(got, golden_csr(csr_golden, case, "add3"), f"{case} add3 (allocating)")
        if z.nnz == 0:
            assert not z.col and not z.val
        for p in (z.row_ptr, z.col, z.val):
            check(lib.nb200_free_async(p, None), "free")


def test_async_entry_points_leave_the_length_on_the_device(nacho, csr_golden):
    """nb200_csr_{add,mul}_f32_async return without waiting; length, status and row count arrive in three device words."""
    import torch
    from nacho_b200 import _capi
    from nacho_b200._capi import CsrStruct, check, lib
    for case in ("medium", "giant_row", "all_empty"):
        a, b = golden_csr(csr_golden, case, "a"), golden_csr(csr_golden, case, "b")
        ga, gb = csr_to_gpu(a), csr_to_gpu(b)
        for fn, tag, cap in ((lib.nb200_csr_add_f32_async, "add", len(a.col) + len(b.col)),
                             (lib.nb200_csr_mul_f32_async, "mul", min(len(a.col), len(b.col)))):
            want = golden_csr(csr_golden, case, tag)
            rp = torch.empty(a.rows + 1, dtype=torch.int32, device="cuda")
            col = torch.empty(max(cap, 1), dtype=torch.int32, device="cuda")
            val = torch.empty(max(cap, 1), dtype=torch.float32, device="cuda")
            res = torch.full((3,), -1, dtype=torch.int64, device="cuda")
            z = CsrStruct(a.rows, a.cols, 0, rp.data_ptr(), col.data_ptr(), val.data_ptr())
            sa, sb = ga._struct(), gb._struct()
            check(fn(C.byref(sa), C.byref(sb), C.byref(z), cap, res.data_ptr(), None), tag)
            n, status, rows = (int(x) for x in res.cpu())
            assert status == _capi.OK and n == len(want.col) and rows == a.rows
            got = CSR(a.rows, a.cols, rp.cpu().numpy(), col[:n].cpu().numpy(), val[:n].cpu().numpy())
            assert_same(got, want, f"{case} {tag} (async)")
            if cap > 0:  # a capacity below the worst case is refused: this form cannot count first
                assert fn(C.byref(sa), C.byref(sb), C.byref(z), cap - 1, res.data_ptr(), None) == _capi.E_CAPACITY


def test_bounded_wait_gives_up_and_reports(nacho, oracle):
    """The look-back of the single-pass kernel, made to wait for a tile that never runs: the wait
    ends after its poll limit, the call reports NB200_E_TIMEOUT, and the context keeps working."""
    import time
    import torch
    from nacho_b200 import _capi, synth
    from nacho_b200._capi import CsrStruct, lib
    ta, tb = synth.random_csr(4000, 30000, 0.004, 71), synth.random_csr(4000, 30000, 0.004, 72)
    ga, gb = synth_to_gpu(ta), synth_to_gpu(tb)
    cap = ga.values.numel() + gb.values.numel()
    assert cap > 5 * 5200, "needs several tiles"
    rp = torch.zeros(4001, dtype=torch.int32, device="cuda")
    col = torch.empty(cap, dtype=torch.int32, device="cuda")
    val = torch.empty(cap, dtype=torch.float32, device="cuda")
    z = CsrStruct(4000, 30000, 0, rp.data_ptr(), col.data_ptr(), val.data_ptr())
    sa, sb = ga._struct(), gb._struct()
    t0 = time.perf_counter()
    status = lib.nb200_selftest_lookback_timeout(C.byref(sa), C.byref(sb), C.byref(z), cap, 50, None)
    torch.cuda.synchronize()
    assert status == _capi.E_TIMEOUT
    assert time.perf_counter() - t0 < 5.0, "the give-up must come after a short, bounded wait"
    assert "wait" in lib.nb200_strerror(status).decode()
    said = lib.nb200_last_cuda_error().decode()   # which wait gave up, and at which tile
    assert "look-back" in said and "tile" in said, said
    # the same context, stream and scratch pool still give exact results
    assert_same(csr_from_gpu(nacho.gpu_csr_add_f32(ga, gb)), oracle.csr_add(synth_csr(ta), synth_csr(tb), 8), "add after a give-up")


@pytest.mark.parametrize("case", ["smoke", "medium", "identical", "giant_row"])
def test_two_pass_route_with_exact_capacity(nacho, csr_golden, case):
    """A capacity below the worst-case bound but large enough for the result takes the
    count -> scan -> fill route; it must give the same arrays as the single-pass route."""
    import torch
    from nacho_b200._capi import CsrStruct, check, lib
    a, b = golden_csr(csr_golden, case, "a"), golden_csr(csr_golden, case, "b")
    ga, gb = csr_to_gpu(a), csr_to_gpu(b)
    for fn, tag in ((lib.nb200_csr_add_f32_into, "add"), (lib.nb200_csr_mul_f32_into, "mul")):
        want = golden_csr(csr_golden, case, tag)
        n = len(want.col)
        rp = torch.empty(a.rows + 1, dtype=torch.int32, device="cuda")
        col = torch.empty(max(n, 1), dtype=torch.int32, device="cuda")
        val = torch.empty(max(n, 1), dtype=torch.float32, device="cuda")
        z = CsrStruct(a.rows, a.cols, 0, rp.data_ptr(), col.data_ptr(), val.data_ptr())
        sa, sb = ga._struct(), gb._struct()
        check(fn(C.byref(sa), C.byref(sb), C.byref(z), n, None), tag)
        torch.cuda.synchronize()
        got = CSR(a.rows, a.cols, rp.cpu().numpy(), col[:n].cpu().numpy(), val[:n].cpu().numpy())
        assert_same(got, want, f"{case} {tag} (two-pass)")


def test_env_knobs_in_a_child_process(tmp_path):
    """NACHO_B200_EXACT_ALLOC=1 (the allocating entry points count first and allocate exactly nnz, as
    the reference's drivers do) and NACHO_B200_ADD3_CHAINED=1 (the three-operand add as two chained
    unions): both read once per process, both must give the golden results."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "knobs.py"
    script.write_text(f'''
import ctypes as C, sys
sys.path.insert(0, {root!r}); sys.path.insert(0, {os.path.join(root, "tests")!r})
import numpy as np, torch
import test_csr_gpu as t
from helpers import assert_same, csr_from_gpu, csr_to_gpu, golden_csr
from nacho_b200 import nacho
from nacho_b200._capi import CsrStruct, check, lib
from oracle.cpu_oracle import CSR
g = np.load({os.path.join(root, "tests", "golden", "csr_golden.npz")!r})
for case in ("smoke", "medium", "all_empty", "giant_row", "cancel"):
    a, b, c = (golden_csr(g, case, tag) for tag in ("a", "b", "c"))
    ga, gb, gc = csr_to_gpu(a), csr_to_gpu(b), csr_to_gpu(c)
    for fn, tag in ((lib.nb200_csr_add_f32, "add"), (lib.nb200_csr_mul_f32, "mul")):
        z = CsrStruct()
        sa, sb = ga._struct(), gb._struct()
        check(fn(C.byref(sa), C.byref(sb), C.byref(z), 256, 256, None), tag)
        torch.cuda.synchronize()
        got = CSR(z.rows, z.cols, t._d2h(z.row_ptr, z.rows + 1, np.int32), t._d2h(z.col, z.nnz, np.int32), t._d2h(z.val, z.nnz, np.float32))
        assert_same(got, golden_csr(g, case, tag), case + " " + tag + " (exact allocation)")
        assert (z.nnz > 0) == bool(z.col) == bool(z.val)
        for p in (z.row_ptr, z.col, z.val):
            check(lib.nb200_free_async(p, None), "free")
    assert_same(csr_from_gpu(nacho.gpu_csr_add_3_f32(ga, gb, gc)), golden_csr(g, case, "add3"), case + " add3 (chained)")
print("knobs ok")
''')
    env = dict(os.environ, NACHO_B200_EXACT_ALLOC="1", NACHO_B200_ADD3_CHAINED="1")
    r = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "knobs ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_capacity_and_argument_errors(nacho, csr_golden):
    import torch
    from nacho_b200 import _capi
    from nacho_b200._capi import CsrStruct, lib
    a, b = golden_csr(csr_golden, "smoke", "a"), golden_csr(csr_golden, "smoke", "b")
    ga, gb = csr_to_gpu(a), csr_to_gpu(b)
    want = golden_csr(csr_golden, "smoke", "add")
    rp = torch.empty(a.rows + 1, dtype=torch.int32, device="cuda")
    col = torch.empty(8, dtype=torch.int32, device="cuda")
    val = torch.empty(8, dtype=torch.float32, device="cuda")
    z = CsrStruct(a.rows, a.cols, 0, rp.data_ptr(), col.data_ptr(), val.data_ptr())
    sa, sb = ga._struct(), gb._struct()
    assert lib.nb200_csr_add_f32_into(C.byref(sa), C.byref(sb), C.byref(z), 8, None) == _capi.E_CAPACITY
    assert z.nnz == len(want.col)
    assert lib.nb200_csr_add_f32_into(None, C.byref(sb), C.byref(z), 8, None) == _capi.E_BADARG
    bad = CsrStruct(a.rows + 1, a.cols, sb.nnz, sb.row_ptr, sb.col, sb.val)
    assert lib.nb200_csr_add_f32_into(C.byref(sa), C.byref(bad), C.byref(z), 8, None) == _capi.E_BADARG
    # a stated capacity without the arrays behind it is refused before anything is launched
    hollow = CsrStruct(a.rows, a.cols, 0, rp.data_ptr(), None, None)
    assert lib.nb200_csr_add_f32_into(C.byref(sa), C.byref(sb), C.byref(hollow), 1 << 20, None) == _capi.E_BADARG
    assert lib.nb200_csr_mul_f32_into(C.byref(sa), C.byref(sb), C.byref(hollow), 1 << 20, None) == _capi.E_BADARG
    with pytest.raises(TypeError):
        nacho.CSR_gpu(ga.dim_j_offsets.cpu(), ga.dim_j_indices, ga.values, ga.shape)
    with pytest.raises(TypeError):
        nacho.CSR_gpu(ga.dim_j_offsets, ga.dim_j_indices.to(torch.int64), ga.values, ga.shape)


def test_launch_counter_and_profile(nacho, csr_golden):
    from nacho_b200 import _capi
    a, b = golden_csr(csr_golden, "medium", "a"), golden_csr(csr_golden, "medium", "b")
    ga, gb = csr_to_gpu(a), csr_to_gpu(b)
    before = _capi.launch_count()
    _capi.profile_reset()
    _capi.profile_enable(True)
    nacho.gpu_csr_add_f32(ga, gb)
    _capi.profile_enable(False)
    assert _capi.launch_count() - before == 2  # partition + single-pass merge
    n, ms = _capi.profile_read("csr_add_fused")
    assert n == 1 and ms > 0
    assert "csr2_partition" in _capi.profile_names()


@pytest.mark.parametrize("op", ["add", "mul"])
def test_host_streaming_entry_points(nacho, oracle, op):
    """Host-resident operands streamed through the GPU in row blocks (several blocks here)."""
    import torch
    from nacho_b200 import host, synth
    ta = synth.c3_csr(0, 2, rows=1 << 16, cols=1 << 20, nnz=1 << 25)
    tb = synth.c3_csr(1, 2, rows=1 << 16, cols=1 << 20, nnz=1 << 25)
    pin = lambda t: (t[0], t[1], t[2].pin_memory(), t[3].pin_memory(), t[4].pin_memory())
    fn = host.csr_add_host if op == "add" else host.csr_mul_host
    rows, cols, rp, col, val = fn(pin(ta), pin(tb))
    got = CSR(rows, cols, rp.numpy(), col.numpy(), val.numpy())
    want = (oracle.csr_add if op == "add" else oracle.csr_mul)(synth_csr(ta), synth_csr(tb), 8)
    assert_same(got, want, f"host {op}")
    # small and empty inputs take the same path with a single block
    small = synth.random_csr(50, 40, 0.1, 3)
    r = fn(pin(small), pin(small))
    w = (oracle.csr_add if op == "add" else oracle.csr_mul)(synth_csr(small), synth_csr(small), 1)
    assert_same(CSR(r[0], r[1], r[2].numpy(), r[3].numpy(), r[4].numpy()), w, f"host {op} small")
