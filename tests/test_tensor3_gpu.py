"""GPU suite: COO3 and CSF3 tensor add through the C ABI against the golden vectors made by the
reference's CPU kernels, against the C oracle on seeded inputs, and through properties at a
size the oracle would not finish quickly."""
import numpy as np
import pytest

from helpers import T3_CASES, assert_same, csf3_levels, golden_coo3, golden_csf3
from oracle.cpu_oracle import COO3, CSF3

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nacho():
    import torch
    assert torch.cuda.is_available(), "GPU suite needs a CUDA device"
    from nacho_b200 import nacho as mod
    return mod


def coo3_to_gpu(nacho, t: COO3):
    coords = np.stack([t.i, t.j, t.k], axis=1).reshape(-1, 3)
    return nacho.to_coo3(coords, t.val, t.dims, "cuda")


def coo3_from_gpu(z) -> COO3:
    import torch
    torch.cuda.synchronize()
    return COO3(tuple(int(x) for x in z.shape), z.dim_i_indices.cpu().numpy(), z.dim_j_indices.cpu().numpy(),
                z.dim_k_indices.cpu().numpy(), z.values.cpu().numpy())


def csf3_from_gpu(z) -> CSF3:
    import torch
    torch.cuda.synchronize()
    return CSF3(tuple(int(x) for x in z.shape), z.dim_i_indices.cpu().numpy(), z.dim_j_offsets.cpu().numpy(),
                z.dim_j_indices.cpu().numpy(), z.dim_k_offsets.cpu().numpy(), z.dim_k_indices.cpu().numpy(),
                z.values.cpu().numpy())


@pytest.mark.parametrize("case", T3_CASES)
def test_golden_coo3_and_csf3(nacho, tensor3_golden, case):
    a, b = golden_coo3(tensor3_golden, case, "a"), golden_coo3(tensor3_golden, case, "b")
    z = nacho.gpu_coo3d_add_f32(coo3_to_gpu(nacho, a), coo3_to_gpu(nacho, b))
    assert_same(coo3_from_gpu(z), golden_coo3(tensor3_golden, case, "coo3"), f"{case} coo3")
    ca, cb = np.stack([a.i, a.j, a.k], 1).reshape(-1, 3), np.stack([b.i, b.j, b.k], 1).reshape(-1, 3)
    f = nacho.gpu_csf_add_f32(nacho.to_csf3(ca, a.val, a.dims, "cuda"), nacho.to_csf3(cb, b.val, b.dims, "cuda"))
    assert_same(csf3_from_gpu(f), golden_csf3(tensor3_golden, case), f"{case} csf3")


def _seeded(dims, n, seed, overlap=0.3):
    rng = np.random.default_rng(seed)
    def draw(m):
        c = np.unique(np.stack([rng.integers(0, e, m) for e in dims], axis=1), axis=0)
        return c
    ca = draw(n)
    keep = ca[rng.random(len(ca)) < overlap]
    cb = np.unique(np.concatenate([keep, draw(n)]), axis=0)
    va = rng.uniform(-1, 1, len(ca)).astype(np.float32)
    vb = rng.uniform(-1, 1, len(cb)).astype(np.float32)
    return (ca.astype(np.int32), va), (cb.astype(np.int32), vb)


@pytest.mark.parametrize("dims,n,seed", [((40, 30, 25), 900, 1), ((1 << 12, 1 << 10, 1 << 8), 200_000, 2),
                                          ((5, 1 << 16, 1 << 12), 150_000, 3), ((1 << 17, 4, 4), 100_000, 4),
                                          ((3, 3, 1 << 20), 50_000, 5)])
def test_seeded_vs_oracle(nacho, oracle, dims, n, seed):
    (ca, va), (cb, vb) = _seeded(dims, n, seed)
    a, b = COO3(dims, ca[:, 0], ca[:, 1], ca[:, 2], va), COO3(dims, cb[:, 0], cb[:, 1], cb[:, 2], vb)
    z = nacho.gpu_coo3d_add_f32(nacho.to_coo3(ca, va, dims, "cuda"), nacho.to_coo3(cb, vb, dims, "cuda"))
    assert_same(coo3_from_gpu(z), oracle.coo3_add(a, b, 8), "coo3")
    fa, fb = CSF3(dims, *csf3_levels(ca), va), CSF3(dims, *csf3_levels(cb), vb)
    f = nacho.gpu_csf_add_f32(nacho.to_csf3(ca, va, dims, "cuda"), nacho.to_csf3(cb, vb, dims, "cuda"))
    assert_same(csf3_from_gpu(f), oracle.csf3_add(fa, fb), "csf3")


def test_config5_reduced_vs_oracle(nacho, oracle):
    """Configuration 5 at one hundredth of its entry count (same extents and slice skew)."""
    from nacho_b200 import synth
    ta, tb = synth.c5_pair(nnz=1_000_000, seed=5100)
    def to_np(t):
        dims, i, j, k, v = synth.to_numpy(t)
        return COO3(dims, i, j, k, v)
    a, b = to_np(ta), to_np(tb)
    z = nacho.gpu_coo3d_add_f32(coo3_to_gpu(nacho, a), coo3_to_gpu(nacho, b))
    want = oracle.coo3_add(a, b, 8)
    assert_same(coo3_from_gpu(z), want, "config 5 (1 M entries) coo3")
    ca, cb = np.stack([a.i, a.j, a.k], 1), np.stack([b.i, b.j, b.k], 1)
    f = nacho.gpu_csf_add_f32(nacho.to_csf3(ca, a.val, a.dims, "cuda"), nacho.to_csf3(cb, b.val, b.dims, "cuda"))
    fa, fb = CSF3(a.dims, *csf3_levels(ca), a.val), CSF3(b.dims, *csf3_levels(cb), b.val)
    assert_same(csf3_from_gpu(f), oracle.csf3_add(fa, fb), "config 5 (1 M entries) csf3")


def test_coo3_properties_at_scale(nacho):
    """20 M entries per operand with configuration 5's extents: properties of a sorted union."""
    import torch
    from nacho_b200 import synth
    ta, tb = synth.c5_pair(nnz=20_000_000, seed=5200, device="cuda")
    mk = lambda t: nacho.COO3_gpu(t[1], t[2], t[3], t[4], torch.tensor(list(t[0]), dtype=torch.int32))
    a, b = mk(ta), mk(tb)
    z = nacho.gpu_coo3d_add_f32(a, b)
    torch.cuda.synchronize()
    d1, d2 = ta[0][1], ta[0][2]
    key = lambda t: (t.dim_i_indices.to(torch.int64) * d1 + t.dim_j_indices.to(torch.int64)) * d2 + t.dim_k_indices.to(torch.int64)
    ka, kb, kz = key(a), key(b), key(z)
    assert bool((kz[1:] > kz[:-1]).all()), "result coordinates not strictly increasing"
    union = torch.unique(torch.cat([ka, kb]))
    assert torch.equal(union, kz)
    s = lambda t: float(t.values.to(torch.float64).sum())
    assert abs(s(z) - (s(a) + s(b))) <= 1e-3
    # adding B again keeps the coordinate set (idempotent structure)
    z2 = nacho.gpu_coo3d_add_f32(z, b)
    assert torch.equal(key(z2), kz)


@pytest.mark.parametrize("dims,n,seed", [((1 << 30, 1 << 30, 1 << 30), 40_000, 61), ((2**31 - 1, 5, 2**31 - 1), 30_000, 62),
                                          ((7, 2**31 - 1, 1 << 29), 9_000, 63), ((1 << 22, 1 << 21, 1 << 21), 60_000, 64)])
def test_wide_extents_vs_oracle(nacho, oracle, dims, n, seed):
    """Extents whose coordinates do not pack into 64 bits (more than 63 bits together) take the
    kernel that compares (i, j) and k as two words; COO3 and CSF3 results equal the oracle's."""
    (ca, va), (cb, vb) = _seeded(dims, n, seed)
    a, b = COO3(dims, ca[:, 0], ca[:, 1], ca[:, 2], va), COO3(dims, cb[:, 0], cb[:, 1], cb[:, 2], vb)
    z = nacho.gpu_coo3d_add_f32(nacho.to_coo3(ca, va, dims, "cuda"), nacho.to_coo3(cb, vb, dims, "cuda"))
    assert_same(coo3_from_gpu(z), oracle.coo3_add(a, b, 8), "coo3, wide extents")
    fa, fb = CSF3(dims, *csf3_levels(ca), va), CSF3(dims, *csf3_levels(cb), vb)
    f = nacho.gpu_csf_add_f32(nacho.to_csf3(ca, va, dims, "cuda"), nacho.to_csf3(cb, vb, dims, "cuda"))
    assert_same(csf3_from_gpu(f), oracle.csf3_add(fa, fb), "csf3, wide extents")
    # identical operands: every coordinate is in both
    z2 = nacho.gpu_coo3d_add_f32(nacho.to_coo3(ca, va, dims, "cuda"), nacho.to_coo3(ca, va, dims, "cuda"))
    assert_same(coo3_from_gpu(z2), oracle.coo3_add(a, a, 8), "coo3, wide extents, identical operands")


def test_allocating_tensor_entry_points(nacho, oracle):
    """nb200_coo3d_add_f32 and nb200_csf_add_f32 allocate their own result arrays, each released
    separately with nb200_free_async, as an adopting binding would."""
    import ctypes as C
    import torch
    from nacho_b200._capi import Coo3Struct, Csf3Struct, check, lib
    rt = C.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]

    def d2h(ptr, count, dtype):
        out = np.empty(count, dtype)
        if count:
            assert rt.cudaMemcpy(out.ctypes.data, ptr, out.nbytes, 2) == 0
        return out

    for dims, n, seed in (((40, 30, 25), 900, 1), ((1 << 12, 1 << 10, 1 << 8), 50_000, 2), ((1 << 30, 1 << 30, 1 << 30), 20_000, 3)):
        (ca, va), (cb, vb) = _seeded(dims, n, seed)
        a, b = COO3(dims, ca[:, 0], ca[:, 1], ca[:, 2], va), COO3(dims, cb[:, 0], cb[:, 1], cb[:, 2], vb)
        ga, gb = nacho.to_coo3(ca, va, dims, "cuda"), nacho.to_coo3(cb, vb, dims, "cuda")
        sa, sb, z = ga._struct(), gb._struct(), Coo3Struct()
        check(lib.nb200_coo3d_add_f32(C.byref(sa), C.byref(sb), C.byref(z), 256, 256, None), "coo3d_add")
        torch.cuda.synchronize()
        got = COO3(tuple(z.dims), d2h(z.i, z.nnz, np.int32), d2h(z.j, z.nnz, np.int32), d2h(z.k, z.nnz, np.int32),
                   d2h(z.val, z.nnz, np.float32))
        assert_same(got, oracle.coo3_add(a, b, 4), f"coo3 allocating, dims {dims}")
        for p in (z.i, z.j, z.k, z.val):
            check(lib.nb200_free_async(p, None), "free")
        fa, fb = nacho.to_csf3(ca, va, dims, "cuda"), nacho.to_csf3(cb, vb, dims, "cuda")
        ta, tb, f = fa._struct(), fb._struct(), Csf3Struct()
        check(lib.nb200_csf_add_f32(C.byref(ta), C.byref(tb), C.byref(f), 256, 256, None), "csf_add")
        torch.cuda.synchronize()
        got = CSF3(tuple(f.dims), d2h(f.i_idx, f.n_i, np.int32), d2h(f.j_ptr, f.n_i + 1, np.int32), d2h(f.j_idx, f.n_j, np.int32),
                   d2h(f.k_ptr, f.n_j + 1, np.int32), d2h(f.k_idx, f.n_k, np.int32), d2h(f.val, f.n_k, np.float32))
        want = oracle.csf3_add(CSF3(dims, *csf3_levels(ca), va), CSF3(dims, *csf3_levels(cb), vb))
        assert_same(got, want, f"csf3 allocating, dims {dims}")
        for p in (f.i_idx, f.j_ptr, f.j_idx, f.k_ptr, f.k_idx, f.val):
            check(lib.nb200_free_async(p, None), "free")


def test_csf3_blocks_through_the_gpu_operator(nacho):
    """The multi-GPU decomposition of the CSF3 add, run block after block on one GPU: cuts on the
    k level, clipped sub-trees through gpu_csf_add_f32, seam-aware reassembly; equals the
    unsharded result bit-for-bit."""
    import torch
    from nacho_b200 import shard
    dims = (9, 50, 400)
    (ca, va), (cb, vb) = _seeded(dims, 60_000, 31)
    la, lb = csf3_levels(ca), csf3_levels(cb)
    whole = csf3_from_gpu(nacho.gpu_csf_add_f32(nacho.to_csf3(ca, va, dims, "cuda"), nacho.to_csf3(cb, vb, dims, "cuda")))
    shape = torch.tensor(list(dims), dtype=torch.int32)
    to_gpu = lambda blk: nacho.CSF3_gpu(*[torch.from_numpy(np.ascontiguousarray(x)).cuda() for x in blk], shape)
    for parts in (2, 5):
        cuts = shard.csf3_cuts(la, lb, dims, parts)
        blocks = []
        for (x0, y0), (x1, y1) in zip(cuts, cuts[1:]):
            z = csf3_from_gpu(nacho.gpu_csf_add_f32(to_gpu(shard.csf3_block(la, va, x0, x1)), to_gpu(shard.csf3_block(lb, vb, y0, y1))))
            blocks.append((z.i_idx, z.j_ptr, z.j_idx, z.k_ptr, z.k_idx, z.val))
        got = shard.concat_csf3_blocks(blocks)
        assert_same(CSF3(dims, *got), whole, f"CSF3 in {parts} blocks")


def test_count_scan_fill_route_in_a_child_process(tmp_path):
    """NACHO_B200_TWO_PASS=1 (read once per process) sends the coordinate merge through count ->
    scan -> fill, and the CSF3 add through its separate compress pass; both must still match the
    C oracle bit-for-bit."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "two_pass.py"
    script.write_text(f'''
import sys
sys.path.insert(0, {root!r}); sys.path.insert(0, {os.path.join(root, "tests")!r})
import numpy as np
import test_tensor3_gpu as t3
from helpers import assert_same, csf3_levels
from nacho_b200 import nacho
from oracle.cpu_oracle import COO3, CSF3, Oracle
oracle = Oracle()
for dims, n, seed in (((40, 30, 25), 900, 1), ((1 << 12, 1 << 10, 1 << 8), 120_000, 2), ((5, 1 << 16, 1 << 12), 90_000, 3)):
    (ca, va), (cb, vb) = t3._seeded(dims, n, seed)
    a, b = COO3(dims, ca[:, 0], ca[:, 1], ca[:, 2], va), COO3(dims, cb[:, 0], cb[:, 1], cb[:, 2], vb)
    z = nacho.gpu_coo3d_add_f32(nacho.to_coo3(ca, va, dims, "cuda"), nacho.to_coo3(cb, vb, dims, "cuda"))
    assert_same(t3.coo3_from_gpu(z), oracle.coo3_add(a, b, 8), "coo3, two passes")
    f = nacho.gpu_csf_add_f32(nacho.to_csf3(ca, va, dims, "cuda"), nacho.to_csf3(cb, vb, dims, "cuda"))
    assert_same(t3.csf3_from_gpu(f), oracle.csf3_add(CSF3(dims, *csf3_levels(ca), va), CSF3(dims, *csf3_levels(cb), vb)), "csf3, compress pass")
print("two-pass ok")
''')
    env = dict(os.environ, NACHO_B200_TWO_PASS="1")
    r = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "two-pass ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.parametrize("route", ["0", "1"])
@pytest.mark.parametrize("dims,n,seed", [((40, 30, 25), 900, 71), ((64, 64, 1 << 12), 400_000, 72),   # fibres of ~100 entries
                                          ((3, 2000, 1 << 10), 300_000, 73), ((1 << 17, 4, 4), 100_000, 74),   # ~1 entry per fibre
                                          ((1 << 30, 1 << 30, 1 << 30), 40_000, 75), ((2, 2, 2**31 - 1), 200_000, 76)])
def test_csf3_both_routes(nacho, oracle, monkeypatch, route, dims, n, seed):
    """CSF3 add through the route over expanded coordinates (0) and through the two-level route (1:
    fibre lists merged first, entries through the CSR union with one row per result fibre); both
    must give the oracle's tree whatever the fibre lengths, also for identical operands (every
    fibre and entry in both) and for operands without a common fibre."""
    monkeypatch.setenv("NACHO_B200_CSF_TWO_LEVEL", route)
    (ca, va), (cb, vb) = _seeded(dims, n, seed)
    fa, fb = CSF3(dims, *csf3_levels(ca), va), CSF3(dims, *csf3_levels(cb), vb)
    ga, gb = nacho.to_csf3(ca, va, dims, "cuda"), nacho.to_csf3(cb, vb, dims, "cuda")
    assert_same(csf3_from_gpu(nacho.gpu_csf_add_f32(ga, gb)), oracle.csf3_add(fa, fb), f"csf3 route {route}")
    assert_same(csf3_from_gpu(nacho.gpu_csf_add_f32(ga, ga)), oracle.csf3_add(fa, fa), f"csf3 route {route}, identical operands")
    # disjoint fibres: B moved to other i (first extent permitting)
    if dims[0] >= 4:
        half = dims[0] // 2
        cl, ch = ca[ca[:, 0] < half], cb[cb[:, 0] >= half]
        vl, vh = va[ca[:, 0] < half], vb[cb[:, 0] >= half]
        if len(cl) and len(ch):
            want = oracle.csf3_add(CSF3(dims, *csf3_levels(cl), vl), CSF3(dims, *csf3_levels(ch), vh))
            got = nacho.gpu_csf_add_f32(nacho.to_csf3(cl, vl, dims, "cuda"), nacho.to_csf3(ch, vh, dims, "cuda"))
            assert_same(csf3_from_gpu(got), want, f"csf3 route {route}, disjoint slices")
