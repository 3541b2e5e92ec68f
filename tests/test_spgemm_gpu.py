"""GPU suite: expand-sort-compress SpGEMM through the C ABI against the C oracle (the
reference has no CPU SpGEMM; the oracle restates its GPU algorithm and is itself pinned
against a float64 product in the CPU suite). Structure must match exactly. Values: rows of
at most 256 products sum in the oracle's order and must match bit-for-bit; longer rows are
held to |x - x64| <= 1e-5 * sum|a*b| (relative 1e-5 per entry wherever there is no
cancellation), the tolerance of the task statement."""
import numpy as np
import pytest

from helpers import csr_from_gpu, csr_to_gpu, synth_csr, synth_to_gpu
from oracle.cpu_oracle import CSR

pytestmark = pytest.mark.gpu

REL_TOL = 1e-5
SORTED_ROW_PRODUCTS = 256   # rows up to here are sorted on chip and summed in the oracle's order


@pytest.fixture(scope="module")
def nacho():
    import torch
    assert torch.cuda.is_available(), "GPU suite needs a CUDA device"
    from nacho_b200 import nacho as mod
    return mod


def check(nacho, oracle, a: CSR, b: CSR, ga=None, gb=None, exact_rows_only=False):
    want, v64, abs64, products = oracle.spgemm(a, b, 8, extras=True)
    got = csr_from_gpu(nacho.gpu_spgemm_f32(ga or csr_to_gpu(a), gb or csr_to_gpu(b)))
    assert got.rows == a.rows and got.cols == b.cols
    assert np.array_equal(got.row_ptr, want.row_ptr), "row offsets differ"
    assert np.array_equal(got.col, want.col), "columns differ"
    # per-row product counts decide which path a row took
    b_len = np.diff(b.row_ptr)
    per_entry = b_len[a.col] if len(a.col) else np.zeros(0, np.int64)
    row_products = np.add.reduceat(np.append(per_entry, 0), a.row_ptr[:-1].clip(max=len(per_entry)))
    row_products[np.diff(a.row_ptr) == 0] = 0
    short = np.repeat(row_products <= SORTED_ROW_PRODUCTS, np.diff(want.row_ptr))
    same = got.val.view(np.uint32) == want.val.view(np.uint32)
    assert same[short].all(), "a row of <= 256 products differs from the fixed-order float32 sum"
    assert np.all(np.abs(got.val.astype(np.float64) - v64) <= REL_TOL * abs64 + 1e-30)
    return got, products


def test_smoke_shape(nacho, oracle):
    from nacho_b200 import synth
    a = synth_csr(synth.random_csr(200, 180, 0.05, 7))
    b = synth_csr(synth.random_csr(180, 150, 0.05, 8))
    check(nacho, oracle, a, b)


def test_empty_and_degenerate(nacho, oracle):
    from nacho_b200 import synth
    a = synth_csr(synth.random_csr(64, 50, 0.0, 1))
    b = synth_csr(synth.random_csr(50, 70, 0.2, 2))
    got, _ = check(nacho, oracle, a, b)
    assert len(got.col) == 0
    a = synth_csr(synth.random_csr(64, 50, 0.2, 3))
    check(nacho, oracle, a, synth_csr(synth.random_csr(50, 70, 0.0, 4)))   # B empty: no products at all
    check(nacho, oracle, synth_csr(synth.random_csr(1, 300, 0.5, 5)), synth_csr(synth.random_csr(300, 1, 0.5, 6)))


def test_exact_cancellation_is_kept(nacho, oracle):
    """C = [1, 1] @ [[1], [-1]] stores an explicit 0.0, as the reference's compress does."""
    a = CSR(1, 2, np.array([0, 2], np.int32), np.array([0, 1], np.int32), np.array([1, 1], np.float32))
    b = CSR(2, 1, np.array([0, 1, 2], np.int32), np.array([0, 0], np.int32), np.array([1, -1], np.float32))
    got, _ = check(nacho, oracle, a, b)
    assert got.row_ptr.tolist() == [0, 1] and got.val.tolist() == [0.0]


def test_medium_and_long_rows(nacho, oracle):
    """Rows in the warp, sorted-CTA and ranked bins (<= 32, <= 256, more products), next to empty rows."""
    rng = np.random.default_rng(3)
    rows, inner, cols = 300, 4000, 6000
    lens = rng.integers(0, 6, rows)
    lens[9] = 25       # sorted in shared memory: about 200 products
    lens[10] = 200      # ranked: 200 entries x ~8 = 1600 products
    lens[20] = 900      # ranked
    lens[21] = 3000     # ranked, most of the inner dimension
    lens[50:60] = 0
    rp = np.zeros(rows + 1, np.int32)
    rp[1:] = np.cumsum(lens)
    col = np.concatenate([np.sort(rng.choice(inner, int(n), replace=False)) for n in lens]).astype(np.int32)
    a = CSR(rows, inner, rp, col, rng.uniform(-1, 1, len(col)).astype(np.float32))
    from nacho_b200 import synth
    b = synth_csr(synth.random_csr(inner, cols, 0.002, 9))
    check(nacho, oracle, a, b)


def test_long_huge_and_giant_rows(nacho, oracle):
    """Rows on both sides of 65535 products (16-bit and 32-bit column ranks) and one row with more
    than 2^20 products (handed out first). A row of explicit zeros against negative values makes
    every product -0.0: its entries must still be stored (as 0.0 sums)."""
    from nacho_b200 import synth
    rng = np.random.default_rng(11)
    rows, inner, cols = 48, 3000, 100_000
    tb = synth.random_csr(inner, cols, 0.005, 12)          # about 500 entries per row of B
    lens = rng.integers(0, 4, rows)
    lens[3], lens[4], lens[5] = 6, 9, 13                   # ranked: about 3000 / 4500 / 6500 products
    lens[8], lens[9], lens[10] = 20, 64, 700               # ranked, ranked, heavy (about 350000 products)
    lens[11] = 600                                         # heavy, all-zero values
    lens[20] = 2600                                        # giant: about 1.3 M products
    rp = np.zeros(rows + 1, np.int32)
    rp[1:] = np.cumsum(lens)
    col = np.concatenate([np.sort(rng.choice(inner, int(n), replace=False)) for n in lens]).astype(np.int32)
    val = rng.uniform(-1, 1, len(col)).astype(np.float32)
    val[rp[11]:rp[12]] = 0.0
    val[rp[10]:rp[11]:7] = 0.0
    a = CSR(rows, inner, rp, col, val)
    b = synth_csr(tb)
    b = CSR(b.rows, b.cols, b.row_ptr, b.col, -np.abs(b.val))
    got, products = check(nacho, oracle, a, b)
    assert products > (1 << 20)
    row11 = got.val[got.row_ptr[11]:got.row_ptr[12]]
    assert len(row11) > 0 and not row11.any()


def test_wider_than_the_shared_bitmap(nacho, oracle):
    """300000 columns: wider than the shared-memory bitmap (262144 columns), so every ranked row
    is walked in two column windows through the window pointer table of B, the second window
    partial."""
    from nacho_b200 import synth
    rng = np.random.default_rng(17)
    rows, inner, cols = 32, 2000, 300_000
    lens = rng.integers(0, 3, rows)
    lens[2], lens[3], lens[4], lens[5], lens[6] = 6, 12, 25, 60, 200   # the last one heavy: about 120000 products
    rp = np.zeros(rows + 1, np.int32)
    rp[1:] = np.cumsum(lens)
    col = np.concatenate([np.sort(rng.choice(inner, int(n), replace=False)) for n in lens]).astype(np.int32)
    a = CSR(rows, inner, rp, col, rng.uniform(-1, 1, len(col)).astype(np.float32))
    check(nacho, oracle, a, synth_csr(synth.random_csr(inner, cols, 0.002, 18)))


def test_hyper_wide_b_without_pointer_table(nacho, oracle):
    """2^30 columns and 70000 rows of B: the window pointer table (70000 x 4097 entries) would
    exceed its budget, so the 4096 column windows of every ranked row are located by binary
    search instead. Almost all windows of a row are empty."""
    rng = np.random.default_rng(23)
    inner, cols, per_row = 70_000, 1 << 30, 100
    keys = np.unique(np.repeat(np.arange(inner, dtype=np.int64), per_row) * cols + rng.integers(0, cols, inner * per_row))
    b_rows, b_col = keys // cols, (keys % cols).astype(np.int32)
    b_rp = np.zeros(inner + 1, np.int32)
    b_rp[1:] = np.cumsum(np.bincount(b_rows, minlength=inner))
    b = CSR(inner, cols, b_rp, b_col, rng.uniform(-1, 1, len(b_col)).astype(np.float32))
    lens = np.array([0, 4, 30, 0, 700, 2])
    rp = np.zeros(len(lens) + 1, np.int32)
    rp[1:] = np.cumsum(lens)
    col = np.concatenate([np.sort(rng.choice(inner, int(n), replace=False)) for n in lens]).astype(np.int32)
    a = CSR(len(lens), inner, rp, col, rng.uniform(-1, 1, len(col)).astype(np.float32))
    check(nacho, oracle, a, b)


def test_single_window_and_partial_last_window(nacho, oracle):
    """Column counts around multiples of the bitmap granularity (8192 columns per 256 words),
    with rows heavy enough to be ranked."""
    from nacho_b200 import synth
    for n, cols in enumerate((16384, 16385, 40000)):
        a = synth_csr(synth.random_csr(40, 600, 0.3, 30 + n))
        b = synth_csr(synth.random_csr(600, cols, 0.02, 40 + n))
        check(nacho, oracle, a, b)


def test_laplacian_squared_reduced(nacho, oracle):
    """Configuration 4b on a 96 x 96 grid: 13-point stencil, at most 13 entries per row."""
    from nacho_b200 import synth
    t = synth.laplacian_csr(96)
    a = synth_csr(t)
    got, products = check(nacho, oracle, a, a, synth_to_gpu(t), synth_to_gpu(t))
    assert np.diff(got.row_ptr).max() == 13
    assert products == int((np.diff(a.row_ptr)[a.col]).sum())


def test_rmat_reduced(nacho, oracle):
    """Configuration 4a at scale 12 (4096 rows, B = A^T): skewed rows in every bin."""
    from nacho_b200 import synth
    ta = synth.rmat_csr(scale=12, seed=4012)
    tb = synth.transpose_csr(ta)
    check(nacho, oracle, synth_csr(ta), synth_csr(tb), synth_to_gpu(ta), synth_to_gpu(tb))


def test_full_size_laplacian_properties(nacho):
    """Configuration 4b at full size (512 x 512 grid): known structure of the squared stencil."""
    import torch
    from nacho_b200 import synth
    t = synth.laplacian_csr(512, device="cuda")
    a = synth_to_gpu(t)
    c = nacho.gpu_spgemm_f32(a, a)
    torch.cuda.synchronize()
    assert c.values.numel() == 3_397_636  # 13-point stencil on a 512 x 512 grid
    rp = c.dim_j_offsets.to(torch.int64)
    rows = torch.repeat_interleave(torch.arange(512 * 512, device="cuda"), rp[1:] - rp[:-1])
    key = rows * (512 * 512) + c.dim_j_indices.to(torch.int64)
    assert bool((key[1:] > key[:-1]).all())
    # the Laplacian has zero row sums away from the boundary, so does its square; all sums are small integers
    dense_sum = float(c.values.to(torch.float64).sum())
    a_sum = torch.zeros(512 * 512, dtype=torch.float64, device="cuda").index_add_(
        0, torch.repeat_interleave(torch.arange(512 * 512, device="cuda"), (a.dim_j_offsets[1:] - a.dim_j_offsets[:-1]).to(torch.int64)),
        a.values.to(torch.float64))
    # sum(C) = 1^T A A 1 = (A^T 1) . (A 1) = |A 1|^2 for symmetric A
    assert abs(dense_sum - float((a_sum * a_sum).sum())) < 1e-6 * max(1.0, abs(dense_sum))
    assert bool((c.values == c.values.round()).all())


def test_allocating_entry_point(nacho, oracle):
    """nb200_spgemm_f32 allocates the three result arrays itself (released one by one)."""
    import ctypes as C
    import torch
    from nacho_b200 import synth
    from nacho_b200._capi import CsrStruct, check as ck, lib
    rt = C.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]

    def d2h(ptr, count, dtype):
        out = np.empty(count, dtype)
        if count:
            assert rt.cudaMemcpy(out.ctypes.data, ptr, out.nbytes, 2) == 0
        return out

    cases = [(synth.random_csr(500, 400, 0.03, 21), synth.random_csr(400, 300, 0.03, 22)),
             (synth.random_csr(64, 50, 0.0, 1), synth.random_csr(50, 70, 0.2, 2))]
    ta = synth.rmat_csr(scale=10, seed=4210)
    cases.append((ta, synth.transpose_csr(ta)))
    for ta, tb in cases:
        want, v64, abs64, _ = oracle.spgemm(synth_csr(ta), synth_csr(tb), 4, extras=True)
        ga, gb = synth_to_gpu(ta), synth_to_gpu(tb)
        sa, sb, c = ga._struct(), gb._struct(), CsrStruct()
        ck(lib.nb200_spgemm_f32(C.byref(sa), C.byref(sb), C.byref(c), 256, 256, None), "spgemm")
        torch.cuda.synchronize()
        assert (c.rows, c.cols, c.nnz) == (want.rows, want.cols, len(want.col))
        assert np.array_equal(d2h(c.row_ptr, c.rows + 1, np.int32), want.row_ptr)
        assert np.array_equal(d2h(c.col, c.nnz, np.int32), want.col)
        val = d2h(c.val, c.nnz, np.float32)
        assert np.all(np.abs(val.astype(np.float64) - v64) <= REL_TOL * abs64 + 1e-30)
        if c.nnz == 0:
            assert not c.col and not c.val
        for p in (c.row_ptr, c.col, c.val):
            ck(lib.nb200_free_async(p, None), "free")


def test_symbolic_reports_products(nacho, oracle):
    import ctypes as C
    import torch
    from nacho_b200 import synth
    from nacho_b200._capi import CsrStruct, check as ck, lib
    ta, tb = synth.random_csr(500, 400, 0.03, 21), synth.random_csr(400, 300, 0.03, 22)
    want, _, _, products = oracle.spgemm(synth_csr(ta), synth_csr(tb), 4, extras=True)
    ga, gb = synth_to_gpu(ta), synth_to_gpu(tb)
    rp = torch.empty(501, dtype=torch.int32, device="cuda")
    c = CsrStruct(0, 0, 0, rp.data_ptr(), None, None)
    p = C.c_int64(0)
    sa, sb = ga._struct(), gb._struct()
    ck(lib.nb200_spgemm_f32_symbolic(C.byref(sa), C.byref(sb), C.byref(c), C.byref(p), None), "symbolic")
    assert p.value == products and c.nnz == len(want.col)
    assert np.array_equal(rp.cpu().numpy(), want.row_ptr)


def test_numeric_after_other_work_on_the_stream(nacho, oracle):
    """The numeric pass reuses what the symbolic pass left in the scratch pool only if nothing
    else used the pool in between; here a CSR add runs between the two passes, and a numeric
    pass is also repeated with new values in A (same structure)."""
    import ctypes as C
    import torch
    from nacho_b200 import synth
    from nacho_b200._capi import CsrStruct, check as ck, lib
    ta = synth.rmat_csr(scale=10, seed=4110)
    tb = synth.transpose_csr(ta)
    a, b = synth_csr(ta), synth_csr(tb)
    want, v64, abs64, _ = oracle.spgemm(a, b, 8, extras=True)
    ga, gb = synth_to_gpu(ta), synth_to_gpu(tb)
    sa, sb = ga._struct(), gb._struct()
    rp = torch.empty(a.rows + 1, dtype=torch.int32, device="cuda")
    c = CsrStruct(0, 0, 0, rp.data_ptr(), None, None)
    ck(lib.nb200_spgemm_f32_symbolic(C.byref(sa), C.byref(sb), C.byref(c), None, None), "symbolic")
    nacho.gpu_csr_add_f32(ga, ga)                      # takes the scratch pool in between
    col = torch.empty(c.nnz, dtype=torch.int32, device="cuda")
    val = torch.empty(c.nnz, dtype=torch.float32, device="cuda")
    c.col, c.val = col.data_ptr(), val.data_ptr()
    ck(lib.nb200_spgemm_f32_numeric(C.byref(sa), C.byref(sb), C.byref(c), None), "numeric")
    torch.cuda.synchronize()
    assert np.array_equal(rp.cpu().numpy(), want.row_ptr) and np.array_equal(col.cpu().numpy(), want.col)
    assert np.all(np.abs(val.cpu().numpy().astype(np.float64) - v64) <= REL_TOL * abs64 + 1e-30)

    # symbolic again, then two numeric passes: the second with A's values doubled in place
    ck(lib.nb200_spgemm_f32_symbolic(C.byref(sa), C.byref(sb), C.byref(c), None, None), "symbolic")
    c.col, c.val = col.data_ptr(), val.data_ptr()
    ck(lib.nb200_spgemm_f32_numeric(C.byref(sa), C.byref(sb), C.byref(c), None), "numeric")
    ga.values.mul_(2.0)
    ck(lib.nb200_spgemm_f32_numeric(C.byref(sa), C.byref(sb), C.byref(c), None), "numeric")
    torch.cuda.synchronize()
    assert np.array_equal(col.cpu().numpy(), want.col)
    assert np.all(np.abs(val.cpu().numpy().astype(np.float64) - 2.0 * v64) <= 2.0 * REL_TOL * abs64 + 1e-30)
