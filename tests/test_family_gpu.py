"""GPU suite: the rest of the reference's element-wise family -- 2-D COO add / multiply, CSR + COO,
DCSR add / multiply -- the two inner products and the masked SpGEMM, through the C ABI.

Index arrays and values of the element-wise kernels must equal, bit for bit, the golden vectors
made by the reference's own CPU kernels (tests/golden/make_family_golden.py), and on larger seeded
inputs what the C oracle's CSR add / multiply give once converted to the format in question. Inner
products are float32 sums whose order the reference does not fix (atomic accumulation): they are
held to 1e-5 of sum|a b| against a float64 sum, and the reference's own value must lie within the
same bound. The masked SpGEMM is held to the SpGEMM tolerance on the mask's positions.
"""
import os

import numpy as np
import pytest

from helpers import CSR_CASES, T3_CASES, assert_same, csf3_levels, csr_from_gpu, csr_to_gpu, golden_csr, synth_csr
from oracle.cpu_oracle import COO, CSR, DCSR, csr_to_coo, csr_to_dcsr

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def nacho():
    import torch
    assert torch.cuda.is_available(), "GPU suite needs a CUDA device"
    from nacho_b200 import nacho as mod
    return mod


@pytest.fixture(scope="module")
def family_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "family_golden.npz"))


def _t(x, dtype):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x, dtype)).cuda()


def coo_to_gpu(nacho, m: COO):
    import torch
    return nacho.COO_gpu(_t(m.i, np.int32), _t(m.j, np.int32), _t(m.val, np.float32), torch.tensor([m.rows, m.cols], dtype=torch.int32))


def dcsr_to_gpu(nacho, m: DCSR):
    import torch
    return nacho.DCSR_gpu(_t(m.i_idx, np.int32), _t(m.j_ptr, np.int32), _t(m.j_idx, np.int32), _t(m.val, np.float32),
                          torch.tensor([m.rows, m.cols], dtype=torch.int32))


def coo_from_gpu(z) -> COO:
    import torch
    torch.cuda.synchronize()
    return COO(int(z.shape[0]), int(z.shape[1]), z.dim_i_indices.cpu().numpy(), z.dim_j_indices.cpu().numpy(), z.values.cpu().numpy())


def dcsr_from_gpu(z) -> DCSR:
    import torch
    torch.cuda.synchronize()
    return DCSR(int(z.shape[0]), int(z.shape[1]), z.dim_i_indices.cpu().numpy(), z.dim_j_offsets.cpu().numpy(),
                z.dim_j_indices.cpu().numpy(), z.values.cpu().numpy())


@pytest.mark.parametrize("case", CSR_CASES)
def test_golden_coo_and_dcsr(nacho, csr_golden, family_golden, case):
    a, b = golden_csr(csr_golden, case, "a"), golden_csr(csr_golden, case, "b")
    g = family_golden
    ca, cb = coo_to_gpu(nacho, csr_to_coo(a)), coo_to_gpu(nacho, csr_to_coo(b))
    for op, fn in (("coo_add", nacho.gpu_coo_add_f32), ("coo_mul", nacho.gpu_coo_mul_f32)):
        want = COO(a.rows, a.cols, g[f"{case}.{op}.i"], g[f"{case}.{op}.j"], g[f"{case}.{op}.val"])
        assert_same(coo_from_gpu(fn(ca, cb)), want, f"{case} {op}")
    want = CSR(a.rows, a.cols, g[f"{case}.coo_csr_add.rp"], g[f"{case}.coo_csr_add.col"], g[f"{case}.coo_csr_add.val"])
    assert_same(csr_from_gpu(nacho.gpu_coo_csr_add_f32(csr_to_gpu(a), cb)), want, f"{case} coo_csr_add")
    da, db = dcsr_to_gpu(nacho, csr_to_dcsr(a)), dcsr_to_gpu(nacho, csr_to_dcsr(b))
    for op, fn in (("dcsr_add", nacho.gpu_dcsr_add_f32), ("dcsr_mul", nacho.gpu_dcsr_mul_f32),
                   ("dcsr_mul", nacho.gpu_dcsr_mul_without_recursive_partitioning_f32)):
        want = DCSR(a.rows, a.cols, *[g[f"{case}.{op}.{f}"] for f in ("i_idx", "j_ptr", "j_idx", "val")])
        assert_same(dcsr_from_gpu(fn(da, db)), want, f"{case} {op}")


def _dcsr_expected(z: CSR, a: CSR, b: CSR, product: bool) -> DCSR:
    """The DCSR form of a CSR result: rows with entries for a sum; for a product the rows both operands
    store (an empty range where their columns do not meet), as the reference's kernels return."""
    la, lb, lz = (np.diff(np.asarray(m.row_ptr, np.int64)) for m in (a, b, z))
    keep = np.flatnonzero((la > 0) & (lb > 0)) if product else np.flatnonzero(lz > 0)
    ptr = np.zeros(len(keep) + 1, np.int32)
    ptr[1:] = np.cumsum(lz[keep])
    return DCSR(z.rows, z.cols, keep.astype(np.int32), ptr, z.col, z.val)


@pytest.mark.parametrize("rows,cols,density,seed", [(3000, 20000, 0.004, 81), (100000, 50, 0.01, 82), (40, 1 << 22, 0.0005, 83),
                                                    (200000, 1 << 16, 0.00002, 84)])
def test_seeded_vs_oracle(nacho, oracle, rows, cols, density, seed):
    from nacho_b200 import synth
    a, b = synth_csr(synth.random_csr(rows, cols, density, seed)), synth_csr(synth.random_csr(rows, cols, density, seed + 500))
    zs, zp = oracle.csr_add(a, b, 8), oracle.csr_mul(a, b, 8)
    ca, cb = coo_to_gpu(nacho, csr_to_coo(a)), coo_to_gpu(nacho, csr_to_coo(b))
    assert_same(coo_from_gpu(nacho.gpu_coo_add_f32(ca, cb)), csr_to_coo(zs), "coo_add")
    assert_same(coo_from_gpu(nacho.gpu_coo_mul_f32(ca, cb)), csr_to_coo(zp), "coo_mul")
    assert_same(csr_from_gpu(nacho.gpu_coo_csr_add_f32(csr_to_gpu(a), cb)), zs, "coo_csr_add")
    da, db = dcsr_to_gpu(nacho, csr_to_dcsr(a)), dcsr_to_gpu(nacho, csr_to_dcsr(b))
    assert_same(dcsr_from_gpu(nacho.gpu_dcsr_add_f32(da, db)), _dcsr_expected(zs, a, b, False), "dcsr_add")
    assert_same(dcsr_from_gpu(nacho.gpu_dcsr_mul_f32(da, db)), _dcsr_expected(zp, a, b, True), "dcsr_mul")


def test_converters(nacho):
    """to_coo / to_dcsr give the buffers the reference's converters give (python/nacho/convert.py:34-67)."""
    import torch
    from nacho_b200 import synth
    rows, cols, rp, col, val = synth.random_csr(500, 300, 0.02, 9)
    t = torch.sparse_csr_tensor(rp.to(torch.int64), col.to(torch.int64), val, size=(rows, cols))
    m = CSR(rows, cols, rp.numpy(), col.numpy(), val.numpy())
    d = nacho.to_dcsr(t, "cuda")
    assert_same(dcsr_from_gpu(d), csr_to_dcsr(m), "to_dcsr")
    c = nacho.to_coo(t.to_sparse_coo(), "cuda")
    assert_same(coo_from_gpu(c), csr_to_coo(m), "to_coo")
    with pytest.raises(ValueError):
        nacho.to_coo(t.to_sparse_coo(), "cpu")


@pytest.mark.parametrize("case", T3_CASES)
def test_inner_products(nacho, tensor3_golden, family_golden, case):
    g = tensor3_golden
    dims = tuple(int(x) for x in g[f"{case}.dims"])
    ca, va = g[f"{case}.a.coords"].reshape(-1, 3), g[f"{case}.a.val"]
    cb, vb = g[f"{case}.b.coords"].reshape(-1, 3), g[f"{case}.b.val"]
    key = lambda c: (c[:, 0].astype(np.int64) * dims[1] + c[:, 1]) * dims[2] + c[:, 2]
    _, ia, ib = np.intersect1d(key(ca), key(cb), return_indices=True)
    prod = (va[ia] * vb[ib]).astype(np.float64)        # float32 products, as both implementations form them
    want, bound = float(prod.sum()), 1e-5 * float(np.abs(prod).sum()) + 1e-30
    z = nacho.gpu_inner_prod_coo_f32(nacho.to_coo3(ca, va, dims, "cuda"), nacho.to_coo3(cb, vb, dims, "cuda"))
    got = float(z.values.cpu()[0])
    assert z.values.numel() == 1 and abs(got - want) <= bound, f"{case} inner_prod_coo: {got} vs {want}"
    assert abs(float(family_golden[f"{case}.inner_prod_coo"][0]) - want) <= bound   # the reference sits in the same bound
    f = nacho.gpu_inner_prod_f32(nacho.to_csf3(ca, va, dims, "cuda"), nacho.to_csf3(cb, vb, dims, "cuda"))
    got = float(f.values.cpu()[0])
    assert abs(got - want) <= bound, f"{case} inner_prod: {got} vs {want}"
    if f"{case}.inner_prod" in family_golden.files:
        assert abs(float(family_golden[f"{case}.inner_prod"][0]) - want) <= bound


def test_inner_product_at_scale(nacho):
    """Two million entries per operand with a shared third: many tiles, one atomic per tile."""
    import torch
    from nacho_b200 import synth
    ta, tb = synth.c5_pair(nnz=2_000_000, seed=5300, device="cuda")
    mk = lambda t: nacho.COO3_gpu(t[1], t[2], t[3], t[4], torch.tensor(list(t[0]), dtype=torch.int32))
    z = nacho.gpu_inner_prod_coo_f32(mk(ta), mk(tb))
    d1, d2 = ta[0][1], ta[0][2]
    key = lambda t: (t[1].to(torch.int64) * d1 + t[2].to(torch.int64)) * d2 + t[3].to(torch.int64)
    ka, kb = key(ta), key(tb)
    pos = torch.searchsorted(kb, ka).clamp(max=kb.numel() - 1)
    hit = kb[pos] == ka
    prod = (ta[4][hit] * tb[4][pos[hit]]).to(torch.float64)
    want, bound = float(prod.sum()), 1e-5 * float(prod.abs().sum())
    assert int(hit.sum()) > 100_000
    assert abs(float(z.values.cpu()[0]) - want) <= bound


def mask_classes_case():
    """A, B, mask with one row for every route of the masked product: mask rows of narrow / medium /
    wide / beyond-bitmap column span, short and long, a row with few products, empty rows."""
    import torch
    rng = np.random.default_rng(977)
    cols, inner = 1 << 22, 64
    spans = [(0, 60_000, 1_500), (5_000, 200_000, 5_000), (1_000, 900_000, 20_000), (0, cols, 6_000),
             (70_000, 120_000, 3_000), (0, 0, 0), (10, 50_000, 40), (300_000, 1_300_000, 9_000)]
    mask_rows = [np.sort(rng.choice(np.arange(lo, hi), n, replace=False)) if n else np.zeros(0, np.int64) for lo, hi, n in spans]
    rows = len(spans)

    def tup(r, c, lists):
        rp = np.zeros(r + 1, np.int32)
        rp[1:] = np.cumsum([len(x) for x in lists])
        col = np.concatenate(lists).astype(np.int32)
        val = rng.uniform(-1, 1, col.size).astype(np.float32)
        return r, c, torch.from_numpy(rp), torch.from_numpy(col), torch.from_numpy(val)

    # B's rows draw half of their columns from the mask rows, so that products land on the mask
    pool = np.unique(np.concatenate(mask_rows))
    b_rows = [np.unique(np.concatenate([rng.choice(pool, 1500), rng.integers(0, cols, 1500)])) for _ in range(inner)]
    a_rows = [np.sort(rng.choice(inner, n, replace=False)) for n in (20, 30, 25, 40, 20, 10, 0, 35)]
    a_rows[6] = np.array([3], np.int64)                 # the light row: one A entry ...
    b_rows[3] = np.sort(rng.choice(mask_rows[6], 30, replace=False))  # ... times a short B row
    return tup(rows, inner, a_rows), tup(inner, cols, b_rows), tup(rows, cols, mask_rows)


@pytest.mark.parametrize("shape", ["uniform", "rmat", "empty_mask", "classes"])
def test_masked_spgemm(nacho, oracle, shape):
    """gpu_sssmm_f32: sum_j a_ij b_jk c_ik on the positions the mask stores that the product reaches."""
    from nacho_b200 import synth
    if shape == "uniform":
        ta, tb, tc = synth.random_csr(400, 300, 0.03, 91), synth.random_csr(300, 400, 0.03, 92), synth.random_csr(400, 400, 0.05, 93)
    elif shape == "rmat":   # skewed rows: a few rows hold most of the products; the mask is A's own pattern squared-ish
        ta = synth.rmat_csr(scale=11, seed=4311)
        tb = synth.transpose_csr(ta)
        tc = synth.random_csr(1 << 11, 1 << 11, 0.01, 94)
    elif shape == "classes":
        ta, tb, tc = mask_classes_case()
    else:
        ta, tb, tc = synth.random_csr(60, 50, 0.1, 95), synth.random_csr(50, 70, 0.1, 96), synth.random_csr(60, 70, 0.0, 97)
    a, b, c = synth_csr(ta), synth_csr(tb), synth_csr(tc)
    full, v64, abs64, _ = oracle.spgemm(a, b, 4, extras=True)
    z = csr_from_gpu(nacho.gpu_sssmm_f32(csr_to_gpu(a), csr_to_gpu(b), csr_to_gpu(c)))
    # expected structure: positions stored by both the product and the mask
    key = lambda m: np.repeat(np.arange(m.rows, dtype=np.int64), np.diff(m.row_ptr)) * m.cols + m.col
    kf, kc, kz = key(full), key(c), key(z)
    common, i_f, i_c = np.intersect1d(kf, kc, return_indices=True)
    assert np.array_equal(kz, common), "masked structure"
    want = v64[i_f] * c.val[i_c].astype(np.float64)
    bound = 1e-5 * abs64[i_f] * np.abs(c.val[i_c]) + 1e-30
    assert np.all(np.abs(z.val.astype(np.float64) - want) <= bound)
