"""CPU suite: the C oracle against the committed golden vectors (made by the reference's own
CPU kernels) and, where the reference checker library is present, against those kernels live
on seeded inputs and for several thread counts."""
import numpy as np
import pytest

from helpers import (CSR_CASES, T3_CASES, assert_same, csf3_levels, golden_coo3, golden_csf3, golden_csr,
                     synth_csr)
from oracle.cpu_oracle import COO3, CSF3, CSR


@pytest.mark.parametrize("case", CSR_CASES)
@pytest.mark.parametrize("threads", [1, 3, 16])
def test_csr_golden(oracle, csr_golden, case, threads):
    a, b, c = (golden_csr(csr_golden, case, t) for t in "abc")
    assert_same(oracle.csr_add(a, b, threads), golden_csr(csr_golden, case, "add"), f"{case} add")
    assert_same(oracle.csr_mul(a, b, threads), golden_csr(csr_golden, case, "mul"), f"{case} mul")
    assert_same(oracle.csr_add_3(a, b, c, threads), golden_csr(csr_golden, case, "add3"), f"{case} add3")


@pytest.mark.parametrize("case", T3_CASES)
def test_tensor3_golden(oracle, tensor3_golden, case):
    a, b = golden_coo3(tensor3_golden, case, "a"), golden_coo3(tensor3_golden, case, "b")
    for threads in (1, 5):
        assert_same(oracle.coo3_add(a, b, threads), golden_coo3(tensor3_golden, case, "coo3"), f"{case} coo3")
    fa = CSF3(a.dims, *csf3_levels(np.stack([a.i, a.j, a.k], 1)), a.val)
    fb = CSF3(b.dims, *csf3_levels(np.stack([b.i, b.j, b.k], 1)), b.val)
    assert_same(oracle.csf3_add(fa, fb), golden_csf3(tensor3_golden, case), f"{case} csf3")


def test_golden_keeps_explicit_zeros(csr_golden):
    z = golden_csr(csr_golden, "cancel", "add")
    a = golden_csr(csr_golden, "cancel", "a")
    assert np.array_equal(z.row_ptr, a.row_ptr) and np.all(z.val == 0.0) and len(z.val) == len(a.val)


def test_oracle_vs_reference_live(oracle, reference):
    from nacho_b200 import synth
    for rows, cols, dens, seed in [(200, 180, 0.05, 1), (1, 50, 0.5, 3), (300, 1000, 0.0, 4), (2000, 2000, 0.01, 5)]:
        a, b, c = (synth_csr(synth.random_csr(rows, cols, dens, seed + 100 * k)) for k in range(3))
        for threads in (1, 4):
            assert_same(oracle.csr_add(a, b, threads), reference.csr_add(a, b), "add")
            assert_same(oracle.csr_mul(a, b, threads), reference.csr_mul(a, b), "mul")
            assert_same(oracle.csr_add_3(a, b, c, threads), reference.csr_add_3(a, b, c), "add3")


def test_oracle_vs_reference_config1(oracle, reference):
    from nacho_b200 import synth
    a, b = synth_csr(synth.c1_csr(0)), synth_csr(synth.c1_csr(1))
    assert_same(oracle.csr_add(a, b, 8), reference.csr_add(a, b), "config 1 add")


def test_spgemm_oracle_against_float64_product(oracle):
    import scipy.sparse as sp
    from nacho_b200 import synth
    a = synth_csr(synth.random_csr(200, 180, 0.05, 7))
    b = synth_csr(synth.random_csr(180, 150, 0.05, 8))
    c, v64, abs64, products = oracle.spgemm(a, b, 4, extras=True)
    ones = lambda m: sp.csr_matrix((np.ones(len(m.col)), m.col, m.row_ptr), shape=(m.rows, m.cols))
    pat = (ones(a) @ ones(b)).tocsr()
    pat.sort_indices()
    assert np.array_equal(pat.indptr, c.row_ptr) and np.array_equal(pat.indices, c.col)
    assert products == int(pat.data.sum())
    full = lambda m: sp.csr_matrix((m.val.astype(np.float64), m.col, m.row_ptr), shape=(m.rows, m.cols))
    ref = (full(a) @ full(b)).toarray()
    got = np.zeros_like(ref)
    got[np.repeat(np.arange(c.rows), np.diff(c.row_ptr)), c.col] = v64
    assert np.allclose(got, ref, rtol=0, atol=1e-12)
    assert np.all(np.abs(c.val - v64) <= 1e-5 * abs64 + 1e-30)
    # thread count does not change the float32 sums (fixed ascending-j order)
    c1 = oracle.spgemm(a, b, 1)
    assert_same(c, c1, "spgemm threads")
