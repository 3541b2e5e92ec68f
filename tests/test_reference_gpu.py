"""GPU suite: the product against the reference's own GPU kernels on the same device.

``oracle/_ref/libnacho_ref_gpu.so`` holds the GPU drivers emitted by the reference's compiler,
compiled unchanged for sm_100a (``make -C oracle ref_gpu``). Index arrays must match exactly for
every kernel; add / multiply values must match bit-for-bit; SpGEMM values are held to the
tolerance of the SpGEMM suite (both sides sum with atomics in no fixed order). It is the only
implementation of SpGEMM the reference has, so this is where its structure is pinned on device.
Inputs are kept small and non-empty, and SpGEMM product counts far below the reference's int32
limit."""
import numpy as np
import pytest

from helpers import synth_csr

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_gpu():
    from oracle.gpu_reference import ReferenceGpu
    if not ReferenceGpu.available():
        pytest.skip("oracle/_ref/libnacho_ref_gpu.so was not built (needs the reference checkout)")
    import torch
    assert torch.cuda.is_available(), "GPU suite needs a CUDA device"
    return ReferenceGpu()


@pytest.fixture(scope="module")
def nacho():
    from nacho_b200 import nacho as mod
    return mod


def dev(t):
    """synth tuple (ints and torch tensors) with its tensors on the GPU."""
    import torch
    return tuple(x.cuda() if isinstance(x, torch.Tensor) else x for x in t)


def as_csr_gpu(nacho, t):
    import torch
    rows, cols, rp, col, val = t
    return nacho.CSR_gpu(rp, col, val, torch.tensor([rows, cols], dtype=torch.int32))


def same_csr(got, want, exact_values=True):
    import torch
    rows, cols, rp, col, val = want
    assert int(got.shape[0]) == rows and int(got.shape[1]) == cols
    assert torch.equal(got.dim_j_offsets, rp), "row offsets differ from the reference's GPU kernel"
    assert torch.equal(got.dim_j_indices, col), "columns differ from the reference's GPU kernel"
    if exact_values:
        assert torch.equal(got.values.view(torch.int32), val.view(torch.int32)), "values differ bit-wise"


@pytest.mark.parametrize("rows,cols,density,seed", [(200, 180, 0.05, 1), (4096, 4096, 0.01, 2), (64, 50, 0.3, 3),
                                                    (50_000, 64, 0.1, 5)])
def test_csr_add_mul_add3(nacho, ref_gpu, rows, cols, density, seed):
    from nacho_b200 import synth
    a, b, c = (dev(synth.random_csr(rows, cols, density, 10 * seed + k)) for k in range(3))
    ga, gb, gc = (as_csr_gpu(nacho, t) for t in (a, b, c))
    same_csr(nacho.gpu_csr_add_f32(ga, gb), ref_gpu.csr_add(a, b))
    same_csr(nacho.gpu_csr_mul_f32(ga, gb), ref_gpu.csr_mul(a, b))
    same_csr(nacho.gpu_csr_add_3_f32(ga, gb, gc), ref_gpu.csr_add_3(a, b, c))


def test_csr_add_skewed_rows(nacho, ref_gpu):
    """Configuration 3 at 1/256 of its size with sigma = 2: a few rows hold most entries."""
    from nacho_b200 import synth
    a = dev(synth.c3_csr(0, 2.0, rows=4096, cols=4096, nnz=250_000))
    b = dev(synth.c3_csr(1, 2.0, rows=4096, cols=4096, nnz=250_000))
    same_csr(nacho.gpu_csr_add_f32(as_csr_gpu(nacho, a), as_csr_gpu(nacho, b)), ref_gpu.csr_add(a, b))


def test_tensor3_add(nacho, ref_gpu):
    import torch
    from nacho_b200 import synth
    ta, tb = synth.c5_pair(nnz=200_000, seed=5200)
    a, b = dev(ta), dev(tb)
    shape = torch.tensor(list(a[0]), dtype=torch.int32)
    z = nacho.gpu_coo3d_add_f32(nacho.COO3_gpu(*a[1:5], shape), nacho.COO3_gpu(*b[1:5], shape))
    dims, i, j, k, val = ref_gpu.coo3_add(a, b)
    assert torch.equal(z.dim_i_indices, i) and torch.equal(z.dim_j_indices, j) and torch.equal(z.dim_k_indices, k)
    assert torch.equal(z.values.view(torch.int32), val.view(torch.int32))

    fa = nacho.to_csf3(torch.stack(a[1:4], 1).cpu().numpy(), a[4].cpu().numpy(), a[0], "cuda")
    fb = nacho.to_csf3(torch.stack(b[1:4], 1).cpu().numpy(), b[4].cpu().numpy(), b[0], "cuda")
    f = nacho.gpu_csf_add_f32(fa, fb)
    as_tuple = lambda t: (tuple(int(x) for x in t.shape), t.dim_i_indices, t.dim_j_offsets, t.dim_j_indices, t.dim_k_offsets,
                          t.dim_k_indices, t.values)
    want = ref_gpu.csf3_add(as_tuple(fa), as_tuple(fb))
    for got_arr, want_arr, name in zip(as_tuple(f)[1:6], want[1:6], ("i_idx", "j_ptr", "j_idx", "k_ptr", "k_idx")):
        assert torch.equal(got_arr, want_arr), f"CSF3 {name} differs from the reference's GPU kernel"
    assert torch.equal(f.values.view(torch.int32), want[6].view(torch.int32))


def check_spgemm(nacho, ref_gpu, oracle, ta, tb):
    import torch
    a, b = dev(ta), dev(tb)
    got = nacho.gpu_spgemm_f32(as_csr_gpu(nacho, a), as_csr_gpu(nacho, b))
    want = ref_gpu.spgemm(a, b)
    same_csr(got, want, exact_values=False)
    # both sides against the float64 product, entry by entry
    _, v64, abs64, _ = oracle.spgemm(synth_csr(ta), synth_csr(tb), 8, extras=True)
    bound = 1e-5 * abs64 + 1e-30
    assert np.all(np.abs(got.values.cpu().numpy().astype(np.float64) - v64) <= bound)
    assert np.all(np.abs(want[4].cpu().numpy().astype(np.float64) - v64) <= 4 * bound), "the reference itself is off"


def test_spgemm_random(nacho, ref_gpu, oracle):
    from nacho_b200 import synth
    check_spgemm(nacho, ref_gpu, oracle, synth.random_csr(500, 400, 0.03, 21), synth.random_csr(400, 300, 0.03, 22))


def test_spgemm_laplacian_and_rmat(nacho, ref_gpu, oracle):
    """Configuration 4b on a 64 x 64 grid and configuration 4a at scale 11 (B = A^T, rows in every
    bin of the product's SpGEMM; about 1.3 M products)."""
    from nacho_b200 import synth
    lap = synth.laplacian_csr(64)
    check_spgemm(nacho, ref_gpu, oracle, lap, lap)
    ta = synth.rmat_csr(scale=11, seed=4011)
    check_spgemm(nacho, ref_gpu, oracle, ta, synth.transpose_csr(ta))


def check_sssmm(nacho, ref_gpu, oracle, ta, tb, tc):
    """Masked product against the reference's own emitted sssmm GPU kernel: same structure (the mask's
    positions a product reaches), values of both sides within 1e-5 of sum|a b c| of a float64 sum."""
    a, b, c = dev(ta), dev(tb), dev(tc)
    if not hasattr(ref_gpu.lib, "ref_gpu_sssmm"):
        pytest.skip("the checker library was built before the reference's sssmm kernel was added to it")
    got = nacho.gpu_sssmm_f32(as_csr_gpu(nacho, a), as_csr_gpu(nacho, b), as_csr_gpu(nacho, c))
    want = ref_gpu.sssmm(a, b, c)
    same_csr(got, want, exact_values=False)
    ha, hb, hc = synth_csr(ta), synth_csr(tb), synth_csr(tc)
    full, v64, abs64, _ = oracle.spgemm(ha, hb, 8, extras=True)
    key = lambda m: np.repeat(np.arange(m.rows, dtype=np.int64), np.diff(m.row_ptr)) * m.cols + m.col
    _, i_f, i_c = np.intersect1d(key(full), key(hc), return_indices=True)
    x64 = v64[i_f] * hc.val[i_c].astype(np.float64)
    bound = 1e-5 * abs64[i_f] * np.abs(hc.val[i_c]) + 1e-30
    assert len(x64) == got.values.numel()
    assert np.all(np.abs(got.values.cpu().numpy().astype(np.float64) - x64) <= bound)
    assert np.all(np.abs(want[4].cpu().numpy().astype(np.float64) - x64) <= 4 * bound), "the reference itself is off"


def test_sssmm_against_the_reference_gpu_kernel(nacho, ref_gpu, oracle):
    from nacho_b200 import synth
    check_sssmm(nacho, ref_gpu, oracle, synth.random_csr(500, 400, 0.03, 31), synth.random_csr(400, 300, 0.03, 32),
                synth.random_csr(500, 300, 0.05, 33))
    ta = synth.rmat_csr(scale=11, seed=4111)   # A A masked by A, as the reference's sssmm benchmark runs square matrices
    check_sssmm(nacho, ref_gpu, oracle, ta, ta, ta)
    lap = synth.laplacian_csr(48)
    check_sssmm(nacho, ref_gpu, oracle, lap, lap, lap)


def test_randomised_shapes_against_the_reference_gpu_kernels(nacho, ref_gpu):
    """Forty seeded draws of shape, density and row skew through all four CSR kernels of both
    sides: index arrays equal, add / multiply values bit-equal, SpGEMM values close (both sides
    sum in no fixed order). Operands are kept non-empty."""
    import torch
    from nacho_b200 import synth
    rng = np.random.default_rng(2024)
    for case in range(40):
        rows = int(rng.integers(1, 3000))
        cols = int(rng.integers(2, 3000))
        density = float(rng.choice([0.002, 0.01, 0.05, 0.2])) if rows * cols > 4000 else 0.3
        if case % 3 == 0:   # skewed rows: lognormal lengths
            lengths = np.minimum(np.round(rng.lognormal(0, 2.0, rows) * density * cols).astype(np.int64), cols)
        else:
            lengths = rng.binomial(cols, density, rows)
        lengths[int(rng.integers(0, rows))] = max(1, int(lengths.max()))   # at least one stored entry
        ops = [dev(synth.csr_from_lengths(np.maximum(lengths if k == 0 else rng.permutation(lengths), 0), cols, 100 * case + k))
               for k in range(3)]
        ga, gb, gc = (as_csr_gpu(nacho, t) for t in ops)
        same_csr(nacho.gpu_csr_add_f32(ga, gb), ref_gpu.csr_add(ops[0], ops[1]))
        same_csr(nacho.gpu_csr_mul_f32(ga, gb), ref_gpu.csr_mul(ops[0], ops[1]))
        same_csr(nacho.gpu_csr_add_3_f32(ga, gb, gc), ref_gpu.csr_add_3(*ops))
        if case % 2 == 0:   # C = A * B^T-shaped product: B gets `cols` rows
            tb = dev(synth.random_csr(cols, int(rng.integers(2, 2000)), float(rng.choice([0.005, 0.03])) , 7000 + case))
            if tb[3].numel() == 0:
                continue
            got = nacho.gpu_spgemm_f32(ga, as_csr_gpu(nacho, tb))
            want = ref_gpu.spgemm(ops[0], tb)
            same_csr(got, want, exact_values=False)
            assert torch.allclose(got.values, want[4], rtol=1e-4, atol=1e-5)
