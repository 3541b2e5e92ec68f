"""GPU suite: seeded random draws of shape, density, row skew and extents through the masked SpGEMM
and through both routes of the CSF3 add, each held to the CPU oracle (structure exact; masked-product
values within 1e-5 of sum|a b c| of a float64 sum; CSF3 trees bit-for-bit)."""
import numpy as np
import pytest

from helpers import assert_same, csf3_levels, csr_from_gpu, csr_to_gpu, synth_csr
from oracle.cpu_oracle import CSF3

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nacho():
    import torch
    assert torch.cuda.is_available(), "GPU suite needs a CUDA device"
    from nacho_b200 import nacho as mod
    return mod


def test_masked_spgemm_random_draws(nacho, oracle):
    """Forty draws: up to 400 x 400 operands, B and the mask 50 to 3 million columns wide (every class
    of mask row: narrow, medium and wide bitmaps, spans beyond the largest bitmap, rows of a few
    products), uniform and log-normal row lengths."""
    from nacho_b200 import synth
    rng = np.random.default_rng(12345)
    key = lambda m: np.repeat(np.arange(m.rows, dtype=np.int64), np.diff(m.row_ptr)) * m.cols + m.col
    for case in range(40):
        rows, inner = int(rng.integers(1, 400)), int(rng.integers(1, 400))
        cols = int(rng.choice([50, 3000, 70000, 300000, 3_000_000]))
        densities = [float(rng.choice([0.002, 0.02, 0.2])) for _ in range(3)]

        def draw(r, c, d, seed):
            if case % 3 == 0:
                lengths = np.minimum(np.round(rng.lognormal(0, 2.0, r) * d * min(c, 5000)).astype(np.int64), c)
            else:
                lengths = rng.binomial(min(c, 20000), d, r)
            return synth.csr_from_lengths(np.maximum(lengths, 0), c, seed)

        a, b, c = (synth_csr(t) for t in (draw(rows, inner, densities[0], 3 * case), draw(inner, cols, densities[1], 3 * case + 1),
                                           draw(rows, cols, densities[2], 3 * case + 2)))
        z = csr_from_gpu(nacho.gpu_sssmm_f32(csr_to_gpu(a), csr_to_gpu(b), csr_to_gpu(c)))
        full, v64, abs64, _ = oracle.spgemm(a, b, 4, extras=True)
        common, i_f, i_c = np.intersect1d(key(full), key(c), return_indices=True)
        assert np.array_equal(key(z), common), f"case {case}: masked structure"
        want = v64[i_f] * c.val[i_c].astype(np.float64)
        bound = 1e-5 * abs64[i_f] * np.abs(c.val[i_c]) + 1e-30
        assert np.all(np.abs(z.val.astype(np.float64) - want) <= bound), f"case {case}: values"


def test_csf3_random_draws_both_routes(nacho, oracle, monkeypatch):
    """Thirty draws of extents (1 to 2^26, 1 to 2^16, 1 to 2^22), entry counts and overlap (disjoint,
    a third shared, identical coordinate sets), each through the route over expanded coordinates and
    through the two-level route."""
    from test_tensor3_gpu import _seeded, csf3_from_gpu
    rng = np.random.default_rng(54321)
    for case in range(30):
        dims = (int(rng.choice([1, 3, 40, 5000, 1 << 20, 1 << 26])), int(rng.choice([1, 7, 300, 1 << 16])),
                int(rng.choice([1, 9, 4096, 1 << 22])))
        n = int(min(rng.choice([10, 500, 20000, 150000]), max(1, dims[0] * dims[1] * dims[2] // 2)))
        (ca, va), (cb, vb) = _seeded(dims, n, 900 + case, overlap=float(rng.choice([0.0, 0.3, 1.0])))
        want = oracle.csf3_add(CSF3(dims, *csf3_levels(ca), va), CSF3(dims, *csf3_levels(cb), vb))
        for route in ("0", "1"):
            monkeypatch.setenv("NACHO_B200_CSF_TWO_LEVEL", route)
            got = csf3_from_gpu(nacho.gpu_csf_add_f32(nacho.to_csf3(ca, va, dims, "cuda"), nacho.to_csf3(cb, vb, dims, "cuda")))
            assert_same(got, want, f"case {case}, dims {dims}, route {route}")
