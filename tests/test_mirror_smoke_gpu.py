"""GPU suite: the mirror package used the way the reference's own smoke script uses ``nacho``
(tests/smoke.py:275-303 of the reference): ``install_as_nacho()`` makes ``import nacho`` resolve to
the mirror, every one of the fifteen kernels the reference's compiler declares is looked up as
``nacho.gpu_<kernel>_f32``, fed through the reference's converters (``to_csr``, ``to_dcsr``,
``to_coo``, ``to_coo3``, ``to_csf3``) with its input shapes (200 x 180 at density 0.05; 900 draws in
40 x 30 x 25) and compared with the scipy / dictionary expression of the same operation under the
reference's absolute tolerance of 1e-4. None may be missing: a script written against the
reference's GPU half finds every name it calls.
"""
import zlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOLERANCE = 1e-4
ROWS, COLS, DENSITY = 200, 180, 0.05
SHAPE_3D = (40, 30, 25)

KERNELS = ["csr_add", "csr_add_3", "csr_mul", "dcsr_add", "dcsr_mul", "dcsr_mul_without_recursive_partitioning", "coo_add",
           "coo_mul", "coo_csr_add", "csf_add", "coo3d_add", "inner_prod", "inner_prod_coo", "spgemm", "sssmm"]


@pytest.fixture(scope="module")
def nacho():
    import torch
    assert torch.cuda.is_available(), "GPU suite needs a CUDA device"
    import nacho_b200
    nacho_b200.install_as_nacho()
    import nacho as installed
    return installed


def _matrix(rng, rows=ROWS, cols=COLS):
    import scipy.sparse as sp
    m = sp.random(rows, cols, density=DENSITY, format="csr", dtype=np.float32, random_state=rng)
    m.sort_indices()
    return m


def _tensor(rng):
    c = np.unique(np.stack([rng.integers(0, e, 900) for e in SHAPE_3D], axis=1), axis=0).astype(np.int32)
    return c, rng.uniform(-1, 1, len(c)).astype(np.float32)


def _torch_csr(m):
    import torch
    return torch.sparse_csr_tensor(torch.from_numpy(m.indptr.astype(np.int32)), torch.from_numpy(m.indices.astype(np.int32)),
                                   torch.from_numpy(m.data.astype(np.float32)), size=m.shape)


def _host(t):
    import torch
    torch.cuda.synchronize()
    return t.cpu().numpy()


def _csr_result(z):
    import scipy.sparse as sp
    return sp.csr_matrix((_host(z.values), _host(z.dim_j_indices), _host(z.dim_j_offsets)), shape=(int(z.shape[0]), int(z.shape[1])))


def _dcsr_result(z, shape):
    import scipy.sparse as sp
    rows, offsets = _host(z.dim_i_indices), _host(z.dim_j_offsets)
    lengths = np.zeros(shape[0] + 1, np.int64)
    lengths[rows + 1] = offsets[1:] - offsets[:-1]
    return sp.csr_matrix((_host(z.values), _host(z.dim_j_indices), np.cumsum(lengths)), shape=shape)


def _coo_result(z):
    import scipy.sparse as sp
    return sp.coo_matrix((_host(z.values), (_host(z.dim_i_indices), _host(z.dim_j_indices))),
                         shape=(int(z.shape[0]), int(z.shape[1]))).tocsr()


def _close(actual, expected):
    if isinstance(actual, dict):
        return actual.keys() == expected.keys() and all(abs(actual[k] - expected[k]) < TOLERANCE for k in expected)
    actual, expected = actual.tocsr(), expected.tocsr()
    expected.eliminate_zeros()
    diff = abs(actual - expected)
    return diff.nnz == 0 or diff.max() < TOLERANCE


def _sum3(ca, va, cb, vb):
    out = {tuple(int(x) for x in c): float(v) for c, v in zip(ca, va)}
    for c, v in zip(cb, vb):
        k = tuple(int(x) for x in c)
        out[k] = out.get(k, 0.0) + float(v)
    return out


def _dot3(ca, va, cb, vb):
    a = {tuple(int(x) for x in c): float(v) for c, v in zip(ca, va)}
    return sum(a[k] * float(v) for c, v in zip(cb, vb) if (k := tuple(int(x) for x in c)) in a)


@pytest.mark.parametrize("name", KERNELS)
def test_kernel_through_the_installed_package(nacho, name):
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    fn = getattr(nacho, f"gpu_{name}_f32", None)
    assert fn is not None, f"nacho.gpu_{name}_f32 is missing from the mirror"
    dev = "cuda"
    csr = lambda m: nacho.to_csr(_torch_csr(m), dev)
    dcsr = lambda m: nacho.to_dcsr(_torch_csr(m), dev)
    coo = lambda m: nacho.to_coo(_torch_csr(m).to_sparse_coo(), dev)
    if name in ("csr_add", "csr_mul"):
        a, b = _matrix(rng), _matrix(rng)
        actual, expected = _csr_result(fn(csr(a), csr(b))), (a + b if name == "csr_add" else a.multiply(b))
    elif name == "csr_add_3":
        a, b, c = _matrix(rng), _matrix(rng), _matrix(rng)
        actual, expected = _csr_result(fn(csr(a), csr(b), csr(c))), a + b + c
    elif name.startswith("dcsr"):
        a, b = _matrix(rng), _matrix(rng)
        actual, expected = _dcsr_result(fn(dcsr(a), dcsr(b)), a.shape), (a + b if name == "dcsr_add" else a.multiply(b))
    elif name in ("coo_add", "coo_mul"):
        a, b = _matrix(rng), _matrix(rng)
        actual, expected = _coo_result(fn(coo(a), coo(b))), (a + b if name == "coo_add" else a.multiply(b))
    elif name == "coo_csr_add":
        a, b = _matrix(rng), _matrix(rng)
        actual, expected = _csr_result(fn(csr(a), coo(b))), a + b
    elif name in ("spgemm", "sssmm"):
        a, b = _matrix(rng, ROWS, COLS), _matrix(rng, COLS, ROWS)
        if name == "spgemm":
            actual, expected = _csr_result(fn(csr(a), csr(b))), a @ b
        else:
            c = _matrix(rng, ROWS, ROWS)
            actual, expected = _csr_result(fn(csr(a), csr(b), csr(c))), (a @ b).multiply(c)
    else:
        (ca, va), (cb, vb) = _tensor(rng), _tensor(rng)
        if name == "coo3d_add":
            z = fn(nacho.to_coo3(ca, va, SHAPE_3D, dev), nacho.to_coo3(cb, vb, SHAPE_3D, dev))
            keys = zip(_host(z.dim_i_indices), _host(z.dim_j_indices), _host(z.dim_k_indices))
            actual, expected = {tuple(int(x) for x in k): float(v) for k, v in zip(keys, _host(z.values))}, _sum3(ca, va, cb, vb)
        elif name == "csf_add":
            z = fn(nacho.to_csf3(ca, va, SHAPE_3D, dev), nacho.to_csf3(cb, vb, SHAPE_3D, dev))
            i_idx, jp, j_idx, kp, k_idx, vals = (_host(x) for x in (z.dim_i_indices, z.dim_j_offsets, z.dim_j_indices,
                                                                   z.dim_k_offsets, z.dim_k_indices, z.values))
            actual = {(int(i), int(j_idx[q]), int(k_idx[p])): float(vals[p])
                      for n, i in enumerate(i_idx) for q in range(jp[n], jp[n + 1]) for p in range(kp[q], kp[q + 1])}
            expected = _sum3(ca, va, cb, vb)
        else:
            conv = nacho.to_csf3 if name == "inner_prod" else nacho.to_coo3
            z = fn(conv(ca, va, SHAPE_3D, dev), conv(cb, vb, SHAPE_3D, dev))
            actual, expected = {(): float(_host(z.values)[0])}, {(): _dot3(ca, va, cb, vb)}
    assert _close(actual, expected), f"gpu_{name}_f32 differs from the scipy expression"


def test_cpu_half_is_absent_by_design(nacho):
    """The product has no CPU kernels: the reference's ``cpu_*`` names do not exist here, and asking
    a converter for a CPU tensor raises instead of handing out a class without kernels."""
    assert not any(hasattr(nacho, f"cpu_{k}_f32") for k in KERNELS)
    with pytest.raises(ValueError):
        nacho.to_csr(_torch_csr(_matrix(np.random.default_rng(1))), "cpu")
