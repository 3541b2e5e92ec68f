"""CPU suite: the file readers and the coalescing step in front of the converters (runs on CPU
tensors here; the same torch code runs on the GPU when asked for device="cuda")."""
import numpy as np
import pytest
import torch


def test_matrix_market_general_and_symmetric(tmp_path):
    from nacho_b200.nacho import io
    p = tmp_path / "g.mtx"
    p.write_text("%%MatrixMarket matrix coordinate real general\n% a comment\n3 4 3\n1 1 1.5\n3 2 -2\n2 4 0.25\n")
    m = io.parse2D(str(p))
    assert (m.N, m.M) == (3, 4)
    assert m.row.tolist() == [0, 2, 1] and m.col.tolist() == [0, 1, 3] and m.data.tolist() == [1.5, -2.0, 0.25]
    assert m.row.dtype == torch.int32 and m.data.dtype == torch.float32
    for sym, sign in (("symmetric", 1.0), ("skew-symmetric", -1.0)):
        p = tmp_path / f"{sym}.mtx"
        p.write_text(f"%%MatrixMarket matrix coordinate real {sym}\n3 3 3\n1 1 2\n2 1 3\n3 2 4\n")
        m = io.parse2D(str(p))
        # mirrored entries are appended after the stored ones, diagonal entries are not repeated
        assert m.row.tolist() == [0, 1, 2, 0, 1] and m.col.tolist() == [0, 0, 1, 1, 2]
        assert m.data.tolist() == [2.0, 3.0, 4.0, sign * 3.0, sign * 4.0]
    bad = tmp_path / "bad.mtx"
    bad.write_text("%%MatrixMarket matrix coordinate complex general\n1 1 1\n1 1 1 0\n")
    with pytest.raises(ValueError):
        io.parse2D(str(bad))


def test_frostt_reader_and_coalescing(tmp_path):
    from nacho_b200.nacho import convert, io
    p = tmp_path / "t.tns"
    p.write_text("2 1 3 1.0\n1 1 1 2.0\n2 1 3 0.5\n1 2 1 -1.0\n")
    t = io.parse3D_i32_f32(str(p), 2, 2, 3)
    assert (t.N, t.M, t.K, t.nnz) == (2, 2, 3, 4)
    assert t.row.tolist() == [1, 0, 1, 0] and t.dep.tolist() == [2, 0, 2, 0]
    with pytest.raises(ValueError):
        io.parse3D_i32_f32(str(p), 1, 2, 3)
    coords, vals = io.coalesce_coo3(t.row, t.col, t.dep, t.data, (2, 2, 3), device="cpu")
    assert coords.tolist() == [[0, 0, 0], [0, 1, 0], [1, 0, 2]] and vals.tolist() == [2.0, -1.0, 1.5]
    # the level build accepts what coalescing returns
    lv = convert.csf3_levels_device(coords[:, 0], coords[:, 1], coords[:, 2])
    assert [x.tolist() for x in lv] == [[0, 1], [0, 2, 3], [0, 1, 0], [0, 1, 2, 3], [0, 0, 2]]


def test_coalesce_matches_numpy_on_random_input():
    from nacho_b200.nacho import io
    rng = np.random.default_rng(3)
    n, shape = 5000, (40, 30)
    r, c = rng.integers(0, shape[0], n), rng.integers(0, shape[1], n)
    v = rng.integers(-8, 9, n).astype(np.float32)          # small integers: sums are exact in any order
    i, j, vals, shp = io.coalesce_coo(r, c, v, shape, device="cpu")
    dense = np.zeros(shape, np.float32)
    np.add.at(dense, (r, c), v)
    keys = np.unique(r * shape[1] + c)
    assert np.array_equal(i.numpy().astype(np.int64) * shape[1] + j.numpy(), keys)
    assert np.array_equal(vals.numpy(), dense.reshape(-1)[keys]) and shp.tolist() == list(shape)
