"""Generates ``family_golden.npz``: results of the reference's own CPU kernels for the rest of its
element-wise family (coo_add, coo_mul, coo_csr_add, dcsr_add, dcsr_mul) and its two inner products,
on the operands already stored in ``csr_golden.npz`` / ``tensor3_golden.npz``.

Run where the reference checker library exists (``make -C oracle ref REF=<reference checkout>``):
``python tests/golden/make_family_golden.py``. Only results are stored; the tests rebuild the
COO / DCSR operands from the stored CSR operands with the converters in ``oracle/cpu_oracle.py``.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from make_golden import csf3_levels  # noqa: E402
from oracle.cpu_oracle import COO3, CSF3, CSR, Reference, csr_to_coo, csr_to_dcsr  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ref = Reference()
    g = np.load(os.path.join(HERE, "csr_golden.npz"))
    out = {}
    cases = sorted({k.split(".")[0] for k in g.files})
    for case in cases:
        rows, cols = (int(x) for x in g[f"{case}.a.shape"])
        a = CSR(rows, cols, g[f"{case}.a.rp"], g[f"{case}.a.col"], g[f"{case}.a.val"])
        b = CSR(rows, cols, g[f"{case}.b.rp"], g[f"{case}.b.col"], g[f"{case}.b.val"])
        for op, fn in (("coo_add", ref.coo_add), ("coo_mul", ref.coo_mul)):
            z = fn(csr_to_coo(a), csr_to_coo(b))
            out[f"{case}.{op}.i"], out[f"{case}.{op}.j"], out[f"{case}.{op}.val"] = z.i, z.j, z.val
        z = ref.coo_csr_add(a, csr_to_coo(b))
        out[f"{case}.coo_csr_add.rp"], out[f"{case}.coo_csr_add.col"], out[f"{case}.coo_csr_add.val"] = z.row_ptr, z.col, z.val
        for op, fn in (("dcsr_add", ref.dcsr_add), ("dcsr_mul", ref.dcsr_mul)):
            z = fn(csr_to_dcsr(a), csr_to_dcsr(b))
            for fld in ("i_idx", "j_ptr", "j_idx", "val"):
                out[f"{case}.{op}.{fld}"] = getattr(z, fld)
    t = np.load(os.path.join(HERE, "tensor3_golden.npz"))
    for case in sorted({k.split(".")[0] for k in t.files}):
        dims = tuple(int(x) for x in t[f"{case}.dims"])
        ca, va = t[f"{case}.a.coords"].reshape(-1, 3), t[f"{case}.a.val"]
        cb, vb = t[f"{case}.b.coords"].reshape(-1, 3), t[f"{case}.b.val"]
        out[f"{case}.inner_prod_coo"] = np.array([ref.inner_prod_coo(COO3(dims, ca[:, 0], ca[:, 1], ca[:, 2], va),
                                                                     COO3(dims, cb[:, 0], cb[:, 1], cb[:, 2], vb))], np.float32)
        if len(va) and len(vb):  # the reference's CSF3 inner product reads past an empty operand's arrays: not run on those
            out[f"{case}.inner_prod"] = np.array([ref.inner_prod(CSF3(dims, *csf3_levels(ca), va), CSF3(dims, *csf3_levels(cb), vb))],
                                                 np.float32)
    np.savez_compressed(os.path.join(HERE, "family_golden.npz"), **out)
    print(f"wrote family_golden.npz ({len(out)} arrays), reference threads = {ref.threads()}")


if __name__ == "__main__":
    main()
