"""CPU suite: the C-ABI library loads without a GPU and exports every function that
include/nacho_b200.h declares; the Python mirror exposes the reference's names."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "nacho_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nb200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(os.path.join(ROOT, "nacho_b200", "libnacho_b200.so"))
    names = declared_functions()
    assert len(names) >= 10
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_binding_covers_every_declared_symbol():
    from nacho_b200 import _capi
    assert sorted(_capi.PROTOTYPES) == declared_functions()
    assert _capi.lib.nb200_version() == 100
    assert _capi.lib.nb200_strerror(4).decode() == "result arrays too small"


def test_mirror_surface():
    import nacho_b200
    from nacho_b200 import nacho
    for name in ("CSR_gpu", "gpu_csr_add_f32", "gpu_csr_mul_f32", "to_csr", "to_coo3", "to_csf3"):
        assert hasattr(nacho, name), name
    nacho_b200.install_as_nacho()
    import nacho as installed
    assert installed is nacho
