"""nacho_b200: B200 (sm_100a) implementation of nacho's sparse-kernel hot path.

``nacho_b200.nacho`` mirrors the reference's Python package (tensor classes ``CSR_gpu`` /
``COO3_gpu`` / ``CSF3_gpu``, operators ``gpu_<kernel>_f32`` and the ``to_*`` converters);
``install_as_nacho()`` registers it under the name ``nacho`` so that scripts written against
the reference run unchanged. All compute goes through ``libnacho_b200.so``: the first use of
``nacho_b200.nacho`` (or ``nacho_b200._capi``) loads it and raises if it is missing or does not
export the whole C ABI -- there is no fallback. ``nacho_b200.build`` and ``nacho_b200.synth``
import without the library, so that it can be (re)built from a clean tree.
"""
from __future__ import annotations

import importlib
import sys

__all__ = ["nacho", "install_as_nacho"]

_LAZY = ("_capi", "nacho", "shard", "host")


def __getattr__(name):
    if name in _LAZY:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def install_as_nacho() -> None:
    """Makes ``import nacho`` resolve to this package's mirror of the reference API."""
    mirror = importlib.import_module(f"{__name__}.nacho")
    sys.modules.setdefault("nacho", mirror)
    sys.modules.setdefault("nacho.nacho_ext", mirror.nacho_ext)
    sys.modules.setdefault("nacho.convert", mirror.convert)
