"""nacho_b200: B200 (sm_100a) implementation of nacho's sparse-kernel hot path.

``nacho_b200.nacho`` mirrors the reference's Python package (tensor classes ``CSR_gpu`` /
``COO3_gpu`` / ``CSF3_gpu``, operators ``gpu_<kernel>_f32`` and the ``to_*`` converters);
``install_as_nacho()`` registers it under the name ``nacho`` so that scripts written against
the reference run unchanged. All compute goes through ``libnacho_b200.so``.
"""
from __future__ import annotations

import sys

from . import _capi  # noqa: F401  (raises if the CUDA library is missing)
from . import nacho  # noqa: F401

__all__ = ["nacho", "install_as_nacho"]


def install_as_nacho() -> None:
    """Makes ``import nacho`` resolve to this package's mirror of the reference API."""
    sys.modules.setdefault("nacho", nacho)
    sys.modules.setdefault("nacho.nacho_ext", nacho.nacho_ext)
    sys.modules.setdefault("nacho.convert", nacho.convert)
