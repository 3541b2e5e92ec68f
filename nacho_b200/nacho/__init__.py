"""Mirror of the reference's ``nacho`` package (python/nacho/__init__.py:1-2): the extension
module's classes and operators, then the torch converters; the file readers the reference's runtime
registers beside them (runtime/register_runtime.cpp:20-39) and device-side coalescing live in ``io``."""
from .nacho_ext import *  # noqa: F401,F403
from .convert import to_csr, to_dcsr, to_coo, to_coo3, to_csf3  # noqa: F401
from .io import COO2D, COO3D_parsed, parse2D, parse3D_i32_f32, coalesce_coo, coalesce_coo3  # noqa: F401
from . import nacho_ext, convert, io  # noqa: F401
