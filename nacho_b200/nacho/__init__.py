"""Mirror of the reference's ``nacho`` package (python/nacho/__init__.py:1-2): the extension
module's classes and operators, then the torch converters."""
from .nacho_ext import *  # noqa: F401,F403
from .convert import to_csr, to_dcsr, to_coo, to_coo3, to_csf3  # noqa: F401
from . import nacho_ext, convert  # noqa: F401
