"""Drop-in alias: ``custom_cuda`` -> ``custom_cuda_kernals_b200``.

Code written against the reference project imports ``custom_cuda.kernels.<op>``
and ``custom_cuda._native``; this package re-exports the B200 implementation
under those names so such code runs unchanged.
"""

import sys as _sys

import custom_cuda_kernals_b200 as _impl
from custom_cuda_kernals_b200 import _native

__version__ = _impl.__version__
_sys.modules[__name__ + "._native"] = _native
