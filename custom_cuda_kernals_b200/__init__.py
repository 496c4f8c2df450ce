"""B200 (sm_100a) kernels for the Llama-block op set, behind the reference's
``custom_cuda.kernels.*`` Python API.

Layers (the reference's four, custom_cuda README.md:53-78, rebuilt):

    kernels/<op>.py      public API: allocates outputs, calls ``_native``
    _native              C++ module: validation, current-stream lookup, FFI
    libcustom_cuda_b200  ``extern "C" launch_*`` launchers (include/custom_cuda_b200.h)
    csrc/*.cu            the CUDA kernels

There is no CPU or library fallback: importing ``_native`` fails if the
extension has not been built (``python -m custom_cuda_kernals_b200._build``).
"""

__version__ = "0.1.0"

from . import _native  # noqa: F401  (fails loudly when the extension is missing)
from . import kernels  # noqa: F401
