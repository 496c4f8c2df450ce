"""Same module layout as the reference's ``custom_cuda.kernels`` package."""

import importlib as _importlib
import sys as _sys

for _name in ("fp8_quant", "linear_cross_entropy", "matmul_add_bias", "moe_router", "rmsnorm_residual", "rope", "swiglu",
              "token_permute"):
    _mod = _importlib.import_module(f"custom_cuda_kernals_b200.kernels.{_name}")
    _sys.modules[f"{__name__}.{_name}"] = _mod
    globals()[_name] = _mod
