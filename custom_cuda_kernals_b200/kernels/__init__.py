"""Python entry points, one module per op, mirroring ``custom_cuda.kernels``:
``kernels.<op>.<op>`` is the function (the package itself re-exports nothing,
so ``kernels.rope`` is the module, as in the reference).
"""

from . import fp8_quant, fused, linear_cross_entropy, matmul_add_bias, rmsnorm_residual, rope, swiglu  # noqa: F401
