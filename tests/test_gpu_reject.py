"""GPU: argument validation - every rejection is a ValueError raised before any launch
(tests/test_*_kernel.py rejection tests; src/kernels/error.rs:9-36)."""

import pytest
import torch

from tests.gpu_util import DEV

pytestmark = pytest.mark.gpu


def test_cpu_tensors_rejected():
    from custom_cuda import _native
    from custom_cuda.kernels import fp8_quant, linear_cross_entropy, matmul_add_bias, rmsnorm_residual, rope, swiglu
    x = torch.randn(4, 8)
    with pytest.raises(ValueError, match="must be a CUDA tensor"):
        rmsnorm_residual.rmsnorm_residual(x, x, torch.randn(8))
    with pytest.raises(ValueError):
        swiglu.swiglu(x, x)
    with pytest.raises(ValueError):
        fp8_quant.fp8_quant(x, "e4m3", "block")
    with pytest.raises(ValueError):
        matmul_add_bias.matmul_add_bias(x, torch.randn(3, 8))
    with pytest.raises(ValueError):
        linear_cross_entropy.linear_cross_entropy(x, torch.randn(10, 8), torch.randint(0, 10, (4,)))
    q = torch.randn(1, 4, 2, 16)
    with pytest.raises(ValueError):
        _native.rope_fwd(q, q, torch.randn(4, 8), torch.randn(4, 8), torch.empty_like(q), torch.empty_like(q))


def test_non_contiguous_rejected():
    from custom_cuda.kernels.rmsnorm_residual import rmsnorm_residual
    from custom_cuda.kernels.swiglu import swiglu
    wide = torch.randn(2, 8, 32, device=DEV)
    x = wide[..., ::2]
    w = torch.randn(16, device=DEV)
    with pytest.raises(ValueError, match="contiguous"):
        rmsnorm_residual(x, x, w)
    with pytest.raises(ValueError, match="contiguous"):
        swiglu(x, x)


def test_dtype_and_shape_mismatch_rejected():
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    from custom_cuda.kernels.rmsnorm_residual import rmsnorm_residual
    from custom_cuda.kernels.rope import rope
    x = torch.randn(4, 16, device=DEV)
    with pytest.raises(ValueError, match="dtype mismatch"):
        rmsnorm_residual(x, x.half(), torch.randn(16, device=DEV))
    with pytest.raises(ValueError, match="shape mismatch"):
        rmsnorm_residual(x, x, torch.randn(15, device=DEV))
    with pytest.raises(ValueError, match="unsupported dtype"):
        rmsnorm_residual(x.double(), x.double(), torch.randn(16, device=DEV).double())
    with pytest.raises(ValueError, match="shape mismatch"):
        matmul_add_bias(x, torch.randn(8, 15, device=DEV))
    q = torch.randn(1, 4, 2, 16, device=DEV)
    cos = torch.randn(4, 8, device=DEV)
    with pytest.raises(ValueError):
        rope(q, q.half(), cos, cos)
    with pytest.raises(ValueError):
        rope(q.half(), q.half(), cos.half(), cos.half())
    q15 = torch.randn(1, 4, 2, 15, device=DEV)
    with pytest.raises(ValueError, match="even"):
        rope(q15, q15, torch.randn(4, 7, device=DEV), torch.randn(4, 7, device=DEV))


def test_bad_strings_rejected():
    from custom_cuda.kernels.fp8_quant import fp8_quant
    from custom_cuda.kernels.linear_cross_entropy import linear_cross_entropy
    x = torch.randn(4, 8, device=DEV)
    with pytest.raises(ValueError):
        fp8_quant(x, "not_a_format", "block")
    with pytest.raises(ValueError):
        fp8_quant(x, "e4m3", "not_a_granularity")
    with pytest.raises(ValueError):
        linear_cross_entropy(x, torch.randn(10, 8, device=DEV),
                             torch.randint(0, 10, (4,), device=DEV), reduction="bogus")


def test_launch_follows_the_current_stream():
    """Work is queued on torch's current stream: a result produced on a side stream is
    correct after synchronising that stream only."""
    from custom_cuda.kernels.swiglu import swiglu
    side = torch.cuda.Stream()
    g = torch.randn(1 << 20, device=DEV)
    u = torch.randn(1 << 20, device=DEV)
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        y = swiglu(g, u)
    side.synchronize()
    torch.testing.assert_close(y, torch.nn.functional.silu(g) * u, rtol=1e-4, atol=1e-5)
