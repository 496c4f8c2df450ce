"""CPU: the shared library loads and exports every symbol include/custom_cuda_b200.h
declares; the Python module exposes the reference's `_native` names."""

import ctypes
import pathlib
import re

ROOT = pathlib.Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "custom_cuda_b200.h"
LIB = ROOT / "custom_cuda_kernals_b200" / "libcustom_cuda_b200.so"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(?:int32_t|int64_t)\s+(\w+)\s*\(", text)))


def test_header_declares_the_reference_launchers():
    names = declared_symbols()
    for want in ("launch_rmsnorm_residual_fwd", "launch_swiglu_fwd", "launch_rope_fwd",
                 "launch_fp8_quant_block_fwd", "launch_fp8_quant_tensor_fwd", "launch_matmul_add_bias_fwd",
                 "launch_linear_ce_chunk_update"):
        assert want in names


def test_library_exports_every_declared_symbol():
    assert LIB.exists(), "build first: python -m custom_cuda_kernals_b200._build"
    lib = ctypes.CDLL(str(LIB))
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_native_module_has_reference_names():
    import custom_cuda
    from custom_cuda import _native
    for name in ("rmsnorm_residual_fwd", "swiglu_fwd", "rope_fwd", "linear_ce_chunk_update",
                 "matmul_add_bias_fwd", "fp8_quant_block_fwd", "fp8_quant_tensor_fwd"):   # src/lib.rs:13-27
        assert callable(getattr(_native, name))
    from custom_cuda.kernels.linear_cross_entropy import DEFAULT_CHUNK_SIZE
    assert DEFAULT_CHUNK_SIZE == 4096
    import inspect

    from custom_cuda.kernels.fp8_quant import fp8_quant
    from custom_cuda.kernels.linear_cross_entropy import linear_cross_entropy
    from custom_cuda.kernels.rmsnorm_residual import rmsnorm_residual
    assert list(inspect.signature(rmsnorm_residual).parameters) == ["x", "residual", "weight", "eps"]
    assert inspect.signature(rmsnorm_residual).parameters["eps"].default == 1e-6
    assert list(inspect.signature(fp8_quant).parameters) == ["x", "fp8_format", "granularity"]
    sig = inspect.signature(linear_cross_entropy)
    assert list(sig.parameters) == ["hidden", "weight", "targets", "ignore_index", "reduction", "chunk_size"]
    assert sig.parameters["ignore_index"].default == -100 and sig.parameters["reduction"].default == "mean"


def test_validation_runs_without_a_gpu():
    import pytest
    import torch

    from custom_cuda.kernels.fp8_quant import fp8_quant
    from custom_cuda.kernels.swiglu import swiglu
    with pytest.raises(ValueError, match="must be a CUDA tensor"):
        swiglu(torch.randn(4), torch.randn(4))
    with pytest.raises(ValueError, match="fp8_format"):
        fp8_quant(torch.randn(4, 4), "e3m4")
    with pytest.raises(ValueError, match="granularity"):
        fp8_quant(torch.randn(4, 4), "e4m3", "row")
