"""GPU parity against the committed golden vectors: outputs of the reference project's own
baselines (tests/golden/make_golden.py) on its seeded inputs, replayed through the CUDA path."""

import pathlib

import pytest
import torch

from oracle import cases, ops
from tests.gpu_util import DEV, check, to_dev

pytestmark = pytest.mark.gpu
golden = torch.load(pathlib.Path(__file__).parent / "golden" / "golden_small.pt")


def _keys(prefix):
    return [k for k in golden if k.startswith(prefix + "/") and "tables" not in k]


@pytest.mark.parametrize("key", _keys("rmsnorm"))
def test_rmsnorm_vs_reference_output(key):
    from custom_cuda.kernels.rmsnorm_residual import rmsnorm_residual
    c = cases.by_name(cases.NORM_CASES, key.split("/")[1])
    y, ro = rmsnorm_residual(*to_dev(*cases.norm_inputs(c)), c.eps)
    check(y, golden[key]["y"], c.dtype)
    check(ro, golden[key]["residual_out"], c.dtype)


@pytest.mark.parametrize("key", _keys("swiglu"))
def test_swiglu_vs_reference_output(key):
    from custom_cuda.kernels.swiglu import swiglu
    c = cases.by_name(cases.GLU_CASES, key.split("/")[1])
    check(swiglu(*to_dev(*cases.glu_inputs(c))), golden[key]["y"], c.dtype)


@pytest.mark.parametrize("key", _keys("rope"))
def test_rope_vs_reference_output(key):
    from custom_cuda.kernels.rope import rope
    c = cases.by_name(cases.ROPE_CASES, key.split("/")[1])
    q, k = rope(*to_dev(*cases.rope_inputs(c)))
    check(q, golden[key]["q"], c.dtype)
    check(k, golden[key]["k"], c.dtype)


@pytest.mark.parametrize("key", _keys("fp8"))
def test_fp8_vs_reference_output_bit_exact(key):
    from custom_cuda.kernels.fp8_quant import fp8_quant
    c = cases.by_name(cases.FP8_CASES, key.split("/")[1])
    codes, scale = fp8_quant(cases.fp8_inputs(c).to(DEV), c.fp8_format, c.granularity)
    assert torch.equal(codes.cpu().view(torch.uint8), golden[key]["codes"])
    assert torch.equal(scale.cpu().reshape(-1), golden[key]["scale"].reshape(-1))


@pytest.mark.parametrize("key", _keys("gemm"))
def test_gemm_vs_reference_output(key):
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    c = cases.by_name(cases.GEMM_CASES, key.split("/")[1])
    check(matmul_add_bias(*to_dev(*cases.gemm_inputs(c))), golden[key]["y"], c.dtype, ops.TOLERANCE_GEMM)


@pytest.mark.parametrize("key", _keys("lce"))
def test_lce_vs_reference_output(key):
    from custom_cuda.kernels.linear_cross_entropy import linear_cross_entropy
    c = cases.by_name(cases.LCE_CASES, key.split("/")[1])
    got = linear_cross_entropy(*to_dev(*cases.lce_inputs(c)), reduction=c.reduction).cpu()
    want64 = golden[key]["loss64"]
    if c.name.startswith("all_ignored"):
        assert torch.isnan(got).all() and torch.isnan(want64).all()
        return
    torch.testing.assert_close(got.double(), want64, rtol=1e-4, atol=1e-6)   # the reference's fp64 ground truth
