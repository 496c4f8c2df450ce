"""GPU parity: fp8_quant codes and scales, bit for bit against the CPU oracle
(block / tensor cases of baselines/fp8_quant.py plus the per-token mode)."""

import hashlib
import json
import pathlib

import pytest
import torch

from oracle import cases, ops, workloads
from tests.gpu_util import DEV

pytestmark = pytest.mark.gpu
DIGESTS = json.loads((pathlib.Path(__file__).parent / "golden" / "fp8_digests.json").read_text())


def _sha(t):
    return hashlib.sha256(t.contiguous().cpu().view(torch.uint8).numpy().tobytes()).hexdigest()


def _assert_bit_exact(x, fmt, gran):
    from custom_cuda.kernels.fp8_quant import fp8_quant
    want_codes, want_scale = ops.fp8_quant(x, fmt, gran)
    codes, scale = fp8_quant(x.to(DEV), fmt, gran)
    assert codes.dtype == ops.FP8_TORCH_DTYPE[fmt] and codes.shape == x.shape
    assert scale.dtype == torch.float32
    assert scale.numel() == want_scale.numel()
    assert torch.equal(scale.cpu().reshape(-1), want_scale.reshape(-1)), "scales differ"
    diff = codes.cpu().view(torch.uint8) != want_codes.view(torch.uint8)
    assert not diff.any(), f"{int(diff.sum())} of {diff.numel()} codes differ"
    return codes, scale


@pytest.mark.parametrize("case", cases.FP8_CASES, ids=lambda c: c.name)
def test_fp8_cases_bit_exact(case):
    x = cases.fp8_inputs(case)
    codes, scale = _assert_bit_exact(x, case.fp8_format, case.granularity)
    if case.granularity == "block":
        assert scale.shape == (ops.ceil_div(case.m, 128), ops.ceil_div(case.n, 128))
    elif case.granularity == "tensor":
        assert scale.shape == (1,)
    else:
        assert scale.shape == (case.m, 1)
    if case.name in DIGESTS:   # the reference's own baseline output, hashed
        assert _sha(codes) == DIGESTS[case.name]["codes"]
        assert _sha(scale.reshape(-1)) == DIGESTS[case.name]["scale"]


@pytest.mark.parametrize("gran", ["token", "block", "tensor"])
@pytest.mark.parametrize("shape", [(3, 16), (5, 48), (7, 1000), (130, 272), (2, 40000), (1, 70000), (4, 140000)])
def test_fp8_odd_shapes(gran, shape):
    g = torch.Generator().manual_seed(shape[1])
    x = (torch.randn(shape, generator=g) * 3).to(torch.bfloat16)
    _assert_bit_exact(x, "e4m3", gran)
    _assert_bit_exact(x.float(), "e5m2", gran)


def test_fp8_special_values():
    from custom_cuda.kernels.fp8_quant import fp8_quant
    for gran in ("token", "block", "tensor"):
        z, s = fp8_quant(torch.zeros(256, 256, device=DEV), "e4m3", gran)
        assert torch.all(z.float() == 0) and torch.isfinite(s).all() and torch.all(s > 0)
    # tiny magnitudes (scale clamps at 1e-12), negative zero, a wide dynamic range per row
    x = torch.tensor([[1e-30, -1e-30, 0.0, -0.0] * 4, [1e-3, -7.0, 448.0, 3e4] * 4, [1e-14, 2e-13, -3e-13, 0.0] * 4])
    for gran in ("token", "block", "tensor"):
        _assert_bit_exact(x, "e4m3", gran)
        _assert_bit_exact(x, "e5m2", gran)


def test_fp8_config2c_full_size_bit_exact_and_roundtrip():
    """Benchmark config 2c: [8192, 4096] bf16 with 0.1 % outliers x50, per-token e4m3."""
    x = workloads.fp8_activations()
    codes, scale = _assert_bit_exact(x, "e4m3", "token")
    deq = codes.float() * scale
    xs = x.to(DEV).float() / scale
    err = (deq / scale - xs).abs()
    bound = 2.0 * (0.5 * 0.125 * xs.abs() + 2.0 ** -6)       # tests/test_fp8_quant.py:56-85
    assert torch.all(err <= bound)
    assert float((codes.float().abs().amax(dim=1) == 448).float().mean()) == 1.0   # every row uses the full range


def test_fp8_block_beats_tensor_on_dynamic_range():
    from custom_cuda.kernels.fp8_quant import fp8_quant
    g = torch.Generator().manual_seed(0)
    x = torch.zeros(256, 256)
    x[:128, :128] = torch.randn(128, 128, generator=g) * 0.01
    x[128:, 128:] = torch.randn(128, 128, generator=g) * 100.0
    xd = x.to(DEV)
    ct, st = fp8_quant(xd, "e4m3", "tensor")
    cb, sb = fp8_quant(xd, "e4m3", "block")
    err_t = (ops.fp8_dequant(ct.cpu(), st.cpu(), "tensor")[:128, :128] - x[:128, :128]).abs().mean()
    err_b = (ops.fp8_dequant(cb.cpu(), sb.cpu(), "block")[:128, :128] - x[:128, :128]).abs().mean()
    assert err_b < err_t
