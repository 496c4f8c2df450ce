"""GPU: the GEMM epilogue that leaves row statistics for the op after it, and the two consumers.

``matmul_add_bias_stats`` must store bit for bit what ``matmul_add_bias`` /
``matmul_add_bias_residual`` store, and its statistics must be exactly the canonical ones (one
fp32 FMA chain per row and 256-column tile, columns ascending; a maximum has no order).  Then

  * ``fp8_quant_token_from_amax(y, row_amax)`` == ``fp8_quant(y, "token")`` bit for bit, and
  * ``rmsnorm_from_stats(y, row_sumsq, w)`` == the norm's rounding chain evaluated with the
    canonical statistic, bit for bit; against ``rmsnorm(y, w)`` (same chain, its own summation
    order) it may differ only where the statistic moved by an ulp: at most 1e-3 of the elements,
    each by at most two units in the last place of the storage type (one from the rounding of the
    normalised value, which the multiplication by the weight and the second rounding can double).

These are the steps either side of o_proj and down_proj in the reference's decoder block
(examples/llama_block.py:163-172); the reference has no fused form, so the unfused chain of this
library - itself checked against the oracle - is the comparator."""

import pytest
import torch

from tests.gpu_util import DEV, device_status_clean

pytestmark = pytest.mark.gpu

SHAPES = [(300, 512, 1024), (1000, 1024, 4096), (130, 64, 264), (77, 128, 256), (4096, 4096, 4096), (1024, 256, 8)]


def _inputs(m, k, n, dtype, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = torch.randn(m, k, device=DEV, generator=g).to(dtype)
    w = (k ** -0.5 * torch.randn(n, k, device=DEV, generator=g)).to(dtype)
    b = (0.1 * torch.randn(n, device=DEV, generator=g)).to(dtype)
    r = torch.randn(m, n, device=DEV, generator=g).to(dtype)
    gw = (1 + 0.1 * torch.randn(n, device=DEV, generator=g)).to(dtype)
    return x, w, b, r, gw


def _canonical_sumsq(y):
    """One fp32 chain per row and 256-column tile, columns ascending (v * v is exact in fp32 for
    16-bit v, so fma(v, v, s) == s + v * v)."""
    m, n = y.shape
    v = y.float()
    tiles = (n + 255) // 256
    out = torch.zeros(tiles, m, device=y.device)
    for t in range(tiles):
        s = torch.zeros(m, device=y.device)
        for c in range(256 * t, min(n, 256 * t + 256)):
            s = s + v[:, c] * v[:, c]
        out[t] = s
    return out


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("with_residual", [True, False])
def test_stats_epilogue_and_its_consumers(shape, dtype, with_residual):
    from custom_cuda.kernels.fp8_quant import fp8_quant
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias
    from custom_cuda_kernals_b200.kernels.fused import (fp8_quant_token_from_amax, matmul_add_bias_residual,
                                                        matmul_add_bias_stats, rmsnorm_from_stats)
    from custom_cuda_kernals_b200.kernels.rmsnorm_residual import rmsnorm
    m, k, n = shape
    x, w, b, r, gw = _inputs(m, k, n, dtype, seed=m + n)
    res = r if with_residual else None
    want = matmul_add_bias_residual(x, w, b, r) if with_residual else matmul_add_bias(x, w, b)
    poison = 7.0
    y, ss, am = matmul_add_bias_stats(x, w, b, res, sumsq=True, amax=True)
    assert torch.equal(y, want)                                              # same stored values, bit for bit
    assert ss.shape == am.shape == ((n + 255) // 256, m)
    assert torch.equal(ss, _canonical_sumsq(y))                              # the canonical statistic, bit for bit
    pad = torch.zeros(m, ss.shape[0] * 256, device=DEV)
    pad[:, :n] = y.float().abs()
    assert torch.equal(am, pad.view(m, -1, 256).amax(dim=2).t().contiguous())
    # only one of the two, the other untouched
    y2, ss2, none = matmul_add_bias_stats(x, w, b, res, sumsq=True, amax=False)
    assert none is None and torch.equal(y2, y) and torch.equal(ss2, ss)
    del poison

    if n % 8 == 0:
        codes, scale = fp8_quant_token_from_amax(y, am)
        codes_w, scale_w = fp8_quant(y, "e4m3", "token")
        assert torch.equal(codes.view(torch.uint8), codes_w.view(torch.uint8)) and torch.equal(scale, scale_w)
        c5, s5 = fp8_quant_token_from_amax(y, am, "e5m2")
        c5w, s5w = fp8_quant(y, "e5m2", "token")
        assert torch.equal(c5.view(torch.uint8), c5w.view(torch.uint8)) and torch.equal(s5, s5w)

        eps = 1e-5
        h = rmsnorm_from_stats(y, ss, gw, eps)
        total = torch.zeros(m, device=DEV)
        for t in range(ss.shape[0]):
            total = total + ss[t]
        # tensor / tensor is an IEEE division on the GPU; tensor / python-scalar is a multiplication by
        # the rounded reciprocal, which differs when n is not a power of two
        cols = torch.tensor(float(n), device=DEV)
        inv = torch.ones((), device=DEV) / torch.sqrt(total / cols + eps)
        chain = (y.float() * inv[:, None]).to(dtype) * gw                    # round, multiply in the storage type
        assert torch.equal(h, chain)
        unfused = rmsnorm(y, gw, eps)
        differ = (h != unfused)
        assert differ.float().mean().item() <= 1e-3
        if differ.any():                                                     # two units in the last place at most
            a, c = h[differ].float(), unfused[differ].float()
            ulp = torch.maximum(a.abs(), c.abs()) * (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10)
            assert torch.all((a - c).abs() <= 2.01 * ulp)
    assert device_status_clean(y)


def test_stats_entry_points_reject_bad_arguments():
    from custom_cuda_kernals_b200 import _native
    from custom_cuda_kernals_b200.kernels.fused import fp8_quant_token_from_amax, matmul_add_bias_stats, rmsnorm_from_stats
    x, w, b, r, gw = _inputs(64, 64, 256, torch.bfloat16, 1)
    with pytest.raises(ValueError, match="float16 or bfloat16"):
        matmul_add_bias_stats(x.float(), w.float())
    with pytest.raises(ValueError, match="residual shape"):
        matmul_add_bias_stats(x, w, None, r[:, :128].contiguous())
    y, ss, am = matmul_add_bias_stats(x, w, amax=True)
    with pytest.raises(ValueError, match="row_sumsq shape"):
        rmsnorm_from_stats(y, ss[:, :32].contiguous(), gw)
    with pytest.raises(ValueError, match="row_amax shape"):
        fp8_quant_token_from_amax(y, am[:, :32].contiguous())
    with pytest.raises(ValueError, match="fp8_format"):
        fp8_quant_token_from_amax(y, am, "e3m4")
    bad = torch.empty(2, 64, device=DEV)
    with pytest.raises(ValueError, match="row_sumsq shape"):
        _native.matmul_add_bias_stats_fwd(x, w, None, None, torch.empty_like(y), bad, None)


@pytest.mark.parametrize("rows,cols", [(300, 1024), (64, 4096), (7, 8), (100, 264), (16, 8192), (3, 32768 + 8)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
def test_rmsnorm_fp8_quant_equals_the_two_kernel_chain(rows, cols, dtype, fmt):
    """norm + per-token quantiser in one pass == fp8_quant(rmsnorm(x)) bit for bit (codes, scales and
    the optional normalised output), also when the sums of squares come from a GEMM epilogue."""
    from custom_cuda.kernels.fp8_quant import fp8_quant
    from custom_cuda_kernals_b200.kernels.fused import matmul_add_bias_stats, rmsnorm_fp8_quant, rmsnorm_from_stats
    from custom_cuda_kernals_b200.kernels.rmsnorm_residual import rmsnorm
    g = torch.Generator(device=DEV).manual_seed(rows + cols)
    x = torch.randn(rows, cols, device=DEV, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(cols, device=DEV, generator=g)).to(dtype)
    normed = rmsnorm(x, w, 1e-5)
    want_codes, want_scale = fp8_quant(normed, fmt, "token")
    codes, scale, y = rmsnorm_fp8_quant(x, w, 1e-5, fmt, want_normed=True)
    assert torch.equal(y, normed)
    assert torch.equal(codes.view(torch.uint8), want_codes.view(torch.uint8)) and torch.equal(scale, want_scale)
    c2, s2 = rmsnorm_fp8_quant(x, w, 1e-5, fmt)
    assert torch.equal(c2.view(torch.uint8), codes.view(torch.uint8)) and torch.equal(s2, scale)
    if cols <= 4096:      # sums of squares from the producing GEMM's epilogue
        a = torch.randn(rows, 64, device=DEV, generator=g).to(dtype)
        wt = (0.125 * torch.randn(cols, 64, device=DEV, generator=g)).to(dtype)
        out, ss, _ = matmul_add_bias_stats(a, wt)
        c3, s3 = rmsnorm_fp8_quant(out, w, 1e-5, fmt, row_sumsq=ss)
        w3, ws3 = fp8_quant(rmsnorm_from_stats(out, ss, w, 1e-5), fmt, "token")
        assert torch.equal(c3.view(torch.uint8), w3.view(torch.uint8)) and torch.equal(s3, ws3)


@pytest.mark.parametrize("shape", [(256, 512, 256), (1000, 1024, 1408), (130, 64, 384), (4096, 4096, 2048)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fp8_fused_epilogues_equal_the_unfused_chains(shape, dtype):
    """FP8 gate-up GEMM + SwiGLU (+ row maxima) and FP8 GEMM + residual against
    matmul_add_bias_fp8 -> swiglu / add, bit for bit; the maxima reproduce fp8_quant(act)."""
    from custom_cuda.kernels.fp8_quant import fp8_quant
    from custom_cuda.kernels.matmul_add_bias import matmul_add_bias_fp8
    from custom_cuda.kernels.swiglu import swiglu
    from custom_cuda_kernals_b200.kernels.fused import (fp8_quant_token_from_amax, interleave_gate_up,
                                                        matmul_add_bias_residual_fp8, matmul_swiglu_fp8)
    m, k, f = shape
    g = torch.Generator(device=DEV).manual_seed(m + f)
    x = torch.randn(m, k, device=DEV, generator=g).to(dtype)
    wg = (k ** -0.5 * torch.randn(f, k, device=DEV, generator=g)).to(dtype)
    wu = (k ** -0.5 * torch.randn(f, k, device=DEV, generator=g)).to(dtype)
    x8, xs = fp8_quant(x, "e4m3", "token")
    wg8, wgs = fp8_quant(wg, "e4m3", "token")
    wu8, wus = fp8_quant(wu, "e4m3", "token")
    wgu8, wgus = fp8_quant(interleave_gate_up(wg, wu), "e4m3", "token")
    want = swiglu(matmul_add_bias_fp8(x8, xs, wg8, wgs, None, dtype), matmul_add_bias_fp8(x8, xs, wu8, wus, None, dtype))
    act, amax = matmul_swiglu_fp8(x8, xs, wgu8, wgus, dtype, amax=True)
    assert torch.equal(act, want)
    assert torch.equal(matmul_swiglu_fp8(x8, xs, wgu8, wgus, dtype), want)
    c, s = fp8_quant_token_from_amax(act, amax)
    cw, sw = fp8_quant(act, "e4m3", "token")
    assert torch.equal(c.view(torch.uint8), cw.view(torch.uint8)) and torch.equal(s, sw)
    # GEMM + bias + residual
    b = (0.1 * torch.randn(f, device=DEV, generator=g)).to(dtype)
    r = torch.randn(m, f, device=DEV, generator=g).to(dtype)
    for bias in (b, None):
        got = matmul_add_bias_residual_fp8(x8, xs, wg8, wgs, bias, r)
        assert torch.equal(got, matmul_add_bias_fp8(x8, xs, wg8, wgs, bias, dtype) + r)
    assert device_status_clean(act)
