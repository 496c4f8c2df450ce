"""GPU parity: rmsnorm_residual, swiglu, rope against the CPU oracle on the
reference's case tables (baselines/<op>.py ALL_CASES), same seeded inputs."""

import pytest
import torch

from oracle import cases, ops, workloads
from tests.gpu_util import DEV, check, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", cases.NORM_CASES, ids=lambda c: c.name)
def test_rmsnorm_residual_cases(case):
    from custom_cuda.kernels.rmsnorm_residual import rmsnorm_residual
    x, r, w = cases.norm_inputs(case)
    y_ref, ro_ref = ops.rmsnorm_residual(x, r, w, case.eps)
    y, ro = rmsnorm_residual(*to_dev(x, r, w), case.eps)
    assert y.shape == x.shape and y.dtype == case.dtype and ro.dtype == case.dtype
    if x.numel() == 0:
        return
    check(ro, ro_ref, case.dtype)
    check(y, y_ref, case.dtype)
    y64, ro64 = ops.rmsnorm_residual_fp64(x, r, w, case.eps)
    check(y.double(), y64, case.dtype)


@pytest.mark.parametrize("hidden", [8, 24, 100, 4096 + 8, 5120, 20000, 40000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_row_widths(hidden, dtype):
    """Register path (4 and 8 vectors per thread), ragged widths and the generic path."""
    from custom_cuda.kernels.rmsnorm_residual import rmsnorm_residual
    g = torch.Generator().manual_seed(hidden)
    x = torch.randn(5, hidden, generator=g).to(dtype)
    r = torch.randn(5, hidden, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
    y_ref, ro_ref = ops.rmsnorm_residual(x, r, w, 1e-5)
    y, ro = rmsnorm_residual(*to_dev(x, r, w), 1e-5)
    check(ro, ro_ref, dtype)
    check(y, y_ref, dtype)


def test_rmsnorm_config1_full_size():
    """Benchmark config 1: fp32 [2048, 4096], eps 1e-5."""
    from custom_cuda.kernels.rmsnorm_residual import rmsnorm_residual
    x, r, w, eps = workloads.rmsnorm_fp32()
    y_ref, ro_ref = ops.rmsnorm_residual(x, r, w, eps)
    y, ro = rmsnorm_residual(*to_dev(x, r, w), eps)
    assert torch.equal(ro.cpu(), ro_ref)
    check(y, y_ref, torch.float32)
    # running it twice gives bitwise identical results (fixed reduction order)
    y2, _ = rmsnorm_residual(*to_dev(x, r, w), eps)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("case", cases.GLU_CASES, ids=lambda c: c.name)
def test_swiglu_cases(case):
    from custom_cuda.kernels.swiglu import swiglu
    gate, up = cases.glu_inputs(case)
    want = ops.swiglu(gate, up)
    got = swiglu(*to_dev(gate, up))
    assert got.shape == gate.shape and got.dtype == case.dtype
    if gate.numel():
        check(got, want, case.dtype)
        check(got.double(), ops.swiglu_fp64(gate, up), case.dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_swiglu_tail_sweep(dtype):
    """Every length 1..129 (tests/test_swiglu_kernel.py:74-93): vector body + ragged tail."""
    from custom_cuda.kernels.swiglu import swiglu
    g = torch.Generator().manual_seed(3)
    for n in range(1, 130):
        gate = torch.randn(n, generator=g).to(dtype)
        up = torch.randn(n, generator=g).to(dtype)
        check(swiglu(*to_dev(gate, up)), ops.swiglu(gate, up), dtype)


def test_swiglu_unaligned_view_and_extremes():
    from custom_cuda.kernels.swiglu import swiglu
    g = torch.Generator().manual_seed(4)
    base_g = torch.randn(1000, generator=g).to(torch.bfloat16).to(DEV)
    base_u = torch.randn(1000, generator=g).to(torch.bfloat16).to(DEV)
    gate, up = base_g[1:], base_u[1:]          # contiguous but only 2-byte aligned
    check(swiglu(gate, up), ops.swiglu(gate.cpu(), up.cpu()), torch.bfloat16)
    ext = torch.tensor([-200.0, -88.0, -20.0, -0.0, 0.0, 20.0, 88.0, 200.0])
    got = swiglu(ext.to(DEV), torch.ones(8, device=DEV))
    torch.testing.assert_close(got.cpu(), ops.swiglu(ext, torch.ones(8)), rtol=1e-5, atol=1e-30)


def test_swiglu_config2a_full_size():
    from custom_cuda.kernels.swiglu import swiglu
    gate, up = workloads.swiglu_bf16()
    got = swiglu(*to_dev(gate, up))
    check(got, ops.swiglu(gate, up), torch.bfloat16)


@pytest.mark.parametrize("case", cases.ROPE_CASES, ids=lambda c: c.name)
def test_rope_cases(case):
    from custom_cuda.kernels.rope import rope
    q, k, cos, sin = cases.rope_inputs(case)
    q_ref, k_ref = ops.rope(q, k, cos, sin)
    q_out, k_out = rope(*to_dev(q, k, cos, sin))
    assert q_out.shape == q.shape and k_out.shape == k.shape and q_out.dtype == case.dtype
    if case.batch == 0:
        return
    check(q_out, q_ref, case.dtype)
    check(k_out, k_ref, case.dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("head_dim", [6, 10, 14, 24])
def test_rope_scalar_path(dtype, head_dim):
    """Half head dims 3, 5, 7, 12 are not a whole number of 16-byte vectors
    (tests/test_rope_kernel.py:59-84)."""
    from custom_cuda.kernels.rope import rope
    g = torch.Generator().manual_seed(head_dim)
    q = torch.randn(2, 5, 3, head_dim, generator=g).to(dtype)
    k = torch.randn(2, 5, 1, head_dim, generator=g).to(dtype)
    cos, sin = ops.rope_tables(5, head_dim)
    q_ref, k_ref = ops.rope(q, k, cos, sin)
    q_out, k_out = rope(*to_dev(q, k, cos, sin))
    check(q_out, q_ref, dtype)
    check(k_out, k_ref, dtype)


def test_rope_preserves_norm_and_many_heads():
    """Rotation keeps each head row's norm (tests/test_rope.py:69-78); 136 heads x 8 vectors
    exceed one CTA's thread count, exercising the item loop."""
    from custom_cuda.kernels.rope import rope
    g = torch.Generator().manual_seed(9)
    q = torch.randn(3, 7, 128, 128, generator=g)
    k = torch.randn(3, 7, 8, 128, generator=g)
    cos, sin = ops.rope_tables(7, 128, 500000.0)
    q_out, k_out = rope(*to_dev(q, k, cos, sin))
    torch.testing.assert_close(q_out.norm(dim=-1).cpu(), q.norm(dim=-1), rtol=1e-4, atol=1e-4)
    q_ref, k_ref = ops.rope(q, k, cos, sin)
    check(q_out, q_ref, torch.float32)
    check(k_out, k_ref, torch.float32)


def test_rope_config2b_full_size_and_position_slices():
    from custom_cuda.kernels.rope import rope
    q, k, cos, sin = workloads.rope_bf16()
    q_ref, k_ref = ops.rope(q, k, cos, sin)
    qd, kd, cd, sd = to_dev(q, k, cos, sin)
    q_out, k_out = rope(qd, kd, cd, sd)
    check(q_out, q_ref, torch.bfloat16)
    check(k_out, k_ref, torch.bfloat16)
    # sequence sharding: a slice of positions with the matching table slice gives the same rows
    s0, s1 = 512, 1024
    q_part, k_part = rope(qd[:, s0:s1].contiguous(), kd[:, s0:s1].contiguous(), cd[s0:s1], sd[s0:s1])
    assert torch.equal(q_part, q_out[:, s0:s1]) and torch.equal(k_part, k_out[:, s0:s1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dims", [(2, 33, 8, 2, 64), (1, 128, 32, 8, 128), (3, 5, 3, 1, 6), (16, 1, 32, 8, 128), (1, 1, 4, 2, 64)])
def test_rope_strided_views_equal_packed_inputs(dims, dtype):
    """q and k as column ranges of one fused QKV buffer [tokens, (Hq + 2 Hkv) * D] give exactly
    what packed copies give (vector path and, for head_dim 6, the scalar path)."""
    from custom_cuda.kernels.rope import rope, rope_strided
    b, s, hq, hkv, d = dims
    g = torch.Generator().manual_seed(sum(dims))
    qkv = torch.randn(b, s, (hq + 2 * hkv) * d, generator=g).to(dtype).to(DEV)
    q = qkv[..., :hq * d].unflatten(-1, (hq, d))
    k = qkv[..., hq * d:(hq + hkv) * d].unflatten(-1, (hkv, d))
    cos, sin = (t.to(DEV) for t in ops.rope_tables(s, d, 500000.0))
    q1, k1 = rope_strided(q, k, cos, sin)
    q2, k2 = rope(q.contiguous(), k.contiguous(), cos, sin)
    assert q1.is_contiguous() and torch.equal(q1, q2) and torch.equal(k1, k2)
    q_ref, k_ref = ops.rope(q.cpu().contiguous(), k.cpu().contiguous(), cos.cpu(), sin.cpu())
    check(q1, q_ref, dtype)
    check(k1, k_ref, dtype)
    with pytest.raises(ValueError):
        rope_strided(q.transpose(1, 2), k.transpose(1, 2), cos, sin)     # heads no longer contiguous per token


@pytest.mark.parametrize("shape", [(5, 100), (64, 768), (300, 4096), (3, 20000), (2, 40000)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_rmsnorm_alone_equals_zero_residual(shape, dtype):
    """The norm without the residual add gives exactly what rmsnorm_residual gives for a zero residual."""
    from custom_cuda.kernels.rmsnorm_residual import rmsnorm, rmsnorm_residual
    g = torch.Generator().manual_seed(shape[1])
    x = torch.randn(shape, generator=g).to(dtype).to(DEV)
    w = (1 + 0.1 * torch.randn(shape[1], generator=g)).to(dtype).to(DEV)
    y = rmsnorm(x, w, 1e-5)
    y_ref, ro = rmsnorm_residual(x, torch.zeros_like(x), w, 1e-5)
    assert torch.equal(y, y_ref) and torch.equal(ro, x)
    want, _ = ops.rmsnorm_residual(x.cpu(), torch.zeros_like(x).cpu(), w.cpu(), 1e-5)
    check(y, want, dtype)
