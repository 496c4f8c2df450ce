"""GPU: gradients of the elementwise block ops against torch autograd.

The reference has no backward; the comparison is autograd through the oracle's op chain on
fp32 copies of the same inputs (the kernels compute in fp32 and round once), within the
forward tolerances of each storage type."""

import pytest
import torch

from custom_cuda_kernals_b200.kernels import autograd as A
from oracle import ops
from tests.gpu_util import DEV, device_status_clean, to_dev

pytestmark = pytest.mark.gpu

TOL = {torch.float32: dict(rtol=1e-4, atol=1e-5), torch.float16: dict(rtol=1e-2, atol=1e-3),
       torch.bfloat16: dict(rtol=2e-2, atol=1e-2)}
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def _gen(seed):
    return torch.Generator().manual_seed(seed)


@pytest.mark.parametrize("shape", [(64, 256), (3, 1000), (1, 7), (257, 4096 + 8), (2, 3, 40)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_gradients(shape, dtype):
    g = _gen(sum(shape))
    gate, up, dy = (torch.randn(shape, generator=g).to(dtype) for _ in range(3))
    g32, u32 = gate.float().clone().requires_grad_(True), up.float().clone().requires_grad_(True)
    (torch.nn.functional.silu(g32) * u32).backward(dy.float())
    dg, du = A.swiglu_backward(*to_dev(gate, up, dy))
    torch.testing.assert_close(dg.float().cpu(), g32.grad, **TOL[dtype])
    torch.testing.assert_close(du.float().cpu(), u32.grad, **TOL[dtype])
    # through autograd
    gd, ud = gate.to(DEV).requires_grad_(True), up.to(DEV).requires_grad_(True)
    y = A.swiglu_trainable(gd, ud)
    y.backward(dy.to(DEV))
    assert torch.equal(gd.grad, dg) and torch.equal(ud.grad, du)
    assert device_status_clean(y)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rope_gradients(dtype):
    g = _gen(11)
    b, s, hq, hkv, d = 2, 33, 4, 2, 64
    q, k = torch.randn(b, s, hq, d, generator=g).to(dtype), torch.randn(b, s, hkv, d, generator=g).to(dtype)
    dq, dk = torch.randn(b, s, hq, d, generator=g).to(dtype), torch.randn(b, s, hkv, d, generator=g).to(dtype)
    cos, sin = ops.rope_tables(s, d, 10000.0)
    q32, k32 = q.float().clone().requires_grad_(True), k.float().clone().requires_grad_(True)
    qo, ko = ops.rope(q32, k32, cos, sin)
    torch.autograd.backward([qo, ko], [dq.float(), dk.float()])
    qd, kd = q.to(DEV).requires_grad_(True), k.to(DEV).requires_grad_(True)
    out = A.rope_trainable(qd, kd, cos.to(DEV), sin.to(DEV))
    torch.autograd.backward(list(out), [dq.to(DEV), dk.to(DEV)])
    torch.testing.assert_close(qd.grad.float().cpu(), q32.grad, **TOL[dtype])
    torch.testing.assert_close(kd.grad.float().cpu(), k32.grad, **TOL[dtype])


def _rmsnorm32(x32, r32, w32, eps):
    ro = x32 + r32
    return ro * torch.rsqrt(ro.pow(2).mean(-1, keepdim=True) + eps) * w32, ro


@pytest.mark.parametrize("shape", [(300, 4096), (5, 64), (1, 8), (2, 17, 1024), (700, 8192)])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("with_residual_grad", [True, False])
def test_rmsnorm_residual_gradients(shape, dtype, with_residual_grad):
    if dtype == torch.float32 and shape[-1] > 4096:
        pytest.skip("fp32 rows wider than 4096 are outside the gradient kernel's register budget")
    g = _gen(sum(shape))
    x, r = torch.randn(shape, generator=g).to(dtype), torch.randn(shape, generator=g).to(dtype)
    w = (1.0 + 0.1 * torch.randn(shape[-1], generator=g)).to(dtype)
    dy, dro = torch.randn(shape, generator=g).to(dtype), torch.randn(shape, generator=g).to(dtype)
    eps = 1e-5
    # autograd reference on the rounded sum the kernel saves (residual_out), in fp32
    ro_saved = (x + r)
    ro32 = ro_saved.float().clone().requires_grad_(True)
    w32 = w.float().clone().requires_grad_(True)
    y32 = ro32 * torch.rsqrt(ro32.pow(2).mean(-1, keepdim=True) + eps) * w32
    y32.backward(dy.float())
    want_dx = ro32.grad + (dro.float() if with_residual_grad else 0.0)
    xd, rd, wd = x.to(DEV).requires_grad_(True), r.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True)
    y, ro = A.rmsnorm_residual_trainable(xd, rd, wd, eps)
    if with_residual_grad:
        torch.autograd.backward([y, ro], [dy.to(DEV), dro.to(DEV)])
    else:
        y.backward(dy.to(DEV))
    tol = TOL[dtype]
    torch.testing.assert_close(xd.grad.float().cpu(), want_dx, **tol)
    assert torch.equal(xd.grad, rd.grad)
    # d_weight sums over rows: compare relative to its scale
    scale = w32.grad.abs().max().item() + 1e-6
    assert (wd.grad.float().cpu() - w32.grad).abs().max().item() <= tol["rtol"] * scale + tol["atol"]
    assert device_status_clean(y)


def test_rmsnorm_gradient_rejects_ragged_width():
    x = torch.randn(4, 102, device=DEV)
    with pytest.raises(ValueError, match="column count"):
        A.rmsnorm_residual_backward(x, None, x, torch.ones(102, device=DEV), 1e-5)
    wide = torch.randn(2, 8192, device=DEV)
    with pytest.raises(ValueError, match="column count"):
        A.rmsnorm_residual_backward(wide, None, wide, torch.ones(8192, device=DEV), 1e-5)
