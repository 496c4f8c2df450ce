"""Autograd-enabled forms of the elementwise block ops.

The reference is forward-only (its tests assert that outputs carry no autograd history,
tests/test_linear_cross_entropy_kernel.py:98-113) and so are the drop-in entry points in this
package.  These are separate calls for training loops: the forward is the same kernel, the
backward is a hand-written kernel too (RoPE's backward is RoPE with the sine negated).

    swiglu_trainable(gate, up)                         -> y
    rope_trainable(q, k, cos, sin)                     -> (q_out, k_out)
    rmsnorm_residual_trainable(x, residual, weight, eps) -> (y, residual_out)

The cross entropy's gradient path is in ``kernels.linear_cross_entropy``.
"""

from __future__ import annotations

import torch

from .. import _native
from .rmsnorm_residual import rmsnorm_residual
from .rope import rope
from .swiglu import swiglu

__all__ = ["swiglu_trainable", "rope_trainable", "rmsnorm_residual_trainable", "swiglu_backward",
           "rope_backward", "rmsnorm_residual_backward"]


def swiglu_backward(gate: torch.Tensor, up: torch.Tensor, dy: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``(d_gate, d_up)`` of ``y = silu(gate) * up`` for the upstream gradient ``dy``."""
    dgate, dup = torch.empty_like(gate), torch.empty_like(up)
    _native.swiglu_bwd(gate, up, dy.contiguous(), dgate, dup)
    return dgate, dup


def rope_backward(dq_out: torch.Tensor, dk_out: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor
                  ) -> tuple[torch.Tensor, torch.Tensor]:
    """The rotation is orthogonal: its transpose is the rotation by the opposite angle."""
    return rope(dq_out.contiguous(), dk_out.contiguous(), cos, -sin)


def rmsnorm_residual_backward(dy: torch.Tensor, d_residual_out: torch.Tensor | None, residual_out: torch.Tensor,
                              weight: torch.Tensor, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    """``(dx, dweight)``; ``dx`` is the gradient of ``x`` and of ``residual`` alike.
    ``d_residual_out`` is the gradient arriving through the second output, or ``None``."""
    cols = dy.shape[-1]
    rows = dy.numel() // cols if cols else 0
    dx, dweight = torch.empty_like(dy), torch.empty_like(weight)
    ws = torch.empty(max(1, _native.rmsnorm_bwd_workspace_bytes(rows, cols)), dtype=torch.uint8, device=dy.device)
    _native.rmsnorm_residual_bwd(dy.contiguous(), None if d_residual_out is None else d_residual_out.contiguous(),
                                 residual_out, weight, dx, dweight, ws, eps)
    return dx, dweight


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        ctx.save_for_backward(gate, up)
        return swiglu(gate, up)

    @staticmethod
    def backward(ctx, dy):
        return swiglu_backward(*ctx.saved_tensors, dy)


class _RoPE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, cos, sin):
        ctx.save_for_backward(cos, sin)
        return rope(q, k, cos, sin)

    @staticmethod
    def backward(ctx, dq, dk):
        cos, sin = ctx.saved_tensors
        return (*rope_backward(dq, dk, cos, sin), None, None)


class _RMSNormResidual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, eps):
        y, residual_out = rmsnorm_residual(x, residual, weight, eps)
        ctx.save_for_backward(residual_out, weight)
        ctx.eps = eps
        return y, residual_out

    @staticmethod
    def backward(ctx, dy, d_residual_out):
        residual_out, weight = ctx.saved_tensors
        dx, dweight = rmsnorm_residual_backward(dy, d_residual_out, residual_out, weight, ctx.eps)
        return dx, dx, dweight, None


def swiglu_trainable(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return _SwiGLU.apply(gate, up)


def rope_trainable(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor
                   ) -> tuple[torch.Tensor, torch.Tensor]:
    return _RoPE.apply(q, k, cos, sin)


def rmsnorm_residual_trainable(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6
                               ) -> tuple[torch.Tensor, torch.Tensor]:
    return _RMSNormResidual.apply(x, residual, weight, eps)
