"""Fused residual add + RMSNorm behind the reference's entry point
(custom_cuda/kernels/rmsnorm_residual.py:17-28), and the norm alone.

Rounding follows the PyTorch baseline (baselines/rmsnorm_residual.py:130-136): the sum ``x +
residual`` is rounded to the storage type, the mean of squares is taken from that rounded sum in
fp32, the normalised value is rounded to the storage type and then multiplied by ``weight``.
One CTA owns a row and keeps it in registers between the reduction and the store
(csrc/rmsnorm_residual.cu), so each input is read from memory once.  The gradient is in
``kernels.autograd.rmsnorm_residual_trainable``.
"""

from __future__ import annotations

import torch

from .. import _native

__all__ = ["rmsnorm_residual", "rmsnorm"]


def rmsnorm_residual(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                     eps: float = 1e-6) -> tuple[torch.Tensor, torch.Tensor]:
    """``(y, residual_out)`` with ``residual_out = x + residual`` and ``y = residual_out *
    rsqrt(mean(residual_out ** 2) + eps) * weight`` over the last dimension.  ``x`` and
    ``residual`` share shape ``[..., hidden]`` and dtype (float32 / float16 / bfloat16) and are
    contiguous CUDA tensors; ``weight`` is ``[hidden]`` of that dtype."""
    y, residual_out = torch.empty_like(x), torch.empty_like(x)     # 1.3 us each on the host; views of one buffer cost more
    _native.rmsnorm_residual_fwd(x, residual, weight, y, residual_out, eps)
    return y, residual_out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``RMSNorm(x) * weight`` alone - what ``rmsnorm_residual(x, 0, weight)[0]`` returns - for
    callers whose residual add was folded into the producing GEMM.  (Not in the reference.)"""
    y = torch.empty_like(x)
    _native.rmsnorm_fwd(x, weight, y, eps)
    return y
