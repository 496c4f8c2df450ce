"""Fused residual add + RMSNorm (custom_cuda/kernels/rmsnorm_residual.py:17-28)."""

from __future__ import annotations

import torch

from .. import _native

__all__ = ["rmsnorm_residual", "rmsnorm"]


def rmsnorm_residual(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                     eps: float = 1e-6) -> tuple[torch.Tensor, torch.Tensor]:
    """``residual_out = x + residual``; ``y = RMSNorm(residual_out) * weight``.

    x, residual: ``[..., hidden]`` contiguous CUDA tensors of one dtype
    (float32/float16/bfloat16); weight: ``[hidden]`` of the same dtype.
    Returns ``(y, residual_out)``.
    """
    y = torch.empty_like(x)
    residual_out = torch.empty_like(x)
    _native.rmsnorm_residual_fwd(x, residual, weight, y, residual_out, eps)
    return y, residual_out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``RMSNorm(x) * weight`` alone - what ``rmsnorm_residual(x, 0, weight)[0]`` returns - for
    callers whose residual add was folded into the producing GEMM.  (Not in the reference.)"""
    y = torch.empty_like(x)
    _native.rmsnorm_fwd(x, weight, y, eps)
    return y
