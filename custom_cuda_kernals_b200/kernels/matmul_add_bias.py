"""``y = x @ weight.T + bias`` (custom_cuda/kernels/matmul_add_bias.py:16-26) and an FP8 variant."""

from __future__ import annotations

import torch

from .. import _native

__all__ = ["matmul_add_bias", "matmul_add_bias_fp8"]


def matmul_add_bias(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """x ``[M, K]``, weight ``[N, K]``, bias ``[N]`` or ``None``; one dtype; returns ``[M, N]``."""
    y = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
    _native.matmul_add_bias_fwd(x, weight, bias, y)
    return y


def matmul_add_bias_fp8(a_fp8: torch.Tensor, a_scale: torch.Tensor, w_fp8: torch.Tensor, w_scale: torch.Tensor,
                        bias: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``(a_fp8 * a_scale) @ (w_fp8 * w_scale).T + bias`` with e4m3 operands.

    a_fp8 ``[M, K]`` with per-token scales ``[M, 1]``; w_fp8 ``[N, K]`` with
    per-output-channel scales ``[N, 1]`` (both as produced by
    ``fp8_quant(..., "e4m3", "token")``); bias ``[N]`` in ``out_dtype``.
    """
    y = torch.empty((a_fp8.shape[0], w_fp8.shape[0]), dtype=out_dtype, device=a_fp8.device)
    _native.matmul_add_bias_fp8_fwd(a_fp8, a_scale, w_fp8, w_scale, bias, y)
    return y
