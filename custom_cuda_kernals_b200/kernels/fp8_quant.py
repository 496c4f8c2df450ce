"""Dynamic FP8 quantisation (custom_cuda/kernels/fp8_quant.py:28-63, plus a per-token mode)."""

from __future__ import annotations

import math

import torch

from .. import _native

__all__ = ["fp8_quant"]

_FP8_TORCH_DTYPES = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
_TILE = 128


def fp8_quant(x: torch.Tensor, fp8_format: str = "e4m3",
              granularity: str = "block") -> tuple[torch.Tensor, torch.Tensor]:
    """``scale = max(amax / FP8_MAX, 1e-12)``; ``x_fp8 = (x / scale) -> fp8``.

    x: ``[M, N]`` contiguous CUDA tensor (float32/float16/bfloat16).
    granularity: ``"block"`` - one scale per 128x128 tile, scale
    ``[ceil(M/128), ceil(N/128)]``; ``"tensor"`` - scale ``[1]``; ``"token"``
    - one scale per row, scale ``[M, 1]`` (not in the reference).  Codes and
    scales equal PyTorch's ``(x.float() / scale).to(fp8)`` bit for bit.
    """
    if fp8_format not in _FP8_TORCH_DTYPES:
        raise ValueError(f"fp8_format must be 'e4m3' or 'e5m2', got {fp8_format!r}")
    if granularity not in ("block", "tensor", "token"):
        raise ValueError(f"granularity must be 'block', 'tensor' or 'token', got {granularity!r}")
    m, n = x.shape
    x_fp8 = torch.empty((m, n), dtype=_FP8_TORCH_DTYPES[fp8_format], device=x.device)
    if granularity == "block":
        scale = torch.empty(math.ceil(m / _TILE), math.ceil(n / _TILE), dtype=torch.float32, device=x.device)
        _native.fp8_quant_block_fwd(x, x_fp8, scale, fp8_format)
    elif granularity == "token":
        scale = torch.empty(m, 1, dtype=torch.float32, device=x.device)
        _native.fp8_quant_token_fwd(x, x_fp8, scale, fp8_format)
    else:
        scale = torch.empty(1, dtype=torch.float32, device=x.device)
        amax_scratch = torch.zeros(1, dtype=torch.int32, device=x.device)
        _native.fp8_quant_tensor_fwd(x, x_fp8, scale, amax_scratch, fp8_format)
    return x_fp8, scale
