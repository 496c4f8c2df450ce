"""Dynamic FP8 quantisation behind the reference's entry point (custom_cuda/kernels/fp8_quant.py:28-63),
with a per-token granularity added.

For every scale group (the whole tensor, a 128 x 128 tile, or a row) the kernels compute
``scale = max(amax / FP8_MAX, 1e-12)`` and ``code = fp8(x / scale)`` and reproduce PyTorch's CPU
result of that chain bit for bit: the division is IEEE-correct (rebuilt from a reciprocal and
fused multiply-adds in csrc/fp8_quant.cu), the cast rounds to nearest even and saturates.  Each
input element is read from memory once in every granularity except "tensor", whose global
maximum needs a first pass.
"""

from __future__ import annotations

import torch

from .. import _native

__all__ = ["fp8_quant"]

_CODE_DTYPE = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
_TILE = 128


def _tiles(extent: int) -> int:
    return -(-extent // _TILE)


def _block(x, codes, fmt):
    scale = x.new_empty((_tiles(x.shape[0]), _tiles(x.shape[1])), dtype=torch.float32)
    _native.fp8_quant_block_fwd(x, codes, scale, fmt)
    return scale


def _token(x, codes, fmt):
    scale = x.new_empty((x.shape[0], 1), dtype=torch.float32)
    _native.fp8_quant_token_fwd(x, codes, scale, fmt)
    return scale


def _tensor(x, codes, fmt):
    scale = x.new_empty(1, dtype=torch.float32)
    running_max = x.new_zeros(1, dtype=torch.int32)          # the kernel's atomic-max cell; must start at 0
    _native.fp8_quant_tensor_fwd(x, codes, scale, running_max, fmt)
    return scale


_BY_GRANULARITY = {"block": _block, "tensor": _tensor, "token": _token}


def fp8_quant(x: torch.Tensor, fp8_format: str = "e4m3",
              granularity: str = "block") -> tuple[torch.Tensor, torch.Tensor]:
    """Quantise ``x`` (``[M, N]``, contiguous, CUDA, float32 / float16 / bfloat16) to FP8.

    Returns ``(x_fp8, scale)``: ``x_fp8`` is ``[M, N]`` in ``torch.float8_e4m3fn`` or
    ``torch.float8_e5m2``; ``scale`` is float32 of shape ``[ceil(M/128), ceil(N/128)]`` for
    ``"block"``, ``[1]`` for ``"tensor"`` and ``[M, 1]`` for ``"token"`` (the last one does not
    exist in the reference).  Unknown formats or granularities raise ``ValueError``.
    """
    codes_dtype = _CODE_DTYPE.get(fp8_format)
    if codes_dtype is None:
        raise ValueError(f"fp8_format must be 'e4m3' or 'e5m2', got {fp8_format!r}")
    run = _BY_GRANULARITY.get(granularity)
    if run is None:
        raise ValueError(f"granularity must be 'block', 'tensor' or 'token', got {granularity!r}")
    if x.dim() != 2:
        raise ValueError(f"shape mismatch: x must be 2-D [M, N], got {tuple(x.shape)}")
    codes = torch.empty(tuple(x.shape), dtype=codes_dtype, device=x.device)
    return codes, run(x, codes, fp8_format)
