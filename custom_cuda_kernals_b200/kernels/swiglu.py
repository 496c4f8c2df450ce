"""SwiGLU gated activation (custom_cuda/kernels/swiglu.py:16-20)."""

from __future__ import annotations

import torch

from .. import _native

__all__ = ["swiglu"]


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``y = silu(gate) * up`` for same-shape contiguous CUDA tensors."""
    y = torch.empty_like(gate)
    _native.swiglu_fwd(gate, up, y)
    return y
