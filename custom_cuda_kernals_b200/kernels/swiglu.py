"""SwiGLU gated activation behind the reference's entry point (custom_cuda/kernels/swiglu.py:16-20).

Rounding follows the PyTorch baseline (baselines/swiglu.py:109-112): ``silu(gate)`` is evaluated in
fp32 and rounded to the storage type, then multiplied by ``up`` and rounded again.  The kernel is
one streaming pass (csrc/swiglu.cu): three tensors of traffic, any shape, any element count - the
ragged tail below one 16-byte vector is handled inside the same launch, and buffers that are not
16-byte aligned (sliced views) take an element-wise kernel instead of being refused.  The
gradient lives in ``kernels.autograd.swiglu_trainable``; this call is forward-only like the
reference's.
"""

from __future__ import annotations

import torch

from .. import _native

__all__ = ["swiglu"]


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``y = silu(gate) * up``: ``gate`` and ``up`` are contiguous CUDA tensors of one shape and
    one dtype (float32, float16 or bfloat16); ``y`` is a new tensor like ``gate``.  Validation
    errors are ``ValueError``, launch failures ``RuntimeError``; launches on the current stream."""
    out = torch.empty_like(gate)
    _native.swiglu_fwd(gate, up, out)
    return out
