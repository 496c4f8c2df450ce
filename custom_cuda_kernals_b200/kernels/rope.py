"""Rotary position embedding, half-split convention (custom_cuda/kernels/rope.py:16-28)."""

from __future__ import annotations

import torch

from .. import _native

__all__ = ["rope", "rope_strided"]


def rope(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor,
         sin: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Rotate ``q [B,S,Hq,D]`` and ``k [B,S,Hkv,D]`` with fp32 tables
    ``cos, sin [S, D/2]``; row ``s`` of the tables is applied to position ``s``.
    To run on a slice of positions, pass the matching slice of the tables.
    """
    q_out = torch.empty_like(q)
    k_out = torch.empty_like(k)
    _native.rope_fwd(q, k, cos, sin, q_out, k_out)
    return q_out, k_out


def rope_strided(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor,
                 sin: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``rope`` for q / k that are views into a wider buffer - e.g. the q and k column ranges of a
    fused QKV projection output viewed as ``[B, S, H, D]``: heads of a token contiguous, tokens
    evenly spaced.  Returns contiguous tensors.  (Not in the reference, which rejects views.)"""
    q_out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    k_out = torch.empty(k.shape, dtype=k.dtype, device=k.device)
    _native.rope_strided_fwd(q, k, cos, sin, q_out, k_out)
    return q_out, k_out
