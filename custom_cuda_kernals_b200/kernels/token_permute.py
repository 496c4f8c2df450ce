"""Row movement around the expert FFNs of a mixture-of-experts layer.

Same entry points as the reference's ``custom_cuda.kernels.token_permute``
(custom_cuda/kernels/token_permute.py:18-42): both directions are gathers, the index arrays
come from ``compute_permutation`` (baselines/token_permute.py:58-72 in the reference: one
stable argsort of the flattened expert assignments and its inverse).
"""

from __future__ import annotations

import torch

from .. import _native

__all__ = ["token_gather", "token_combine", "compute_permutation"]


def token_gather(src: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """``dst[i] = src[indices[i]]``.  src: ``[S, H]`` contiguous CUDA tensor, indices: ``[N]``
    int64 with values in ``[0, S)``.  Returns ``dst: [N, H]``."""
    n = indices.shape[0]
    dst = torch.empty((n, src.shape[1]), dtype=src.dtype, device=src.device)
    _native.token_gather_fwd(src, indices, dst)
    return dst


def token_combine(expert_output: torch.Tensor, unpermute_index: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """``combined[t] = sum_j weights[t, j] * expert_output[unpermute_index[t, j]]`` (fp32
    accumulation).  expert_output: ``[N, H]``; unpermute_index: ``[T, k]`` int64; weights:
    ``[T, k]`` float32.  Returns ``combined: [T, H]`` in expert_output's dtype."""
    t, k = unpermute_index.shape
    combined = torch.empty((t, expert_output.shape[1]), dtype=expert_output.dtype, device=expert_output.device)
    if k == 0:
        return combined.zero_()
    _native.token_combine_fwd(expert_output, unpermute_index, weights, combined)
    return combined


def compute_permutation(topk_indices: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """From the router's ``topk_indices: [T, k]``: ``permute_index: [T * k]`` (source token of
    every slot of the expert-sorted order; stable, so tokens keep their order inside an expert)
    and ``unpermute_index: [T, k]`` (the slot each (token, choice) landed in)."""
    t, k = topk_indices.shape
    order = torch.argsort(topk_indices.reshape(-1), stable=True)
    inverse = torch.empty_like(order)
    inverse[order] = torch.arange(t * k, device=topk_indices.device)
    return order // k, inverse.reshape(t, k)
