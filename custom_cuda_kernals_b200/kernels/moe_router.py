"""Top-k softmax router of a mixture-of-experts layer.

Same entry point as the reference's ``custom_cuda.kernels.moe_router.moe_router``
(custom_cuda/kernels/moe_router.py:18-30); semantics of baselines/moe_router.py:109-119:
softmax in fp32 whatever the storage type, the k largest probabilities with their expert
ids, optionally renormalised to sum to 1.
"""

from __future__ import annotations

import torch

from .. import _native

__all__ = ["moe_router"]


def moe_router(logits: torch.Tensor, k: int, renormalize: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """``topk_weights, topk_indices = topk(softmax(logits, dim=-1), k)``, optionally renormalised.

    logits: ``[T, E]`` contiguous CUDA tensor, ``E <= 256``.  Returns ``topk_weights: [T, k]``
    (float32, descending) and ``topk_indices: [T, k]`` (int64; equal probabilities go to the
    lower expert id).  ``k > E`` raises ``RuntimeError`` as ``torch.topk`` does.
    """
    n_tokens = logits.shape[0]
    topk_weights = torch.empty((n_tokens, k), dtype=torch.float32, device=logits.device)
    topk_indices = torch.empty((n_tokens, k), dtype=torch.long, device=logits.device)
    _native.moe_router_fwd(logits, topk_weights, topk_indices, renormalize)
    return topk_weights, topk_indices
