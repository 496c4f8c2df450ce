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
    """Routes every token to its ``k`` most probable experts.

    ``logits`` holds one row of ``E`` gate scores per token (2-D, contiguous, on the GPU; at most
    256 experts).  Each row goes through a softmax evaluated in fp32; the ``k`` largest
    probabilities come back in descending order as ``[T, k]`` float32 together with their expert
    ids as ``[T, k]`` int64, ties going to the lower id.  With ``renormalize`` the kept
    probabilities are divided by their sum.  Asking for more experts than there are raises
    ``RuntimeError``, like ``torch.topk``.
    """
    shape = (logits.shape[0], k)
    weights = torch.empty(shape, dtype=torch.float32, device=logits.device)
    experts = torch.empty(shape, dtype=torch.long, device=logits.device)
    _native.moe_router_fwd(logits, weights, experts, renormalize)
    return weights, experts
