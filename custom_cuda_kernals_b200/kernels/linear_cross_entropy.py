"""Linear + cross entropy without materialising the logits
(custom_cuda/kernels/linear_cross_entropy.py:32-82).

float16/bfloat16 inputs run one fused kernel (tensor-core GEMM tiles folded
into per-row online-softmax state).  float32 inputs, or a hidden size that is
not a multiple of 8, use the reference's structure instead: a loop over
vocabulary chunks of ``chunk_size`` columns, each chunk's logits produced by
``matmul_add_bias`` and folded in by ``linear_ce_chunk_update``.  Forward only:
the result carries no autograd history.
"""

from __future__ import annotations

import torch

from .. import _native

__all__ = ["linear_cross_entropy", "lce_row_stats", "lce_loss_from_stats", "DEFAULT_CHUNK_SIZE"]

DEFAULT_CHUNK_SIZE = 4096
IGNORE_INDEX = -100


def _fused_ok(hidden: torch.Tensor, weight: torch.Tensor) -> bool:
    return (hidden.dtype in (torch.float16, torch.bfloat16) and hidden.dim() == 2
            and hidden.shape[1] % 8 == 0 and hidden.shape[1] > 0
            and hidden.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def lce_row_stats(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, v_start: int = 0,
                  chunk_size: int = DEFAULT_CHUNK_SIZE) -> torch.Tensor:
    """Per-row ``[3, N]`` fp32 statistics (max logit, sum exp(logit - max),
    target logit or 0) of ``hidden @ weight.T`` where ``weight`` holds rows
    ``v_start ...`` of the full LM head.  This is what one rank of a
    vocabulary-sharded run computes.
    """
    n = hidden.shape[0]
    v = weight.shape[0]
    dev = hidden.device
    stats = torch.empty(3, n, dtype=torch.float32, device=dev)
    if n == 0:
        return stats
    if _fused_ok(hidden, weight) and hidden.is_cuda:
        ws = torch.empty(max(1, _native.lce_workspace_bytes(hidden, n, v)), dtype=torch.uint8, device=dev)
        _native.linear_cross_entropy_fwd(hidden, weight, targets, v_start, stats, ws)
        return stats
    stats[0].fill_(float("-inf"))
    stats[1:].zero_()
    for c0 in range(0, v, chunk_size):
        c1 = min(c0 + chunk_size, v)
        logits = torch.empty(n, c1 - c0, dtype=hidden.dtype, device=dev)
        _native.matmul_add_bias_fwd(hidden, weight[c0:c1], None, logits)
        _native.linear_ce_chunk_update(logits, targets, v_start + c0, stats[0], stats[1], stats[2])
    return stats


def lce_loss_from_stats(stats: torch.Tensor, targets: torch.Tensor, ignore_index: int = IGNORE_INDEX,
                        reduction: str = "mean") -> torch.Tensor:
    """Merge ``[shards, 3, N]`` statistics and reduce to the loss."""
    n = targets.shape[0]
    dev = targets.device
    loss_rows = torch.empty(n, dtype=torch.float32, device=dev) if reduction == "none" else None
    reduce_out = torch.empty(2, dtype=torch.float32, device=dev)
    _native.lce_finalize(stats, targets, ignore_index, loss_rows, reduce_out)
    if reduction == "none":
        return loss_rows
    if reduction == "sum":
        return reduce_out[0]
    return reduce_out[0] / reduce_out[1]   # 0/0 -> nan when every row is ignored, as F.cross_entropy


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor,
                         ignore_index: int = IGNORE_INDEX, reduction: str = "mean",
                         chunk_size: int = DEFAULT_CHUNK_SIZE) -> torch.Tensor:
    """``cross_entropy(hidden @ weight.T, targets)`` as an fp32 scalar (or ``[N]``).

    hidden ``[N, H]``, weight ``[V, H]`` (no bias), targets ``[N]`` int64.
    Rows whose target equals ``ignore_index`` contribute 0 and are left out of
    the mean; a target outside ``[0, V)`` that is not ``ignore_index`` yields
    a target logit of 0, as in the reference kernel.
    """
    if reduction not in ("mean", "sum", "none"):
        raise ValueError(f"reduction must be 'mean', 'sum', or 'none', got {reduction!r}")
    n, _ = hidden.shape
    if n == 0:
        for name, t in (("hidden", hidden), ("weight", weight), ("targets", targets)):
            if not t.is_cuda:
                raise ValueError(f"argument '{name}' must be a CUDA tensor, got device type '{t.device.type}'")
        empty = torch.zeros(0, dtype=torch.float32, device=hidden.device)
        if reduction == "none":
            return empty
        return empty.sum() if reduction == "sum" else empty.sum() / 0.0
    stats = lce_row_stats(hidden, weight, targets, 0, chunk_size)
    return lce_loss_from_stats(stats.unsqueeze(0), targets, ignore_index, reduction)
