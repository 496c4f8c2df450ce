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

__all__ = ["linear_cross_entropy", "lce_row_stats", "lce_loss_from_stats", "linear_cross_entropy_fwd_bwd", "lce_stats_and_gradients", "lce_lse_from_stats", "lce_grad_scale",
           "linear_cross_entropy_trainable", "DEFAULT_CHUNK_SIZE"]

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


def lce_lse_from_stats(stats: torch.Tensor) -> torch.Tensor:
    """Row-wise log-sum-exp over the whole vocabulary from ``[shards, 3, N]`` statistics."""
    m = stats[:, 0].amax(dim=0)
    total = (stats[:, 1] * torch.exp(stats[:, 0] - m)).sum(dim=0)
    return (m + torch.log(total)).contiguous()


_IGNORED, _ELSEWHERE = -1, -2


def _local_targets(targets: torch.Tensor, v_start: int, v: int, ignore_index: int) -> tuple[torch.Tensor, int]:
    """Targets as column indices of a vocabulary shard, and the value that marks an ignored row
    in them.  "Ignored" is decided on the GLOBAL ids: with ``ignore_index >= 0`` (a pad id, say 0)
    a real target whose local index happens to equal ``ignore_index`` must not be dropped on the
    shard that starts ``ignore_index`` columns below it.  So on a shard with ``v_start > 0``
    ignored rows become -1 and rows whose target lies in another shard -2 (matches no column)."""
    if v_start == 0:
        return targets, ignore_index       # local == global; out-of-range targets match no column already
    local = targets - v_start
    local = torch.where((local >= 0) & (local < v), local, torch.full_like(local, _ELSEWHERE))
    return torch.where(targets == ignore_index, torch.full_like(local, _IGNORED), local).contiguous(), _IGNORED


def lce_grad_scale(targets: torch.Tensor, ignore_index: int, reduction: str) -> float:
    """d(loss)/d(loss_i): 1 for 'sum', 1 / (rows not ignored) for 'mean' (nan when all are)."""
    if reduction not in ("mean", "sum"):
        raise ValueError(f"reduction must be 'mean' or 'sum' for the gradient path, got {reduction!r}")
    if reduction == "sum":
        return 1.0
    valid = int((targets != ignore_index).sum().item())
    return 1.0 / valid if valid else float("nan")


def lce_stats_and_gradients(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, grad_scale: float,
                            v_start: int = 0, ignore_index: int = IGNORE_INDEX, rows_per_chunk: int = 8192,
                            weight_t: torch.Tensor | None = None, gather=None, recompute: bool = False
                            ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Forward statistics and gradients of ``grad_scale * sum_i loss_i`` for the vocabulary
    rows ``weight`` holds (``v_start ...`` of the LM head), ``rows_per_chunk`` rows at a time:

    1. the fused forward kernel, which here also leaves the chunk's fp32 logits in a scratch
       buffer ``[rows, V]`` (with ``recompute`` it does not, and step 2 runs the contraction a
       second time instead - no fp32 buffer, one more GEMM);
    2. ``gather`` (the statistics all-gather of a vocabulary-sharded run) and the row-wise
       log-sum-exp; ``dlogits = (exp(logit - lse) - onehot) * grad_scale`` written once, row-major,
       in the storage type, by one bandwidth-bound pass over the logits (6 bytes per logit);
    3. ``d_hidden[chunk] = dlogits @ W`` and ``d_weight (+)= dlogits^T @ hidden[chunk]`` on the
       tcgen05 GEMM, which reads ``dlogits``, ``W`` and ``hidden`` as they are stored (MN-major
       operand descriptors): no transposed copy of any of them exists.  ``d_weight`` is written
       directly when one chunk covers all rows, else accumulated in fp32 across the chunks.

    Scratch memory: ``rows_per_chunk * V * 6`` bytes (fp32 logits + dlogits of one chunk; ``* 2``
    with ``recompute``), plus a ``V * H`` fp32 accumulator when there are several chunks.
    ``weight_t`` is accepted for compatibility and ignored (no transposed weight is needed).

    Returns ``(stats [shards, 3, N], d_hidden - this shard's contribution, d_weight)``."""
    from .fused import matmul_general
    n, h = hidden.shape
    v = weight.shape[0]
    if not (_fused_ok(hidden, weight) and hidden.is_cuda) or v % 8 != 0:
        raise ValueError("the gradient path needs float16/bfloat16 CUDA inputs with H and V multiples of 8")
    dev, dt = hidden.device, hidden.dtype
    local, local_ignore = _local_targets(targets, v_start, v, ignore_index)
    d_hidden = torch.empty_like(hidden)
    one_chunk = n <= rows_per_chunk
    d_weight = torch.empty(v, h, dtype=dt, device=dev) if one_chunk else torch.zeros(v, h, dtype=torch.float32, device=dev)
    rows_max = min(n, rows_per_chunk)
    logits = None if recompute else torch.empty(rows_max, v, dtype=torch.float32, device=dev)
    dl_buf = torch.empty(rows_max, v, dtype=dt, device=dev)
    stats_parts = []
    for r0 in range(0, n, rows_per_chunk):
        r1 = min(n, r0 + rows_per_chunk)
        rows = r1 - r0
        hc, tc = hidden[r0:r1], targets[r0:r1]
        dl = dl_buf[:rows]
        stats = torch.empty(3, rows, dtype=torch.float32, device=dev)
        ws = torch.empty(max(1, _native.lce_workspace_bytes(hidden, rows, v)), dtype=torch.uint8, device=dev)
        _native.linear_cross_entropy_fwd(hc, weight, tc, v_start, stats, ws, None if recompute else logits[:rows])
        stats = gather(stats) if gather is not None else stats.unsqueeze(0)
        stats_parts.append(stats)
        lse = lce_lse_from_stats(stats)
        if recompute:
            _native.lce_dlogits_fwd(hc, weight, local[r0:r1], lse, local_ignore, grad_scale, dl)
        else:
            _native.lce_dlogits_from_logits(logits[:rows], local[r0:r1], lse, local_ignore, grad_scale, dl, None)
        matmul_general(dl, weight, b_transposed=True, out=d_hidden[r0:r1])                     # [r, V] x [V, H]
        matmul_general(dl, hc, a_transposed=True, b_transposed=True, out=d_weight,            # [r, V]^T x [r, H]
                       accumulate=not one_chunk)
    stats_all = stats_parts[0] if one_chunk else torch.cat(stats_parts, dim=2)
    return stats_all, d_hidden, d_weight if d_weight.dtype == dt else d_weight.to(dt)


def linear_cross_entropy_fwd_bwd(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor,
                                 ignore_index: int = IGNORE_INDEX, reduction: str = "mean",
                                 rows_per_chunk: int = 8192, weight_t: torch.Tensor | None = None,
                                 recompute: bool = False) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Loss and its gradients with respect to ``hidden`` and ``weight`` (for an upstream gradient
    of 1) - what the reference names as its missing piece (custom_cuda/kernels/
    linear_cross_entropy.py:11-18).  float16/bfloat16, ``H`` and ``V`` multiples of 8.

    See ``lce_stats_and_gradients``; scratch memory is ``rows_per_chunk * V * 6`` bytes (fp32
    logits and dlogits of a chunk; ``* 2`` bytes with ``recompute``) plus a ``V * H`` fp32
    accumulator when ``N > rows_per_chunk``.  ``weight_t`` is ignored (kept for compatibility: no
    transposed weight is needed).  Returns ``(loss, d_hidden, d_weight)``."""
    scale = lce_grad_scale(targets, ignore_index, reduction)
    stats, d_hidden, d_weight = lce_stats_and_gradients(hidden, weight, targets, scale, 0, ignore_index,
                                                        rows_per_chunk, weight_t, None, recompute)
    return lce_loss_from_stats(stats, targets, ignore_index, reduction), d_hidden, d_weight


class _LinearCrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, ignore_index, reduction, rows_per_chunk):
        loss, d_hidden, d_weight = linear_cross_entropy_fwd_bwd(
            hidden.detach(), weight.detach(), targets, ignore_index, reduction, rows_per_chunk)
        ctx.save_for_backward(d_hidden, d_weight)
        return loss

    @staticmethod
    def backward(ctx, grad_out):
        d_hidden, d_weight = ctx.saved_tensors
        return d_hidden * grad_out.to(d_hidden.dtype), d_weight * grad_out.to(d_weight.dtype), None, None, None, None


def linear_cross_entropy_trainable(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor,
                                   ignore_index: int = IGNORE_INDEX, reduction: str = "mean",
                                   rows_per_chunk: int = 8192) -> torch.Tensor:
    """``linear_cross_entropy`` with autograd support: the gradients are computed together with
    the loss (see ``linear_cross_entropy_fwd_bwd``) and handed to autograd in ``backward``.
    ``linear_cross_entropy`` itself stays forward-only, as in the reference."""
    return _LinearCrossEntropyFn.apply(hidden, weight, targets, ignore_index, reduction, rows_per_chunk)
