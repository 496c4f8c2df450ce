"""Partitioning of the op path across the GPUs of one node, one process per GPU.

The reference is single-GPU (no distributed code anywhere in it); this module
adds the three partitions the ops admit and the one collective any of them needs:

  * token rows   (rmsnorm_residual, swiglu, rope, fp8_quant per token, the decoder
                  block): contiguous row / sequence ranges, weights replicated,
                  no communication;
  * GEMM columns (matmul_add_bias): rank i owns ``weight[n0:n1]`` and ``bias[n0:n1]``
                  and writes ``y[:, n0:n1]``; no communication for the op itself;
  * vocabulary   (linear_cross_entropy): rank i owns whole 128-row tiles of the LM
                  head, produces per-row (max, sum-exp, target-logit) statistics for
                  its slice, and ONE all-gather of ``[3, N]`` fp32 per call lets every
                  rank merge them into the same loss.

Plumbing is ``torch.distributed`` (NCCL over NVLink/NVSwitch on GPUs, gloo on CPU
for tests).  The payload of the collective is tens of kilobytes, so latency, not
link bandwidth, is what it costs.
"""

from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist

__all__ = ["init_from_env", "row_range", "sequence_range", "column_range", "vocab_range",
           "gather_row_stats", "vocab_parallel_linear_cross_entropy",
           "vocab_parallel_linear_cross_entropy_fwd_bwd", "max_over_ranks"]

VOCAB_TILE = 128


def init_from_env(timeout_s: float = 120.0) -> tuple[int, int, int]:
    """Join the process group described by RANK / WORLD_SIZE / LOCAL_RANK / MASTER_*.
    Returns ``(rank, world_size, local_rank)``; a single process needs no group."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if torch.cuda.is_available():
        torch.cuda.set_device(local % torch.cuda.device_count())
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        backend = "nccl" if torch.cuda.is_available() else "gloo"
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return rank, world, local


def _even_range(total: int, rank: int, world: int, multiple: int = 1) -> tuple[int, int]:
    """Contiguous range of ``total`` items for ``rank``; boundaries fall on multiples of
    ``multiple`` (the last range absorbs a ragged end), sizes differ by at most one unit."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    if total < 0 or multiple < 1:
        raise ValueError("total must be >= 0 and multiple >= 1")
    units = -(-total // multiple)
    lo = min(total, (units * rank // world) * multiple)
    hi = min(total, (units * (rank + 1) // world) * multiple)
    return lo, hi


def row_range(rows: int, rank: int, world: int) -> tuple[int, int]:
    """Token-row partition for the row-independent ops."""
    return _even_range(rows, rank, world)


def sequence_range(batch: int, rank: int, world: int) -> tuple[int, int]:
    """Whole sequences per rank (RoPE positions and causal attention stay local).
    ``batch`` must be a multiple of ``world`` so that every rank has work."""
    if batch % world != 0:
        raise ValueError(f"batch {batch} is not a multiple of world size {world}")
    return _even_range(batch, rank, world)


def column_range(n: int, rank: int, world: int, multiple: int = 8) -> tuple[int, int]:
    """Output-column partition of ``weight [N, K]`` for matmul_add_bias; boundaries on
    multiples of 8 keep every shard's rows of y 16-byte aligned for bf16."""
    return _even_range(n, rank, world, multiple)


def vocab_range(vocab: int, rank: int, world: int) -> tuple[int, int]:
    """Vocabulary partition by whole 128-row tiles of the LM head (128256 = 1002 tiles
    -> 125 or 126 tiles per rank at 8 ranks)."""
    return _even_range(vocab, rank, world, VOCAB_TILE)


def gather_row_stats(stats: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather per-rank ``[3, N]`` statistics into ``[world, 3, N]`` - the single
    collective of the vocabulary-parallel cross entropy.  Works on any backend."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return stats.unsqueeze(0)
    world = dist.get_world_size(group)
    flat = torch.empty((world * stats.shape[0], *stats.shape[1:]), dtype=stats.dtype, device=stats.device)
    dist.all_gather_into_tensor(flat, stats.contiguous(), group=group)   # concatenation along dim 0
    return flat.view(world, *stats.shape)


def vocab_parallel_linear_cross_entropy(hidden: torch.Tensor, weight_shard: torch.Tensor, targets: torch.Tensor,
                                        v_start: int, ignore_index: int = -100, reduction: str = "mean",
                                        group=None) -> torch.Tensor:
    """Cross entropy of ``hidden @ W.T`` where this rank holds ``W[v_start : v_start +
    len(weight_shard)]``; hidden and targets are replicated.  Every rank returns the
    same fp32 loss."""
    from .kernels.linear_cross_entropy import lce_loss_from_stats, lce_row_stats
    if reduction not in ("mean", "sum", "none"):
        raise ValueError(f"reduction must be 'mean', 'sum', or 'none', got {reduction!r}")
    stats = lce_row_stats(hidden, weight_shard, targets, v_start)
    return lce_loss_from_stats(gather_row_stats(stats, group), targets, ignore_index, reduction)


def vocab_parallel_linear_cross_entropy_fwd_bwd(hidden: torch.Tensor, weight_shard: torch.Tensor,
                                                targets: torch.Tensor, v_start: int, ignore_index: int = -100,
                                                reduction: str = "mean", rows_per_chunk: int = 8192,
                                                scatter_rows: bool = False, group=None
                                                ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Loss, ``d_hidden`` and this rank's ``d_weight`` rows for a vocabulary-sharded LM head.

    Collectives: the ``[3, rows]`` statistics all-gather of the forward (one per row chunk),
    and one reduction of the per-shard ``d_hidden`` contributions - an all-reduce, or with
    ``scatter_rows`` (``N`` divisible by the world size) a reduce-scatter that leaves each rank
    with its ``row_range`` of ``d_hidden``.  ``d_weight`` needs no exchange: every rank owns its
    rows."""
    from .kernels import linear_cross_entropy as lce
    scale = lce.lce_grad_scale(targets, ignore_index, reduction)
    stats, d_hidden, d_weight = lce.lce_stats_and_gradients(
        hidden, weight_shard, targets, scale, v_start, ignore_index, rows_per_chunk,
        gather=lambda st: gather_row_stats(st, group))
    loss = lce.lce_loss_from_stats(stats, targets, ignore_index, reduction)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        world = dist.get_world_size(group)
        if scatter_rows:
            if hidden.shape[0] % world:
                raise ValueError(f"scatter_rows needs N ({hidden.shape[0]}) divisible by the world size ({world})")
            mine = torch.empty(hidden.shape[0] // world, hidden.shape[1], dtype=d_hidden.dtype, device=d_hidden.device)
            dist.reduce_scatter_tensor(mine, d_hidden, group=group)
            d_hidden = mine
        else:
            dist.all_reduce(d_hidden, group=group)
    return loss, d_hidden, d_weight


def max_over_ranks(value: float, device=None) -> float:
    """MAX all-reduce of a host scalar (used for device-timed durations)."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device or ("cuda" if torch.cuda.is_available() else "cpu"))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
