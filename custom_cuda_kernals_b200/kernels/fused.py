"""GEMMs with the neighbouring elementwise op folded into the epilogue (additions; the
reference runs gate_proj, up_proj, swiglu, down_proj and the residual add as separate
kernels, examples/llama_block.py:168-172).  Results equal the unfused chains bit for bit."""

from __future__ import annotations

import torch

from .. import _native

__all__ = ["interleave_gate_up", "matmul_swiglu", "matmul_add_bias_residual", "GATE_UP_BLOCK"]

GATE_UP_BLOCK = 128


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """``[F, K]`` gate and up weights -> one ``[2F, K]`` weight in which every block of 128
    gate rows is followed by the matching 128 up rows (the layout ``matmul_swiglu`` reads).
    ``F`` must be a multiple of 128.  Done once, when the weights are loaded."""
    f, k = w_gate.shape
    if w_up.shape != w_gate.shape or f % GATE_UP_BLOCK != 0:
        raise ValueError(f"gate/up weights must share a shape [F, K] with F a multiple of {GATE_UP_BLOCK}; "
                         f"got {tuple(w_gate.shape)} and {tuple(w_up.shape)}")
    g = w_gate.reshape(f // GATE_UP_BLOCK, GATE_UP_BLOCK, k)
    u = w_up.reshape(f // GATE_UP_BLOCK, GATE_UP_BLOCK, k)
    return torch.stack([g, u], dim=1).reshape(2 * f, k).contiguous()


def matmul_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(x @ Wg.T) * (x @ Wu.T)`` for ``w_gate_up = interleave_gate_up(Wg, Wu)``;
    x ``[M, K]`` float16/bfloat16, returns ``[M, F]``."""
    y = torch.empty((x.shape[0], w_gate_up.shape[0] // 2), dtype=x.dtype, device=x.device)
    _native.matmul_swiglu_fwd(x, w_gate_up, y)
    return y


def matmul_add_bias_residual(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
                             residual: torch.Tensor) -> torch.Tensor:
    """``x @ weight.T + bias + residual`` (residual ``[M, N]``), float16/bfloat16."""
    y = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
    _native.matmul_add_bias_residual_fwd(x, weight, bias, residual, y)
    return y
