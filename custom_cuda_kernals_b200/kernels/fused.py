"""GEMMs with the neighbouring elementwise op folded into the epilogue (additions; the
reference runs gate_proj, up_proj, swiglu, down_proj and the residual add as separate
kernels, examples/llama_block.py:168-172).  Results equal the unfused chains bit for bit."""

from __future__ import annotations

import torch

from .. import _native

__all__ = ["interleave_gate_up", "matmul_swiglu", "matmul_add_bias_residual", "matmul_add_bias_rope", "matmul_add_bias_stats",
           "rmsnorm_from_stats", "fp8_quant_token_from_amax", "matmul_general", "rmsnorm_fp8_quant",
           "matmul_swiglu_fp8", "matmul_add_bias_residual_fp8", "matmul_add_bias_rope_fp8", "GATE_UP_BLOCK"]

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


def matmul_add_bias_rope(x: torch.Tensor, w_qkv: torch.Tensor, bias: torch.Tensor | None, cos: torch.Tensor,
                         sin: torch.Tensor, rope_cols: int) -> torch.Tensor:
    """One projection for q, k and v with the rotary embedding applied in the GEMM epilogue:
    ``y = x @ w_qkv.T + bias`` (``x [B*S, K]``, rows ordered sequence by sequence; ``w_qkv`` = q, k
    and v weights concatenated along the output dimension, heads of 128), then RoPE with
    ``cos, sin [S, 64]`` (row ``r`` is position ``r % S``) on the first ``rope_cols`` output columns
    - the q and k heads.  Equals ``rope_strided`` applied to the q / k column ranges of
    ``matmul_add_bias(x, w_qkv, bias)`` bit for bit, without the extra pass over q and k
    (examples/llama_block.py:147-156 run three projections and a separate rope kernel).
    Returns ``[B*S, N]``; q, k and v are column ranges of it."""
    y = torch.empty((x.shape[0], w_qkv.shape[0]), dtype=x.dtype, device=x.device)
    _native.matmul_add_bias_rope_fwd(x, w_qkv, bias, cos, sin, y, rope_cols)
    return y


def matmul_add_bias_stats(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                          residual: torch.Tensor | None = None, sumsq: bool = True, amax: bool = False
                          ) -> tuple[torch.Tensor, torch.Tensor | None, torch.Tensor | None]:
    """``y = x @ weight.T + bias (+ residual)`` - bit for bit what ``matmul_add_bias`` (or
    ``matmul_add_bias_residual``) returns - together with what the op after it needs, computed in
    the same epilogue from the stored values: ``row_sumsq`` and / or ``row_amax``, each
    ``[ceil(N / 256), M]`` float32 (one value per row and 256-column output tile; the tiles of a row
    are computed by different CTAs).  Feed them to ``rmsnorm_from_stats`` /
    ``fp8_quant_token_from_amax``, which then skip their own row reduction.  These are the steps
    either side of o_proj and down_proj in the reference's block (examples/llama_block.py:163-172).
    Returns ``(y, row_sumsq or None, row_amax or None)``."""
    m, n = x.shape[0], weight.shape[0]
    tiles = _native.gemm_stat_tiles(n)
    y = torch.empty((m, n), dtype=x.dtype, device=x.device)
    stats = torch.empty((int(sumsq) + int(amax), tiles, m), dtype=torch.float32, device=x.device)
    ss = stats[0] if sumsq else None
    am = stats[int(sumsq)] if amax else None
    _native.matmul_add_bias_stats_fwd(x, weight, bias, residual, y, ss, am)
    return y, ss, am


def rmsnorm_from_stats(x: torch.Tensor, row_sumsq: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``rmsnorm(x, weight, eps)`` for an ``x`` that came out of ``matmul_add_bias_stats``: the
    sum of squares of every row is the sum of its ``row_sumsq`` partials (added in tile order),
    so this pass only scales.  Same rounding chain as ``rmsnorm``; the two can differ where the
    order of the fp32 additions moves the statistic by an ulp."""
    y = torch.empty_like(x)
    _native.rmsnorm_from_stats_fwd(x, row_sumsq, weight, y, eps)
    return y


def fp8_quant_token_from_amax(x: torch.Tensor, row_amax: torch.Tensor, fp8_format: str = "e4m3"
                              ) -> tuple[torch.Tensor, torch.Tensor]:
    """``fp8_quant(x, fp8_format, "token")`` for an ``x`` that came out of
    ``matmul_add_bias_stats(..., amax=True)``: bit-identical codes and ``[M, 1]`` scales, without
    the row-wide maximum (it is the maximum of the row's ``row_amax`` partials)."""
    if fp8_format not in ("e4m3", "e5m2"):
        raise ValueError(f"fp8_format must be 'e4m3' or 'e5m2', got {fp8_format!r}")
    fp8_dtype = torch.float8_e4m3fn if fp8_format == "e4m3" else torch.float8_e5m2
    codes = torch.empty(x.shape, dtype=fp8_dtype, device=x.device)
    scale = torch.empty((x.shape[0], 1), dtype=torch.float32, device=x.device)
    _native.fp8_quant_token_from_amax_fwd(x, row_amax, codes, scale, fp8_format)
    return codes, scale


def matmul_general(a: torch.Tensor, b: torch.Tensor, a_transposed: bool = False, b_transposed: bool = False,
                   out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """``A @ B.T`` on the tensor cores with either operand read as stored.

    ``a`` holds ``A [M, K]``, or with ``a_transposed`` its transpose ``[K, M]``; ``b`` holds
    ``B [N, K]`` (the ``nn.Linear`` weight layout), or with ``b_transposed`` ``[K, N]``.  The
    gradients of ``y = x @ W.T`` are the transposed forms - ``dx = matmul_general(dy, W,
    b_transposed=True)``, ``dW = matmul_general(dy, x, a_transposed=True, b_transposed=True)`` - and
    no transposed copy of ``dy``, ``W`` or ``x`` is made.  With ``accumulate`` the product is added
    to the float32 tensor ``out`` (a gradient summed over row chunks); otherwise the result is in
    the operands' dtype (written to ``out`` if given).  float16 / bfloat16; the contiguous
    dimension of each operand must be a multiple of 8."""
    m = a.shape[1] if a_transposed else a.shape[0]
    n = b.shape[1] if b_transposed else b.shape[0]
    if accumulate and out is None:
        raise ValueError("accumulate=True needs the float32 tensor to accumulate into (out=...)")
    if out is None:
        out = torch.empty((m, n), dtype=a.dtype, device=a.device)
    _native.matmul_general_fwd(a, b, out, a_transposed, b_transposed, accumulate)
    return out


def _fp8_dtype(fp8_format: str) -> torch.dtype:
    if fp8_format not in ("e4m3", "e5m2"):
        raise ValueError(f"fp8_format must be 'e4m3' or 'e5m2', got {fp8_format!r}")
    return torch.float8_e4m3fn if fp8_format == "e4m3" else torch.float8_e5m2


def rmsnorm_fp8_quant(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, fp8_format: str = "e4m3",
                      row_sumsq: torch.Tensor | None = None, want_normed: bool = False):
    """``fp8_quant(rmsnorm(x, weight, eps), fp8_format, "token")`` in one pass over ``x``: the
    normalised row never goes to memory (unless ``want_normed`` asks for it too), so the norm that
    feeds an FP8 projection costs 3 bytes of HBM traffic per element instead of 7.  Codes and
    ``[M, 1]`` scales are bit-identical to the two-kernel chain.  ``row_sumsq`` (from
    ``matmul_add_bias_stats``) replaces the row reduction, as in ``rmsnorm_from_stats``.
    Returns ``(codes, scale)`` or ``(codes, scale, normed)``."""
    codes = torch.empty(x.shape, dtype=_fp8_dtype(fp8_format), device=x.device)
    scale = torch.empty((x.shape[0], 1), dtype=torch.float32, device=x.device)
    y = torch.empty_like(x) if want_normed else None
    _native.rmsnorm_fp8_quant_token_fwd(x, weight, row_sumsq, y, codes, scale, eps, fp8_format)
    return (codes, scale, y) if want_normed else (codes, scale)


def matmul_swiglu_fp8(a_fp8: torch.Tensor, a_scale: torch.Tensor, w_gate_up_fp8: torch.Tensor, w_scale: torch.Tensor,
                      out_dtype: torch.dtype = torch.bfloat16, amax: bool = False):
    """``matmul_swiglu`` with e4m3 operands: ``a_fp8 [M, K]`` with per-token scales, ``w_gate_up_fp8
    [2F, K]`` = the per-row quantisation of ``interleave_gate_up(Wg, Wu)`` with its ``[2F]`` scales.
    Equals ``swiglu(matmul_add_bias_fp8(a, Wg), matmul_add_bias_fp8(a, Wu))`` bit for bit.  With
    ``amax`` also returns ``row_amax [F / 128, M]`` for ``fp8_quant_token_from_amax``."""
    m, f = a_fp8.shape[0], w_gate_up_fp8.shape[0] // 2
    y = torch.empty((m, f), dtype=out_dtype, device=a_fp8.device)
    am = torch.empty((f // GATE_UP_BLOCK, m), dtype=torch.float32, device=a_fp8.device) if amax else None
    _native.matmul_swiglu_fp8_fwd(a_fp8, a_scale, w_gate_up_fp8, w_scale, y, am)
    return (y, am) if amax else y


def matmul_add_bias_rope_fp8(a_fp8: torch.Tensor, a_scale: torch.Tensor, w_fp8: torch.Tensor, w_scale: torch.Tensor,
                             bias: torch.Tensor | None, cos: torch.Tensor, sin: torch.Tensor, rope_cols: int,
                             out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``matmul_add_bias_rope`` with e4m3 operands (per-token / per-output-channel scales): equals
    ``rope_strided`` on the q / k column ranges of ``matmul_add_bias_fp8(...)`` bit for bit."""
    y = torch.empty((a_fp8.shape[0], w_fp8.shape[0]), dtype=out_dtype, device=a_fp8.device)
    _native.matmul_add_bias_rope_fp8_fwd(a_fp8, a_scale, w_fp8, w_scale, bias, cos, sin, y, rope_cols)
    return y


def matmul_add_bias_residual_fp8(a_fp8: torch.Tensor, a_scale: torch.Tensor, w_fp8: torch.Tensor, w_scale: torch.Tensor,
                                 bias: torch.Tensor | None, residual: torch.Tensor) -> torch.Tensor:
    """``matmul_add_bias_fp8(a, w, bias) + residual`` in one kernel (same roundings)."""
    y = torch.empty((a_fp8.shape[0], w_fp8.shape[0]), dtype=residual.dtype, device=a_fp8.device)
    _native.matmul_add_bias_residual_fp8_fwd(a_fp8, a_scale, w_fp8, w_scale, bias, residual, y)
    return y
