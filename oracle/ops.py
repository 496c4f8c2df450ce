"""CPU restatement of the six Llama-block ops (test infrastructure only).

Every function runs on CPU tensors and follows the reference baseline's chain
of casts exactly, because for bf16/fp16 storage the position of each rounding
is part of the result.  Citations are ``path:line`` inside the reference
project (BhargavKumarNath/custom_cuda_kernals).
"""

from __future__ import annotations

import math

import torch

F32 = torch.float32
F64 = torch.float64

FP8_TORCH_DTYPE = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
FP8_TILE = 128          # side of one scale tile in "block" granularity
FP8_SCALE_FLOOR = 1e-12  # lower clamp on every scale
IGNORE_INDEX = -100


# --------------------------------------------------------------------------- rmsnorm + residual
def rmsnorm_residual(x, residual, weight, eps):
    """``ro = x + residual`` (rounded to the storage dtype), then the norm of
    that *rounded* sum in fp32, cast back, times ``weight`` in the storage
    dtype.  Follows baselines/rmsnorm_residual.py:130-136.
    """
    store = x.dtype
    ro = x + residual
    wide = ro.to(F32)
    mean_sq = (wide * wide).mean(dim=-1, keepdim=True)
    y = (wide * torch.rsqrt(mean_sq + eps)).to(store) * weight
    return y, ro


def rmsnorm_residual_fp64(x, residual, weight, eps):
    """fp64 ground truth, baselines/rmsnorm_residual.py:158-169."""
    ro = x.to(F64) + residual.to(F64)
    inv = torch.rsqrt((ro * ro).mean(dim=-1, keepdim=True) + eps)
    return ro * inv * weight.to(F64), ro


# --------------------------------------------------------------------------- swiglu
def swiglu(gate, up):
    """``silu(gate)`` in fp32, rounded to the storage dtype, then multiplied by
    ``up`` in the storage dtype.  Follows baselines/swiglu.py:109-112.
    """
    g = gate.to(F32)
    return (g * torch.sigmoid(g)).to(gate.dtype) * up


def swiglu_fp64(gate, up):
    """baselines/swiglu.py:127-132."""
    g = gate.to(F64)
    return g * torch.sigmoid(g) * up.to(F64)


# --------------------------------------------------------------------------- rope
def rope_tables(seq_len, head_dim, theta=10000.0, pos_offset=0):
    """fp32 cos/sin tables ``[seq_len, head_dim/2]`` for positions
    ``pos_offset .. pos_offset+seq_len-1``.  With ``pos_offset=0`` this is
    baselines/rope.py:103-115: ``inv_freq = 1/theta**(2i/D)`` in fp32, outer
    product with fp32 positions, then cos and sin.
    """
    exponents = torch.arange(0, head_dim, 2, dtype=F32) / head_dim
    inv_freq = 1.0 / (theta ** exponents)
    pos = torch.arange(pos_offset, pos_offset + seq_len, dtype=F32)
    angle = torch.outer(pos, inv_freq)
    return angle.cos().contiguous(), angle.sin().contiguous()


def _rotate(x, cos, sin, wide):
    half = x.shape[-1] // 2
    xw = x.to(wide)
    lo, hi = xw[..., :half], xw[..., half:]
    c = cos.to(wide)[None, :, None, :]
    s = sin.to(wide)[None, :, None, :]
    return torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1)


def rope(q, k, cos, sin):
    """Half-split rotation of ``q [B,S,Hq,D]`` and ``k [B,S,Hkv,D]`` in fp32
    with one rounding to the storage dtype.  baselines/rope.py:129-145.
    """
    return _rotate(q, cos, sin, F32).to(q.dtype), _rotate(k, cos, sin, F32).to(k.dtype)


def rope_fp64(q, k, cos, sin):
    """baselines/rope.py:159-176."""
    return _rotate(q, cos, sin, F64), _rotate(k, cos, sin, F64)


# --------------------------------------------------------------------------- fp8 quantisation
def _tile_amax(mag, tile):
    """amax of every ``tile x tile`` block of a non-negative matrix; ragged
    edge tiles are padded with zeros (which cannot change a max of
    magnitudes).  baselines/fp8_quant.py:126-146.
    """
    m, n = mag.shape
    pm, pn = (-m) % tile, (-n) % tile
    if pm or pn:
        mag = torch.nn.functional.pad(mag, (0, pn, 0, pm))
    rows, cols = mag.shape[0] // tile, mag.shape[1] // tile
    return mag.reshape(rows, tile, cols, tile).amax(dim=(1, 3))


def fp8_spread_scale(scale, granularity, m, n, tile=FP8_TILE):
    """Broadcast a scale tensor of any granularity to ``[m, n]``."""
    if granularity == "tensor":
        return scale.reshape(1, 1).expand(m, n)
    if granularity == "token":
        return scale.reshape(m, 1).expand(m, n)
    wide = scale.repeat_interleave(tile, dim=0).repeat_interleave(tile, dim=1)
    return wide[:m, :n]


def fp8_quant(x, fp8_format="e4m3", granularity="block", tile=FP8_TILE):
    """Dynamic FP8 quantisation: ``scale = max(amax / FP8_MAX, 1e-12)`` and
    ``codes = (x32 / scale) -> fp8`` with IEEE fp32 divisions and a
    round-to-nearest-even cast.  ``"tensor"`` and ``"block"`` follow
    baselines/fp8_quant.py:152-178 (scale is 0-D resp. ``[ceil(M/128),
    ceil(N/128)]``).  ``"token"`` is the same chain with a row-wise amax and
    ``scale [M, 1]``; the reference has no baseline for it, so that mode is
    unpinned by the reference.
    """
    fp8 = FP8_TORCH_DTYPE[fp8_format]
    top = torch.finfo(fp8).max
    x32 = x.to(F32)
    mag = x32.abs()
    m, n = x.shape
    if granularity == "tensor":
        scale = torch.clamp(mag.max() / top, min=FP8_SCALE_FLOOR)
        return (x32 / scale).to(fp8), scale
    if granularity == "token":
        scale = torch.clamp(mag.amax(dim=-1, keepdim=True) / top, min=FP8_SCALE_FLOOR)
        return (x32 / scale).to(fp8), scale
    if granularity == "block":
        scale = torch.clamp(_tile_amax(mag, tile) / top, min=FP8_SCALE_FLOOR)
        return (x32 / fp8_spread_scale(scale, "block", m, n, tile)).to(fp8), scale
    raise ValueError(f"unknown granularity {granularity!r}")


def fp8_dequant(codes, scale, granularity, tile=FP8_TILE):
    """``codes.float() * scale`` (baselines/fp8_quant.py:181-189)."""
    m, n = codes.shape
    return codes.to(F32) * fp8_spread_scale(scale, granularity, m, n, tile)


def fp8_scale_fp64(x, fp8_format, granularity, tile=FP8_TILE):
    """fp64 ground truth for the scale only (baselines/fp8_quant.py:192-210)."""
    top = torch.finfo(FP8_TORCH_DTYPE[fp8_format]).max
    mag = x.to(F64).abs()
    if granularity == "tensor":
        amax = mag.max()
    elif granularity == "token":
        amax = mag.amax(dim=-1, keepdim=True)
    else:
        amax = _tile_amax(mag, tile)
    return torch.clamp(amax / top, min=FP8_SCALE_FLOOR)


# --------------------------------------------------------------------------- matmul + bias
def matmul_add_bias(x, weight, bias=None):
    """``x @ weight.T`` rounded to the storage dtype, then ``+ bias`` in the
    storage dtype (two roundings).  baselines/matmul_add_bias.py:117-126.
    """
    y = x @ weight.T
    return y if bias is None else y + bias


def matmul_add_bias_fp64(x, weight, bias=None):
    """baselines/matmul_add_bias.py:149-156."""
    y = x.to(F64) @ weight.to(F64).T
    return y if bias is None else y + bias.to(F64)


def matmul_add_bias_fp8(a_codes, a_scale, w_codes, w_scale, bias=None, out_dtype=torch.bfloat16):
    """FP8 GEMM with per-token activation scales ``[M,1]`` and per-output-
    channel weight scales ``[N,1]``: dequantise both operands to fp32, matmul
    in fp32, add the bias in fp32, round once.  The reference has no FP8 GEMM
    (csrc/kernels/matmul_add_bias.cu:200-219 accepts f32/f16/bf16 only), so
    this variant is unpinned by the reference.
    """
    a = a_codes.to(F32) * a_scale.reshape(-1, 1)
    w = w_codes.to(F32) * w_scale.reshape(-1, 1)
    y = a @ w.T
    if bias is not None:
        y = y + bias.to(F32)
    return y.to(out_dtype)


# --------------------------------------------------------------------------- linear + cross entropy
def linear_cross_entropy(hidden, weight, targets, ignore_index=IGNORE_INDEX, reduction="mean"):
    """Full logits in the storage dtype, then ``F.cross_entropy``; the loss
    comes back in the storage dtype.  baselines/linear_cross_entropy.py:133-146.
    """
    logits = hidden @ weight.T
    return torch.nn.functional.cross_entropy(
        logits, targets, ignore_index=ignore_index, reduction=reduction)


def linear_cross_entropy_fp64(hidden, weight, targets, ignore_index=IGNORE_INDEX, reduction="mean"):
    """baselines/linear_cross_entropy.py:171-180."""
    logits = hidden.to(F64) @ weight.to(F64).T
    return torch.nn.functional.cross_entropy(
        logits, targets, ignore_index=ignore_index, reduction=reduction)


def linear_cross_entropy_rowblocked(hidden, weight, targets, ignore_index=IGNORE_INDEX,
                                    reduction="mean", rows_per_block=1024, wide=F64):
    """The same function evaluated ``rows_per_block`` rows at a time so the
    ``[N, V]`` logits never exist at once (rows are independent).  Per-row
    losses are computed in ``wide`` precision and reduced in fp64.
    """
    n = hidden.shape[0]
    w = weight.to(wide)
    per_row = torch.zeros(n, dtype=F64)
    for r0 in range(0, n, rows_per_block):
        r1 = min(n, r0 + rows_per_block)
        logits = hidden[r0:r1].to(wide) @ w.T
        per_row[r0:r1] = torch.nn.functional.cross_entropy(
            logits, targets[r0:r1], ignore_index=ignore_index, reduction="none").to(F64)
    if reduction == "none":
        return per_row
    total = per_row.sum()
    if reduction == "sum":
        return total
    return total / (targets != ignore_index).sum().to(F64)


def lce_partials(hidden, weight_slice, targets, v_start):
    """Per-row ``(max, sum exp(l - max), target logit or 0)`` of the logits
    against one vocabulary slice ``weight[v_start : v_start+len]``, in fp64.
    This is the quantity one rank of a vocabulary-sharded run produces.
    """
    logits = hidden.to(F64) @ weight_slice.to(F64).T
    mx = logits.max(dim=1).values
    sm = torch.exp(logits - mx[:, None]).sum(dim=1)
    local = targets - v_start
    inside = (local >= 0) & (local < weight_slice.shape[0])
    tg = torch.zeros_like(mx)
    if inside.any():
        rows = torch.nonzero(inside).squeeze(1)
        tg[rows] = logits[rows, local[rows]]
    return mx, sm, tg


def lce_merge(partials):
    """Merge per-slice ``(max, sumexp, target)`` triples into per-row loss."""
    mx = torch.stack([p[0] for p in partials]).max(dim=0).values
    sm = sum(p[1] * torch.exp(p[0] - mx) for p in partials)
    tg = sum(p[2] for p in partials)
    return mx + torch.log(sm) - tg


# --------------------------------------------------------------------------- Llama decoder block
def llama_block(x, w, n_heads=32, n_kv_heads=8, eps=1e-5, theta=500000.0):
    """Llama-3 style pre-norm decoder block built from the ops above plus
    torch SDPA, structured as examples/llama_block.py:158-173 (norm ->
    q/k/v projections -> rope -> causal GQA attention -> o_proj -> norm ->
    gate/up -> swiglu -> down -> + residual).  ``w`` maps the reference's
    parameter names to tensors ``[out_features, in_features]``.
    """
    b, s, hid = x.shape
    d = hid // n_heads
    cos, sin = rope_tables(s, d, theta)
    h, res = rmsnorm_residual(x, torch.zeros_like(x), w["input_layernorm_weight"], eps)
    q = (h @ w["q_proj"].T).view(b, s, n_heads, d)
    k = (h @ w["k_proj"].T).view(b, s, n_kv_heads, d)
    v = (h @ w["v_proj"].T).view(b, s, n_kv_heads, d)
    q, k = rope(q, k, cos, sin)
    rep = n_heads // n_kv_heads
    if rep > 1:
        k = k[:, :, :, None, :].expand(b, s, n_kv_heads, rep, d).reshape(b, s, n_heads, d)
        v = v[:, :, :, None, :].expand(b, s, n_kv_heads, rep, d).reshape(b, s, n_heads, d)
    att = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
    att = att.transpose(1, 2).contiguous().view(b, s, hid) @ w["o_proj"].T
    h2, res2 = rmsnorm_residual(att, res, w["post_attention_layernorm_weight"], eps)
    mlp = swiglu(h2 @ w["gate_proj"].T, h2 @ w["up_proj"].T) @ w["down_proj"].T
    return mlp + res2


# --------------------------------------------------------------------------- comparison helper
# --------------------------------------------------------------------------- mixture-of-experts neighbours
def moe_router(logits, k, renormalize=True, wide=False):
    """baselines/moe_router.py:109-119 (eager) and :139-148 (fp64 when ``wide``): softmax in
    fp32, top-k probabilities and their expert ids, optional renormalisation."""
    probs = torch.softmax(logits.to(torch.float64 if wide else torch.float32), dim=-1)
    topk_weights, topk_indices = torch.topk(probs, k, dim=-1)
    if renormalize:
        topk_weights = topk_weights / topk_weights.sum(dim=-1, keepdim=True)
    return topk_weights, topk_indices


def compute_permutation(topk_indices):
    """baselines/token_permute.py:58-72: stable argsort of the flattened expert assignments
    and its inverse."""
    t, k = topk_indices.shape
    order = torch.argsort(topk_indices.reshape(-1), stable=True)
    inverse = torch.empty_like(order)
    inverse[order] = torch.arange(t * k, device=topk_indices.device)
    return order // k, inverse.reshape(t, k)


def token_gather(src, indices, wide=False):
    """baselines/token_permute.py:196-198 (:209-210 when ``wide``)."""
    return (src.to(torch.float64) if wide else src).index_select(0, indices)


def token_combine(expert_output, unpermute_index, weights, wide=False):
    """baselines/token_permute.py:213-226 (:240-248 when ``wide``): gather each token's k
    expert rows, scale by the fp32 gate weights, sum in fp32, round once."""
    if unpermute_index.numel() == 0:
        return torch.zeros(unpermute_index.shape[0], expert_output.shape[-1],
                           dtype=torch.float64 if wide else expert_output.dtype, device=expert_output.device)
    if wide:
        return (expert_output.to(torch.float64)[unpermute_index] * weights.to(torch.float64).unsqueeze(-1)).sum(dim=1)
    gathered = expert_output[unpermute_index]
    return (gathered.to(torch.float32) * weights.unsqueeze(-1)).sum(dim=1).to(expert_output.dtype)


def assert_close_with_outliers(actual, expected, *, rtol, atol, max_outlier_fraction=0.0):
    """``|a-e| <= atol + rtol*|e|`` for all but ``max_outlier_fraction`` of the
    elements (bf16 results sitting on a rounding boundary can flip by one ulp
    between two valid evaluation orders; tests/numerics.py:26-60).
    """
    a, e = actual.detach().cpu().double(), expected.detach().cpu().double()
    if a.shape != e.shape:
        raise AssertionError(f"shape {tuple(a.shape)} != {tuple(e.shape)}")
    if a.numel() == 0:
        return
    bad = (a - e).abs() > (atol + rtol * e.abs())
    bad |= torch.isnan(a) != torch.isnan(e)
    frac = bad.double().mean().item()
    if frac > max_outlier_fraction:
        worst = ((a - e).abs() - (atol + rtol * e.abs())).max().item()
        raise AssertionError(
            f"{int(bad.sum())} of {a.numel()} elements ({frac:.3e}) outside rtol={rtol} "
            f"atol={atol} (allowed fraction {max_outlier_fraction}); worst excess {worst:.3e}")


TOLERANCE = {
    # storage dtype -> (rtol, atol, outlier fraction); project_plan.md:475-481
    torch.float32: (1e-4, 1e-4, 0.0),
    torch.float16: (1e-2, 1e-3, 0.0),
    torch.bfloat16: (1e-2, 1e-2, 1e-5),
}
TOLERANCE_GEMM = {
    # tests/test_matmul_add_bias_kernel.py:23-27, tests/test_linear_cross_entropy_kernel.py:25-29
    torch.float32: (1e-4, 1e-4, 0.0),
    torch.float16: (1e-2, 1e-2, 0.0),
    torch.bfloat16: (1e-2, 2e-2, 1e-5),
}


def ceil_div(a, b):
    return math.ceil(a / b)
