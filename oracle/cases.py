"""Shape/dtype case tables and seeded input generators (test infrastructure).

The tables list the same shapes the reference project's tests sweep (its
``STANDARD_CASES`` + ``EDGE_CASES`` in baselines/<op>.py), crossed with
f32/f16/bf16, and the generators draw from one ``torch.Generator`` in the same
order as the reference's ``make_inputs`` so that a CPU run with the same seed
yields the very tensors the reference's baselines would see.
"""

from __future__ import annotations

from collections import namedtuple

import torch

DTYPES = (torch.float32, torch.float16, torch.bfloat16)


def _short(dt):
    return str(dt).replace("torch.", "")


def _cross(kind, rows, fields, extra=()):
    out = []
    for row in rows:
        name, *vals = row
        for dt in DTYPES:
            out.append(kind(f"{name}_{_short(dt)}", *vals[:len(fields)], dt, *vals[len(fields):], *extra))
    return out


# --------------------------------------------------------------------------- rmsnorm + residual
# baselines/rmsnorm_residual.py:76-93
NormCase = namedtuple("NormCase", "name batch seq_len hidden_dim dtype eps", defaults=(1e-6,))
NORM_CASES = _cross(NormCase, [
    ("small", 4, 128, 768), ("medium", 2, 2048, 4096), ("large", 1, 4096, 4096),
    ("npot_batch", 3, 17, 4096), ("npot_hidden", 2, 64, 100), ("seq_len_1", 8, 1, 4096),
    ("long_seq", 1, 8192, 2048), ("empty_batch", 0, 128, 4096), ("single_elem", 1, 1, 128),
], "bsh")


def norm_inputs(case, seed=0, device="cpu"):
    """x, residual, weight ~ N(0,1) in that draw order (baselines/rmsnorm_residual.py:96-120)."""
    g = torch.Generator(device=device).manual_seed(seed)
    shape = (case.batch, case.seq_len, case.hidden_dim)
    x = torch.randn(shape, dtype=case.dtype, device=device, generator=g)
    r = torch.randn(shape, dtype=case.dtype, device=device, generator=g)
    w = torch.randn(case.hidden_dim, dtype=case.dtype, device=device, generator=g)
    return x, r, w


# --------------------------------------------------------------------------- swiglu
# baselines/swiglu.py:66-83
GluCase = namedtuple("GluCase", "name batch seq_len intermediate_dim dtype")
GLU_CASES = _cross(GluCase, [
    ("small", 4, 128, 3072), ("medium", 2, 2048, 11008), ("large", 1, 4096, 11008),
    ("npot_batch", 3, 17, 11008), ("npot_dim", 2, 64, 100), ("seq_len_1", 8, 1, 11008),
    ("long_seq", 1, 8192, 4096), ("empty_batch", 0, 128, 11008), ("single_elem", 1, 1, 128),
], "bsd")


def glu_inputs(case, seed=0, device="cpu"):
    """gate, up ~ N(0,1) (baselines/swiglu.py:85-104)."""
    g = torch.Generator(device=device).manual_seed(seed)
    shape = (case.batch, case.seq_len, case.intermediate_dim)
    gate = torch.randn(shape, dtype=case.dtype, device=device, generator=g)
    up = torch.randn(shape, dtype=case.dtype, device=device, generator=g)
    return gate, up


# --------------------------------------------------------------------------- rope
# baselines/rope.py:83-100
RopeCase = namedtuple("RopeCase", "name batch seq_len n_q_heads n_kv_heads head_dim dtype theta",
                      defaults=(10000.0,))
ROPE_CASES = _cross(RopeCase, [
    ("small_mha", 4, 128, 12, 12, 64), ("medium_gqa", 2, 2048, 32, 8, 128),
    ("large_gqa", 1, 4096, 32, 8, 128), ("npot_batch", 3, 17, 8, 2, 64),
    ("seq_len_1", 8, 1, 8, 8, 64), ("long_seq", 1, 8192, 8, 8, 64),
    ("empty_batch", 0, 128, 8, 8, 64), ("single_elem", 1, 1, 1, 1, 64),
    ("small_head_dim", 2, 32, 4, 1, 16),
], "bsqkd")


def rope_inputs(case, seed=0, device="cpu"):
    """q, k ~ N(0,1) plus the fp32 tables (baselines/rope.py:118-126)."""
    from .ops import rope_tables
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn((case.batch, case.seq_len, case.n_q_heads, case.head_dim),
                    dtype=case.dtype, device=device, generator=g)
    k = torch.randn((case.batch, case.seq_len, case.n_kv_heads, case.head_dim),
                    dtype=case.dtype, device=device, generator=g)
    cos, sin = rope_tables(case.seq_len, case.head_dim, case.theta)
    return q, k, cos.to(device), sin.to(device)


# --------------------------------------------------------------------------- fp8 quantisation
# baselines/fp8_quant.py:96-118 ("token" granularity is this library's addition)
Fp8Case = namedtuple("Fp8Case", "name m n dtype fp8_format granularity")
_FP8_SHAPES = [
    ("small", 256, 256), ("medium", 1024, 1024), ("large", 4096, 4096),
    ("npot_ragged", 257, 513), ("smaller_than_tile", 64, 64), ("single_row", 1, 256),
    ("single_col", 256, 1), ("tall_skinny", 2048, 128),
]
FP8_CASES = [
    Fp8Case(f"{name}_{_short(dt)}_{fmt}_{gran}", m, n, dt, fmt, gran)
    for name, m, n in _FP8_SHAPES for dt in DTYPES
    for fmt in ("e4m3", "e5m2") for gran in ("tensor", "block", "token")
]


def fp8_inputs(case, seed=0, device="cpu"):
    """x ~ N(0,1) (baselines/fp8_quant.py:121-123)."""
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn((case.m, case.n), dtype=case.dtype, device=device, generator=g)


# --------------------------------------------------------------------------- matmul + bias
# baselines/matmul_add_bias.py:80-101
GemmCase = namedtuple("GemmCase", "name m k n dtype has_bias", defaults=(True,))
GEMM_CASES = _cross(GemmCase, [
    ("qkv_proj", 2048, 4096, 4096), ("mlp_up", 2048, 4096, 11008), ("mlp_down", 2048, 11008, 4096),
    ("npot_dims", 257, 513, 129), ("tall_skinny", 4096, 64, 64), ("short_wide", 64, 64, 4096),
    ("k_eq_1", 128, 1, 128), ("single_row", 1, 256, 256), ("empty_m", 0, 256, 256),
], "mkn") + _cross(GemmCase, [("no_bias", 256, 512, 256)], "mkn", extra=(False,))


def gemm_inputs(case, seed=0, device="cpu"):
    """x, weight[N,K], bias, each 0.02*N(0,1) (baselines/matmul_add_bias.py:104-114)."""
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn((case.m, case.k), dtype=case.dtype, device=device, generator=g) * 0.02
    w = torch.randn((case.n, case.k), dtype=case.dtype, device=device, generator=g) * 0.02
    b = None
    if case.has_bias:
        b = torch.randn(case.n, dtype=case.dtype, device=device, generator=g) * 0.02
    return x, w, b


# --------------------------------------------------------------------------- linear cross entropy
# baselines/linear_cross_entropy.py:82-108
LceCase = namedtuple("LceCase", "name n_tokens hidden_dim vocab_size dtype ignore_fraction reduction",
                     defaults=(0.0, "mean"))
LCE_CASES = _cross(LceCase, [
    ("small_vocab", 256, 768, 8000), ("llama2_vocab", 512, 4096, 32000),
    ("llama3_vocab", 256, 4096, 128256), ("npot_tokens", 257, 256, 1009),
    ("with_ignored", 256, 256, 4000, 0.3), ("all_ignored", 64, 128, 1000, 1.0),
    ("single_token", 1, 128, 1000), ("empty_batch", 0, 128, 1000), ("tiny_vocab", 64, 64, 3),
    ("reduction_sum", 128, 128, 2000, 0.0, "sum"), ("reduction_none", 128, 128, 2000, 0.0, "none"),
], "nhv")


def lce_inputs(case, seed=0, device="cpu"):
    """hidden, weight = 0.02*N(0,1); labels uniform; an ``ignore_fraction`` of
    them replaced by -100 (baselines/linear_cross_entropy.py:111-130).
    """
    g = torch.Generator(device=device).manual_seed(seed)
    hidden = torch.randn((case.n_tokens, case.hidden_dim), dtype=case.dtype, device=device, generator=g) * 0.02
    weight = torch.randn((case.vocab_size, case.hidden_dim), dtype=case.dtype, device=device, generator=g) * 0.02
    if case.n_tokens == 0:
        return hidden, weight, torch.empty(0, dtype=torch.long, device=device)
    targets = torch.randint(0, case.vocab_size, (case.n_tokens,), device=device, generator=g, dtype=torch.long)
    if case.ignore_fraction > 0:
        drop = torch.rand(case.n_tokens, device=device, generator=g) < case.ignore_fraction
        targets = torch.where(drop, torch.full_like(targets, -100), targets)
    return hidden, weight, targets


# --------------------------------------------------------------------------- MoE router
# baselines/moe_router.py:78-100
RouterCase = namedtuple("RouterCase", "name n_tokens n_experts k dtype renormalize", defaults=(True,))
ROUTER_CASES = _cross(RouterCase, [
    ("mixtral_like", 2048, 8, 2), ("deepseek_like", 2048, 160, 6), ("ksweep_k1", 1024, 32, 1),
    ("ksweep_k2", 1024, 32, 2), ("ksweep_k4", 1024, 32, 4), ("ksweep_k8", 1024, 32, 8),
    ("npot_experts", 256, 100, 4), ("npot_tokens", 257, 16, 2), ("single_expert", 64, 1, 1),
    ("k_eq_experts", 64, 8, 8), ("large_expert_count", 128, 256, 8),
], "tek") + _cross(RouterCase, [("no_renorm", 256, 16, 2)], "tek", extra=(False,)) + _cross(RouterCase, [
    ("single_token", 1, 16, 2), ("empty_batch", 0, 16, 2)], "tek")


def router_inputs(case, seed=0, device="cpu"):
    """logits ~ N(0,1) (baselines/moe_router.py:103-106)."""
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn((case.n_tokens, case.n_experts), dtype=case.dtype, device=device, generator=g)


# --------------------------------------------------------------------------- token gather / combine
# baselines/token_permute.py:139-167
GatherCase = namedtuple("GatherCase", "name n_src_rows n_dst_rows hidden_dim dtype")
GATHER_CASES = _cross(GatherCase, [
    ("mixtral_like", 2048, 4096, 4096), ("large_hidden", 2048, 4096, 11008), ("npot_hidden", 257, 513, 100),
    ("single_row", 1, 1, 256), ("empty_dst", 64, 0, 256), ("small_hidden", 128, 256, 16),
], "sdh")
CombineCase = namedtuple("CombineCase", "name n_tokens k hidden_dim dtype")
COMBINE_CASES = _cross(CombineCase, [
    ("mixtral_like", 2048, 2, 4096), ("deepseek_like", 2048, 6, 4096), ("k1", 256, 1, 512), ("k8", 256, 8, 512),
    ("npot_hidden", 257, 3, 100), ("single_token", 1, 2, 256), ("empty_batch", 0, 2, 256), ("small_hidden", 128, 4, 16),
], "tkh")


def gather_inputs(case, seed=0, device="cpu"):
    """src ~ N(0,1), then uniform row indices (baselines/token_permute.py:170-182)."""
    g = torch.Generator(device=device).manual_seed(seed)
    src = torch.randn((case.n_src_rows, case.hidden_dim), dtype=case.dtype, device=device, generator=g)
    if case.n_dst_rows == 0 or case.n_src_rows == 0:
        indices = torch.empty(case.n_dst_rows, dtype=torch.long, device=device)
    else:
        indices = torch.randint(0, case.n_src_rows, (case.n_dst_rows,), device=device, generator=g, dtype=torch.long)
    return src, indices


def combine_inputs(case, seed=0, device="cpu"):
    """expert_output ~ N(0,1), weights ~ U(0,1) fp32, then a random permutation of the expert
    rows as the index (baselines/token_permute.py:185-204).  Returns (expert_output,
    unpermute_index, weights)."""
    g = torch.Generator(device=device).manual_seed(seed)
    n = case.n_tokens * case.k
    expert_output = torch.randn((n, case.hidden_dim), dtype=case.dtype, device=device, generator=g)
    weights = torch.rand(case.n_tokens, case.k, dtype=torch.float32, device=device, generator=g)
    if n == 0:
        index = torch.empty(case.n_tokens, case.k, dtype=torch.long, device=device)
    else:
        index = torch.randperm(n, device=device, generator=g).reshape(case.n_tokens, case.k)
    return expert_output, index, weights


def by_name(table, name):
    for case in table:
        if case.name == name:
            return case
    raise KeyError(name)
