"""Seeded synthetic inputs for the five benchmark configurations (test
infrastructure; also used by ``bench.py`` to build its host-side inputs).

Every generator draws on the CPU from ``torch.Generator().manual_seed(seed)``
so that the GPU path and the CPU oracle see identical tensors.  ``scale``
arguments shrink the row count for parity tests without changing the
distributions.
"""

from __future__ import annotations

import torch

from .ops import rope_tables

SEEDS = {"rmsnorm": 1001, "swiglu": 1002, "rope": 1003, "fp8": 1004, "gemm": 1005,
         "block": 1006, "lce": 1007}

LLAMA3_8B = dict(hidden=4096, ffn=14336, n_heads=32, n_kv_heads=8, head_dim=128,
                 eps=1e-5, theta=500000.0, vocab=128256)


def _gen(key, salt=0):
    return torch.Generator().manual_seed(SEEDS[key] + 7919 * salt)


def rmsnorm_fp32(tokens=2048, hidden=4096, salt=0):
    """Config 1: x, residual ~ N(0,1) fp32, weight = 1 + 0.1 N(0,1), eps 1e-5."""
    g = _gen("rmsnorm", salt)
    x = torch.randn(tokens, hidden, generator=g)
    r = torch.randn(tokens, hidden, generator=g)
    w = 1.0 + 0.1 * torch.randn(hidden, generator=g)
    return x, r, w, 1e-5


def swiglu_bf16(rows=8192, ffn=14336, salt=0):
    """Config 2a: gate, up ~ N(0,1) bf16."""
    g = _gen("swiglu", salt)
    gate = torch.randn(rows, ffn, generator=g).to(torch.bfloat16)
    up = torch.randn(rows, ffn, generator=g).to(torch.bfloat16)
    return gate, up


def rope_bf16(batch=4, seq=2048, n_q=32, n_kv=8, head_dim=128, theta=500000.0, salt=0):
    """Config 2b: q, k ~ N(0,1) bf16; fp32 tables for positions 0..seq-1."""
    g = _gen("rope", salt)
    q = torch.randn(batch, seq, n_q, head_dim, generator=g).to(torch.bfloat16)
    k = torch.randn(batch, seq, n_kv, head_dim, generator=g).to(torch.bfloat16)
    cos, sin = rope_tables(seq, head_dim, theta)
    return q, k, cos, sin


def fp8_activations(rows=8192, cols=4096, salt=0, outlier_fraction=1e-3, outlier_gain=50.0):
    """Config 2c: x ~ N(0,1) bf16 with 0.1 % of the elements multiplied by 50."""
    g = _gen("fp8", salt)
    x = torch.randn(rows, cols, generator=g)
    hot = torch.rand(rows, cols, generator=g) < outlier_fraction
    x = torch.where(hot, x * outlier_gain, x)
    return x.to(torch.bfloat16)


def gemm_bf16(m=8192, k=4096, n=14336, salt=0):
    """Config 3: A ~ N(0,1), W[N,K] ~ N(0,0.02), bias ~ N(0,0.02), bf16."""
    g = _gen("gemm", salt)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    b = (0.02 * torch.randn(n, generator=g)).to(torch.bfloat16)
    return a, w, b


def block_weights(cfg=LLAMA3_8B, salt=0, dtype=torch.bfloat16):
    """Config 4 parameters: every projection N(0, 0.02), norm weights 1."""
    g = _gen("block", salt)
    hid, ffn = cfg["hidden"], cfg["ffn"]
    kv = cfg["n_kv_heads"] * cfg["head_dim"]

    def lin(out_f, in_f):
        return (0.02 * torch.randn(out_f, in_f, generator=g)).to(dtype)

    return {
        "input_layernorm_weight": torch.ones(hid, dtype=dtype),
        "post_attention_layernorm_weight": torch.ones(hid, dtype=dtype),
        "q_proj": lin(hid, hid), "k_proj": lin(kv, hid), "v_proj": lin(kv, hid),
        "o_proj": lin(hid, hid), "gate_proj": lin(ffn, hid), "up_proj": lin(ffn, hid),
        "down_proj": lin(hid, ffn),
    }


def block_input(batch=8, seq=2048, hidden=4096, salt=0, dtype=torch.bfloat16):
    """Config 4 activations: 0.02 * N(0,1)."""
    g = _gen("block", 1000 + salt)
    return (0.02 * torch.randn(batch, seq, hidden, generator=g)).to(dtype)


# decoder-block pins: name -> (architecture overrides of LLAMA3_8B, batch, seq)
BLOCK_PINS = {
    "small_gqa": (dict(hidden=256, ffn=512, n_heads=8, n_kv_heads=2, head_dim=32), 2, 48),
    "small_mha": (dict(hidden=128, ffn=384, n_heads=4, n_kv_heads=4, head_dim=32), 3, 17),
    "llama3_8b_seq64": (dict(), 1, 64),
}


def block_pin_inputs(name):
    """Weights and input of one decoder-block pin: the benchmark's seeded generators, with
    norm weights 1 + 0.1 N(0,1) instead of ones so that the norm-weight multiply is exercised."""
    over, batch, seq = BLOCK_PINS[name]
    cfg = dict(LLAMA3_8B, **over)
    w = block_weights(cfg)
    g = torch.Generator().manual_seed(4242)
    for key in ("input_layernorm_weight", "post_attention_layernorm_weight"):
        w[key] = (1.0 + 0.1 * torch.randn(cfg["hidden"], generator=g)).to(torch.bfloat16)
    return cfg, w, block_input(batch, seq, cfg["hidden"])


def lce_bf16(tokens=16384, hidden=4096, vocab=128256, ignore_fraction=0.05, salt=0):
    """Config 5: hidden ~ N(0,1), LM-head W[V,H] ~ N(0,0.02), labels uniform
    with 5 % replaced by -100.
    """
    g = _gen("lce", salt)
    h = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    w = torch.empty(vocab, hidden, dtype=torch.bfloat16)
    step = 8192
    for v0 in range(0, vocab, step):           # bounded fp32 staging
        v1 = min(vocab, v0 + step)
        w[v0:v1] = (0.02 * torch.randn(v1 - v0, hidden, generator=g)).to(torch.bfloat16)
    t = torch.randint(0, vocab, (tokens,), generator=g, dtype=torch.long)
    drop = torch.rand(tokens, generator=g) < ignore_fraction
    t = torch.where(drop, torch.full_like(t, -100), t)
    return h, w, t
