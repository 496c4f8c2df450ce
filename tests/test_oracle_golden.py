"""CPU: the oracle replayed against the committed golden vectors.

The golden files were produced by the reference project's own baselines
(``tests/golden/make_golden.py``); these tests need no reference checkout.
"""

import hashlib
import json
import pathlib

import pytest
import torch

from oracle import cases, ops

GOLD = pathlib.Path(__file__).parent / "golden"
golden = torch.load(GOLD / "golden_small.pt")
digests = json.loads((GOLD / "fp8_digests.json").read_text())
pin = json.loads((GOLD / "pin_report.json").read_text())


def _sha(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def _near(a, b, dtype):
    # elementwise chains are IEEE-exact on any CPU except libm-level functions
    # (exp, cos, sin, rsqrt) and reduction order; allow 2 ulp of the storage type.
    ulp = {torch.float32: 2 ** -22, torch.float16: 2 ** -9, torch.bfloat16: 2 ** -6}[dtype]
    torch.testing.assert_close(a.float(), b.float(), rtol=ulp, atol=ulp * 1e-2)


def test_pin_report_is_clean():
    assert set(pin["ops"]) == {"rmsnorm", "swiglu", "rope", "fp8", "gemm", "lce", "router", "gather", "combine",
                               "block"}
    for op, r in pin["ops"].items():
        assert r["cases"] >= (3 if op == "block" else 18), op
        assert not r["input_mismatch"] and not r["output_mismatch"], op


@pytest.mark.parametrize("key", [k for k in golden if k.startswith("rmsnorm/")])
def test_rmsnorm(key):
    c = cases.by_name(cases.NORM_CASES, key.split("/")[1])
    y, ro = ops.rmsnorm_residual(*cases.norm_inputs(c), c.eps)
    assert torch.equal(ro, golden[key]["residual_out"])
    _near(y, golden[key]["y"], c.dtype)


@pytest.mark.parametrize("key", [k for k in golden if k.startswith("swiglu/")])
def test_swiglu(key):
    c = cases.by_name(cases.GLU_CASES, key.split("/")[1])
    _near(ops.swiglu(*cases.glu_inputs(c)), golden[key]["y"], c.dtype)


@pytest.mark.parametrize("key", [k for k in golden if k.startswith("rope/") and "tables" not in k])
def test_rope(key):
    c = cases.by_name(cases.ROPE_CASES, key.split("/")[1])
    q, k = ops.rope(*cases.rope_inputs(c))
    _near(q, golden[key]["q"], c.dtype)
    _near(k, golden[key]["k"], c.dtype)


def test_rope_tables_llama3():
    cos, sin = ops.rope_tables(64, 128, 500000.0)
    torch.testing.assert_close(cos, golden["rope/tables_theta500000"]["cos"], rtol=0, atol=2e-6)
    torch.testing.assert_close(sin, golden["rope/tables_theta500000"]["sin"], rtol=0, atol=2e-6)


def test_rope_tables_offset_is_a_slice():
    cos, sin = ops.rope_tables(48, 64, 10000.0)
    c2, s2 = ops.rope_tables(16, 64, 10000.0, pos_offset=32)
    assert torch.equal(cos[32:], c2) and torch.equal(sin[32:], s2)


@pytest.mark.parametrize("name", sorted(digests))
def test_fp8_bit_exact_against_reference_digest(name):
    """Codes and scales of every reference FP8 case (tensor + block), bit for bit."""
    c = cases.by_name(cases.FP8_CASES, name)
    if c.m * c.n > 1 << 22:
        pytest.skip("large case kept for the GPU suite")
    codes, scale = ops.fp8_quant(cases.fp8_inputs(c), c.fp8_format, c.granularity)
    assert _sha(codes) == digests[name]["codes"]
    assert _sha(scale.reshape(-1)) == digests[name]["scale"]


@pytest.mark.parametrize("key", [k for k in golden if k.startswith("fp8/")])
def test_fp8_small_vectors(key):
    c = cases.by_name(cases.FP8_CASES, key.split("/")[1])
    codes, scale = ops.fp8_quant(cases.fp8_inputs(c), c.fp8_format, c.granularity)
    assert torch.equal(codes.view(torch.uint8), golden[key]["codes"])
    assert torch.equal(scale, golden[key]["scale"])


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
def test_fp8_token_mode_properties(fmt):
    """Per-token mode is unpinned by the reference; check it against the
    tensor-mode chain row by row (a 1-row matrix's tensor scale is its token scale)."""
    x = torch.randn(37, 200, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    codes, scale = ops.fp8_quant(x, fmt, "token")
    assert scale.shape == (37, 1) and scale.dtype == torch.float32
    for r in (0, 17, 36):
        c1, s1 = ops.fp8_quant(x[r:r + 1], fmt, "tensor")
        assert torch.equal(c1.view(torch.uint8), codes[r:r + 1].view(torch.uint8))
        assert s1.item() == scale[r].item()
    z, zs = ops.fp8_quant(torch.zeros(4, 16), fmt, "token")
    assert torch.all(z.float() == 0) and torch.all(zs > 0) and torch.isfinite(zs).all()


def test_fp8_e4m3_cast_rules():
    """Ties to even incl. subnormals, sign of zero kept, (448,464] saturates by rounding."""
    v = torch.tensor([2.0 ** -10, 1.5 * 2.0 ** -9, -0.0, 448.00003, 460.0, 0.4375 + 2 ** -6])
    got = v.to(torch.float8_e4m3fn).view(torch.uint8).tolist()
    assert got[0] == 0x00 and got[1] == 0x02 and got[2] == 0x80 and got[3] == 0x7E and got[4] == 0x7E


@pytest.mark.parametrize("key", [k for k in golden if k.startswith("gemm/")])
def test_gemm(key):
    c = cases.by_name(cases.GEMM_CASES, key.split("/")[1])
    y = ops.matmul_add_bias(*cases.gemm_inputs(c))
    rtol, atol, frac = ops.TOLERANCE_GEMM[c.dtype]
    ops.assert_close_with_outliers(y, golden[key]["y"], rtol=rtol, atol=atol, max_outlier_fraction=frac)


@pytest.mark.parametrize("key", [k for k in golden if k.startswith("lce/")])
def test_lce(key):
    c = cases.by_name(cases.LCE_CASES, key.split("/")[1])
    h, w, t = cases.lce_inputs(c)
    loss = ops.linear_cross_entropy(h, w, t, reduction=c.reduction)
    want, want64 = golden[key]["loss"], golden[key]["loss64"]
    if c.name.startswith("all_ignored"):
        assert torch.isnan(loss) and torch.isnan(want)
        return
    rtol, atol, _ = ops.TOLERANCE_GEMM[c.dtype]
    torch.testing.assert_close(loss.float(), want.float(), rtol=rtol, atol=atol)
    blocked = ops.linear_cross_entropy_rowblocked(h, w, t, reduction=c.reduction, rows_per_block=100)
    torch.testing.assert_close(blocked, want64, rtol=1e-9, atol=1e-9)


def test_lce_partials_merge_equals_full():
    c = cases.by_name(cases.LCE_CASES, "with_ignored_float32")
    h, w, t = cases.lce_inputs(c)
    cuts = [0, 1024, 2048, 3000, 4000]
    parts = [ops.lce_partials(h, w[a:b], t, a) for a, b in zip(cuts[:-1], cuts[1:])]
    per_row = ops.lce_merge(parts)
    want = ops.linear_cross_entropy_fp64(h, w, t, reduction="none")
    keep = t != -100
    torch.testing.assert_close(per_row[keep], want[keep], rtol=1e-10, atol=1e-10)


@pytest.mark.parametrize("key", [k for k in golden if k.startswith("block/")])
def test_block_against_reference_block_output(key):
    """The oracle block against the stored output of the reference's own BaselineLlamaBlock
    (examples/llama_block.py:83-189) on the same seeded weights and input.  On the machine that
    wrote the file the two are bit-equal (pin_report.json); another CPU may pick other bf16 GEMM
    kernels, so the replay uses the reference's block bar (examples/llama_block.py:271-283:
    rtol 1e-2, atol 2e-2) with the outlier budget two bf16 evaluations of the chain need."""
    from oracle import workloads
    cfg, w, x = workloads.block_pin_inputs(key.split("/")[1])
    with torch.no_grad():
        y = ops.llama_block(x, w, n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"], eps=cfg["eps"],
                            theta=cfg["theta"])
    want = golden[key]["y"]
    assert y.shape == want.shape and y.dtype == want.dtype
    if torch.equal(y, want):
        return
    ops.assert_close_with_outliers(y, want, rtol=1e-2, atol=2e-2, max_outlier_fraction=0.05)


def test_block_oracle_runs_and_is_finite():
    from oracle import workloads
    cfg = dict(workloads.LLAMA3_8B, hidden=256, ffn=512, n_heads=4, n_kv_heads=2, head_dim=64)
    w = workloads.block_weights(cfg)
    x = workloads.block_input(2, 16, 256)
    y = ops.llama_block(x, w, n_heads=4, n_kv_heads=2)
    assert y.shape == x.shape and y.dtype == torch.bfloat16 and torch.isfinite(y.float()).all()


@pytest.mark.parametrize("key", [k for k in golden if k.startswith("router/")])
def test_moe_router(key):
    c = cases.by_name(cases.ROUTER_CASES, key.split("/")[1])
    w, i = ops.moe_router(cases.router_inputs(c), c.k, c.renormalize)
    assert w.dtype == torch.float32 and i.dtype == torch.int64
    _near(w, golden[key]["weights"], torch.float32)
    assert torch.equal(i, golden[key]["indices"])


@pytest.mark.parametrize("key", [k for k in golden if k.startswith("gather/")])
def test_token_gather(key):
    c = cases.by_name(cases.GATHER_CASES, key.split("/")[1])
    assert torch.equal(ops.token_gather(*cases.gather_inputs(c)), golden[key]["dst"])


@pytest.mark.parametrize("key", [k for k in golden if k.startswith("combine/") and "permutation" not in k])
def test_token_combine(key):
    c = cases.by_name(cases.COMBINE_CASES, key.split("/")[1])
    _near(ops.token_combine(*cases.combine_inputs(c)), golden[key]["combined"], c.dtype)


def test_compute_permutation_golden_and_round_trip():
    g = golden["combine/compute_permutation"]
    perm, unperm = ops.compute_permutation(g["topk"])
    assert torch.equal(perm, g["permute_index"]) and torch.equal(unperm, g["unpermute_index"])
    # gather into expert order, combine back with unit weight on one choice: the identity
    t, k = g["topk"].shape
    x = torch.randn(t, 16, generator=torch.Generator().manual_seed(1))
    expert_rows = ops.token_gather(x, perm)
    assert torch.all(g["topk"].reshape(-1)[torch.argsort(g["topk"].reshape(-1), stable=True)].diff() >= 0)
    w = torch.zeros(t, k)
    w[:, 1] = 1.0
    assert torch.equal(ops.token_combine(expert_rows, unperm, w), x)
