"""Pin the CPU oracle to the reference project and write the golden vectors.

Run once, on a machine that has a checkout of the reference project
(BhargavKumarNath/custom_cuda_kernals):

    python tests/golden/make_golden.py --reference /path/to/reference

It imports the reference's own ``baselines`` package, and for EVERY case of
the reference's ``ALL_CASES`` tables (on CPU, seed 0):

  1. checks that ``oracle.cases.*_inputs`` reproduces the reference's
     ``make_inputs`` tensors bit for bit;
  2. checks that ``oracle.ops.*`` reproduces the reference's ``eager_*``
     (and ``reference_fp64``) outputs bit for bit;

  3. builds the reference's own decoder block (``BaselineLlamaBlock`` of
     ``examples/llama_block.py:83-189``, ``device="cpu"``) on a small and on a
     Llama-3-8B-shaped configuration, loads the oracle's seeded weights into
     it and checks that ``oracle.ops.llama_block`` reproduces its output bit
     for bit (the example imports ``custom_cuda.kernels``; this repository's
     alias package of that name is imported first, so the built ``_native``
     module must exist, no GPU is needed);

then stores, for a set of small cases, the reference's outputs in
``golden_small.pt`` and, for every FP8 case, a SHA-256 of the reference's code
bytes and scale bytes in ``fp8_digests.json``.  ``pin_report.json`` records
what was compared.  ``tests/test_oracle_golden.py`` replays these files with no
reference checkout present.
"""

from __future__ import annotations

import argparse
import hashlib
import importlib
import json
import pathlib
import sys

import torch

HERE = pathlib.Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from oracle import cases, ops, workloads  # noqa: E402

SMALL = {
    "rmsnorm": ["npot_hidden", "single_elem"],
    "swiglu": ["npot_dim", "single_elem"],
    "rope": ["npot_batch", "single_elem", "small_head_dim"],
    "fp8": ["smaller_than_tile", "single_row", "single_col"],
    "gemm": ["npot_dims", "single_row"],
    "lce": ["npot_tokens", "with_ignored", "all_ignored", "tiny_vocab", "reduction_sum",
            "reduction_none", "single_token"],
    "router": ["npot_tokens", "single_expert", "k_eq_experts", "no_renorm", "single_token"],
    "gather": ["npot_hidden", "single_row", "small_hidden"],
    "combine": ["npot_hidden", "single_token", "small_hidden"],
}
SKIP_HEAVY = {"mlp_up", "mlp_down", "llama3_vocab", "llama2_vocab"}  # minutes of CPU GEMM each


def digest(t):
    raw = t.contiguous().view(torch.uint8) if t.dtype != torch.uint8 else t.contiguous()
    return hashlib.sha256(raw.numpy().tobytes()).hexdigest()


def same(a, b):
    if a is None or b is None:
        return a is None and b is None
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    if a.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    return torch.equal(a, b) or bool(((a == b) | (a.isnan() & b.isnan())).all())


def base_of(name):
    for suffix in ("_float32", "_float16", "_bfloat16"):
        if suffix in name:
            return name.split(suffix)[0]
    return name


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    # this repository's alias package, before the reference checkout goes first on sys.path:
    # the reference's decoder-block example imports the same names
    import custom_cuda.kernels.rmsnorm_residual  # noqa: F401
    import custom_cuda.kernels.rope  # noqa: F401
    import custom_cuda.kernels.swiglu  # noqa: F401
    sys.path.insert(0, args.reference)
    ref = {k: importlib.import_module(f"baselines.{m}") for k, m in {
        "rmsnorm": "rmsnorm_residual", "swiglu": "swiglu", "rope": "rope", "fp8": "fp8_quant",
        "gemm": "matmul_add_bias", "lce": "linear_cross_entropy", "router": "moe_router",
        "permute": "token_permute"}.items()}
    torch.manual_seed(0)

    golden, digests = {}, {}
    report = {"torch": torch.__version__, "ops": {}}

    def note(op, ok_inputs, ok_outputs, name):
        r = report["ops"].setdefault(op, {"cases": 0, "input_mismatch": [], "output_mismatch": []})
        r["cases"] += 1
        if not ok_inputs:
            r["input_mismatch"].append(name)
        if not ok_outputs:
            r["output_mismatch"].append(name)

    # ---- rmsnorm
    mine = {c.name: c for c in cases.NORM_CASES}
    for rc in ref["rmsnorm"].ALL_CASES:
        c = mine[rc.name]
        ri = ref["rmsnorm"].make_inputs(rc, device="cpu", seed=0)
        mi = cases.norm_inputs(c, seed=0)
        ro = ref["rmsnorm"].eager_rmsnorm_residual(*ri, rc.eps)
        mo = ops.rmsnorm_residual(*mi, c.eps)
        r64 = ref["rmsnorm"].reference_fp64(*ri, rc.eps)
        m64 = ops.rmsnorm_residual_fp64(*mi, c.eps)
        note("rmsnorm", all(same(a, b) for a, b in zip(ri, mi)),
             all(same(a, b) for a, b in zip(ro + r64, mo + m64)), rc.name)
        if base_of(rc.name) in SMALL["rmsnorm"]:
            golden[f"rmsnorm/{rc.name}"] = {"y": ro[0], "residual_out": ro[1]}

    # ---- swiglu
    mine = {c.name: c for c in cases.GLU_CASES}
    for rc in ref["swiglu"].ALL_CASES:
        c = mine[rc.name]
        ri = ref["swiglu"].make_inputs(rc, device="cpu", seed=0)
        mi = cases.glu_inputs(c, seed=0)
        ro, mo = ref["swiglu"].eager_swiglu(*ri), ops.swiglu(*mi)
        note("swiglu", all(same(a, b) for a, b in zip(ri, mi)),
             same(ro, mo) and same(ref["swiglu"].reference_fp64(*ri), ops.swiglu_fp64(*mi)), rc.name)
        if base_of(rc.name) in SMALL["swiglu"]:
            golden[f"swiglu/{rc.name}"] = {"y": ro}

    # ---- rope
    mine = {c.name: c for c in cases.ROPE_CASES}
    for rc in ref["rope"].ALL_CASES:
        c = mine[rc.name]
        ri = ref["rope"].make_inputs(rc, device="cpu", seed=0)
        mi = cases.rope_inputs(c, seed=0)
        ro, mo = ref["rope"].eager_rope(*ri), ops.rope(*mi)
        r64, m64 = ref["rope"].reference_fp64(*ri), ops.rope_fp64(*mi)
        note("rope", all(same(a, b) for a, b in zip(ri, mi)),
             all(same(a, b) for a, b in zip(ro + r64, mo + m64)), rc.name)
        if base_of(rc.name) in SMALL["rope"]:
            golden[f"rope/{rc.name}"] = {"q": ro[0], "k": ro[1]}
    # the Llama-3 table (theta 500000) used by the benchmark configs
    rc_cos, rc_sin = ref["rope"].compute_cos_sin(64, 128, 500000.0, device="cpu")
    mc, ms = ops.rope_tables(64, 128, 500000.0)
    note("rope", True, same(rc_cos, mc) and same(rc_sin, ms), "tables_theta500000")
    golden["rope/tables_theta500000"] = {"cos": rc_cos, "sin": rc_sin}

    # ---- fp8 (tensor + block exist in the reference; token is this library's addition)
    mine = {c.name: c for c in cases.FP8_CASES}
    for rc in ref["fp8"].ALL_CASES:
        c = mine[rc.name]
        ri = ref["fp8"].make_inputs(rc, device="cpu", seed=0)
        mi = cases.fp8_inputs(c, seed=0)
        rcodes, rscale = ref["fp8"].eager_fp8_quant(ri, rc.fp8_format, rc.granularity)
        mcodes, mscale = ops.fp8_quant(mi, c.fp8_format, c.granularity)
        r64 = ref["fp8"].reference_fp64(ri, rc.fp8_format, rc.granularity)
        m64 = ops.fp8_scale_fp64(mi, c.fp8_format, c.granularity)
        rdq = ref["fp8"].dequantize(rcodes, rscale, rc.granularity)
        mdq = ops.fp8_dequant(mcodes, mscale, c.granularity)
        note("fp8", same(ri, mi), same(rcodes, mcodes) and same(rscale, mscale) and same(r64, m64)
             and same(rdq, mdq), rc.name)
        digests[rc.name] = {"codes": digest(rcodes), "scale": digest(rscale.reshape(-1))}
        if base_of(rc.name) in SMALL["fp8"]:
            golden[f"fp8/{rc.name}"] = {"codes": rcodes.view(torch.uint8), "scale": rscale}

    # ---- matmul + bias
    mine = {c.name: c for c in cases.GEMM_CASES}
    for rc in ref["gemm"].ALL_CASES:
        if base_of(rc.name) in SKIP_HEAVY:
            continue
        c = mine[rc.name]
        ri = ref["gemm"].make_inputs(rc, device="cpu", seed=0)
        mi = cases.gemm_inputs(c, seed=0)
        ro = ref["gemm"].eager_matmul_add_bias_unfused(*ri)
        mo = ops.matmul_add_bias(*mi)
        note("gemm", all(same(a, b) for a, b in zip(ri, mi)),
             same(ro, mo) and same(ref["gemm"].reference_fp64(*ri), ops.matmul_add_bias_fp64(*mi)),
             rc.name)
        if base_of(rc.name) in SMALL["gemm"]:
            golden[f"gemm/{rc.name}"] = {"y": ro}

    # ---- linear cross entropy
    mine = {c.name: c for c in cases.LCE_CASES}
    for rc in ref["lce"].ALL_CASES:
        if base_of(rc.name) in SKIP_HEAVY:
            continue
        c = mine[rc.name]
        ri = ref["lce"].make_inputs(rc, device="cpu", seed=0)
        mi = cases.lce_inputs(c, seed=0)
        ro = ref["lce"].eager_linear_cross_entropy(*ri, reduction=rc.reduction)
        mo = ops.linear_cross_entropy(*mi, reduction=c.reduction)
        r64 = ref["lce"].reference_fp64(*ri, reduction=rc.reduction)
        m64 = ops.linear_cross_entropy_fp64(*mi, reduction=c.reduction)
        note("lce", all(same(a, b) for a, b in zip(ri, mi)), same(ro, mo) and same(r64, m64), rc.name)
        if base_of(rc.name) in SMALL["lce"]:
            golden[f"lce/{rc.name}"] = {"loss": ro, "loss64": r64}

    # ---- MoE router
    mine = {c.name: c for c in cases.ROUTER_CASES}
    for rc in ref["router"].ALL_CASES:
        c = mine[rc.name]
        ri = ref["router"].make_inputs(rc, device="cpu", seed=0)
        mi = cases.router_inputs(c, seed=0)
        ro = ref["router"].eager_moe_router(ri, rc.k, rc.renormalize)
        mo = ops.moe_router(mi, c.k, c.renormalize)
        r64 = ref["router"].reference_fp64(ri, rc.k, rc.renormalize)
        m64 = ops.moe_router(mi, c.k, c.renormalize, wide=True)
        note("router", same(ri, mi) and rc.renormalize == c.renormalize,
             all(same(a, b) for a, b in zip(ro + r64, mo + m64)), rc.name)
        if base_of(rc.name) in SMALL["router"]:
            golden[f"router/{rc.name}"] = {"weights": ro[0], "indices": ro[1]}

    # ---- token gather / combine and the permutation bookkeeping
    mine = {c.name: c for c in cases.GATHER_CASES}
    for rc in ref["permute"].GATHER_ALL_CASES:
        c = mine[rc.name]
        ri = ref["permute"].make_gather_inputs(rc, device="cpu", seed=0)
        mi = cases.gather_inputs(c, seed=0)
        ro, mo = ref["permute"].eager_token_gather(*ri), ops.token_gather(*mi)
        note("gather", all(same(a, b) for a, b in zip(ri, mi)),
             same(ro, mo) and same(ref["permute"].reference_gather_fp64(*ri), ops.token_gather(*mi, wide=True)), rc.name)
        if base_of(rc.name) in SMALL["gather"]:
            golden[f"gather/{rc.name}"] = {"dst": ro}
    mine = {c.name: c for c in cases.COMBINE_CASES}
    for rc in ref["permute"].COMBINE_ALL_CASES:
        c = mine[rc.name]
        ri = ref["permute"].make_combine_inputs(rc, device="cpu", seed=0)
        mi = cases.combine_inputs(c, seed=0)
        ro, mo = ref["permute"].eager_token_combine(*ri), ops.token_combine(*mi)
        note("combine", all(same(a, b) for a, b in zip(ri, mi)),
             same(ro, mo) and same(ref["permute"].reference_combine_fp64(*ri), ops.token_combine(*mi, wide=True)), rc.name)
        if base_of(rc.name) in SMALL["combine"]:
            golden[f"combine/{rc.name}"] = {"combined": ro}
    topk = torch.randint(0, 8, (37, 3), generator=torch.Generator().manual_seed(3))
    rp, mp = ref["permute"].compute_permutation(topk), ops.compute_permutation(topk)
    note("combine", True, all(same(a, b) for a, b in zip(rp, mp)), "compute_permutation")
    golden["combine/compute_permutation"] = {"topk": topk, "permute_index": rp[0], "unpermute_index": rp[1]}

    # ---- the decoder block (examples/llama_block.py:83-189; acceptance check :271-283)
    example = importlib.import_module("examples.llama_block")
    for name in workloads.BLOCK_PINS:
        cfg, w, x = workloads.block_pin_inputs(name)
        blk = example.BaselineLlamaBlock(
            hidden_size=cfg["hidden"], intermediate_size=cfg["ffn"], num_heads=cfg["n_heads"],
            num_kv_heads=cfg["n_kv_heads"], seq_len=x.shape[1], rms_eps=cfg["eps"], rope_theta=cfg["theta"],
            dtype=torch.bfloat16, device="cpu")
        with torch.no_grad():
            for key, t in w.items():
                target = getattr(blk, key)
                (target.weight if isinstance(target, torch.nn.Linear) else target).copy_(t)
            ro = blk(x)
            mo = ops.llama_block(x, w, n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"], eps=cfg["eps"],
                                 theta=cfg["theta"])
        note("block", True, same(ro, mo), name)
        golden[f"block/{name}"] = {"y": ro}

    torch.save(golden, HERE / "golden_small.pt")
    (HERE / "fp8_digests.json").write_text(json.dumps(digests, indent=0, sort_keys=True))
    (HERE / "pin_report.json").write_text(json.dumps(report, indent=1, sort_keys=True))
    bad = {op: r for op, r in report["ops"].items() if r["input_mismatch"] or r["output_mismatch"]}
    print(json.dumps({op: r["cases"] for op, r in report["ops"].items()}))
    if bad:
        print("MISMATCH", json.dumps(bad, indent=1))
        raise SystemExit(1)
    print("oracle == reference baselines on every compared case; golden files written")


if __name__ == "__main__":
    main()
