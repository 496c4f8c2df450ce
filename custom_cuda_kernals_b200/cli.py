"""Developer command line: ``python -m custom_cuda_kernals_b200.cli <command>``.

Plain-``argparse`` counterparts of the reference's typer/rich tool (custom_cuda/cli/app.py:126-511)
for the operators this library covers:

    list                      the operators, their entry points and test files
    doctor                    environment check: Python, nvcc, PyTorch, GPU, the built libraries, and
                              a live probe of ``_native.rmsnorm_residual_fwd`` / ``fp8_quant_block_fwd``
                              (the two entry points the reference's doctor probes,
                              custom_cuda/cli/env_checks.py:128)
    verify [op] [--cpu]       run the op's parity tests (pytest), all ops when omitted
    benchmark <op> [...]      the op's shape sweep in the reference's CSV format (benchmarks.py) as a table
    profile <op> [-o trace]   torch.profiler Chrome trace of the op on representative inputs

Exit status 0 when everything asked for succeeded, 1 otherwise.  Output is plain text, one table
per command, so it can be read in a terminal or parsed.
"""

from __future__ import annotations

import argparse
import dataclasses
import pathlib
import re
import shutil
import subprocess
import sys
import time

ROOT = pathlib.Path(__file__).resolve().parent.parent
PKG = pathlib.Path(__file__).resolve().parent


@dataclasses.dataclass(frozen=True)
class OpSpec:
    id: str
    title: str
    entry: str                    # public function
    launchers: tuple[str, ...]    # C-ABI entry points
    gpu_tests: tuple[str, ...]
    bench: str | None             # CSV stem of benchmarks.py


OPS = [
    OpSpec("rmsnorm_residual", "Fused RMSNorm + residual add", "custom_cuda.kernels.rmsnorm_residual.rmsnorm_residual",
           ("launch_rmsnorm_residual_fwd", "launch_rmsnorm_fwd", "launch_rmsnorm_from_stats_fwd"),
           ("tests/test_gpu_elementwise.py", "tests/test_gpu_golden.py"), "rmsnorm_residual"),
    OpSpec("swiglu", "Fused SwiGLU", "custom_cuda.kernels.swiglu.swiglu", ("launch_swiglu_fwd",),
           ("tests/test_gpu_elementwise.py",), "swiglu"),
    OpSpec("rope", "Fused RoPE (q and k in one launch)", "custom_cuda.kernels.rope.rope",
           ("launch_rope_fwd", "launch_rope_strided_fwd"), ("tests/test_gpu_elementwise.py",), "rope"),
    OpSpec("fp8_quant", "Dynamic FP8 quantisation (token / block / tensor)", "custom_cuda.kernels.fp8_quant.fp8_quant",
           ("launch_fp8_quant_token_fwd", "launch_fp8_quant_block_fwd", "launch_fp8_quant_tensor_fwd",
            "launch_fp8_quant_token_from_amax_fwd"), ("tests/test_gpu_fp8.py",), "fp8_quant"),
    OpSpec("matmul_add_bias", "tcgen05 GEMM + bias (16-bit and FP8), fused epilogues",
           "custom_cuda.kernels.matmul_add_bias.matmul_add_bias",
           ("launch_matmul_add_bias_fwd", "launch_matmul_add_bias_fp8_fwd", "launch_matmul_swiglu_fwd",
            "launch_matmul_add_bias_residual_fwd", "launch_matmul_add_bias_stats_fwd"),
           ("tests/test_gpu_gemm.py", "tests/test_gpu_fused_stats.py", "tests/test_gpu_wait_limit.py"), "matmul_add_bias"),
    OpSpec("linear_cross_entropy", "Fused linear + cross entropy (logits stay in tensor memory)",
           "custom_cuda.kernels.linear_cross_entropy.linear_cross_entropy",
           ("launch_linear_cross_entropy_fwd", "launch_lce_finalize", "launch_linear_ce_chunk_update"),
           ("tests/test_gpu_lce.py",), "linear_cross_entropy"),
    OpSpec("moe_router", "Top-k softmax router", "custom_cuda.kernels.moe_router.moe_router", ("launch_moe_router_fwd",),
           ("tests/test_gpu_moe.py",), "moe_router"),
    OpSpec("token_permute", "Token gather / weighted combine", "custom_cuda.kernels.token_permute.token_gather",
           ("launch_token_gather_fwd", "launch_token_combine_fwd"), ("tests/test_gpu_moe.py",), "token_permute"),
    OpSpec("llama_block", "Llama-3 decoder block built from the ops above", "custom_cuda_kernals_b200.llama_block.LlamaBlock",
           (), ("tests/test_gpu_block.py",), None),
]
CPU_TESTS = ("tests/test_oracle_golden.py", "tests/test_cabi_symbols.py", "tests/test_dist_cpu.py")


def find_op(name: str) -> OpSpec:
    for op in OPS:
        if op.id == name:
            return op
    raise SystemExit(f"unknown op {name!r}; choose from: {', '.join(o.id for o in OPS)}")


def table(rows: list[tuple], header: tuple) -> str:
    cells = [tuple(str(c) for c in header)] + [tuple(str(c) for c in r) for r in rows]
    widths = [max(len(r[i]) for r in cells) for i in range(len(header))]
    lines = ["  ".join(c.ljust(w) for c, w in zip(r, widths)).rstrip() for r in cells]
    lines.insert(1, "  ".join("-" * w for w in widths))
    return "\n".join(lines)


# ------------------------------------------------------------------------------------------- doctor
@dataclasses.dataclass(frozen=True)
class Check:
    name: str
    status: str      # ok | warn | fail
    detail: str


def run_checks() -> list[Check]:
    """Same ground as custom_cuda/cli/env_checks.py: interpreter, compiler, PyTorch, GPU, extension."""
    out = [Check("Python interpreter", "ok", f"{sys.version.split()[0]} ({sys.executable})")]
    nvcc = shutil.which("nvcc") or ("/usr/local/cuda/bin/nvcc" if pathlib.Path("/usr/local/cuda/bin/nvcc").exists() else None)
    if nvcc is None:
        out.append(Check("nvcc (CUDA compiler)", "warn", "not found: prebuilt libraries still run, a rebuild cannot"))
    else:
        try:
            text = subprocess.run([nvcc, "--version"], capture_output=True, text=True, timeout=20).stdout
            rel = re.search(r"release (\d+\.\d+)", text)
            out.append(Check("nvcc (CUDA compiler)", "ok", f"release {rel.group(1) if rel else '?'} ({nvcc})"))
        except (OSError, subprocess.SubprocessError) as e:
            out.append(Check("nvcc (CUDA compiler)", "warn", f"found at {nvcc} but failed to run: {e}"))
    try:
        import torch
        out.append(Check("PyTorch", "ok", f"{torch.__version__} (CUDA runtime {torch.version.cuda})"))
    except Exception as e:  # pragma: no cover
        out.append(Check("PyTorch", "fail", repr(e)))
        return out
    from . import _build
    for path, what in ((_build.LIB, "kernel library (C ABI)"), (_build.native_path(), "_native module")):
        out.append(Check(what, "ok" if path.exists() else "fail",
                         str(path.relative_to(ROOT)) if path.exists() else f"{path.name} missing: run python -m custom_cuda_kernals_b200._build"))
    try:
        from . import _native
        have = [n for n in ("rmsnorm_residual_fwd", "fp8_quant_block_fwd") if hasattr(_native, n)]
        out.append(Check("_native entry points", "ok" if len(have) == 2 else "fail", ", ".join(have) or "none found"))
    except Exception as e:
        out.append(Check("_native entry points", "fail", repr(e)))
        return out
    if not torch.cuda.is_available():
        out.append(Check("GPU", "fail", "no CUDA device visible: the kernels need a B200 (sm_100a); there is no CPU fallback"))
        return out
    props = torch.cuda.get_device_properties(0)
    cc = f"sm_{props.major}{props.minor}"
    out.append(Check("GPU", "ok" if (props.major, props.minor) == (10, 0) else "fail",
                     f"{props.name}, {cc}, {props.multi_processor_count} SMs, {props.total_memory / 2 ** 30:.0f} GiB"
                     + ("" if cc == "sm_100" else " - the kernels are built for sm_100a only")))
    try:        # live probe: one tiny launch of each probed entry point, checked against plain torch
        x = torch.randn(8, 256, device="cuda")
        y, ro = torch.empty_like(x), torch.empty_like(x)
        _native.rmsnorm_residual_fwd(x, torch.zeros_like(x), torch.ones(256, device="cuda"), y, ro, 1e-6)
        want = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
        codes = torch.empty(8, 256, dtype=torch.float8_e4m3fn, device="cuda")
        scale = torch.empty(1, 2, device="cuda")
        _native.fp8_quant_block_fwd(x, codes, scale, "e4m3")
        torch.cuda.synchronize()
        good = torch.allclose(y, want, rtol=1e-4, atol=1e-4) and bool((scale > 0).all())
        status = _native.take_device_status(x)
        out.append(Check("kernel launch probe", "ok" if good and status == 0 else "fail",
                         "rmsnorm_residual_fwd and fp8_quant_block_fwd ran and match torch"
                         if good else f"results differ from torch (device status {status})"))
    except Exception as e:
        out.append(Check("kernel launch probe", "fail", repr(e)))
    return out


def cmd_doctor(_args) -> int:
    checks = run_checks()
    print(table([(c.name, c.status.upper(), c.detail) for c in checks], ("check", "status", "detail")))
    fails = sum(c.status == "fail" for c in checks)
    warns = sum(c.status == "warn" for c in checks)
    print(f"\n{fails} failed, {warns} warning(s)" if fails or warns else "\nEverything looks good.")
    return 1 if fails else 0


# ------------------------------------------------------------------------------------------- list / verify
def cmd_list(_args) -> int:
    print(table([(o.id, o.title, o.entry.rsplit(".", 1)[1], ", ".join(o.launchers) or "-") for o in OPS],
                ("id", "title", "function", "C-ABI entry points")))
    return 0


@dataclasses.dataclass
class PytestSummary:
    passed: int = 0
    failed: int = 0
    errors: int = 0
    skipped: int = 0
    duration_s: float = 0.0
    returncode: int = 0
    stdout: str = ""


def run_pytest(files, extra_args=(), timeout=1800) -> PytestSummary:
    t0 = time.monotonic()
    proc = subprocess.run([sys.executable, "-m", "pytest", "-q", *files, *extra_args], cwd=ROOT, capture_output=True,
                          text=True, timeout=timeout)
    s = PytestSummary(returncode=proc.returncode, stdout=proc.stdout, duration_s=time.monotonic() - t0)
    tail = proc.stdout.strip().splitlines()[-1] if proc.stdout.strip() else ""
    for key, attr in (("passed", "passed"), ("failed", "failed"), ("error", "errors"), ("skipped", "skipped"),
                      ("deselected", "skipped")):
        m = re.search(rf"(\d+) {key}", tail)
        if m:
            setattr(s, attr, getattr(s, attr) + int(m.group(1)))
    return s


def cmd_verify(args) -> int:
    if args.cpu:
        files, marker, title = list(CPU_TESTS), "not gpu", "CPU suite (oracle vs golden vectors, C ABI symbols, host logic)"
    elif args.op:
        op = find_op(args.op)
        files, marker, title = list(op.gpu_tests), "gpu", op.title
    else:
        files, marker, title = ["tests/"], "gpu", "every operator"
    try:
        s = run_pytest(files, ["-m", marker], timeout=args.timeout)
    except subprocess.TimeoutExpired:
        print(f"pytest did not finish within {args.timeout} s")
        return 1
    print(table([("passed", s.passed), ("failed", s.failed), ("errors", s.errors), ("skipped / deselected", s.skipped),
                 ("duration", f"{s.duration_s:.1f} s")], ("metric", "value")))
    ok = s.returncode == 0 and s.failed == 0 and s.errors == 0
    if not ok:
        for line in [ln for ln in s.stdout.splitlines() if ln.startswith(("FAILED", "ERROR"))][:25]:
            print("  " + line)
    print(f"\n{'OK' if ok else 'FAIL'} - {title}")
    return 0 if ok else 1


# ------------------------------------------------------------------------------------------- benchmark / profile
def cmd_benchmark(args) -> int:
    import csv

    import torch
    op = find_op(args.op)
    if op.bench is None:
        print(f"{op.id} has no shape sweep; run bench.py at the repository root for the block step")
        return 1
    if not torch.cuda.is_available():
        print("no CUDA device available; run `doctor` to diagnose")
        return 1
    from . import benchmarks
    out_dir = pathlib.Path(args.out)
    argv = ["--op", op.bench, "--out", str(out_dir), "--iters", str(args.iters)]
    for d in args.dtype or []:
        argv += ["--dtype", d]
    rc = benchmarks.main(argv)
    path = out_dir / f"{op.bench}_results.csv"
    if rc != 0 or not path.exists():
        return 1
    rows = list(csv.DictReader(path.open()))
    keep = [c for c in ("impl", "case_name", "dtype", "fp8_format", "granularity", "k", "median_ms", "bandwidth_gb_s",
                        "tflops", "bandwidth_pct_peak") if rows and c in rows[0]]
    print(table([tuple(r[c] for c in keep) for r in rows[:args.max_rows]], tuple(keep)))
    print(f"\n{len(rows)} rows in {path}")
    return 0


def profile_target(op_id: str, dev="cuda"):
    """Representative inputs per op (the role of custom_cuda/cli/registry.py:55-173's profile builders)."""
    import torch
    bf = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *s, scale=1.0: (scale * torch.randn(*s, device=dev, generator=g)).to(bf)
    if op_id == "rmsnorm_residual":
        from .kernels.rmsnorm_residual import rmsnorm_residual
        x, r, w = rn(4096, 4096), rn(4096, 4096), rn(4096)
        return lambda: rmsnorm_residual(x, r, w, 1e-5), "rmsnorm_residual bf16 [4096, 4096]"
    if op_id == "swiglu":
        from .kernels.swiglu import swiglu
        a, b = rn(4096, 14336), rn(4096, 14336)
        return lambda: swiglu(a, b), "swiglu bf16 [4096, 14336]"
    if op_id == "rope":
        from .kernels.rope import rope
        from .llama_block import rope_tables
        q, k = rn(4, 2048, 32, 128), rn(4, 2048, 8, 128)
        cos, sin = rope_tables(2048, 128, 500000.0, dev)
        return lambda: rope(q, k, cos, sin), "rope bf16 q[4,2048,32,128] k[4,2048,8,128]"
    if op_id == "fp8_quant":
        from .kernels.fp8_quant import fp8_quant
        x = rn(8192, 4096)
        return lambda: fp8_quant(x, "e4m3", "token"), "fp8_quant per token bf16 [8192, 4096]"
    if op_id == "matmul_add_bias":
        from .kernels.matmul_add_bias import matmul_add_bias
        a, w, b = rn(4096, 4096), rn(8192, 4096, scale=0.02), rn(8192, scale=0.02)
        return lambda: matmul_add_bias(a, w, b), "matmul_add_bias bf16 4096 x 4096 x 8192"
    if op_id == "linear_cross_entropy":
        from .kernels.linear_cross_entropy import linear_cross_entropy
        h, w = rn(2048, 4096), rn(32064, 4096, scale=0.02)
        t = torch.randint(0, 32064, (2048,), device=dev)
        return lambda: linear_cross_entropy(h, w, t), "linear_cross_entropy bf16 2048 x 4096 x 32064"
    if op_id == "moe_router":
        from .kernels.moe_router import moe_router
        lg = rn(16384, 256)
        return lambda: moe_router(lg, 8), "moe_router bf16 [16384, 256] top-8"
    if op_id == "token_permute":
        from .kernels.token_permute import compute_permutation, token_gather
        x = rn(16384, 4096)
        perm, _ = compute_permutation(torch.randint(0, 8, (16384, 2), device=dev))
        return lambda: token_gather(x, perm), "token_gather bf16 32768 rows of 4096"
    if op_id == "llama_block":
        from .llama_block import PARAM_NAMES, LlamaBlock
        shapes = {"q_proj": (4096, 4096), "k_proj": (1024, 4096), "v_proj": (1024, 4096), "o_proj": (4096, 4096),
                  "gate_proj": (14336, 4096), "up_proj": (14336, 4096), "down_proj": (4096, 14336)}
        w = {n: (rn(*shapes[n], scale=0.02) if n in shapes else torch.ones(4096, device=dev, dtype=bf)) for n in PARAM_NAMES}
        block, x = LlamaBlock(w, max_seq_len=2048), rn(2, 2048, 4096, scale=0.02)
        return lambda: block(x), "Llama-3-8B block forward, batch 2 x seq 2048"
    raise SystemExit(f"no profile target for {op_id!r}")


def cmd_profile(args) -> int:
    import torch
    from torch.profiler import ProfilerActivity, profile
    find_op(args.op)
    if not torch.cuda.is_available():
        print("no CUDA device available; run `doctor` to diagnose")
        return 1
    fn, what = profile_target(args.op)
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], record_shapes=True) as prof:
        for _ in range(args.iters):
            fn()
        torch.cuda.synchronize()
    out = pathlib.Path(args.output or f"{args.op}_{time.strftime('%Y%m%d_%H%M%S')}.json")
    out.parent.mkdir(parents=True, exist_ok=True)
    prof.export_chrome_trace(str(out))
    print(f"{what}: {args.warmup} warm-up + {args.iters} traced calls")
    print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=15))
    print(f"trace written to {out} (open in chrome://tracing or ui.perfetto.dev)")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m custom_cuda_kernals_b200.cli", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    sub.add_parser("list").set_defaults(fn=cmd_list)
    sub.add_parser("doctor").set_defaults(fn=cmd_doctor)
    v = sub.add_parser("verify")
    v.add_argument("op", nargs="?")
    v.add_argument("--cpu", action="store_true", help="the CPU suite instead of the GPU parity tests")
    v.add_argument("--timeout", type=int, default=1800)
    v.set_defaults(fn=cmd_verify)
    b = sub.add_parser("benchmark")
    b.add_argument("op")
    b.add_argument("--out", default="bench_csv")
    b.add_argument("--dtype", action="append")
    b.add_argument("--iters", type=int, default=100)
    b.add_argument("--max-rows", type=int, default=40)
    b.set_defaults(fn=cmd_benchmark)
    p = sub.add_parser("profile")
    p.add_argument("op")
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("-o", "--output")
    p.set_defaults(fn=cmd_profile)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
