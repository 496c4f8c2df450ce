"""Per-op benchmark sweeps that write the reference project's CSV files.

The reference ships one script per kernel (benchmarks/<op>_bench.py) that times PyTorch eager
and its kernel over a shape sweep and writes ``<op>_results.csv``; its plot scripts read those
files.  This module produces files with the same names, columns, ``impl`` labels ("eager",
"cuda_kernel") and case names for this library, with the same method - 10 warm-up calls, 100
timed calls, an L2 flush between calls, CUDA events around the wrapper call, median and
inter-quartile range - and two parameters where the reference has constants sized for a laptop
GPU: the bandwidth peak (``--peak-gbs``, default: the measured copy bandwidth in
MEASURED_PEAKS.json next to the package if present, else 7700) and the flush buffer
(``--flush-mb``, default 512, larger than the 126 MB L2).

    python -m custom_cuda_kernals_b200.benchmarks --out bench_csv                # every op
    python -m custom_cuda_kernals_b200.benchmarks --op rope --op swiglu --dtype bfloat16

Byte and flop counts follow the reference's formulas (benchmarks/rmsnorm_residual_bench.py:
105-121, swiglu_bench.py:75-86, rope_bench.py:79-95, fp8_quant_bench.py:85-91,
matmul_add_bias_bench.py:87-94, linear_cross_entropy_bench.py:121-125, moe_router_bench.py:76-84,
token_permute_bench.py).  The linear cross entropy also gets ``linear_cross_entropy_memory.csv``
(peak incremental device memory), as in the reference.
"""

from __future__ import annotations

import argparse
import csv
import json
import pathlib
import statistics
from collections.abc import Callable
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

WARMUP_ITERS = 10
MEASURE_ITERS = 100
DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def default_peak_gbs() -> float:
    path = pathlib.Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 7700.0


@dataclass
class Case:
    name: str                      # without the dtype suffix
    dims: dict                     # the op's shape fields, in CSV column order


@dataclass
class Op:
    name: str                      # CSV stem: <name>_results.csv
    cases: list[Case]
    make: Callable                 # (dims, dtype, device, generator) -> tuple of call arguments
    eager: Callable                # (*args) -> result, plain PyTorch on the GPU
    kernel: Callable               # (*args) -> result, this library
    nbytes: Callable               # (dims, element size) -> bytes moved, ideal
    flops: Callable | None = None
    columns: list[str] = field(default_factory=list)     # shape columns, in order
    extra: Callable | None = None  # (dims, seconds) -> dict of further columns
    with_bandwidth: bool = True
    with_pct: bool = True
    with_tflops: bool = True
    extra_keys: dict = field(default_factory=dict)       # fixed columns (e.g. fp8_format)


def time_call(fn: Callable[[], object], flush: torch.Tensor, warmup: int, iters: int) -> list[float]:
    """The reference's loop (benchmarks/rmsnorm_residual_bench.py:124-140)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(iters):
        flush.fill_(1.0)
        torch.cuda.synchronize()
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
    return times


def median_iqr(times_ms: list[float]) -> tuple[float, float]:
    s = sorted(times_ms)
    return statistics.median(s), s[int(0.75 * len(s))] - s[int(0.25 * len(s))]


# ---------------------------------------------------------------------------- the ops
def _randn(shape, dtype, dev, g, scale=1.0):
    x = torch.randn(shape, dtype=torch.float32, device=dev, generator=g)
    return (x * scale).to(dtype) if scale != 1.0 else x.to(dtype)


def _eager_rmsnorm(x, r, w, eps):
    ro = x + r
    ro32 = ro.float()
    return (ro32 * torch.rsqrt(ro32.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w, ro


def _eager_rope(q, k, cos, sin):
    def rot(t):
        half = t.shape[-1] // 2
        a, b = t[..., :half].float(), t[..., half:].float()
        c, s = cos[None, :, None, :], sin[None, :, None, :]
        return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(t.dtype)
    return rot(q), rot(k)


def _eager_fp8(x, fmt, gran):
    dt = torch.float8_e4m3fn if fmt == "e4m3" else torch.float8_e5m2
    x32 = x.float()
    if gran == "tensor":
        scale = (x32.abs().amax() / torch.finfo(dt).max).clamp(min=1e-12)
        return (x32 / scale).to(dt), scale.reshape(1)
    m, n = x.shape
    tiles = x32.reshape(m // 128, 128, n // 128, 128)
    scale = (tiles.abs().amax(dim=(1, 3)) / torch.finfo(dt).max).clamp(min=1e-12)
    return (tiles / scale[:, None, :, None]).reshape(m, n).to(dt), scale


def _eager_router(logits, k):
    w, i = torch.topk(torch.softmax(logits.float(), dim=-1), k, dim=-1)
    return w / w.sum(-1, keepdim=True), i


def _eager_combine(rows, index, weights):
    return (rows[index].float() * weights.unsqueeze(-1)).sum(1).to(rows.dtype)


def build_ops() -> dict[str, Op]:
    from .kernels.fp8_quant import fp8_quant
    from .kernels.linear_cross_entropy import linear_cross_entropy
    from .kernels.matmul_add_bias import matmul_add_bias
    from .kernels.moe_router import moe_router
    from .kernels.rmsnorm_residual import rmsnorm_residual
    from .kernels.rope import rope
    from .kernels.swiglu import swiglu
    from .kernels.token_permute import token_combine, token_gather
    from .llama_block import rope_tables

    ops: dict[str, Op] = {}
    act = [("bs4_seq128", 4, 128, 0), ("bs2_seq2048", 2, 2048, 1), ("bs1_seq4096", 1, 4096, 1),
           ("seqsweep_128", 1, 128, 1), ("seqsweep_512", 1, 512, 1), ("seqsweep_2048", 1, 2048, 1),
           ("seqsweep_8192", 1, 8192, 1), ("batchsweep_1", 1, 1024, 1), ("batchsweep_4", 4, 1024, 1),
           ("batchsweep_16", 16, 1024, 1)]

    def act_cases(small, large, tag):
        out = []
        for name, b, s, big in act:
            width = large if big else small
            label = f"{name}_{tag}{width}" if name.startswith("bs") else name
            out.append(Case(label, {"rows": b * s, "cols": width}))
        return out

    ops["rmsnorm_residual"] = Op(
        "rmsnorm_residual", act_cases(768, 4096, "h"),
        make=lambda d, dt, dev, g: (_randn((d["rows"], d["cols"]), dt, dev, g), _randn((d["rows"], d["cols"]), dt, dev, g),
                                    _randn((d["cols"],), dt, dev, g), 1e-6),
        eager=_eager_rmsnorm, kernel=rmsnorm_residual,
        nbytes=lambda d, e: d["rows"] * d["cols"] * e * 4, flops=lambda d: d["rows"] * d["cols"] * 5,
        columns=["rows", "cols"])
    ops["swiglu"] = Op(
        "swiglu", act_cases(3072, 11008, "d"),
        make=lambda d, dt, dev, g: (_randn((d["rows"], d["cols"]), dt, dev, g), _randn((d["rows"], d["cols"]), dt, dev, g)),
        eager=lambda a, b: F.silu(a.float()).to(a.dtype) * b, kernel=swiglu,
        nbytes=lambda d, e: d["rows"] * d["cols"] * e * 3, flops=lambda d: d["rows"] * d["cols"] * 5,
        columns=["rows", "cols"])

    rope_shapes = [("bs4_seq128_mha", 4, 128, 12, 12, 64), ("bs2_seq2048_gqa", 2, 2048, 32, 8, 128),
                   ("bs1_seq4096_gqa", 1, 4096, 32, 8, 128)] + [
        (n, b, s, 32, 8, 128) for n, b, s, _ in act[3:]]

    def rope_make(d, dt, dev, g):
        cos, sin = rope_tables(d["seq"], d["cols"], 10000.0, dev)
        return (_randn((d["batch"], d["seq"], d["hq"], d["cols"]), dt, dev, g),
                _randn((d["batch"], d["seq"], d["hkv"], d["cols"]), dt, dev, g), cos, sin)

    ops["rope"] = Op(
        "rope", [Case(n, {"rows": b * s * (hq + hkv), "cols": hd, "batch": b, "seq": s, "hq": hq, "hkv": hkv})
                 for n, b, s, hq, hkv, hd in rope_shapes],
        make=rope_make, eager=_eager_rope, kernel=rope,
        nbytes=lambda d, e: d["rows"] * d["cols"] * e * 2, flops=lambda d: d["rows"] * d["cols"] * 3,
        columns=["rows", "cols"])

    for fmt in ("e4m3", "e5m2"):
        for gran in ("tensor", "block"):
            ops[f"fp8_quant/{fmt}_{gran}"] = Op(
                "fp8_quant", [Case(n, {"m": m, "n": m}) for n, m in (("small", 256), ("medium", 1024), ("large", 4096),
                                                                      ("xlarge", 8192))],
                make=lambda d, dt, dev, g: (_randn((d["m"], d["n"]), dt, dev, g),),
                eager=lambda x, fmt=fmt, gran=gran: _eager_fp8(x, fmt, gran),
                kernel=lambda x, fmt=fmt, gran=gran: fp8_quant(x, fmt, gran),
                nbytes=lambda d, e: d["m"] * d["n"] * (e + 1), columns=["m", "n"], with_tflops=False,
                extra_keys={"fp8_format": fmt, "granularity": gran})

    gemm_shapes = [("qkv_proj", 2048, 4096, 4096), ("mlp_up", 2048, 4096, 11008), ("mlp_down", 2048, 11008, 4096),
                   ("msweep_128", 128, 4096, 4096), ("msweep_512", 512, 4096, 4096), ("msweep_2048", 2048, 4096, 4096),
                   ("msweep_8192", 8192, 4096, 4096)]
    ops["matmul_add_bias"] = Op(
        "matmul_add_bias", [Case(n, {"m": m, "k": k, "n": nn}) for n, m, k, nn in gemm_shapes],
        make=lambda d, dt, dev, g: (_randn((d["m"], d["k"]), dt, dev, g), _randn((d["n"], d["k"]), dt, dev, g, 0.02),
                                    _randn((d["n"],), dt, dev, g, 0.02)),
        eager=lambda x, w, b: x @ w.T + b, kernel=matmul_add_bias,
        nbytes=lambda d, e: (d["m"] * d["k"] + d["n"] * d["k"] + d["m"] * d["n"]) * e,
        flops=lambda d: 2 * d["m"] * d["k"] * d["n"], columns=["m", "k", "n"], with_pct=False)

    lce_shapes = [("small_vocab", 512, 1024, 8000), ("llama2_vocab", 512, 4096, 32000), ("llama3_vocab", 512, 4096, 128256)]
    ops["linear_cross_entropy"] = Op(
        "linear_cross_entropy",
        [Case(n, {"n_tokens": t, "hidden_dim": h, "vocab_size": v}) for n, t, h, v in lce_shapes],
        make=lambda d, dt, dev, g: (_randn((d["n_tokens"], d["hidden_dim"]), dt, dev, g),
                                    _randn((d["vocab_size"], d["hidden_dim"]), dt, dev, g, 0.02),
                                    torch.randint(0, d["vocab_size"], (d["n_tokens"],), device=dev, generator=g)),
        eager=lambda h, w, t: F.cross_entropy(h @ w.T, t), kernel=linear_cross_entropy,
        nbytes=lambda d, e: 0, flops=lambda d: 2 * d["n_tokens"] * d["vocab_size"] * d["hidden_dim"],
        columns=["n_tokens", "hidden_dim", "vocab_size"], with_bandwidth=False, with_pct=False)

    router_shapes = [("mixtral_like", 4096, 8, 2), ("deepseek_like", 4096, 160, 6)] + [
        (f"ksweep_k{k}", 4096, 32, k) for k in (1, 2, 4, 8)] + [(f"tsweep_{t}", t, 8, 2) for t in (512, 2048, 8192, 32768)]
    ops["moe_router"] = Op(
        "moe_router", [Case(n, {"n_tokens": t, "n_experts": e, "k": k}) for n, t, e, k in router_shapes],
        make=lambda d, dt, dev, g: (_randn((d["n_tokens"], d["n_experts"]), dt, dev, g), d["k"]),
        eager=_eager_router, kernel=moe_router,
        nbytes=lambda d, e: d["n_tokens"] * (d["n_experts"] * e + d["k"] * 12),
        columns=["n_tokens", "n_experts", "k"], with_pct=False, with_tflops=False,
        extra=lambda d, secs: {"tokens_per_sec": d["n_tokens"] / secs})

    gather_shapes = [("mixtral_like", 2048, 4096, 4096), ("large_hidden", 2048, 4096, 11008)] + [
        (f"nsweep_{n}", n, n, 4096) for n in (1024, 4096, 16384, 65536)]
    ops["token_permute_gather"] = Op(
        "token_permute_gather", [Case(n, {"n_dst_rows": dst, "hidden_dim": h, "n_src": src}) for n, src, dst, h in gather_shapes],
        make=lambda d, dt, dev, g: (_randn((d["n_src"], d["hidden_dim"]), dt, dev, g),
                                    torch.randint(0, d["n_src"], (d["n_dst_rows"],), device=dev, generator=g)),
        eager=lambda s, i: s.index_select(0, i), kernel=token_gather,
        nbytes=lambda d, e: 2 * d["n_dst_rows"] * d["hidden_dim"] * e, columns=["n_dst_rows", "hidden_dim"],
        with_tflops=False)
    combine_shapes = [("mixtral_like", 2048, 2), ("deepseek_like", 2048, 6)] + [(f"tsweep_{t}", t, 2) for t in (512, 2048, 8192, 32768)]
    ops["token_permute_combine"] = Op(
        "token_permute_combine", [Case(n, {"n_tokens": t, "k": k, "hidden_dim": 4096}) for n, t, k in combine_shapes],
        make=lambda d, dt, dev, g: (_randn((d["n_tokens"] * d["k"], d["hidden_dim"]), dt, dev, g),
                                    torch.randperm(d["n_tokens"] * d["k"], device=dev, generator=g).reshape(d["n_tokens"], d["k"]),
                                    torch.rand(d["n_tokens"], d["k"], device=dev, generator=g)),
        eager=_eager_combine, kernel=token_combine,
        nbytes=lambda d, e: (d["k"] + 1) * d["n_tokens"] * d["hidden_dim"] * e, columns=["n_tokens", "k", "hidden_dim"],
        with_tflops=False)
    return ops


# ---------------------------------------------------------------------------- running and writing
def csv_columns(op: Op) -> list[str]:
    cols = ["impl", "case_name", "dtype", *op.extra_keys, *op.columns, "median_ms", "iqr_ms"]
    if op.with_bandwidth:
        cols.append("bandwidth_gb_s")
        if op.with_pct:
            cols.append("bandwidth_pct_peak")
    if op.extra is not None:
        cols.append("tokens_per_sec")
    if op.with_tflops and op.flops is not None:
        cols.append("tflops")
    return cols


def run_op(op: Op, dtypes: list[str], peak_gbs: float, flush: torch.Tensor, warmup: int, iters: int,
           impls: tuple[str, ...] = ("eager", "cuda_kernel"), device: str = "cuda", log=print) -> list[dict]:
    rows = []
    suffix = "".join(f"_{v}" for v in op.extra_keys.values())
    for case in op.cases:
        for dname in dtypes:
            dtype = DTYPES[dname]
            g = torch.Generator(device=device).manual_seed(0)
            args = op.make(case.dims, dtype, device, g)
            for impl in impls:
                fn = op.eager if impl == "eager" else op.kernel
                with torch.no_grad():
                    median, iqr = median_iqr(time_call(lambda: fn(*args), flush, warmup, iters))
                secs = median * 1e-3
                row = {"impl": impl, "case_name": f"{case.name}_{dname}{suffix}", "dtype": str(dtype), **op.extra_keys,
                       **{c: case.dims[c] for c in op.columns}, "median_ms": median, "iqr_ms": iqr}
                if op.with_bandwidth:
                    bw = op.nbytes(case.dims, torch.empty(0, dtype=dtype).element_size()) / secs / 1e9
                    row["bandwidth_gb_s"] = bw
                    if op.with_pct:
                        row["bandwidth_pct_peak"] = 100.0 * bw / peak_gbs
                if op.extra is not None:
                    row.update(op.extra(case.dims, secs))
                if op.with_tflops and op.flops is not None:
                    row["tflops"] = op.flops(case.dims) / secs / 1e12
                rows.append(row)
                log(f"{op.name:24s} {impl:12s} {row['case_name']:34s} median={median:9.4f}ms iqr={iqr:8.4f}ms")
            del args
    return rows


def lce_memory_rows(op: Op, device: str = "cuda", log=print) -> list[dict]:
    """Peak incremental device memory of one call, eager against the fused kernel, on the
    reference's float16 training-batch shapes (benchmarks/linear_cross_entropy_bench.py:67-72,
    159-172)."""
    rows = []
    for name, t, h, v in (("mem_llama2_2k_tokens", 2048, 4096, 32000), ("mem_llama3_2k_tokens", 2048, 4096, 128256),
                          ("mem_llama3_4k_tokens", 4096, 4096, 128256), ("mem_llama3_8k_tokens", 8192, 4096, 128256)):
        g = torch.Generator(device=device).manual_seed(0)
        args = op.make({"n_tokens": t, "hidden_dim": h, "vocab_size": v}, torch.float16, device, g)
        for impl, fn in (("eager", op.eager), ("cuda_kernel", op.kernel)):
            with torch.no_grad():
                fn(*args)
                torch.cuda.synchronize()
                torch.cuda.reset_peak_memory_stats(device)
                before = torch.cuda.memory_allocated(device)
                fn(*args)
                torch.cuda.synchronize()
                peak_mb = (torch.cuda.max_memory_allocated(device) - before) / (1 << 20)
            rows.append({"impl": impl, "case_name": name, "dtype": "torch.float16", "n_tokens": t, "hidden_dim": h,
                         "vocab_size": v, "peak_incremental_mb": peak_mb})
            log(f"linear_cross_entropy memory {impl:12s} {name:24s} peak_incremental={peak_mb:9.1f} MB")
        del args
    return rows


def write_csv(path: pathlib.Path, columns: list[str], rows: list[dict]) -> None:
    with open(path, "w", newline="") as f:
        writer = csv.DictWriter(f, fieldnames=columns)
        writer.writeheader()
        writer.writerows(rows)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", action="append", help="CSV stem to run (repeatable); default: all")
    ap.add_argument("--dtype", action="append", choices=list(DTYPES), help="default: all three")
    ap.add_argument("--out", default="bench_csv")
    ap.add_argument("--peak-gbs", type=float, default=None)
    ap.add_argument("--flush-mb", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=WARMUP_ITERS)
    ap.add_argument("--iters", type=int, default=MEASURE_ITERS)
    ap.add_argument("--kernel-only", action="store_true", help="skip the PyTorch eager rows")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("a CUDA device is required")
    ops = build_ops()
    stems = sorted({op.name for op in ops.values()})
    for want in a.op or []:
        if want not in stems:
            raise SystemExit(f"unknown op {want!r}; choose from {stems}")
    peak = a.peak_gbs if a.peak_gbs is not None else default_peak_gbs()
    out = pathlib.Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    flush = torch.empty(a.flush_mb << 18, dtype=torch.float32, device="cuda")
    impls = ("cuda_kernel",) if a.kernel_only else ("eager", "cuda_kernel")
    for stem in (a.op or stems):
        rows, columns = [], None
        for op in ops.values():
            if op.name == stem:
                columns = csv_columns(op)
                rows += run_op(op, a.dtype or list(DTYPES), peak, flush, a.warmup, a.iters, impls)
        write_csv(out / f"{stem}_results.csv", columns, rows)
        print(f"wrote {len(rows)} rows to {out / (stem + '_results.csv')}")
        if stem == "linear_cross_entropy":
            mem = lce_memory_rows(ops["linear_cross_entropy"])
            write_csv(out / "linear_cross_entropy_memory.csv", list(mem[0]), mem)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
