"""The reference-shaped CSV harness: column lists and case names on CPU (no kernel runs),
one short sweep on the GPU."""

import csv

import pytest
import torch

from custom_cuda_kernals_b200 import benchmarks as B

# the reference's result dataclasses, field for field (benchmarks/*_bench.py)
WANT = {
    "rmsnorm_residual": "impl case_name dtype rows cols median_ms iqr_ms bandwidth_gb_s bandwidth_pct_peak tflops",
    "swiglu": "impl case_name dtype rows cols median_ms iqr_ms bandwidth_gb_s bandwidth_pct_peak tflops",
    "rope": "impl case_name dtype rows cols median_ms iqr_ms bandwidth_gb_s bandwidth_pct_peak tflops",
    "fp8_quant": "impl case_name dtype fp8_format granularity m n median_ms iqr_ms bandwidth_gb_s bandwidth_pct_peak",
    "matmul_add_bias": "impl case_name dtype m k n median_ms iqr_ms bandwidth_gb_s tflops",
    "linear_cross_entropy": "impl case_name dtype n_tokens hidden_dim vocab_size median_ms iqr_ms tflops",
    "moe_router": "impl case_name dtype n_tokens n_experts k median_ms iqr_ms bandwidth_gb_s tokens_per_sec",
    "token_permute_gather": "impl case_name dtype n_dst_rows hidden_dim median_ms iqr_ms bandwidth_gb_s bandwidth_pct_peak",
    "token_permute_combine": "impl case_name dtype n_tokens k hidden_dim median_ms iqr_ms bandwidth_gb_s bandwidth_pct_peak",
}


def test_columns_and_case_names_follow_the_reference_files():
    ops = B.build_ops()
    assert {op.name for op in ops.values()} == set(WANT)
    for op in ops.values():
        assert B.csv_columns(op) == WANT[op.name].split(), op.name
    names = [c.name for c in ops["rmsnorm_residual"].cases]
    assert names[:3] == ["bs4_seq128_h768", "bs2_seq2048_h4096", "bs1_seq4096_h4096"] and "batchsweep_16" in names
    assert [c.name for c in ops["swiglu"].cases][0] == "bs4_seq128_d3072"
    assert ops["rope"].cases[1].dims["rows"] == 2 * 2048 * 40 and ops["rope"].cases[1].dims["cols"] == 128
    assert ops["matmul_add_bias"].flops({"m": 2, "k": 3, "n": 5}) == 60
    assert ops["token_permute_combine"].nbytes({"n_tokens": 4, "k": 2, "hidden_dim": 8}, 2) == 3 * 4 * 8 * 2
    assert B.median_iqr([4.0, 1.0, 3.0, 2.0]) == (2.5, 2.0)


@pytest.mark.gpu
def test_short_sweep_writes_the_csv_files(tmp_path):
    rc = B.main(["--op", "moe_router", "--op", "fp8_quant", "--dtype", "bfloat16", "--iters", "3", "--warmup", "1",
                 "--flush-mb", "16", "--out", str(tmp_path), "--peak-gbs", "6500"])
    assert rc == 0
    rows = list(csv.DictReader(open(tmp_path / "moe_router_results.csv")))
    assert list(rows[0]) == WANT["moe_router"].split()
    assert len(rows) == 10 * 2 and {r["impl"] for r in rows} == {"eager", "cuda_kernel"}
    assert rows[0]["case_name"] == "mixtral_like_bfloat16" and rows[0]["dtype"] == "torch.bfloat16"
    assert all(float(r["median_ms"]) > 0 and float(r["tokens_per_sec"]) > 0 for r in rows)
    fp8 = list(csv.DictReader(open(tmp_path / "fp8_quant_results.csv")))
    assert len(fp8) == 4 * 4 * 2 and fp8[0]["case_name"] == "small_bfloat16_e4m3_tensor"
    assert all(0 < float(r["bandwidth_pct_peak"]) < 200 for r in fp8)
    assert torch.cuda.is_available()
