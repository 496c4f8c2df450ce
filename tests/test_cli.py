"""CPU: the developer command line (counterpart of custom_cuda/cli/app.py) - registry, the
environment check without a GPU, and `verify --cpu` on one test file."""

import pathlib

from custom_cuda_kernals_b200 import cli

ROOT = pathlib.Path(__file__).resolve().parent.parent


def test_registry_names_existing_files_and_declared_entry_points():
    header = (ROOT / "include" / "custom_cuda_b200.h").read_text()
    assert [o.id for o in cli.OPS][:6] == ["rmsnorm_residual", "swiglu", "rope", "fp8_quant", "matmul_add_bias",
                                           "linear_cross_entropy"]
    for op in cli.OPS:
        for f in op.gpu_tests:
            assert (ROOT / f).exists(), f
        for name in op.launchers:
            assert f"{name}(" in header, name
    for f in cli.CPU_TESTS:
        assert (ROOT / f).exists()


def test_list_and_doctor_run_without_a_gpu(capsys):
    import torch
    assert cli.main(["list"]) == 0
    assert "launch_rmsnorm_residual_fwd" in capsys.readouterr().out
    rc = cli.main(["doctor"])
    out = capsys.readouterr().out
    assert "_native entry points" in out and "rmsnorm_residual_fwd, fp8_quant_block_fwd" in out
    checks = {c.name: c for c in cli.run_checks()}
    assert checks["kernel library (C ABI)"].status == "ok" and checks["_native module"].status == "ok"
    if torch.cuda.is_available():
        assert rc == 0 and checks["kernel launch probe"].status == "ok"
    else:       # no GPU: said so, as a failure, and nothing pretends to have run
        assert rc == 1 and checks["GPU"].status == "fail" and "kernel launch probe" not in checks


def test_verify_runs_pytest_and_reports(monkeypatch, capsys):
    monkeypatch.setattr(cli, "CPU_TESTS", ("tests/test_cabi_symbols.py",))
    assert cli.main(["verify", "--cpu"]) == 0
    out = capsys.readouterr().out
    assert "passed" in out and "OK - CPU suite" in out
