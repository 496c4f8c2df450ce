"""GPU: `doctor` with its live launch probe, and a `profile` trace of one op."""

import json

import pytest

from custom_cuda_kernals_b200 import cli

pytestmark = pytest.mark.gpu


def test_doctor_passes_on_a_b200_and_probes_the_two_entry_points(capsys):
    assert cli.main(["doctor"]) == 0
    out = capsys.readouterr().out
    assert "kernel launch probe" in out and "match torch" in out and "Everything looks good" in out


def test_profile_writes_a_chrome_trace_that_names_our_kernel(tmp_path, capsys):
    trace = tmp_path / "swiglu.json"
    assert cli.main(["profile", "swiglu", "--warmup", "2", "--iters", "3", "-o", str(trace)]) == 0
    assert "swiglu_kernel" in capsys.readouterr().out
    events = json.loads(trace.read_text())["traceEvents"]
    assert any("swiglu_kernel" in str(e.get("name", "")) for e in events)
