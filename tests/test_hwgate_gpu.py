"""The start-up correctness gate (GEMM layouts, fp8 quantizer and scaled products, attention, two training steps
against the PyTorch operators) passes on the device, and its report names every check."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_hardware_gate_passes_and_reports_every_check():
    from nanochat_cpp_b200.hwgate import run_hardware_gate
    ok, report = run_hardware_gate("cuda:0")
    failed = [r for r in report if not r["ok"]]
    assert ok and not failed, failed
    names = {r["name"] for r in report}
    assert {"gemm.forward", "gemm.dgrad", "gemm.wgrad", "fp8.quantize.codes", "fp8.quantize.scales",
            "attention.forward", "attention.backward.dq", "train.two_steps"} <= names
    assert sum(n.startswith("fp8.scaled_gemm.") for n in names) == 3
