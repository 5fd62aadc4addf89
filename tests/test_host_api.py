"""Runs the C++ test program of the host classes (kudnn_b200/host/test_host_api.cpp): the reference's API-contract
cases without a device, and its numeric Linear+activation / Linear+residual / Gemm cases on the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "kudnn_b200", "kudnn_host_tests")


def _run(args):
    if not os.path.exists(BIN):
        from kudnn_b200 import build
        build.build_all()
    res = subprocess.run([BIN] + args, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=900)
    print(res.stdout)
    return res


def test_api_contract_cases_without_a_device():
    res = _run(["--no-gpu"])
    assert res.returncode == 0, res.stdout
    assert "0 failed" in res.stdout


@pytest.mark.gpu
def test_reference_numeric_cases_on_the_gpu():
    res = _run([])
    assert res.returncode == 0, res.stdout
    assert "0 failed" in res.stdout
