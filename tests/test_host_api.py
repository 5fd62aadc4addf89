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


def test_reference_include_paths_compile(tmp_path):
    """Code written against the reference's include tree (types/..., operations/..., service/...) compiles unchanged
    against the forwarding headers."""
    if not os.path.exists(BIN):
        from kudnn_b200 import build
        build.build_all()
    src = tmp_path / "include_paths.cpp"
    src.write_text(
        '#include "types/kudnn_tensor_info.hpp"\n#include "types/kudnn_normalization.hpp"\n'
        '#include "service/kudnn_err_codes.hpp"\n#include "service/kudnn_exception.hpp"\n'
        '#include "operations/kudnn_gemm.hpp"\n#include "operations/kudnn_linear_activationlayer.hpp"\n'
        '#include "operations/kudnn_linear_res.hpp"\n#include "operations/kudnn_eltwise.hpp"\n'
        '#include "operations/kudnn_rms_normalization.hpp"\n'
        'int main() {\n'
        '    KuDNN::TensorInfo a({4, 8}, KuDNN::Element::TypeT::F32, KuDNN::Layout::AB), b({8, 6}, KuDNN::Element::TypeT::F32,\n'
        '                       KuDNN::Layout::AB), c({4, 6}, KuDNN::Element::TypeT::F32, KuDNN::Layout::AB);\n'
        '    return KuDNN::Gemm::ValidateInput(a, b, c) == KuDNN::Status::SUCCESS ? 0 : 1;\n}\n')
    pkg = os.path.join(ROOT, "kudnn_b200")
    exe = tmp_path / "include_paths"
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(pkg, "host"), str(src),
                    "-L", pkg, "-lkudnn", "-lkudnn_b200", "-Wl,-rpath," + pkg, "-o", str(exe)], check=True)
    assert subprocess.run([str(exe)]).returncode == 0
