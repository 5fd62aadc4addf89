"""CPU checks of the oracle itself: converters against torch, the post-GEMM chain against the committed golden
vectors, the two accumulation modes against each other, and the acceptance criteria of the reference's own
test files (test/dnn/llt/gtest/src/linear_activation_gtest.cpp:120-198, linear_res_gtest.cpp:255-283) on the
shapes those files use."""
import os

import numpy as np
import pytest
import torch

import kudnn_b200 as kb
from oracle import ko
from tests import helpers

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "linear_golden.npz")


def test_converters_match_torch(oracle_lib):
    rng = np.random.default_rng(7)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-8, 6, 20000).astype(np.float32),
        np.array([0.0, -0.0, 1.0, -1.0, 65504.0, 65519.9, 65520.0, 70000.0, 6.1e-5, 5.96e-8, 2.98e-8, 2.981e-8, 1e-9,
                  np.inf, -np.inf, 3.3895314e38, 1.0039062, 1.0117188], dtype=np.float32),
    ])
    t = torch.from_numpy(x)
    bf = ko.to_storage(x, ko.BF16)
    assert np.array_equal(bf, t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16))
    hf = ko.to_storage(x, ko.F16)
    assert np.array_equal(hf, t.to(torch.float16).view(torch.int16).numpy().view(np.uint16))
    # and back
    assert np.array_equal(ko.to_f32(bf, ko.BF16), t.to(torch.bfloat16).to(torch.float32).numpy())
    back = ko.to_f32(hf, ko.F16)
    ref = t.to(torch.float16).to(torch.float32).numpy()
    assert np.array_equal(back[np.isfinite(ref)], ref[np.isfinite(ref)])


def test_all_half_patterns_round_trip(oracle_lib):
    h = np.arange(65536, dtype=np.uint16)
    f = ko.to_f32(h, ko.F16)
    finite = np.isfinite(f)
    assert np.array_equal(ko.to_storage(f[finite], ko.F16), h[finite])
    t = torch.from_numpy(h.view(np.int16)).view(torch.float16).to(torch.float32).numpy()
    assert np.array_equal(f[finite], t[finite])


def _golden_cases():
    z = np.load(GOLDEN)
    return [str(n) for n in z["names"]]


@pytest.mark.parametrize("name", _golden_cases())
def test_oracle_reproduces_golden(oracle_lib, name):
    z = np.load(GOLDEN)
    m, n, k, code, act, res_op, bias_kind = [int(v) for v in z[name + "/meta"]]
    act_alpha, gamma = [float(v) for v in z[name + "/scalars"]]
    bias_strides = {0: (0, 0), 1: (0, 1), 2: (1, 0), 3: (0, 0), 4: (n, 1)}[bias_kind]
    desc = kb.make_desc(m, n, k, code, has_bias=bias_kind != 0, bias_strides=bias_strides, act=act, act_alpha=act_alpha,
                        res_op=res_op)
    a, b = z[name + "/a"], z[name + "/b"]
    bias = z[name + "/bias"] if bias_kind else None
    res = z[name + "/res"] if res_op else None
    c = np.zeros((m, n), dtype=ko.np_dtype(code))
    out = np.zeros((m, n), dtype=ko.np_dtype(code)) if res_op else None
    ko.linear(helpers.oracle_desc(desc), a, b, c, bias, res, out, gamma=gamma, acc=ko.ACC_F64)
    for got, key in ((c, "/c"), (out, "/out")):
        if got is None:
            continue
        want = z[name + key]
        g, w = ko.to_f32(got, code), ko.to_f32(want, code)
        if code == kb.F32:
            scale = np.max(np.abs(w))
            assert np.max(np.abs(g - w)) <= 2e-6 * scale
        else:
            same = (got == want) | (g == w)
            # libm-in-fp32 versus fp64 activations may flip a rounding now and then, never by more than one unit
            assert same.mean() >= 0.995, same.mean()
            ulp = np.abs(got.astype(np.int32) - want.astype(np.int32))
            assert ulp[~same].max(initial=0) <= 1


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_accumulation_modes_agree(oracle_lib, dtype):
    case = dict(m=37, n=53, k=300, dtype=dtype, bias="row", act=kb.ACT_SWISH, seed=3)
    desc, arrays, c = helpers.build_case(case)
    c32, _ = helpers.run_oracle(desc, arrays, c, acc=ko.ACC_F32)
    c64, _ = helpers.run_oracle(desc, arrays, c, acc=ko.ACC_F64)
    info = helpers.compare(c32, c64, desc.c_dtype)
    if dtype != "f32":
        assert info["bit_exact_fraction"] > 0.98


def test_blocked_and_edge_paths_are_the_same_sum(oracle_lib):
    # the 4x4 register block and the single-element path must give identical bits (same lane order)
    case = dict(m=9, n=10, k=70, dtype="f32", seed=5)
    desc, arrays, c = helpers.build_case(case)
    full, _ = helpers.run_oracle(desc, arrays, c)
    for mi in range(9):
        sub = dict(case)
        d1, arr1, c1 = helpers.build_case(sub)
        arr1["a"] = arrays["a"][:, mi:mi + 1, :].copy()
        d1.m = 1
        row, _ = helpers.run_oracle(d1, arr1, c1)
        assert np.array_equal(row[0, 0], full[0, mi])


def _naive_reference(a, w, bias, act, alpha):
    """The test-file reference of linear_activation_gtest.cpp:24-88, in float64."""
    y = a.astype(np.float64) @ w.astype(np.float64).T
    if bias is not None:
        y = y + bias
    if act == kb.ACT_RELU:
        y = np.where(y > 0, y, alpha * y)
    elif act == kb.ACT_SWISH:
        y = y / (1.0 + np.exp(-alpha * y))
    elif act == kb.ACT_GELU_ERF:
        y = 0.5 * y * (1.0 + torch.erf(torch.from_numpy(y / np.sqrt(2.0))).numpy())
    elif act == kb.ACT_GELU_TANH:
        y = 0.5 * y * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (y + 0.044715 * y ** 3)))
    return y


@pytest.mark.parametrize("dtype,eps", [("f32", 1e-4), ("f16", 1e-3 * 20), ("bf16", 1e-2 * 20)])
@pytest.mark.parametrize("act,alpha", [(kb.ACT_RELU, 0.0), (kb.ACT_SWISH, 1.0), (kb.ACT_GELU_ERF, 1.0),
                                        (kb.ACT_GELU_TANH, 1.0)])
def test_reference_gtest_criterion_2d(oracle_lib, dtype, eps, act, alpha):
    # FWD_LINEAR_*_2D_*: 110x20 . 20x200, full [m,n] bias, |dst - ref| / max|input| <= eps
    case = dict(m=110, n=200, k=20, dtype=dtype, bias="full", act=act, act_alpha=alpha, seed=11)
    desc, arrays, c = helpers.build_case(case)
    got, _ = helpers.run_oracle(desc, arrays, c)
    code = desc.c_dtype
    a = ko.to_f32(arrays["a"], code)[0]
    w = ko.to_f32(arrays["b"], code)[0]
    bias = ko.to_f32(arrays["bias"], code)
    ref = _naive_reference(a, w, bias, act, alpha)
    max_input = max(np.abs(a).max(), np.abs(w).max())
    assert np.max(np.abs(ko.to_f32(got, code)[0] - ref)) / max_input <= eps


def test_bad_arguments_are_rejected(oracle_lib):
    desc = kb.make_desc(4, 4, 4, kb.F32, has_bias=True)
    a = np.zeros((4, 4), np.float32)
    with pytest.raises(RuntimeError):
        ko.linear(helpers.oracle_desc(desc), a, a, a.copy(), None)
