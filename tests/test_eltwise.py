"""The operators either side of Linear: the stand-alone activation pass and RMS normalisation over the last axis,
CUDA kernels against the CPU oracle (oracle/kudnn_linear_oracle.c: ko_activation_run, ko_rmsnorm)."""
import numpy as np
import pytest
import torch

import kudnn_b200 as kb
from oracle import ko
from tests import helpers

DT = {"f32": kb.F32, "f16": kb.F16, "bf16": kb.BF16}
ACTS = [(kb.ACT_RELU, 0.0), (kb.ACT_RELU, 0.1), (kb.ACT_SWISH, 1.0), (kb.ACT_GELU_TANH, 0.0), (kb.ACT_GELU_ERF, 0.0),
        (kb.ACT_SIGMOID, 0.0), (kb.ACT_TANH, 0.0)]


def test_oracle_rmsnorm_against_numpy_float64():
    rng = np.random.default_rng(3)
    rows, axis = 7, 200
    x = ko.to_storage(rng.standard_normal((rows, axis), dtype=np.float32) * 3, ko.F16)
    g = ko.to_storage(rng.standard_normal((axis,), dtype=np.float32), ko.F16)
    y = np.zeros_like(x)
    var = np.zeros(rows, dtype=np.float32)
    ko.rmsnorm(x, y, g, var, rows, axis, ko.F16, 2, True, 1e-5)
    xf, gf = ko.to_f32(x, ko.F16).astype(np.float64), ko.to_f32(g, ko.F16).astype(np.float64)
    v64 = (xf * xf).mean(axis=1)
    want = xf * gf / np.sqrt(v64 + 1e-5)[:, None]
    assert np.allclose(var, v64, rtol=1e-6)
    assert np.max(np.abs(ko.to_f32(y, ko.F16) - want) / (np.abs(want) + 1)) < 1e-3


def test_oracle_activation_types():
    x = ko.to_storage(np.linspace(-6, 6, 97, dtype=np.float32), ko.BF16)
    same = np.zeros_like(x)
    ko.activation(x, same, ko.BF16, ko.BF16, ko.ACT_SWISH, 1.0)
    wide = np.zeros(x.shape, dtype=np.float32)
    ko.activation(x, wide, ko.BF16, ko.F32, ko.ACT_SWISH, 1.0)
    # the typed kernel truncates the bf16 result: it never exceeds the fp32 result in magnitude, and is within one unit
    assert np.all(np.abs(ko.to_f32(same, ko.BF16)) <= np.abs(wide) + 1e-30)
    assert np.max(np.abs(ko.to_f32(same, ko.BF16) - wide) / (np.abs(wide) + 1e-3)) < 1.0 / 128


@pytest.mark.gpu
@pytest.mark.parametrize("src,dst", [("f32", "f32"), ("f16", "f16"), ("bf16", "bf16"), ("bf16", "f32"), ("f32", "f16")])
@pytest.mark.parametrize("act,alpha", ACTS)
@pytest.mark.parametrize("count", [5, 4096, 1000003])
def test_activation_matches_the_oracle(cuda_device, src, dst, act, alpha, count):
    rng = np.random.default_rng(11)
    x = ko.to_storage(rng.standard_normal(count, dtype=np.float32) * 3, DT[src])
    want = np.zeros(count, dtype=ko.np_dtype(DT[dst]))
    ko.activation(x, want, DT[src], DT[dst], act, alpha)
    d_x = helpers._to_torch(x, cuda_device)
    d_y = helpers._to_torch(np.zeros(count, dtype=ko.np_dtype(DT[dst])), cuda_device)
    kb.activation(d_x, d_y, count, DT[src], DT[dst], act, alpha, stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    info = helpers.compare(helpers._from_torch(d_y), want, DT[dst])
    if DT[dst] != kb.F32:
        # gelu_erf = 0.5 x erf(x / sqrt 2) + 0.5 x cancels for x << 0, which amplifies the 1-2 ulp by which the two erf
        # implementations (libm, CUDA) differ; the results there are tiny and well inside the tolerance
        assert info["bit_exact_fraction"] > (0.97 if act == kb.ACT_GELU_ERF else 0.99), info
    if act == kb.ACT_RELU:
        assert np.array_equal(helpers._from_torch(d_y), want)
    # host pointers, as the reference's callers pass them
    if count <= 4096:
        h_y = np.zeros(count, dtype=ko.np_dtype(DT[dst]))
        kb.activation(x, h_y, count, DT[src], DT[dst], act, alpha)
        assert np.array_equal(h_y, helpers._from_torch(d_y))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("rows,axis", [(3, 7), (64, 4096), (33, 8192), (5, 20000), (2, 16384), (4, 1000)])
@pytest.mark.parametrize("flags,save", [(0, False), (kb.NORM_USE_SCALE, True), (kb.NORM_USE_SCALE | kb.NORM_USE_GLOBAL_STATS, False)])
def test_rmsnorm_matches_the_oracle(cuda_device, dtype, rows, axis, flags, save):
    rng = np.random.default_rng(12)
    code = DT[dtype]
    x = ko.to_storage(rng.standard_normal((rows, axis), dtype=np.float32) * 2, code)
    g = ko.to_storage(1.0 + 0.1 * rng.standard_normal(axis, dtype=np.float32), code)
    var_in = (0.5 + rng.random(rows)).astype(np.float32)
    want = np.zeros_like(x)
    var_ref = var_in.copy()
    ko.rmsnorm(x, want, g, var_ref, rows, axis, code, flags, save, 1e-5)
    d_x, d_g = helpers._to_torch(x, cuda_device), helpers._to_torch(g, cuda_device)
    d_y = helpers._to_torch(np.zeros_like(x), cuda_device)
    d_var = torch.from_numpy(var_in.copy()).to(cuda_device)
    kb.rmsnorm(d_x, d_y, rows, axis, code, scale=d_g if flags & kb.NORM_USE_SCALE else None, variance=d_var, flags=flags,
               save_stats=save, eps=1e-5, stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    info = helpers.compare(helpers._from_torch(d_y), want, code)
    if code != kb.F32:
        assert info["bit_exact_fraction"] > 0.99
    if save:
        assert np.allclose(d_var.cpu().numpy(), var_ref, rtol=1e-5)
    else:
        assert np.array_equal(d_var.cpu().numpy(), var_in)
    if rows * axis <= 300000:
        h_y = np.zeros_like(x)
        h_var = var_in.copy()
        kb.rmsnorm(x, h_y, rows, axis, code, scale=g if flags & kb.NORM_USE_SCALE else None, variance=h_var, flags=flags,
                   save_stats=save, eps=1e-5)
        assert np.array_equal(h_y, helpers._from_torch(d_y))


@pytest.mark.gpu
def test_eltwise_argument_checks(cuda_device):
    x = torch.zeros(64, dtype=torch.float16, device=cuda_device)
    with pytest.raises(kb.KudnnError) as e:
        kb.activation(x, x, 64, kb.F16, kb.F16, 1)  # ABS: one of the functions that are not implemented
    assert e.value.status == 1
    with pytest.raises(kb.KudnnError) as e:
        kb.rmsnorm(x, x, 4, 16, kb.F16, flags=kb.NORM_USE_SCALE)  # scale flag without a scale tensor
    assert e.value.status == 2
    with pytest.raises(kb.KudnnError) as e:
        kb.rmsnorm(x, x, 4, 16, kb.F16, flags=8)
    assert e.value.status == 1
