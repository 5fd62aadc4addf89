"""Generates tests/golden/linear_golden.npz.

The reference library cannot run on this host (aarch64 SVE/SME + closed KML BLAS) and ships no golden vectors,
so these fixtures come from an implementation that shares no code with the oracle or the CUDA library: torch on
the CPU, contraction in float64, every rounding step through torch's own dtype casts, activations evaluated in
float64.  They pin the ORDER and the ROUNDING MODE of the post-GEMM chain (bias, rounding, activation, second
output) as read from the reference sources; they do not pin KML's summation order, which nobody outside Huawei
can know.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os

import numpy as np
import torch

F32, F16, BF16 = 1, 2, 3
ACT_NONE, ACT_RELU, ACT_GELU_TANH, ACT_SWISH, ACT_GELU_ERF = 0, 5, 20, 25, 27
RES_NONE, RES_EXT, RES_IDENTICAL, RES_ELTWISE_MUL = 0, 1, 2, 3

TORCH_DT = {F32: torch.float32, F16: torch.float16, BF16: torch.bfloat16}


def rne(t32, code):
    """float32 -> storage type -> float32, round to nearest even."""
    return t32.to(TORCH_DT[code]).to(torch.float32)


def trunc_bf16(t32):
    bits = t32.contiguous().view(torch.int32) & -65536
    return bits.view(torch.float32)


def act64(x32, act, alpha):
    x = x32.double()
    if act == ACT_RELU:
        return torch.where(x <= 0, x * alpha, x)
    if act == ACT_SWISH:
        return x / (1.0 + torch.exp(-(x * alpha)))
    if act == ACT_GELU_TANH:
        y = (1.0 + x * x * float(np.float32(0.044715))) * x * float(np.float32(0.7978845608))
        return (1.0 + torch.tanh(y)) * 0.5 * x
    if act == ACT_GELU_ERF:
        return 0.5 * x * (1.0 + torch.erf(x * float(np.float32(0.70710678118))))
    return x


def golden_linear(a, w, bias, res, code, act, act_alpha, res_op, gamma):
    """a [m,k], w [n,k], bias broadcastable to [m,n], res [m,n]; all float32 tensors holding storage-exact values."""
    acc = (a.double() @ w.double().t()).to(torch.float32)
    if code == F16:
        c1 = rne(acc, F16)
        if bias is not None:
            c1 = rne(c1 + bias, F16)
    else:
        t = acc + bias if bias is not None else acc
        c1 = rne(t, code)
    c2 = c1
    if act != ACT_NONE:
        y = act64(c1, act, act_alpha).to(torch.float32)
        c2 = y if code == F32 else (rne(y, F16) if code == F16 else trunc_bf16(y))
    out = None
    if res_op == RES_IDENTICAL:
        out = rne(c2 + res, code)
    elif res_op == RES_EXT:
        out = rne((c2.double() + res.double() * gamma).to(torch.float32), code)
    elif res_op == RES_ELTWISE_MUL:
        out = rne(c2 * res, code)
    return c2, out


def store(t32, code):
    """float32 tensor of storage-exact values -> numpy storage array."""
    if code == F32:
        return t32.numpy().copy()
    return t32.to(TORCH_DT[code]).view(torch.int16).numpy().view(np.uint16).copy()


CASES = [
    # name, m, n, k, dtype, bias, act, act_alpha, res_op, gamma, x ~, w std
    ("c1_f32_relu", 24, 40, 96, F32, "row", ACT_RELU, 0.0, RES_NONE, 1.0, "uniform", 0.02),
    ("c2_bf16_silu", 32, 48, 128, BF16, "row", ACT_SWISH, 1.0, RES_NONE, 1.0, "normal", 0.02),
    ("c3_f16_gelu_tanh_res", 32, 40, 128, F16, "row", ACT_GELU_TANH, 1.0, RES_IDENTICAL, 1.0, "normal", 0.02),
    ("c4_bf16_gate", 4, 64, 256, BF16, None, ACT_NONE, 1.0, RES_ELTWISE_MUL, 1.0, "normal", 0.02),
    ("c5_bf16_silu_bias", 40, 56, 160, BF16, "row", ACT_SWISH, 1.0, RES_NONE, 1.0, "normal", 0.02),
    ("f32_gelu_erf", 17, 23, 50, F32, "row", ACT_GELU_ERF, 1.0, RES_NONE, 1.0, "uniform", None),
    ("f16_relu_colbias", 20, 30, 20, F16, "col", ACT_RELU, 0.0, RES_NONE, 1.0, "uniform", None),
    ("bf16_res_ext", 21, 33, 20, BF16, "full", ACT_NONE, 1.0, RES_EXT, 0.5, "uniform", None),
    ("f16_res_ext", 21, 33, 20, F16, "scalar", ACT_NONE, 1.0, RES_EXT, 2.0, "uniform", None),
    ("f32_res_identical", 110, 200, 20, F32, "row", ACT_NONE, 1.0, RES_IDENTICAL, 1.0, "uniform", None),
    ("bf16_gelu_erf", 16, 24, 64, BF16, None, ACT_GELU_ERF, 1.0, RES_NONE, 1.0, "normal", 0.05),
    ("f16_silu_beta2", 16, 24, 64, F16, "row", ACT_SWISH, 2.0, RES_NONE, 1.0, "normal", 0.05),
]


def main():
    out = {}
    names = []
    for idx, (name, m, n, k, code, bias_kind, act, act_alpha, res_op, gamma, xdist, wstd) in enumerate(CASES):
        g = torch.Generator().manual_seed(1000 + idx)
        x = torch.randn(m, k, generator=g) if xdist == "normal" else torch.rand(m, k, generator=g) * 2 - 1
        w = torch.randn(n, k, generator=g) * wstd if wstd else torch.rand(n, k, generator=g) * 2 - 1
        shape = {None: None, "row": (1, n), "col": (m, 1), "scalar": (1, 1), "full": (m, n)}[bias_kind]
        bias = None
        if shape is not None:
            bias = torch.randn(*shape, generator=g) * (wstd if wstd else 1.0)
        res = torch.randn(m, n, generator=g) if res_op != RES_NONE else None
        a = rne(x, code)
        w = rne(w, code)
        bias = rne(bias, code) if bias is not None else None
        res = rne(res, code) if res is not None else None
        c, o = golden_linear(a, w, bias, res, code, act, act_alpha, res_op, gamma)
        names.append(name)
        out[name + "/meta"] = np.array([m, n, k, code, act, res_op, {None: 0, "row": 1, "col": 2, "scalar": 3,
                                                                      "full": 4}[bias_kind]], dtype=np.int64)
        out[name + "/scalars"] = np.array([act_alpha, gamma], dtype=np.float32)
        out[name + "/a"] = store(a, code)
        out[name + "/b"] = store(w, code)
        if bias is not None:
            out[name + "/bias"] = store(bias, code)
        if res is not None:
            out[name + "/res"] = store(res, code)
        out[name + "/c"] = store(c, code)
        if o is not None:
            out[name + "/out"] = store(o, code)
    out["names"] = np.array(names)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "linear_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(names), "cases")


if __name__ == "__main__":
    main()
