"""Shared machinery of the parity tests: seeded inputs, one call into the CPU oracle, one call into the CUDA
library through its C ABI, and the comparison rules.

A "case" is a plain dict:
    m, n, k            extents
    dtype              "f32" | "f16" | "bf16"  (a, b; also c, res, out unless c_dtype is given; bias unless bias_dtype)
    c_dtype            element type of c, res and out when it differs from the inputs' (f16 / bf16 inputs -> f32)
    bias               None | "row" ([1,n]) | "col" ([m,1]) | "scalar" ([1,1]) | "full" ([m,n])
    act, act_alpha     activation code (kudnn_b200.ACT_*) and its parameter
    res_op             kudnn_b200.RES_* ; gamma
    a_layout           "AB" (k contiguous) | "BA" (m contiguous)
    b_layout           "BA" (W[n,k], k contiguous) | "AB" ([k,n], n contiguous)
    x_dist / w_std     input distributions: x ~ U(-1,1) ("uniform") or N(0,1) ("normal"); W ~ N(0, w_std)
    alpha, beta        GEMM scalars
    batch              tuple of up to three leading extents, with a_bcast / b_bcast flags
    seed
"""
import ctypes

import numpy as np

import kudnn_b200 as kb
from oracle import ko

DT = {"f32": kb.F32, "f16": kb.F16, "bf16": kb.BF16}


def case_defaults(case):
    c = dict(dtype="bf16", bias=None, act=kb.ACT_NONE, act_alpha=1.0, res_op=kb.RES_NONE, gamma=1.0, a_layout="AB",
             b_layout="BA", x_dist="uniform", w_std=None, alpha=1.0, beta=0.0, batch=(), a_bcast=False, b_bcast=True,
             seed=0, bias_dtype=None, c_dtype=None, want_c=True)
    c.update(case)
    return c


def _storage(rng_values, code):
    return ko.to_storage(rng_values.astype(np.float32), code)


def build_case(case):
    """Returns (desc, arrays) where arrays holds numpy storage arrays a, b, bias, res, c0 (initial c)."""
    c = case_defaults(case)
    m, n, k = c["m"], c["n"], c["k"]
    code = DT[c["dtype"]]
    rng = np.random.default_rng(c["seed"])
    batch = tuple(c["batch"])
    nb = int(np.prod(batch)) if batch else 1
    a_batch = 1 if (c["a_bcast"] or not batch) else nb
    b_batch = 1 if (c["b_bcast"] or not batch) else nb

    def draw_x(shape):
        if c["x_dist"] == "normal":
            return rng.standard_normal(shape, dtype=np.float32)
        return rng.uniform(-1.0, 1.0, shape).astype(np.float32)

    # draw order x -> W -> bias -> residual / gate
    x = draw_x((a_batch, m, k))
    w_std = c["w_std"]
    if w_std is None:
        w = rng.uniform(-1.0, 1.0, (b_batch, n, k)).astype(np.float32)
    else:
        w = (rng.standard_normal((b_batch, n, k), dtype=np.float32) * np.float32(w_std)).astype(np.float32)
    bias_shape = {None: None, "row": (1, n), "col": (m, 1), "scalar": (1, 1), "full": (m, n)}[c["bias"]]
    bias = None
    if bias_shape is not None:
        std = np.float32(w_std if w_std is not None else 1.0)
        bias = rng.standard_normal(bias_shape, dtype=np.float32) * std if w_std is not None else \
            rng.uniform(-1.0, 1.0, bias_shape).astype(np.float32)
    res = None
    if c["res_op"] != kb.RES_NONE:
        res = draw_x((nb, m, n))
    c0 = None
    if c["beta"] != 0.0:
        c0 = draw_x((nb, m, n))

    bias_code = DT[c["bias_dtype"]] if c["bias_dtype"] else code
    c_code = DT[c["c_dtype"]] if c["c_dtype"] else code
    arrays = {}
    # a: [batch, m, k] logical; memory layout AB (k fastest) or BA (m fastest)
    if c["a_layout"] == "AB":
        arrays["a"] = _storage(x, code)
        a_sm, a_sk, a_mat = k, 1, m * k
    else:
        arrays["a"] = _storage(np.ascontiguousarray(x.transpose(0, 2, 1)), code)
        a_sm, a_sk, a_mat = 1, m, m * k
    if c["b_layout"] == "BA":
        arrays["b"] = _storage(w, code)  # [batch, n, k]
        b_sk, b_sn, b_mat = 1, k, n * k
    else:
        arrays["b"] = _storage(np.ascontiguousarray(w.transpose(0, 2, 1)), code)  # [batch, k, n]
        b_sk, b_sn, b_mat = n, 1, n * k
    if bias is not None:
        arrays["bias"] = _storage(bias, bias_code)
        bias_sm = bias_shape[1] if bias_shape[0] > 1 else 0
        bias_sn = 1 if bias_shape[1] > 1 else 0
    else:
        bias_sm = bias_sn = 0
    if res is not None:
        arrays["res"] = _storage(res, c_code)
    if c0 is not None:
        arrays["c0"] = _storage(c0, c_code)

    def bstrides(per_matrix, broadcast):
        # contiguous batch strides for up to three leading dims, aligned to the right of batch[3]
        sb = [0, 0, 0]
        if not batch or broadcast:
            return tuple(sb)
        ext = [1] * (3 - len(batch)) + list(batch)
        stride = per_matrix
        for i in (2, 1, 0):
            sb[i] = stride if ext[i] > 1 else 0
            stride *= ext[i]
        return tuple(sb)

    ext3 = tuple([0] * (3 - len(batch)) + list(batch)) if batch else (0, 0, 0)
    desc = kb.make_desc(
        m, n, k, code, a_strides=(a_sm, a_sk), b_strides=(b_sk, b_sn), has_bias=bias is not None,
        bias_strides=(bias_sm, bias_sn), bias_dtype=bias_code, c_dtype=c_code, act=c["act"], act_alpha=c["act_alpha"],
        res_op=c["res_op"], batch=ext3, a_sb=bstrides(a_mat, c["a_bcast"]), b_sb=bstrides(b_mat, c["b_bcast"]),
        c_sb=bstrides(m * n, False), bias_sb=(0, 0, 0), res_sb=bstrides(m * n, False), out_sb=bstrides(m * n, False))
    return desc, arrays, c


def oracle_desc(desc):
    """The oracle's descriptor has the same field layout as the library's."""
    return ko.Desc.from_buffer_copy(bytes(desc))


def run_oracle(desc, arrays, c, acc=ko.ACC_F32):
    m, n = desc.m, desc.n
    nb = int(np.prod(c["batch"])) if c["batch"] else 1
    code = desc.c_dtype
    out_c = arrays["c0"].copy() if "c0" in arrays else np.zeros((nb, m, n), dtype=ko.np_dtype(code))
    out_o = np.zeros((nb, m, n), dtype=ko.np_dtype(desc.out_dtype)) if c["res_op"] != kb.RES_NONE else None
    ko.linear(oracle_desc(desc), arrays["a"], arrays["b"], out_c, arrays.get("bias"), arrays.get("res"), out_o,
              alpha=c["alpha"], beta=c["beta"], gamma=c["gamma"], acc=acc)
    return out_c, out_o


def _to_torch(arr, device):
    import torch
    if arr.dtype == np.uint16:
        return torch.from_numpy(arr.view(np.int16)).to(device)
    return torch.from_numpy(arr).to(device)


def _from_torch(t):
    arr = t.cpu().numpy()
    if arr.dtype == np.int16:
        return arr.view(np.uint16)
    return arr


def run_gpu(desc, arrays, c, device, kernel=kb.KERNEL_AUTO, prepack=False, host=False):
    """One call through the C ABI.  Returns (c, out, kernel_used)."""
    import torch
    m, n = desc.m, desc.n
    nb = int(np.prod(c["batch"])) if c["batch"] else 1
    lin = kb.Linear(desc)
    if kernel != kb.KERNEL_AUTO:
        lin.force_kernel(kernel)
    has_res = c["res_op"] != kb.RES_NONE
    if host:
        out_c = arrays["c0"].copy() if "c0" in arrays else np.zeros((nb, m, n), dtype=ko.np_dtype(desc.c_dtype))
        out_o = np.zeros((nb, m, n), dtype=ko.np_dtype(desc.out_dtype)) if has_res else None
        if prepack:
            lin.prepack(arrays["b"])
        lin.run_host(arrays["a"], arrays["b"], out_c if c["want_c"] else None, arrays.get("bias"), arrays.get("res"),
                     out_o, alpha=c["alpha"], beta=c["beta"], gamma=c["gamma"])
        used = lin.last_kernel
        lin.close()
        return out_c, out_o, used
    d = {k: _to_torch(v, device) for k, v in arrays.items()}
    np_c = ko.np_dtype(desc.c_dtype)
    t_c = d["c0"].clone() if "c0" in d else _to_torch(np.full((nb, m, n), 0x7fc0 if np_c == np.uint16 else np.nan,
                                                              dtype=np_c), device)
    t_o = None
    if has_res:
        np_o = ko.np_dtype(desc.out_dtype)
        t_o = _to_torch(np.full((nb, m, n), 0x7fc0 if np_o == np.uint16 else np.nan, dtype=np_o), device)
    stream = torch.cuda.current_stream().cuda_stream
    if prepack:
        lin.prepack(d["b"], stream=stream)
    lin.run(d["a"], d["b"], t_c if c["want_c"] else None, d.get("bias"), d.get("res"), t_o, alpha=c["alpha"],
            beta=c["beta"], gamma=c["gamma"], stream=stream)
    lin.check(stream=stream)
    used = lin.last_kernel
    out_c = _from_torch(t_c)
    out_o = _from_torch(t_o) if t_o is not None else None
    lin.close()
    return out_c, out_o, used


# ----------------------------------------------------------------------------------------------- comparison rules

FP32_NORMWISE_TOL = 1e-5      # max |y - ref| / max |ref|
HALF_ABS_REL_TOL = 1e-2       # |y - ref| <= 1e-2 * (|ref| + 1), element-wise, for fp16 / bf16 results
# bf16 keeps 8 significant bits: two units in the last place are up to 1.56 % of the value.  The reference chain
# rounds twice after the GEMM (RNE after the bias, truncation after the activation), so a last-bit difference in
# the fp32 accumulator (summation order) can move a result by one unit at each rounding.  Such elements cannot
# always meet 1e-2 * (|ref| + 1); they are allowed if they are rare and within two units.
HALF_OUTLIER_FRACTION = 1e-4
HALF_OUTLIER_MAX_ULP = 2


def _ordered(bits16):
    """Maps 16-bit float patterns to integers whose difference is the distance in units in the last place."""
    b = bits16.astype(np.int32)
    return np.where(b & 0x8000, -(b & 0x7fff), b & 0x7fff)


def compare(got, ref, code):
    """Returns a dict of error figures and raises AssertionError when the tolerance of the type is exceeded."""
    g = ko.to_f32(got, code).astype(np.float64)
    r = ko.to_f32(ref, code).astype(np.float64)
    assert g.shape == r.shape
    assert np.all(np.isfinite(g)), "non-finite values (or untouched output elements) in the result"
    err = np.abs(g - r)
    scale = max(float(np.max(np.abs(r))), 1e-30)
    info = {"max_abs": float(err.max()), "normwise": float(err.max() / scale)}
    # the per-element form with a floor of 1e-3 * max|ref|: reported beside the figure that is enforced
    info["strict_fp32_rel"] = float(np.max(err / np.maximum(np.abs(r), 1e-3 * scale)))
    if code == kb.F32:
        assert info["normwise"] <= FP32_NORMWISE_TOL, "fp32 normwise error %.3e" % info["normwise"]
    else:
        bound = HALF_ABS_REL_TOL * (np.abs(r) + 1.0)
        over = err > bound
        ulp = np.abs(_ordered(got.view(np.uint16)) - _ordered(ref.view(np.uint16)))
        info["worst_over_bound"] = float(np.max(err / bound))
        info["over_bound_fraction"] = float(np.mean(over))
        info["over_bound_count"] = int(np.count_nonzero(over))
        info["elements"] = int(over.size)
        info["max_ulp"] = int(ulp.max())
        info["bit_exact_fraction"] = float(np.mean(ulp == 0))
        assert info["over_bound_fraction"] <= HALF_OUTLIER_FRACTION, \
            "%.2e of the elements exceed 1e-2*(|ref|+1)" % info["over_bound_fraction"]
        if over.any():
            assert int(ulp[over].max()) <= HALF_OUTLIER_MAX_ULP, \
                "an element beyond 1e-2*(|ref|+1) is %d units away from the oracle" % int(ulp[over].max())
    return info


def parity(case, device, kernel=kb.KERNEL_AUTO, acc=ko.ACC_F32, prepack=False, host=False, expect_kernel=None):
    desc, arrays, c = build_case(case)
    ref_c, ref_o = run_oracle(desc, arrays, c, acc=acc)
    got_c, got_o, used = run_gpu(desc, arrays, c, device, kernel=kernel, prepack=prepack, host=host)
    if expect_kernel is not None:
        assert used == expect_kernel, "kernel %s ran, expected %s" % (kb.KERNEL_NAMES.get(used), kb.KERNEL_NAMES.get(
            expect_kernel))
    info = {"kernel": kb.KERNEL_NAMES.get(used)}
    if c["want_c"]:
        info["c"] = compare(got_c, ref_c, desc.c_dtype)
    if ref_o is not None:
        info["out"] = compare(got_o, ref_o, desc.out_dtype)
    return info
