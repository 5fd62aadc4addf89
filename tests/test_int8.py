"""The integer rows of the reference's type table (src/dnn/src/kudnn_gemm.cpp:590-601): fp16 activations with 8-bit
weights (W8A16, :336-372) and the 8-bit integer products with 32-bit results (:259-334), against the CPU oracle.
Integer results must be bit-exact."""
import numpy as np
import pytest
import torch

import kudnn_b200 as kb
from oracle import ko
from tests import helpers

pytestmark = pytest.mark.gpu


def _w8a16_case(m, n, k, wcode, bias, act, res_op, b_layout, seed):
    rng = np.random.default_rng(seed)
    x = ko.to_storage(rng.standard_normal((1, m, k), dtype=np.float32), kb.F16)
    lo, hi = (-128, 128) if wcode == kb.S8 else (0, 256)
    w = rng.integers(lo, hi, (1, n, k)).astype(ko.np_dtype(wcode))
    arrays = {"a": x}
    if b_layout == "BA":
        arrays["b"], b_strides = w, (1, k)
    else:
        arrays["b"], b_strides = np.ascontiguousarray(w.transpose(0, 2, 1)), (n, 1)
    bias_dt = None
    if bias is not None:
        bias_dt = kb.F32 if bias == "f32" else kb.F16
        arrays["bias"] = ko.to_storage(rng.standard_normal((1, n), dtype=np.float32) * 4, bias_dt)
    if res_op != kb.RES_NONE:
        arrays["res"] = ko.to_storage(rng.standard_normal((1, m, n), dtype=np.float32), kb.F16)
    desc = kb.make_desc(m, n, k, kb.F16, b_dtype=wcode, b_strides=b_strides, has_bias=bias is not None, bias_dtype=bias_dt,
                        act=act, res_op=res_op)
    c = helpers.case_defaults(dict(m=m, n=n, k=k, res_op=res_op))
    return desc, arrays, c


@pytest.mark.parametrize("wcode", [kb.S8, kb.U8])
@pytest.mark.parametrize("m,n,k,kernel", [(260, 264, 136, kb.KERNEL_TC), (4, 1003, 1048, kb.KERNEL_GEMV_MMA),
                                           (1, 520, 264, kb.KERNEL_GEMV_FMA), (67, 45, 33, kb.KERNEL_SIMT)])
@pytest.mark.parametrize("bias,act,res_op", [(None, kb.ACT_NONE, kb.RES_NONE), ("f32", kb.ACT_SWISH, kb.RES_IDENTICAL),
                                              ("f16", kb.ACT_RELU, kb.RES_NONE)])
@pytest.mark.parametrize("prepack", [False, True])
def test_w8a16(cuda_device, wcode, m, n, k, kernel, bias, act, res_op, prepack):
    """fp16 x int8 -> fp16: the weights are widened to fp16 (exactly) when they are packed, fp32 accumulation, the bias
    is added in fp32 and the result rounded once, whatever the bias type."""
    b_layout = "BA" if (k % 8 == 0) else "AB"
    desc, arrays, c = _w8a16_case(m, n, k, wcode, bias, act, res_op, b_layout, 91)
    ref_c, ref_o = helpers.run_oracle(desc, arrays, c, acc=ko.ACC_F64)
    got_c, got_o, used = helpers.run_gpu(desc, arrays, c, cuda_device, kernel=kernel, prepack=prepack)
    assert used == kernel
    helpers.compare(got_c, ref_c, desc.c_dtype)
    if res_op != kb.RES_NONE:
        helpers.compare(got_o, ref_o, desc.out_dtype)


def test_w8a16_host_pointers_and_default_dispatch(cuda_device):
    desc, arrays, c = _w8a16_case(300, 520, 264, kb.S8, "f32", kb.ACT_GELU_TANH, kb.RES_NONE, "AB", 92)
    ref_c, _ = helpers.run_oracle(desc, arrays, c, acc=ko.ACC_F64)
    got_c, _, used = helpers.run_gpu(desc, arrays, c, cuda_device, host=True, prepack=True)
    assert used == kb.KERNEL_TC
    helpers.compare(got_c, ref_c, desc.c_dtype)


@pytest.mark.parametrize("acode,bcode", [(kb.S8, kb.S8), (kb.S8, kb.U8), (kb.U8, kb.S8), (kb.U8, kb.U8)])
@pytest.mark.parametrize("bias", [None, "row", "col", "scalar", "full"])
@pytest.mark.parametrize("batch", [(), (3, 2)])
def test_int8_products_are_exact(cuda_device, acode, bcode, bias, batch):
    rng = np.random.default_rng(93)
    m, n, k = 70, 90, 200
    nb = int(np.prod(batch)) if batch else 1

    def draw(code, shape):
        lo, hi = (-128, 128) if code == kb.S8 else (0, 256)
        return rng.integers(lo, hi, shape).astype(ko.np_dtype(code))
    a, b = draw(acode, (nb, m, k)), draw(bcode, (nb, k, n))  # weights [k, n], n contiguous, as the reference's tests store them
    shape = {None: None, "row": (1, n), "col": (m, 1), "scalar": (1, 1), "full": (m, n)}[bias]
    ext3 = tuple([0] * (3 - len(batch)) + list(batch)) if batch else (0, 0, 0)

    def sb(per):
        out, stride = [0, 0, 0], per
        ext = [1] * (3 - len(batch)) + list(batch)
        for i in (2, 1, 0):
            out[i] = stride if ext[i] > 1 else 0
            stride *= ext[i]
        return tuple(out) if batch else (0, 0, 0)
    desc = kb.make_desc(m, n, k, acode, b_dtype=bcode, c_dtype=kb.S32, b_strides=(n, 1), has_bias=shape is not None,
                        bias_dtype=kb.S32, bias_strides=(0, 0) if shape is None else (shape[1] if shape[0] > 1 else 0,
                                                                                     1 if shape[1] > 1 else 0),
                        batch=ext3, a_sb=sb(m * k), b_sb=sb(k * n), c_sb=sb(m * n))
    bias_arr = None if shape is None else rng.integers(-100000, 100000, shape).astype(np.int32)
    want = np.zeros((nb, m, n), dtype=np.int32)
    ko.linear(helpers.oracle_desc(desc), a, b, want, bias_arr)
    # independent check of the oracle itself
    ref = np.einsum("bmk,bkn->bmn", a.astype(np.int64), b.astype(np.int64))
    if bias_arr is not None:
        ref = ref + bias_arr.astype(np.int64)
    assert np.array_equal(want, ref.astype(np.int32))
    d_a, d_b = torch.from_numpy(a).to(cuda_device), torch.from_numpy(b).to(cuda_device)
    d_c = torch.zeros((nb, m, n), dtype=torch.int32, device=cuda_device)
    d_bias = torch.from_numpy(bias_arr).to(cuda_device) if bias_arr is not None else None
    lin = kb.Linear(desc)
    lin.run(d_a, d_b, d_c, d_bias, stream=torch.cuda.current_stream().cuda_stream)
    lin.check(stream=torch.cuda.current_stream().cuda_stream)
    assert np.array_equal(d_c.cpu().numpy(), want)
    if not batch:  # host pointers too
        h_c = np.zeros((1, m, n), dtype=np.int32)
        lin.run_host(a, b, h_c, bias_arr)
        assert np.array_equal(h_c, want)


def test_integer_products_refuse_post_operations(cuda_device):
    assert kb.capi.validate(kb.make_desc(8, 8, 8, kb.S8, c_dtype=kb.S32, act=kb.ACT_RELU)) == 1
    assert kb.capi.validate(kb.make_desc(8, 8, 8, kb.S8, c_dtype=kb.F16)) == 1
    assert kb.capi.validate(kb.make_desc(8, 8, 8, kb.BF16, b_dtype=kb.S8)) == 1
    assert kb.capi.validate(kb.make_desc(8, 8, 8, kb.F16, b_dtype=kb.U8)) == 0


def _int_case(rng, m, n, k, acode, bcode, b_layout, bias):
    def draw(code, shape):
        lo, hi = (-128, 128) if code == kb.S8 else (0, 256)
        return rng.integers(lo, hi, shape).astype(ko.np_dtype(code))
    a = draw(acode, (m, k))
    w = draw(bcode, (n, k))  # logical weights W[n, k]
    if b_layout == "BA":      # K-major, as a transposed nn.Linear weight is stored
        b_arr, b_strides = w, (1, k)
    else:                      # [k, n], n contiguous, as the reference's tests store them
        b_arr, b_strides = np.ascontiguousarray(w.T), (n, 1)
    shape = {None: None, "row": (1, n), "col": (m, 1), "scalar": (1, 1), "full": (m, n)}[bias]
    bias_arr = None if shape is None else rng.integers(-100000, 100000, shape).astype(np.int32)
    desc = kb.make_desc(m, n, k, acode, b_dtype=bcode, c_dtype=kb.S32, b_strides=b_strides, has_bias=shape is not None,
                        bias_dtype=kb.S32, bias_strides=(0, 0) if shape is None else (shape[1] if shape[0] > 1 else 0,
                                                                                     1 if shape[1] > 1 else 0))
    # sums of at most k * 255 * 255 < 2^53: the float64 product is exact
    ref = a.astype(np.float64) @ w.astype(np.float64).T
    if bias_arr is not None:
        ref = ref + bias_arr.astype(np.float64)
    return desc, a, b_arr, bias_arr, ref.astype(np.int64).astype(np.int32)


@pytest.mark.parametrize("acode,bcode", [(kb.S8, kb.S8), (kb.S8, kb.U8), (kb.U8, kb.S8), (kb.U8, kb.U8)])
@pytest.mark.parametrize("m,n,k,b_layout", [(260, 264, 136, "BA"),    # tails in m, n and k; operands need padding
                                            (260, 264, 144, "AB"),    # weights transposed by the pack kernel
                                            (128, 512, 256, "BA"),    # everything read in place
                                            (300, 1000, 1040, "AB"),
                                            (2560, 4096, 272, "BA")])  # CTA pairs, last wave in half-width pieces
@pytest.mark.parametrize("bias", [None, "row", "full"])
@pytest.mark.parametrize("prepack", [False, True])
def test_int8_products_on_tensor_cores(cuda_device, acode, bcode, m, n, k, b_layout, bias, prepack):
    """s8/u8 x s8/u8 -> s32 through tcgen05.mma kind::i8: bit-exact against an exact float64 product, and against the
    C oracle on the small shapes."""
    rng = np.random.default_rng(97)
    desc, a, b_arr, bias_arr, want = _int_case(rng, m, n, k, acode, bcode, b_layout, bias)
    if m * n * k < 2.0e7:
        w_kn = b_arr.T if b_layout == "BA" else b_arr
        odesc = kb.make_desc(m, n, k, acode, b_dtype=bcode, c_dtype=kb.S32, b_strides=(n, 1), has_bias=bias is not None,
                             bias_dtype=kb.S32, bias_strides=(desc.bias_sm, desc.bias_sn))
        oc = np.zeros((1, m, n), dtype=np.int32)
        ko.linear(helpers.oracle_desc(odesc), a[None], np.ascontiguousarray(w_kn)[None], oc, bias_arr)
        assert np.array_equal(oc[0], want)
    stream = torch.cuda.current_stream().cuda_stream
    d_a, d_b = torch.from_numpy(a).to(cuda_device), torch.from_numpy(b_arr).to(cuda_device)
    d_c = torch.full((m, n), -7, dtype=torch.int32, device=cuda_device)
    d_bias = torch.from_numpy(bias_arr).to(cuda_device) if bias_arr is not None else None
    lin = kb.Linear(desc)
    lin.force_kernel(kb.KERNEL_TC)
    if prepack:
        lin.prepack(d_b, stream=stream)
    for _ in range(2):  # the second run reuses the plan
        lin.run(d_a, d_b, d_c, d_bias, stream=stream)
    lin.check(stream=stream)
    assert lin.last_kernel == kb.KERNEL_TC
    assert np.array_equal(d_c.cpu().numpy(), want)
    lin.close()


def test_int8_default_dispatch_and_host_pointers(cuda_device):
    rng = np.random.default_rng(98)
    desc, a, b_arr, bias_arr, want = _int_case(rng, 1024, 2048, 4096, kb.U8, kb.S8, "BA", "row")
    lin = kb.Linear(desc)
    lin.prepack(b_arr)
    h_c = np.zeros((1024, 2048), dtype=np.int32)
    lin.run_host(a, b_arr, h_c, bias_arr)
    assert lin.last_kernel == kb.KERNEL_TC
    assert np.array_equal(h_c, want)
    # alpha != 1 is not a tensor-core case: the general integer kernel takes it
    d_a, d_b = torch.from_numpy(a).to(cuda_device), torch.from_numpy(b_arr).to(cuda_device)
    d_c = torch.zeros((1024, 2048), dtype=torch.int32, device=cuda_device)
    lin2 = kb.Linear(desc)
    lin2.run(d_a, d_b, d_c, torch.from_numpy(bias_arr).to(cuda_device), alpha=2.0, stream=torch.cuda.current_stream().cuda_stream)
    lin2.check(stream=torch.cuda.current_stream().cuda_stream)
    assert lin2.last_kernel == kb.KERNEL_SIMT
    ref = 2 * (a.astype(np.float64) @ b_arr.astype(np.float64).T) + bias_arr
    assert np.array_equal(d_c.cpu().numpy(), ref.astype(np.int64).astype(np.int32))


@pytest.mark.parametrize("wcode", [kb.S8, kb.U8])
@pytest.mark.parametrize("m,n,k", [(1, 520, 272), (1, 1003, 1040), (1, 96, 8192), (2, 264, 528), (4, 1003, 1040),
                                   (8, 96, 2064), (12, 264, 528), (16, 520, 1040)])
@pytest.mark.parametrize("b_layout,prepack", [("BA", False), ("BA", True), ("AB", True)])
@pytest.mark.parametrize("bias,act,res_op", [(None, kb.ACT_NONE, kb.RES_NONE), ("f32", kb.ACT_SWISH, kb.RES_ELTWISE_MUL),
                                              ("f16", kb.ACT_GELU_TANH, kb.RES_NONE)])
def test_w8a16_decode_streams_the_8_bit_weights(cuda_device, wcode, m, n, k, b_layout, prepack, bias, act, res_op):
    """Decode shapes with K a multiple of 16: the streaming kernels read the 8-bit weights themselves (the caller's
    K-major buffer, or the K-major copy pre-packing makes of another layout) and widen them in registers: the FMA kernel
    for one activation row, the MMA kernel for 2 to 16."""
    desc, arrays, c = _w8a16_case(m, n, k, wcode, bias, act, res_op, b_layout, 94)
    ref_c, ref_o = helpers.run_oracle(desc, arrays, c, acc=ko.ACC_F64)
    got_c, got_o, used = helpers.run_gpu(desc, arrays, c, cuda_device, prepack=prepack)   # default dispatch
    assert used == (kb.KERNEL_GEMV_FMA if m == 1 else kb.KERNEL_GEMV_MMA)
    helpers.compare(got_c, ref_c, desc.c_dtype)
    if res_op != kb.RES_NONE:
        helpers.compare(got_o, ref_o, desc.out_dtype)
    # the same primitive on another kernel (widened from the 8-bit state) agrees within the tolerance too
    got2_c, _, used2 = helpers.run_gpu(desc, arrays, c, cuda_device, kernel=kb.KERNEL_SIMT, prepack=prepack)
    assert used2 == kb.KERNEL_SIMT
    helpers.compare(got2_c, ref_c, desc.c_dtype)
