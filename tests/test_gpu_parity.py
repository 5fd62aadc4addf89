"""Parity of the CUDA kernels with the CPU oracle, through the C ABI, on a B200.

Small and medium cases are compared element by element on the full output.  The five benchmark
configurations run at full size; there the oracle evaluates a seeded sample of rows (rows are independent), and
size-independent properties cover the whole output: sum over rows of a linear layer equals the layer applied to the
summed input, and an m-sharded run reproduces the unsharded one bit for bit."""
import os

import numpy as np
import pytest
import torch

import kudnn_b200 as kb
from oracle import ko
from tests import helpers

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "linear_golden.npz")
ACTS = [(kb.ACT_NONE, 1.0), (kb.ACT_RELU, 0.0), (kb.ACT_RELU, 0.1), (kb.ACT_SWISH, 1.0), (kb.ACT_GELU_TANH, 1.0),
        (kb.ACT_GELU_ERF, 1.0), (kb.ACT_SIGMOID, 1.0), (kb.ACT_TANH, 1.0)]


# ------------------------------------------------------------------------------------------- general kernel

@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("act,alpha", ACTS)
def test_simt_activations(cuda_device, dtype, act, alpha):
    # the shape class of FWD_LINEAR_*_2D_* (linear_activation_gtest.cpp:462-1095): 110x20 . 20x200, full bias
    case = dict(m=110, n=200, k=20, dtype=dtype, bias="full", act=act, act_alpha=alpha, seed=21)
    info = helpers.parity(case, cuda_device, kernel=kb.KERNEL_SIMT, acc=ko.ACC_F64, expect_kernel=kb.KERNEL_SIMT)
    if dtype != "f32":
        assert info["c"]["bit_exact_fraction"] > 0.99


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("bias", [None, "row", "col", "scalar", "full"])
@pytest.mark.parametrize("a_layout,b_layout", [("AB", "AB"), ("AB", "BA"), ("BA", "AB"), ("BA", "BA")])
def test_simt_bias_kinds_and_layouts(cuda_device, dtype, bias, a_layout, b_layout):
    case = dict(m=67, n=45, k=33, dtype=dtype, bias=bias, a_layout=a_layout, b_layout=b_layout, seed=22)
    helpers.parity(case, cuda_device, kernel=kb.KERNEL_SIMT, acc=ko.ACC_F64)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("res_op,gamma", [(kb.RES_IDENTICAL, 1.0), (kb.RES_EXT, 0.5), (kb.RES_ELTWISE_MUL, 1.0)])
def test_simt_second_output(cuda_device, dtype, res_op, gamma):
    # LinearResTests shapes (linear_res_gtest.cpp:768-1181): 400x200 . 200x500
    case = dict(m=400, n=500, k=200, dtype=dtype, bias="row", res_op=res_op, gamma=gamma, seed=23)
    helpers.parity(case, cuda_device, kernel=kb.KERNEL_SIMT)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("batch,a_bcast,b_bcast", [((2,), False, True), ((3, 2), False, False), ((4, 3, 2), False, True),
                                                    ((2, 2), True, False)])
def test_simt_batched_with_broadcast(cuda_device, dtype, batch, a_bcast, b_bcast):
    case = dict(m=23, n=31, k=20, dtype=dtype, bias="row", act=kb.ACT_RELU, act_alpha=0.0, batch=batch, a_bcast=a_bcast,
                b_bcast=b_bcast, seed=24)
    helpers.parity(case, cuda_device, acc=ko.ACC_F64, expect_kernel=kb.KERNEL_SIMT)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("batch,m,expect", [((2, 3), 100, kb.KERNEL_TC), ((4,), 130, kb.KERNEL_TC),
                                            ((2, 2), 1, "streaming")])
def test_batched_shared_weights_run_as_rows(cuda_device, dtype, batch, m, expect):
    """[B, S, K] x [K, N] with contiguous batches is one 2-D problem of B*S rows and takes the fast kernels."""
    case = dict(m=m, n=264, k=512, dtype=dtype, bias="row", act=kb.ACT_SWISH, res_op=kb.RES_IDENTICAL, batch=batch,
                b_bcast=True, x_dist="normal", w_std=0.03, seed=25)
    info = helpers.parity(case, cuda_device, acc=ko.ACC_F64, expect_kernel=None if expect == "streaming" else expect)
    if expect == "streaming":  # four rows: one of the streaming kernels, whichever the dispatcher prefers
        assert info["kernel"] in [kb.KERNEL_NAMES[i] for i in (kb.KERNEL_GEMV_FMA, kb.KERNEL_GEMV_MMA)]


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_alpha_beta(cuda_device, dtype):
    case = dict(m=50, n=70, k=64, dtype=dtype, bias="row", alpha=0.5, beta=0.25, seed=25)
    helpers.parity(case, cuda_device, kernel=kb.KERNEL_SIMT)


# ------------------------------------------------------------------------------------------- streaming kernels

@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("m", [1, 2, 3, 4])
def test_gemv_fma(cuda_device, dtype, m):
    case = dict(m=m, n=1000, k=1032, dtype=dtype, bias="row", act=kb.ACT_SWISH, x_dist="normal", w_std=0.05, seed=31)
    helpers.parity(case, cuda_device, kernel=kb.KERNEL_GEMV_FMA, expect_kernel=kb.KERNEL_GEMV_FMA)


@pytest.mark.parametrize("staged,wide", [("1", "1"), ("0", "1"), ("0", "0")])
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("m", [1, 3, 4, 7, 8, 9, 16])
def test_gemv_mma(cuda_device, monkeypatch, staged, wide, dtype, m):
    monkeypatch.setenv("KUDNN_B200_GEMV_STAGED", staged)  # weight feed: through per-warp staging, or fragment-shaped loads
    monkeypatch.setenv("KUDNN_B200_GEMV_WIDE", wide)      # fragment-shaped loads of 32 or 16 bytes per lane (m > 8)
    case = dict(m=m, n=1003, k=1048, dtype=dtype, res_op=kb.RES_ELTWISE_MUL, x_dist="normal", w_std=0.05, seed=32)
    helpers.parity(case, cuda_device, kernel=kb.KERNEL_GEMV_MMA, expect_kernel=kb.KERNEL_GEMV_MMA)


@pytest.mark.parametrize("staged,wide", [("1", "1"), ("0", "1"), ("0", "0")])
@pytest.mark.parametrize("kernel", [kb.KERNEL_GEMV_FMA, kb.KERNEL_GEMV_MMA])
@pytest.mark.parametrize("n,k", [(8, 8), (5, 4096), (40000, 64), (777, 2504), (2600, 16384), (300, 8192)])
def test_gemv_shapes_that_cut_units(cuda_device, monkeypatch, staged, wide, kernel, n, k):
    monkeypatch.setenv("KUDNN_B200_GEMV_STAGED", staged)
    monkeypatch.setenv("KUDNN_B200_GEMV_WIDE", wide)
    # tiny, one long row, many short rows, odd sizes: exercise whole units, split units and idle warps
    case = dict(m=2, n=n, k=k, dtype="bf16", bias="row", x_dist="normal", w_std=0.05, seed=33)
    helpers.parity(case, cuda_device, kernel=kernel, expect_kernel=kernel)


@pytest.mark.parametrize("wide", ["1", "0"])
@pytest.mark.parametrize("n,k", [(8, 8), (5, 4096), (4000, 72), (777, 2504), (2600, 16384)])
def test_gemv_mma_sixteen_rows_shapes(cuda_device, monkeypatch, wide, n, k):
    monkeypatch.setenv("KUDNN_B200_GEMV_WIDE", wide)
    case = dict(m=12, n=n, k=k, dtype="bf16", bias="row", act=kb.ACT_SWISH, x_dist="normal", w_std=0.05, seed=37)
    helpers.parity(case, cuda_device, kernel=kb.KERNEL_GEMV_MMA, expect_kernel=kb.KERNEL_GEMV_MMA)


@pytest.mark.parametrize("staged,wide", [(None, None), ("1", "1"), ("0", "1"), ("0", "0")])
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("m", [2, 4, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(1003, 1048), (300, 8192), (2600, 16384), (8, 8), (4000, 72)])
def test_gemv_mma_decode_packed_weights(cuda_device, monkeypatch, staged, wide, dtype, m, n, k):
    """Pre-packing a decode-shaped primitive stores the weights once more in blocks of 8 rows x 64 k, which is what
    the MMA streaming kernels then read (every feed variant); results must not change."""
    if staged is not None:
        monkeypatch.setenv("KUDNN_B200_GEMV_STAGED", staged)
        monkeypatch.setenv("KUDNN_B200_GEMV_WIDE", wide)
    case = dict(m=m, n=n, k=k, dtype=dtype, bias="row", act=kb.ACT_SWISH, res_op=kb.RES_ELTWISE_MUL, x_dist="normal",
                w_std=0.03, seed=40)
    desc, arrays, c = helpers.build_case(case)
    ref_c, ref_o = helpers.run_oracle(desc, arrays, c)
    packed = helpers.run_gpu(desc, arrays, c, cuda_device, kernel=kb.KERNEL_GEMV_MMA, prepack=True)
    plain = helpers.run_gpu(desc, arrays, c, cuda_device, kernel=kb.KERNEL_GEMV_MMA)
    assert packed[2] == kb.KERNEL_GEMV_MMA
    helpers.compare(packed[0], ref_c, desc.c_dtype)
    helpers.compare(packed[1], ref_o, desc.out_dtype)
    if staged is not None:  # same feed on both layouts: same arithmetic in the same order, only the addresses differ
        assert np.array_equal(packed[0], plain[0]) and np.array_equal(packed[1], plain[1])
    else:                   # the default feed depends on the layout
        helpers.compare(plain[0], ref_c, desc.c_dtype)
        helpers.compare(plain[1], ref_o, desc.out_dtype)


@pytest.mark.parametrize("m", [4, 16])
def test_decode_default_is_deterministic(cuda_device, m):
    case = dict(m=m, n=4096, k=4096, dtype="bf16", res_op=kb.RES_ELTWISE_MUL, x_dist="normal", w_std=0.02, seed=36)
    desc, arrays, c = helpers.build_case(case)
    d = {k: helpers._to_torch(v, cuda_device) for k, v in arrays.items()}
    lin = kb.Linear(desc)
    outs = []
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        t_o = torch.zeros((1, m, 4096), dtype=torch.int16, device=cuda_device)
        lin.run(d["a"], d["b"], None, None, d["res"], t_o, stream=stream)
        lin.check(stream=stream)
        outs.append(helpers._from_torch(t_o))
    assert lin.last_kernel == kb.KERNEL_GEMV_MMA
    _, ref_o = helpers.run_oracle(desc, arrays, c)
    helpers.compare(outs[0], ref_o, desc.out_dtype)
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[1], outs[2])


def test_gemv_repeated_calls_leave_counters_clean(cuda_device):
    case = dict(m=16, n=3000, k=4096, dtype="bf16", res_op=kb.RES_ELTWISE_MUL, x_dist="normal", w_std=0.02, seed=34)
    desc, arrays, c = helpers.build_case(case)
    ref_c, ref_o = helpers.run_oracle(desc, arrays, c)
    d = {k: helpers._to_torch(v, cuda_device) for k, v in arrays.items()}
    lin = kb.Linear(desc)
    outs = []
    for _ in range(3):
        t_c = torch.zeros((1, 16, 3000), dtype=torch.int16, device=cuda_device)
        t_o = torch.zeros_like(t_c)
        lin.run(d["a"], d["b"], t_c, None, d["res"], t_o, stream=torch.cuda.current_stream().cuda_stream)
        lin.check(stream=torch.cuda.current_stream().cuda_stream)
        outs.append(helpers._from_torch(t_o))
    assert lin.last_kernel in (kb.KERNEL_GEMV_MMA,)
    helpers.compare(outs[0], ref_o, desc.out_dtype)
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[1], outs[2])  # slot-ordered sums: deterministic


# ------------------------------------------------------------------------------------------- tensor-core kernel

@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 512), (256, 512, 256), (100, 200, 72), (300, 520, 264),
                                    (1024, 1024, 1024), (129, 257, 8), (2048, 384, 4096)])
def test_tc_16bit_shapes(cuda_device, dtype, m, n, k):
    case = dict(m=m, n=n, k=k, dtype=dtype, bias="row", act=kb.ACT_SWISH, x_dist="normal", w_std=0.05, seed=41)
    helpers.parity(case, cuda_device, kernel=kb.KERNEL_TC, expect_kernel=kb.KERNEL_TC)


@pytest.mark.parametrize("m,n,k", [(128, 256, 32), (128, 1024, 1024), (100, 200, 72), (300, 130, 1000)])
def test_tc_fp32_split(cuda_device, m, n, k):
    case = dict(m=m, n=n, k=k, dtype="f32", bias="row", act=kb.ACT_RELU, act_alpha=0.0, w_std=0.02, seed=42)
    info = helpers.parity(case, cuda_device, kernel=kb.KERNEL_TC, acc=ko.ACC_F64, expect_kernel=kb.KERNEL_TC)
    print("fp32 split-TF32 normwise error", info["c"]["normwise"])


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("a_layout,b_layout", [("AB", "AB"), ("BA", "BA"), ("BA", "AB")])
def test_tc_packs_other_layouts(cuda_device, dtype, a_layout, b_layout):
    case = dict(m=200, n=300, k=136, dtype=dtype, bias="row", a_layout=a_layout, b_layout=b_layout, w_std=0.05, seed=43)
    helpers.parity(case, cuda_device, kernel=kb.KERNEL_TC, acc=ko.ACC_F64, expect_kernel=kb.KERNEL_TC)


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("bias", [None, "col", "scalar", "full"])
@pytest.mark.parametrize("res_op,gamma", [(kb.RES_NONE, 1.0), (kb.RES_IDENTICAL, 1.0), (kb.RES_EXT, 0.5),
                                           (kb.RES_ELTWISE_MUL, 1.0)])
def test_tc_epilogue_variants(cuda_device, dtype, bias, res_op, gamma):
    case = dict(m=260, n=264, k=128, dtype=dtype, bias=bias, act=kb.ACT_GELU_TANH, res_op=res_op, gamma=gamma,
                x_dist="normal", w_std=0.05, seed=44)
    helpers.parity(case, cuda_device, kernel=kb.KERNEL_TC, acc=ko.ACC_F64, expect_kernel=kb.KERNEL_TC)


def test_tc_unaligned_n_and_only_second_output(cuda_device):
    case = dict(m=130, n=203, k=64, dtype="bf16", bias="row", res_op=kb.RES_IDENTICAL, want_c=False, w_std=0.05, seed=45)
    helpers.parity(case, cuda_device, kernel=kb.KERNEL_TC, expect_kernel=kb.KERNEL_TC)


def test_tc_alpha_beta(cuda_device):
    case = dict(m=256, n=256, k=256, dtype="bf16", bias="row", alpha=0.5, beta=0.25, w_std=0.05, seed=46)
    helpers.parity(case, cuda_device, kernel=kb.KERNEL_TC, expect_kernel=kb.KERNEL_TC)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("splits", [None, "1", "3", "64"])
@pytest.mark.parametrize("m,n,k", [(128, 1024, 1024), (100, 200, 2056), (300, 130, 1000)])
def test_tc_split_k(cuda_device, monkeypatch, dtype, splits, m, n, k):
    """Few tiles and a long K: the CTAs of a cluster cut K between them, keep their partial tiles in shared memory and
    add them in rank order through distributed shared memory.  The result must not depend on the cut beyond fp32
    summation order, and repeated calls must agree bit for bit."""
    if splits is not None:
        monkeypatch.setenv("KUDNN_B200_TC_SPLITS", splits)
    case = dict(m=m, n=n, k=k, dtype=dtype, bias="row", act=kb.ACT_SWISH, res_op=kb.RES_EXT, gamma=0.5, x_dist="normal",
                w_std=0.02, seed=48)
    desc, arrays, c = helpers.build_case(case)
    ref_c, ref_o = helpers.run_oracle(desc, arrays, c, acc=ko.ACC_F64)
    first = helpers.run_gpu(desc, arrays, c, cuda_device, kernel=kb.KERNEL_TC)
    second = helpers.run_gpu(desc, arrays, c, cuda_device, kernel=kb.KERNEL_TC)
    helpers.compare(first[0], ref_c, desc.c_dtype)
    helpers.compare(first[1], ref_o, desc.out_dtype)
    assert np.array_equal(first[0], second[0]) and np.array_equal(first[1], second[1])


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("m,n,k", [(2560, 2048, 136), (2400, 2300, 64), (512, 9000, 128)])
def test_tc_cta_pairs(cuda_device, dtype, m, n, k):
    """Large problems run on clusters of two CTAs (256 x 256 tiles); the first two shapes leave a short last wave,
    whose tiles are then cut into two pieces of half the width.  Ragged edges in m and n included."""
    case = dict(m=m, n=n, k=k, dtype=dtype, bias="row", act=kb.ACT_GELU_TANH, res_op=kb.RES_IDENTICAL, x_dist="normal",
                w_std=0.05, seed=49)
    helpers.parity(case, cuda_device, kernel=kb.KERNEL_TC, acc=ko.ACC_F64, expect_kernel=kb.KERNEL_TC)


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("batch,a_bcast,b_bcast", [((2,), False, False), ((3, 2), False, False), ((4, 3, 2), False, False),
                                                    ((2, 2), True, False), ((5,), False, True)])
@pytest.mark.parametrize("a_layout,b_layout", [("AB", "BA"), ("AB", "AB"), ("BA", "AB")])
def test_tc_batched(cuda_device, dtype, batch, a_bcast, b_bcast, a_layout, b_layout):
    """Batched N-D Linear on the tensor-core kernel: the batch entry is a coordinate of its tile scheduler.  Per-batch
    weights (the reference's 3-D to 5-D cases, linear_activation_gtest.cpp:475-512, N-major as its tests store them, or
    K-major), one shared activation matrix, one shared weight matrix; operands that are not K-major are packed, all
    batch entries in one launch."""
    if b_bcast and (a_layout, b_layout) == ("AB", "BA"):
        pytest.skip("shared K-major weights with row-major activations collapse into one 2-D problem (tested elsewhere)")
    case = dict(m=130, n=264, k=136, dtype=dtype, bias="row", act=kb.ACT_RELU, act_alpha=0.0, res_op=kb.RES_IDENTICAL,
                batch=batch, a_bcast=a_bcast, b_bcast=b_bcast, a_layout=a_layout, b_layout=b_layout, x_dist="normal",
                w_std=0.05, seed=56)
    helpers.parity(case, cuda_device, acc=ko.ACC_F64, expect_kernel=kb.KERNEL_TC)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_tc_batched_split_k_and_activations(cuda_device, dtype):
    # few tiles and a long k in every batch entry: cluster split-K with a batch coordinate; general epilogue
    case = dict(m=100, n=200, k=2056, dtype=dtype, bias="full", act=kb.ACT_GELU_ERF, batch=(3,), b_bcast=False,
                x_dist="normal", w_std=0.02, seed=57)
    helpers.parity(case, cuda_device, acc=ko.ACC_F64, expect_kernel=kb.KERNEL_TC)
    # the reference's own batched shape class (110 x 20 . 20 x 200 per entry) is too small to be worth a tensor-core
    # launch and stays on the general kernel
    small = dict(m=110, n=200, k=20, dtype=dtype, bias="full", act=kb.ACT_RELU, act_alpha=0.0, batch=(4, 3, 2),
                 b_bcast=False, b_layout="AB", seed=58)
    helpers.parity(small, cuda_device, acc=ko.ACC_F64, expect_kernel=kb.KERNEL_SIMT)


def test_tc_agrees_with_general_kernel(cuda_device):
    case = dict(m=512, n=768, k=512, dtype="bf16", bias="row", act=kb.ACT_SWISH, x_dist="normal", w_std=0.03, seed=47)
    desc, arrays, c = helpers.build_case(case)
    tc, _, _ = helpers.run_gpu(desc, arrays, c, cuda_device, kernel=kb.KERNEL_TC)
    simt, _, _ = helpers.run_gpu(desc, arrays, c, cuda_device, kernel=kb.KERNEL_SIMT)
    info = helpers.compare(tc, simt, desc.c_dtype)
    assert info["bit_exact_fraction"] > 0.99



# The tensor-core kernel's epilogue comes in two forms: one with the activation and the element type fixed at compile
# time (relu / swish / gelu_tanh, every tensor in the input type) and a general one that reads both from the
# descriptor.  These cases take the general form on each launch shape: a single CTA per tile, CTA pairs, and the
# cluster split-K whose last pass runs the chain from shared memory.
TC_SHAPES = {"single": (260, 264, 128), "pair": (2560, 2048, 136), "splitk": (128, 1024, 1024)}
TC_GENERAL = {
    "gelu_erf": dict(dtype="bf16", bias="row", act=kb.ACT_GELU_ERF),
    "sigmoid": dict(dtype="f16", bias="row", act=kb.ACT_SIGMOID, res_op=kb.RES_IDENTICAL),
    "tanh": dict(dtype="bf16", bias="row", act=kb.ACT_TANH, res_op=kb.RES_EXT, gamma=0.5),
    "gelu_erf_f32": dict(dtype="f32", bias="row", act=kb.ACT_GELU_ERF),
    # the reference's <bf16, bf16, bf16, float> instance (kudnn_gemm.cpp:208-227): fp32 bias, bf16 everything else
    "bf16_f32bias": dict(dtype="bf16", bias="row", bias_dtype="f32", act=kb.ACT_SWISH),
    # <fp16, fp16, float, float> and <bf16, bf16, float, float> (kudnn_gemm.cpp:195-206, :229-241)
    "f16_to_f32": dict(dtype="f16", c_dtype="f32", bias="row", bias_dtype="f32", act=kb.ACT_GELU_TANH,
                       res_op=kb.RES_IDENTICAL),
    "bf16_to_f32": dict(dtype="bf16", c_dtype="f32", bias="row", bias_dtype="f32", act=kb.ACT_RELU, act_alpha=0.0),
    "bf16_to_f32_nobias": dict(dtype="bf16", c_dtype="f32"),
    # fp16 result with an fp32 bias has no exact instance: product and bias add in fp32, one rounding
    "f16_f32bias": dict(dtype="f16", bias="row", bias_dtype="f32", act=kb.ACT_SWISH, res_op=kb.RES_ELTWISE_MUL),
}


@pytest.mark.parametrize("shape", sorted(TC_SHAPES))
@pytest.mark.parametrize("variant", sorted(TC_GENERAL))
def test_tc_general_epilogue(cuda_device, shape, variant):
    m, n, k = TC_SHAPES[shape]
    case = dict(m=m, n=n, k=k, x_dist="normal", w_std=0.05, seed=53, **TC_GENERAL[variant])
    info = helpers.parity(case, cuda_device, kernel=kb.KERNEL_TC, acc=ko.ACC_F64, expect_kernel=kb.KERNEL_TC)
    print("tc general epilogue", shape, variant, info)


@pytest.mark.parametrize("variant", ["bf16_f32bias", "f16_to_f32", "bf16_to_f32", "f16_f32bias"])
@pytest.mark.parametrize("kernel,m", [(kb.KERNEL_SIMT, 67), (kb.KERNEL_GEMV_MMA, 7), (kb.KERNEL_GEMV_FMA, 2)])
def test_mixed_type_tuples_other_kernels(cuda_device, variant, kernel, m):
    case = dict(m=m, n=520, k=264, x_dist="normal", w_std=0.05, seed=54, **TC_GENERAL[variant])
    helpers.parity(case, cuda_device, kernel=kernel, acc=ko.ACC_F64, expect_kernel=kernel)


def test_bf16_scalars_of_the_bias_free_product(cuda_device):
    # without a bias the reference multiplies bf16 operands with cblas_bgemm, whose alpha and beta are bf16
    # (kudnn_gemm.cpp:222-226): 0.3 becomes 0.30078125
    for kernel, m in ((kb.KERNEL_TC, 256), (kb.KERNEL_SIMT, 50)):
        case = dict(m=m, n=256, k=256, dtype="bf16", alpha=0.3, beta=0.7, w_std=0.05, seed=55)
        helpers.parity(case, cuda_device, kernel=kernel, acc=ko.ACC_F64, expect_kernel=kernel)


def test_relu_bf16_overflow_rounds_to_infinity(cuda_device):
    # relu with a negative slope on a huge negative bf16 value: the product lies between the largest bf16 and
    # infinity, and the reference stores infinity instead of truncating (vml_sve_base.h:97-109)
    m, n, k = 128, 256, 64
    a = np.zeros((m, k), dtype=np.float32)
    b = np.zeros((n, k), dtype=np.float32)
    a[:, 0] = -1.0
    b[:, 0] = 3.3895313892515355e38  # 0x7f7f0000, the largest finite bf16
    desc = kb.make_desc(m, n, k, kb.BF16, act=kb.ACT_RELU, act_alpha=-1.0029296875)
    arrays = {"a": ko.to_storage(a, kb.BF16), "b": ko.to_storage(b, kb.BF16)}
    c = helpers.case_defaults(dict(m=m, n=n, k=k))
    ref_c, _ = helpers.run_oracle(desc, arrays, c)
    assert np.all(ref_c == 0x7f80)
    for kernel in (kb.KERNEL_TC, kb.KERNEL_SIMT):
        got_c, _, used = helpers.run_gpu(desc, arrays, c, cuda_device, kernel=kernel)
        assert used == kernel and np.array_equal(got_c.reshape(m, n), ref_c.reshape(m, n))

# ------------------------------------------------------------------------------------------- golden vectors, host path

def _golden_names():
    return [str(n) for n in np.load(GOLDEN)["names"]]


@pytest.mark.parametrize("name", _golden_names())
@pytest.mark.parametrize("kernel", [kb.KERNEL_AUTO, kb.KERNEL_SIMT])
def test_golden_vectors(cuda_device, name, kernel):
    z = np.load(GOLDEN)
    m, n, k, code, act, res_op, bias_kind = [int(v) for v in z[name + "/meta"]]
    act_alpha, gamma = [float(v) for v in z[name + "/scalars"]]
    bias_strides = {0: (0, 0), 1: (0, 1), 2: (1, 0), 3: (0, 0), 4: (n, 1)}[bias_kind]
    desc = kb.make_desc(m, n, k, code, has_bias=bias_kind != 0, bias_strides=bias_strides, act=act, act_alpha=act_alpha,
                        res_op=res_op)
    arrays = {"a": z[name + "/a"], "b": z[name + "/b"]}
    if bias_kind:
        arrays["bias"] = z[name + "/bias"]
    if res_op:
        arrays["res"] = z[name + "/res"]
    c = helpers.case_defaults(dict(m=m, n=n, k=k, res_op=res_op, gamma=gamma))
    got_c, got_o, _ = helpers.run_gpu(desc, arrays, c, cuda_device, kernel=kernel)
    helpers.compare(got_c.reshape(m, n), z[name + "/c"], code)
    if res_op:
        helpers.compare(got_o.reshape(m, n), z[name + "/out"], code)


@pytest.mark.parametrize("dtype,m,n,k", [("f32", 128, 1024, 1024), ("bf16", 256, 512, 512), ("bf16", 4, 512, 1024),
                                          ("f16", 33, 47, 20), ("bf16", 1500, 520, 264), ("f32", 1100, 300, 72)])
@pytest.mark.parametrize("prepack", [False, True])
def test_host_pointer_path(cuda_device, dtype, m, n, k, prepack):
    case = dict(m=m, n=n, k=k, dtype=dtype, bias="row", act=kb.ACT_RELU, act_alpha=0.0, res_op=kb.RES_IDENTICAL,
                w_std=0.05, seed=51)
    helpers.parity(case, cuda_device, acc=ko.ACC_F64, prepack=prepack, host=True)


@pytest.mark.parametrize("dtype,b_layout", [("bf16", "AB"), ("bf16", "BA"), ("f32", "AB"), ("f32", "BA")])
@pytest.mark.parametrize("m", [2, 200])
def test_prepacked_weights_on_device(cuda_device, dtype, b_layout, m):
    case = dict(m=m, n=300, k=264, dtype=dtype, bias="row", b_layout=b_layout, w_std=0.05, seed=52)
    helpers.parity(case, cuda_device, acc=ko.ACC_F64, prepack=True)


# ------------------------------------------------------------------------------------------- benchmark configurations

def _device_inputs(m, n, k, dtype, device, seed, x_dist="normal", bias_std=0.02, res=False):
    g = torch.Generator(device=device).manual_seed(seed)
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[dtype]
    if x_dist == "normal":
        x = torch.randn(m, k, generator=g, device=device, dtype=torch.float32).to(tdt)
    else:
        x = (torch.rand(m, k, generator=g, device=device, dtype=torch.float32) * 2 - 1).to(tdt)
    w = (torch.randn(n, k, generator=g, device=device, dtype=torch.float32) * 0.02).to(tdt)
    bias = (torch.randn(n, generator=g, device=device, dtype=torch.float32) * bias_std).to(tdt)
    r = torch.randn(m, n, generator=g, device=device, dtype=torch.float32).to(tdt) if res else None
    return x, w, bias, r


def _np_storage(t):
    if t.dtype == torch.float32:
        return t.cpu().numpy()
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _check_rows(desc, x, w, bias, res, got_c, got_o, rows, gamma=1.0):
    """Oracle on a sample of rows of the problem described by desc."""
    d = kb.LinearDesc.from_buffer_copy(bytes(desc))
    d.m = len(rows)
    idx = torch.as_tensor(rows, device=x.device)
    a_s = _np_storage(x.index_select(0, idx))
    r_s = _np_storage(res.index_select(0, idx)) if res is not None else None
    c_ref = np.zeros((len(rows), d.n), dtype=ko.np_dtype(d.c_dtype))
    o_ref = np.zeros((len(rows), d.n), dtype=ko.np_dtype(d.out_dtype)) if res is not None else None
    ko.linear(helpers.oracle_desc(d), a_s, _np_storage(w), c_ref, _np_storage(bias) if bias is not None else None, r_s,
              o_ref, gamma=gamma)
    info = {}
    if got_c is not None:
        info["c"] = helpers.compare(_np_storage(got_c.index_select(0, idx)), c_ref, d.c_dtype)
    if got_o is not None:
        info["out"] = helpers.compare(_np_storage(got_o.index_select(0, idx)), o_ref, d.out_dtype)
    return info


def _sample_rows(m, count, seed):
    rng = np.random.default_rng(seed)
    rows = set(rng.integers(0, m, count).tolist()) | {0, m - 1}
    if m > 128:
        rows |= {127, 128}
    return sorted(rows)


def test_config1_fp32_relu_full(cuda_device):
    case = dict(m=128, n=1024, k=1024, dtype="f32", bias="row", act=kb.ACT_RELU, act_alpha=0.0, x_dist="uniform",
                w_std=0.02, seed=0)
    info = helpers.parity(case, cuda_device, acc=ko.ACC_F64, expect_kernel=kb.KERNEL_TC)
    print("config 1 vs fp64 oracle:", info["c"])


def test_config2_bf16_silu_full(cuda_device):
    m, n, k = 4096, 11008, 4096
    x, w, _, _ = _device_inputs(m, n, k, "bf16", cuda_device, 0)
    bias = torch.zeros(n, dtype=torch.bfloat16, device=cuda_device)
    y = torch.empty(m, n, dtype=torch.bfloat16, device=cuda_device)
    desc = kb.make_desc(m, n, k, kb.BF16, has_bias=True, act=kb.ACT_SWISH)
    lin = kb.Linear(desc)
    lin.run(x, w, y, bias, stream=torch.cuda.current_stream().cuda_stream)
    lin.check(stream=torch.cuda.current_stream().cuda_stream)
    assert lin.last_kernel == kb.KERNEL_TC
    info = _check_rows(desc, x, w, bias, None, y, None, _sample_rows(m, 96, 1))
    print("config 2:", info["c"])
    assert info["c"]["bit_exact_fraction"] > 0.98


def test_config3_fp16_gelu_residual_full(cuda_device):
    m, n, k = 8192, 4096, 4096
    x, w, bias, res = _device_inputs(m, n, k, "f16", cuda_device, 0, res=True)
    out = torch.empty(m, n, dtype=torch.float16, device=cuda_device)
    desc = kb.make_desc(m, n, k, kb.F16, has_bias=True, act=kb.ACT_GELU_TANH, res_op=kb.RES_IDENTICAL)
    lin = kb.Linear(desc)
    lin.run(x, w, None, bias, res, out, stream=torch.cuda.current_stream().cuda_stream)
    lin.check(stream=torch.cuda.current_stream().cuda_stream)
    assert lin.last_kernel == kb.KERNEL_TC
    info = _check_rows(desc, x, w, bias, res, None, out, _sample_rows(m, 96, 2))
    print("config 3:", info["out"])


@pytest.mark.parametrize("m", [1, 4, 16])
def test_config4_decode_gate_full(cuda_device, m):
    n, k = 28672, 8192
    x, w, _, gate = _device_inputs(m, n, k, "bf16", cuda_device, 0, res=True)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=cuda_device)
    desc = kb.make_desc(m, n, k, kb.BF16, res_op=kb.RES_ELTWISE_MUL)
    lin = kb.Linear(desc)
    lin.run(x, w, None, None, gate, out, stream=torch.cuda.current_stream().cuda_stream)
    lin.check(stream=torch.cuda.current_stream().cuda_stream)
    assert lin.last_kernel == (kb.KERNEL_GEMV_FMA if m == 1 else kb.KERNEL_GEMV_MMA)
    info = _check_rows(desc, x, w, None, gate, None, out, list(range(m)))
    print("config 4, m = %d:" % m, info["out"])
    assert info["out"]["bit_exact_fraction"] > 0.98


def test_config5_sharded_rows_full(cuda_device):
    # one GPU's share of the 8-way m-sharded run (4096 rows), plus the shard-equals-whole property on 2 shards
    m_total, n, k = 32768, 28672, 8192
    begin, count = kb.shard_range(m_total, 8, 3, 128)
    assert (begin, count) == (12288, 4096)
    x, w, bias, _ = _device_inputs(count, n, k, "bf16", cuda_device, 0)
    y = torch.empty(count, n, dtype=torch.bfloat16, device=cuda_device)
    desc = kb.make_desc(count, n, k, kb.BF16, has_bias=True, act=kb.ACT_SWISH)
    lin = kb.Linear(desc)
    stream = torch.cuda.current_stream().cuda_stream
    lin.run(x, w, y, bias, stream=stream)
    lin.check(stream=stream)
    assert lin.last_kernel == kb.KERNEL_TC
    _check_rows(desc, x, w, bias, None, y, None, _sample_rows(count, 32, 3))
    # two half-size shards give the same bits as the whole
    half = count // 2
    dh = kb.make_desc(half, n, k, kb.BF16, has_bias=True, act=kb.ACT_SWISH)
    lh = kb.Linear(dh)
    y2 = torch.empty_like(y)
    lh.run(x[:half], w, y2[:half], bias, stream=stream)
    lh.run(x[half:], w, y2[half:], bias, stream=stream)
    lh.check(stream=stream)
    assert torch.equal(y.view(torch.int16), y2.view(torch.int16))


def test_config5_full_size_one_gpu(cuda_device):
    """The whole 32768-row layer on one GPU (2.9 GB of operands): the oracle on sampled rows, among them both sides of
    the first tile boundaries and the last row of the last tile, and the size-independent linearity property."""
    m, n, k = 32768, 28672, 8192
    x, w, bias, _ = _device_inputs(m, n, k, "bf16", cuda_device, 0)
    y = torch.empty(m, n, dtype=torch.bfloat16, device=cuda_device)
    desc = kb.make_desc(m, n, k, kb.BF16, has_bias=True, act=kb.ACT_SWISH)
    lin = kb.Linear(desc)
    stream = torch.cuda.current_stream().cuda_stream
    lin.run(x, w, y, bias, stream=stream)
    lin.check(stream=stream)
    assert lin.last_kernel == kb.KERNEL_TC
    rows = sorted(set(_sample_rows(m, 24, 7)) | {127, 128, 255, 256, 257, m - 256, m - 129, m - 128, m - 1})
    info = _check_rows(desc, x, w, bias, None, y, None, rows)
    print("config 5, 32768 rows on one GPU:", info["c"])
    assert info["c"]["bit_exact_fraction"] > 0.98
    del y
    # no activation, fp32 result: the column sums of x . W^T equal (sum of the rows of x) . W^T
    y32 = torch.empty(m, n, dtype=torch.float32, device=cuda_device)
    lin2 = kb.Linear(kb.make_desc(m, n, k, kb.BF16, c_dtype=kb.F32))
    lin2.run(x, w, y32, stream=stream)
    lin2.check(stream=stream)
    col_sums = y32.sum(dim=0, dtype=torch.float64).cpu().numpy()
    want = w.double().cpu().numpy() @ x.sum(dim=0, dtype=torch.float64).cpu().numpy()
    assert np.max(np.abs(col_sums - want)) <= 2e-5 * np.abs(want).max()


def test_row_sum_property_full_size(cuda_device):
    # linearity over the whole output of a full-size problem: sum_m (x . W^T)[m, :] == (sum_m x[m, :]) . W^T
    m, n, k = 4096, 11008, 4096
    x, w, _, _ = _device_inputs(m, n, k, "bf16", cuda_device, 5)
    y = torch.empty(m, n, dtype=torch.float32, device=cuda_device)
    desc = kb.make_desc(m, n, k, kb.BF16, c_dtype=kb.F32)
    lin = kb.Linear(desc)
    stream = torch.cuda.current_stream().cuda_stream
    lin.run(x, w, y, stream=stream)
    lin.check(stream=stream)
    col_sums = y.double().sum(dim=0).cpu().numpy()
    xs = x.double().sum(dim=0).cpu().numpy()
    want = w.double().cpu().numpy() @ xs
    scale = np.abs(want).max()
    assert np.max(np.abs(col_sums - want)) <= 2e-5 * scale
