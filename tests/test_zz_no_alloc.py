"""The entry point that allocates no device memory (kudnn_b200_linear_run_static_scratch).

It serves callers that cannot call cudaMalloc at the moment they need a decode-shaped Linear: engines that gave all
of HBM to their own pools at start-up, and plug-ins whose host forbids allocation inside an operator call.  Its
split-K scratch is one fixed array per device that every call shares and that keeps the previous call's contents,
so the checks that matter are that two calls in a row, on problems of different sizes, each reproduce what the
regular (allocating) entry point and the CPU oracle compute, and that a call, once its kernel variant has been
loaded, leaves the amount of free device memory unchanged.  This file sorts last on purpose: when a run stops at
the first failure, every other test has already run.
"""
import numpy as np
import pytest
import torch

import kudnn_b200 as kb
from tests import helpers

pytestmark = pytest.mark.gpu


def _both_ways(case, device):
    desc, arrays, c = helpers.build_case(case)
    d = {k: helpers._to_torch(v, device) for k, v in arrays.items()}
    stream = torch.cuda.current_stream().cuda_stream
    m, n = desc.m, desc.n
    has_res = c["res_op"] != kb.RES_NONE

    def outputs():
        t_c = torch.zeros((m, n), dtype=torch.int16, device=device)
        t_o = torch.zeros((m, n), dtype=torch.int16, device=device) if has_res else None
        return t_c, t_o

    ref_c, ref_o = outputs()
    lin = kb.Linear(desc)
    lin.run(d["a"], d["b"], ref_c, d.get("bias"), d.get("res"), ref_o, stream=stream)
    lin.check(stream=stream)
    assert lin.last_kernel in (kb.KERNEL_GEMV_FMA, kb.KERNEL_GEMV_MMA)
    got_c, got_o = outputs()
    kb.run_static_scratch(desc, d["a"], d["b"], got_c, d.get("bias"), d.get("res"), got_o, stream=stream)
    torch.cuda.synchronize()
    helpers.compare(helpers._from_torch(got_c), helpers._from_torch(ref_c), desc.c_dtype)
    if has_res:
        helpers.compare(helpers._from_torch(got_o), helpers._from_torch(ref_o), desc.out_dtype)
    # and against the CPU oracle, not only against the library's other entry point
    ora_c, ora_o = helpers.run_oracle(desc, arrays, c)
    helpers.compare(helpers._from_torch(got_c).reshape(ora_c.shape), ora_c, desc.c_dtype)
    if has_res:
        helpers.compare(helpers._from_torch(got_o).reshape(ora_o.shape), ora_o, desc.out_dtype)


def test_two_calls_in_a_row_match_the_allocating_entry_point(cuda_device):
    # the second problem is smaller and cut differently, so it lands on scratch the first call has written
    first = dict(m=16, n=3000, k=4096, dtype="bf16", res_op=kb.RES_ELTWISE_MUL, x_dist="normal", w_std=0.02, seed=61)
    second = dict(m=3, n=1003, k=1048, dtype="f16", bias="row", act=kb.ACT_SWISH, x_dist="normal", w_std=0.05, seed=62)
    _both_ways(first, cuda_device)
    _both_ways(second, cuda_device)
    _both_ways(first, cuda_device)


def test_later_calls_take_no_device_memory(cuda_device):
    """What the entry point exists for.  The first call on a device creates the scratch array and loads the kernel
    variant it launches (the CUDA runtime loads device code lazily), which takes memory from the driver once; every
    later call of that variant must leave the free device memory exactly as it found it."""
    case = dict(m=16, n=3000, k=4096, dtype="bf16", res_op=kb.RES_ELTWISE_MUL, x_dist="normal", w_std=0.02, seed=64)
    desc, arrays, c = helpers.build_case(case)
    d = {k: helpers._to_torch(v, cuda_device) for k, v in arrays.items()}
    smaller = kb.make_desc(16, 2000, 4096, kb.BF16, res_op=kb.RES_ELTWISE_MUL)  # same variant, cut differently
    out = torch.zeros((16, 3000), dtype=torch.int16, device=cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    kb.run_static_scratch(desc, d["a"], d["b"], None, None, d["res"], out, stream=stream)  # warm-up: loads the variant
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for i in range(6):
        kb.run_static_scratch(desc if i % 2 == 0 else smaller, d["a"], d["b"], None, None, d["res"], out, stream=stream)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    kb.run_static_scratch(desc, d["a"], d["b"], None, None, d["res"], out, stream=stream)
    torch.cuda.synchronize()
    _, ref_o = helpers.run_oracle(desc, arrays, c)
    helpers.compare(helpers._from_torch(out).reshape(ref_o.shape), ref_o, desc.out_dtype)


def test_single_row_fp32(cuda_device):
    desc, arrays, c = helpers.build_case(dict(m=1, n=777, k=2504, dtype="f32", bias="row", w_std=0.05, seed=63))
    d = {k: helpers._to_torch(v, cuda_device) for k, v in arrays.items()}
    stream = torch.cuda.current_stream().cuda_stream
    ref = torch.zeros((1, 777), dtype=torch.float32, device=cuda_device)
    got = torch.zeros_like(ref)
    lin = kb.Linear(desc)
    lin.run(d["a"], d["b"], ref, d["bias"], stream=stream)
    kb.run_static_scratch(desc, d["a"], d["b"], got, d["bias"], stream=stream)
    torch.cuda.synchronize()
    helpers.compare(got.cpu().numpy(), ref.cpu().numpy(), desc.c_dtype)


def test_oversized_and_unsuitable_problems_are_refused(cuda_device):
    x = torch.zeros(16, 8192, dtype=torch.bfloat16, device=cuda_device)
    w = torch.zeros(8, dtype=torch.bfloat16, device=cuda_device)  # never read: the call must fail before any launch
    y = torch.zeros(8, dtype=torch.bfloat16, device=cuda_device)
    too_big = kb.make_desc(16, 200000, 8192, kb.BF16)
    with pytest.raises(kb.KudnnError) as e:
        kb.run_static_scratch(too_big, x, w, y)
    assert e.value.status == 1 and "scratch" in str(e.value)
    prefill = kb.make_desc(128, 256, 256, kb.BF16)
    with pytest.raises(kb.KudnnError) as e:
        kb.run_static_scratch(prefill, x, w, y)
    assert e.value.status == 1
    with pytest.raises(kb.KudnnError) as e:
        kb.run_static_scratch(kb.make_desc(4, 256, 256, kb.BF16), None, w, y)
    assert e.value.status == 2
