"""Failure paths, in forms that leave the GPU healthy: a bounded device-side wait that is made to run out, and a
device allocation that is made to fail on the host.  Nothing here faults, traps or hangs a kernel; the timed-out
launch drains, frees its tensor memory and reports through the handle's status block, and the handle is used again
afterwards.  The reference's error convention these map onto: src/dnn/src/service.cpp:32-46, 418-431."""
import numpy as np
import pytest
import torch

import kudnn_b200 as kb
from oracle import ko
from tests import helpers

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_the_handle_recovers(cuda_device):
    # four 128 x 128 tiles, four k-blocks each, one CTA per tile: the plain launch shape the hook applies to
    case = dict(m=256, n=256, k=256, dtype="bf16", bias="row", act=kb.ACT_SWISH, x_dist="normal", w_std=0.05, seed=71)
    desc, arrays, c = helpers.build_case(case)
    ref_c, _ = helpers.run_oracle(desc, arrays, c)
    d = {k: helpers._to_torch(v, cuda_device) for k, v in arrays.items()}
    y = torch.zeros((256, 256), dtype=torch.int16, device=cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    lin = kb.Linear(desc)
    lin.force_kernel(kb.KERNEL_TC)
    # CTA 0 never loads k-block 2 of its tile; every wait gives up after two million SM cycles (about a millisecond)
    lin.debug_set_wait(2_000_000, 2)
    lin.run(d["a"], d["b"], y, d["bias"], stream=stream)
    with pytest.raises(kb.KudnnError) as err:
        lin.check(stream=stream)
    assert err.value.status == 5 and "gave up" in str(err.value)
    # the status block is clear again, the context and the handle are usable, tensor memory was handed back
    lin.debug_set_wait(0, -1)
    for _ in range(2):
        y.zero_()
        lin.run(d["a"], d["b"], y, d["bias"], stream=stream)
        lin.check(stream=stream)
        helpers.compare(helpers._from_torch(y).reshape(ref_c.shape), ref_c, desc.c_dtype)
    assert lin.last_kernel == kb.KERNEL_TC


def test_device_allocation_failure_is_reported_and_survived(cuda_device):
    case = dict(m=4, n=1000, k=1032, dtype="bf16", bias="row", x_dist="normal", w_std=0.05, seed=72)
    desc, arrays, c = helpers.build_case(case)
    ref_c, _ = helpers.run_oracle(desc, arrays, c)
    d = {k: helpers._to_torch(v, cuda_device) for k, v in arrays.items()}
    y = torch.zeros((4, 1000), dtype=torch.int16, device=cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    lin = kb.Linear(desc)
    try:
        for nth in (0, 1):  # the status block, then the streaming kernel's scratch
            kb.debug_fail_allocation(nth)
            with pytest.raises(kb.KudnnError) as err:
                lin.run(d["a"], d["b"], y, d["bias"], stream=stream)
            assert err.value.status == 3
    finally:
        kb.debug_fail_allocation(-1)
    lin.run(d["a"], d["b"], y, d["bias"], stream=stream)
    lin.check(stream=stream)
    helpers.compare(helpers._from_torch(y).reshape(ref_c.shape), ref_c, desc.c_dtype)


def test_prepacked_weights_follow_an_in_place_update(cuda_device):
    """A packed copy is recognised by the weight pointer alone: after the weights change in place, prepack again (or
    unpack) and the new values are used."""
    case = dict(m=200, n=300, k=264, dtype="bf16", bias="row", b_layout="AB", w_std=0.05, seed=73)
    desc, arrays, c = helpers.build_case(case)
    d = {k: helpers._to_torch(v, cuda_device) for k, v in arrays.items()}
    y = torch.zeros((200, 300), dtype=torch.int16, device=cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    lin = kb.Linear(desc)
    lin.prepack(d["b"], stream=stream)
    lin.run(d["a"], d["b"], y, d["bias"], stream=stream)
    lin.check(stream=stream)
    ref_c, _ = helpers.run_oracle(desc, arrays, c)
    helpers.compare(helpers._from_torch(y).reshape(ref_c.shape), ref_c, desc.c_dtype)
    # new weights at the same address
    arrays2 = dict(arrays)
    arrays2["b"] = helpers.build_case(dict(case, seed=74))[1]["b"]
    d["b"].copy_(helpers._to_torch(arrays2["b"], cuda_device))
    ref2, _ = helpers.run_oracle(desc, arrays2, c)
    lin.prepack(d["b"], stream=stream)
    lin.run(d["a"], d["b"], y, d["bias"], stream=stream)
    lin.check(stream=stream)
    helpers.compare(helpers._from_torch(y).reshape(ref2.shape), ref2, desc.c_dtype)
    # and once more through unpack: the run reads the caller's buffer
    arrays3 = dict(arrays)
    arrays3["b"] = helpers.build_case(dict(case, seed=75))[1]["b"]
    d["b"].copy_(helpers._to_torch(arrays3["b"], cuda_device))
    ref3, _ = helpers.run_oracle(desc, arrays3, c)
    lin.unpack()
    lin.run(d["a"], d["b"], y, d["bias"], stream=stream)
    lin.check(stream=stream)
    helpers.compare(helpers._from_torch(y).reshape(ref3.shape), ref3, desc.c_dtype)
