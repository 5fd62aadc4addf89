"""kudnn_b200_linear_run_sharded: one process drives several GPUs (or, on a one-GPU box, several shards on the same
device: the split, the staging and the strided copies are the same), host pointers in and out, against the oracle."""
import numpy as np
import pytest

import kudnn_b200 as kb
from oracle import ko
from tests import helpers

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [kb.SHARD_ROWS, kb.SHARD_COLS])
@pytest.mark.parametrize("nshards", [1, 2, 3, 8])
@pytest.mark.parametrize("dtype,b_layout", [("bf16", "BA"), ("f16", "AB"), ("f32", "BA")])
def test_sharded_run_matches_the_oracle(cuda_device, mode, nshards, dtype, b_layout):
    case = dict(m=700, n=520, k=264, dtype=dtype, bias="row", act=kb.ACT_SWISH, res_op=kb.RES_IDENTICAL, b_layout=b_layout,
                x_dist="normal", w_std=0.05, seed=81)
    desc, arrays, c = helpers.build_case(case)
    ref_c, ref_o = helpers.run_oracle(desc, arrays, c, acc=ko.ACC_F64)
    lin = kb.Linear(desc)
    for _ in range(2):  # the second call finds the children and their packed weights
        out_c = np.zeros((700, 520), dtype=ko.np_dtype(desc.c_dtype))
        out_o = np.zeros((700, 520), dtype=ko.np_dtype(desc.out_dtype))
        lin.run_sharded(arrays["a"], arrays["b"], out_c, arrays["bias"], arrays["res"], out_o, nshards=nshards, mode=mode)
        helpers.compare(out_c.reshape(ref_c.shape), ref_c, desc.c_dtype)
        helpers.compare(out_o.reshape(ref_o.shape), ref_o, desc.out_dtype)
    lin.close()


def test_sharded_run_decode_shape_by_columns(cuda_device):
    # a decode-shaped layer split by columns: every shard streams its slab of the weights
    case = dict(m=4, n=4096, k=1024, dtype="bf16", res_op=kb.RES_ELTWISE_MUL, x_dist="normal", w_std=0.03, seed=82)
    desc, arrays, c = helpers.build_case(case)
    _, ref_o = helpers.run_oracle(desc, arrays, c)
    lin = kb.Linear(desc)
    out_o = np.zeros((4, 4096), dtype=np.uint16)
    lin.run_sharded(arrays["a"], arrays["b"], None, None, arrays["res"], out_o, nshards=4, mode=kb.SHARD_COLS)
    helpers.compare(out_o.reshape(ref_o.shape), ref_o, desc.out_dtype)
    assert lin.last_kernel in (kb.KERNEL_GEMV_FMA, kb.KERNEL_GEMV_MMA)
    lin.close()


def test_sharded_run_refuses_what_it_cannot_split(cuda_device):
    import torch
    desc = kb.make_desc(256, 256, 64, kb.BF16)
    lin = kb.Linear(desc)
    x = torch.zeros(256, 64, dtype=torch.bfloat16, device=cuda_device)
    w = torch.zeros(256, 64, dtype=torch.bfloat16, device=cuda_device)
    y = torch.zeros(256, 256, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(kb.KudnnError) as e:
        lin.run_sharded(x, w, y, nshards=2)  # device pointers
    assert e.value.status == 1
    with pytest.raises(kb.KudnnError) as e:
        lin.run_sharded(np.zeros((256, 64), np.uint16), np.zeros((256, 64), np.uint16), np.zeros((256, 256), np.uint16), nshards=0)
    assert e.value.status == 2
    lin.close()
