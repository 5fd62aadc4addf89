"""The torch.library operator kudnn_b200::linear and the nn.Linear drop-in module (kudnn_b200/torch_ops.py): the
documented PyTorch integration point of the reference (docs/zh/KuDNN_development_guide.md:1748-1775) on this side."""
import numpy as np
import pytest
import torch

import kudnn_b200 as kb
from kudnn_b200 import torch_ops
from oracle import ko
from tests import helpers


def test_fake_implementation_propagates_shapes_without_a_device():
    x = torch.empty(3, 7, 64, dtype=torch.bfloat16, device="meta")
    w = torch.empty(96, 64, dtype=torch.bfloat16, device="meta")
    b = torch.empty(96, dtype=torch.bfloat16, device="meta")
    y = torch.ops.kudnn_b200.linear(x, w, b, kb.ACT_SWISH)
    assert y.shape == (3, 7, 96) and y.dtype == torch.bfloat16 and y.device.type == "meta"
    r = torch.empty(3, 7, 96, dtype=torch.bfloat16, device="meta")
    assert torch.ops.kudnn_b200.linear(x, w, None, 0, 1.0, r, kb.RES_IDENTICAL).shape == (3, 7, 96)


def _oracle(x, w, b, act, res, res_op):
    code = {torch.float32: kb.F32, torch.float16: kb.F16, torch.bfloat16: kb.BF16}[x.dtype]
    m, k = x.reshape(-1, x.shape[-1]).shape
    n = w.shape[0]
    desc = kb.make_desc(m, n, k, code, has_bias=b is not None, act=act, res_op=res_op)

    def st(t):
        t = t.detach().cpu().contiguous()
        return t.numpy() if t.dtype == torch.float32 else t.view(torch.int16).numpy().view(np.uint16)
    c = np.zeros((m, n), dtype=ko.np_dtype(code))
    o = np.zeros((m, n), dtype=ko.np_dtype(code)) if res_op else None
    ko.linear(helpers.oracle_desc(desc), st(x.reshape(m, k)), st(w), c, st(b) if b is not None else None,
              st(res.reshape(m, n)) if res is not None else None, o)
    return (o if res_op else c), code, st


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_linear_silu_module_matches_the_oracle(cuda_device, dtype):
    torch.manual_seed(5)
    layer = torch.nn.Linear(512, 1024, bias=True, device=cuda_device, dtype=dtype)
    with torch.no_grad():
        layer.weight.mul_(0.5)
    mod = torch_ops.Linear.from_torch(layer, act="silu")
    x = torch.randn(4, 50, 512, device=cuda_device, dtype=dtype)
    with torch.no_grad():
        y = mod(x)
    assert y.shape == (4, 50, 1024)
    ref, code, st = _oracle(x, layer.weight, layer.bias, kb.ACT_SWISH, None, kb.RES_NONE)
    helpers.compare(st(y.reshape(200, 1024)), ref, code)
    # decode shape with a gate operand, and weights updated in place (a fresh primitive packs the new values)
    gate = torch.randn(2, 1024, device=cuda_device, dtype=dtype)
    mul = torch_ops.Linear.from_torch(layer, residual="mul")
    with torch.no_grad():
        layer.weight.add_(0.01)
        y2 = mul(x[0, :2], gate)
    ref2, code, st = _oracle(x[0, :2], layer.weight, layer.bias, kb.ACT_NONE, gate, kb.RES_ELTWISE_MUL)
    helpers.compare(st(y2), ref2, code)
    torch_ops.clear_cache()


@pytest.mark.gpu
def test_operator_passes_opcheck(cuda_device):
    x = torch.randn(6, 64, device=cuda_device, dtype=torch.bfloat16)
    w = torch.randn(48, 64, device=cuda_device, dtype=torch.bfloat16)
    b = torch.randn(48, device=cuda_device, dtype=torch.bfloat16)
    torch.library.opcheck(torch.ops.kudnn_b200.linear.default, (x, w, b, kb.ACT_RELU, 0.0),
                          test_utils=("test_schema", "test_faketensor"))
    torch_ops.clear_cache()
