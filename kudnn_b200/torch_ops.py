"""PyTorch glue over the C ABI: the custom operator ``kudnn_b200::linear`` and a drop-in module for ``nn.Linear``.

The reference reaches PyTorch through a patched build in which ``torch._C._set_kdnn_enabled(True)`` routes
``torch.nn.Linear`` to KuDNN (docs/zh/KuDNN_development_guide.md:1407-1486, 1748-1775).  Here the same dispatch point
is an ordinary ``torch.library`` operator: ``y = act(x . W^T + b) (+) residual`` on CUDA tensors, forward only (the
reference classes are FWD primitives too), with a fake (meta) implementation so that shape propagation, FakeTensor
tracing and ``torch.compile`` graph capture see the right output without touching the GPU.  All arithmetic happens in
libkudnn_b200.so; torch supplies the tensors, the current stream and the output allocation.
"""
import collections
from typing import Optional

import torch

from . import capi

_DTYPES = {torch.float32: capi.F32, torch.float16: capi.F16, torch.bfloat16: capi.BF16}
ACTIVATIONS = {None: capi.ACT_NONE, "none": capi.ACT_NONE, "relu": capi.ACT_RELU, "silu": capi.ACT_SWISH,
               "swish": capi.ACT_SWISH, "gelu_tanh": capi.ACT_GELU_TANH, "gelu": capi.ACT_GELU_ERF,
               "gelu_erf": capi.ACT_GELU_ERF, "sigmoid": capi.ACT_SIGMOID, "tanh": capi.ACT_TANH}
RESIDUALS = {None: capi.RES_NONE, "none": capi.RES_NONE, "add": capi.RES_IDENTICAL, "ext": capi.RES_EXT,
             "mul": capi.RES_ELTWISE_MUL}

# Created primitives, keyed by everything the descriptor holds plus the weight's address (a primitive pre-packs the
# weights it first sees and recognises them by pointer).  Bounded: the oldest handle is destroyed when full.
_HANDLES = collections.OrderedDict()
_MAX_HANDLES = 128


def _handle(m, n, k, x, weight, bias, act, act_alpha, residual, res_op):
    code = _DTYPES[x.dtype]
    key = (x.device.index, m, n, k, code, x.stride(-2) if x.dim() > 1 else k, weight.data_ptr(), weight.stride(0),
           weight.stride(1), weight._version, None if bias is None else _DTYPES[bias.dtype], act, act_alpha, res_op)
    lin = _HANDLES.get(key)
    if lin is not None:
        _HANDLES.move_to_end(key)
        return lin
    desc = capi.make_desc(m, n, k, code, a_strides=(k, 1), b_strides=(weight.stride(1), weight.stride(0)),
                          has_bias=bias is not None, bias_dtype=None if bias is None else _DTYPES[bias.dtype], act=act,
                          act_alpha=act_alpha, res_op=res_op)
    lin = capi.Linear(desc)
    lin.prepack(weight, stream=torch.cuda.current_stream(x.device).cuda_stream)
    _HANDLES[key] = lin
    while len(_HANDLES) > _MAX_HANDLES:
        _, old = _HANDLES.popitem(last=False)
        old.close()
    return lin


def clear_cache():
    """Destroys every cached primitive (and the packed weight copies they own)."""
    while _HANDLES:
        _, lin = _HANDLES.popitem()
        lin.close()


@torch.library.custom_op("kudnn_b200::linear", mutates_args=(), device_types="cuda")
def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, act: int = 0,
           act_alpha: float = 1.0, residual: Optional[torch.Tensor] = None, res_op: int = 0,
           gamma: float = 1.0) -> torch.Tensor:
    """act(x . weight^T + bias), then (+) residual when res_op is given.  x [..., k], weight [n, k] as nn.Linear keeps
    it, bias [n], residual [..., n].  act / res_op are the KUDNN_B200_ACT_* / KUDNN_B200_RES_* codes."""
    if x.dtype not in _DTYPES or weight.dtype != x.dtype:
        raise TypeError("kudnn_b200::linear takes float32 / float16 / bfloat16 tensors of one type")
    if weight.dim() != 2 or x.shape[-1] != weight.shape[1]:
        raise ValueError("kudnn_b200::linear: x [..., k] and weight [n, k] do not match")
    n, k = weight.shape
    x2 = x.reshape(-1, k)
    if x2.stride(-1) != 1 or (x2.shape[0] > 1 and x2.stride(0) != k):
        x2 = x2.contiguous()
    m = x2.shape[0]
    out = torch.empty(x.shape[:-1] + (n,), dtype=x.dtype, device=x.device)
    if m == 0:
        return out
    if bias is not None:
        bias = bias.contiguous()
    res2 = None
    if res_op != capi.RES_NONE:
        if residual is None or residual.shape != out.shape or residual.dtype != x.dtype:
            raise ValueError("kudnn_b200::linear: residual must have the output's shape and type")
        res2 = residual.contiguous()
    with torch.cuda.device(x.device):
        lin = _handle(m, n, k, x2, weight, bias, act, act_alpha, res2, res_op)
        stream = torch.cuda.current_stream(x.device).cuda_stream
        if res_op != capi.RES_NONE:
            lin.run(x2, weight, None, bias, res2, out, gamma=gamma, stream=stream)
        else:
            lin.run(x2, weight, out, bias, stream=stream)
    return out


@linear.register_fake
def _linear_fake(x, weight, bias=None, act=0, act_alpha=1.0, residual=None, res_op=0, gamma=1.0):
    return x.new_empty(x.shape[:-1] + (weight.shape[0],))


class Linear(torch.nn.Module):
    """``nn.Linear`` whose forward pass (inference) runs through ``kudnn_b200::linear``, optionally fused with an
    activation and a residual operand:  ``Linear.from_torch(layer, act="silu")(x)`` or ``(x, residual)``."""

    def __init__(self, in_features, out_features, bias=True, act=None, act_alpha=1.0, residual=None, gamma=1.0,
                 device=None, dtype=None):
        super().__init__()
        self.inner = torch.nn.Linear(in_features, out_features, bias=bias, device=device, dtype=dtype)
        self.act, self.act_alpha = ACTIVATIONS[act], float(act_alpha)
        self.res_op, self.gamma = RESIDUALS[residual], float(gamma)

    @classmethod
    def from_torch(cls, layer, act=None, act_alpha=1.0, residual=None, gamma=1.0):
        mod = cls.__new__(cls)
        torch.nn.Module.__init__(mod)
        mod.inner = layer
        mod.act, mod.act_alpha = ACTIVATIONS[act], float(act_alpha)
        mod.res_op, mod.gamma = RESIDUALS[residual], float(gamma)
        return mod

    def forward(self, x, residual=None):
        return torch.ops.kudnn_b200.linear(x, self.inner.weight, self.inner.bias, self.act, self.act_alpha, residual,
                                           self.res_op, self.gamma)
