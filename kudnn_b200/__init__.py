"""kudnn_b200: B200 (sm_100a) Linear(+post-op) kernels behind the KuDNN Linear API.

The product is the CUDA library ``libkudnn_b200.so`` (C ABI, ``include/kudnn_b200.h``) and the C++ classes of the
reference API on top of it (``kudnn_b200/host``).  This Python package is a thin ctypes front end used by the tests
and the benchmark; it adds no compute of its own and has no CPU fallback: if the CUDA library is missing or no
sm_100 device is present, calls fail with an error.
"""
from .capi import (  # noqa: F401
    ACT_GELU_ERF, ACT_GELU_TANH, ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_SWISH, ACT_TANH,
    BF16, F16, F32, S32, S8, U8,
    KERNEL_AUTO, KERNEL_GEMV_FMA, KERNEL_GEMV_MMA, KERNEL_SIMT, KERNEL_TC, KERNEL_NAMES,
    RES_ELTWISE_MUL, RES_EXT, RES_IDENTICAL, RES_NONE,
    KudnnError, Linear, LinearDesc, activation, debug_fail_allocation, library, library_path, make_desc, run_static_scratch, shard_range,
    peer_buffer_close, peer_buffer_create, peer_buffer_destroy, peer_buffer_open, rmsnorm,
    NORM_USE_GLOBAL_STATS, NORM_USE_SCALE, SHARD_COLS, SHARD_ROWS,
)

__all__ = [
    "ACT_GELU_ERF", "ACT_GELU_TANH", "ACT_NONE", "ACT_RELU", "ACT_SIGMOID", "ACT_SWISH", "ACT_TANH",
    "BF16", "F16", "F32", "S32", "S8", "U8",
    "KERNEL_AUTO", "KERNEL_GEMV_FMA", "KERNEL_GEMV_MMA", "KERNEL_SIMT", "KERNEL_TC", "KERNEL_NAMES",
    "RES_ELTWISE_MUL", "RES_EXT", "RES_IDENTICAL", "RES_NONE",
    "KudnnError", "Linear", "LinearDesc", "activation", "debug_fail_allocation", "library", "library_path", "make_desc", "run_static_scratch", "shard_range",
    "peer_buffer_close", "peer_buffer_create", "peer_buffer_destroy", "peer_buffer_open", "rmsnorm",
    "NORM_USE_GLOBAL_STATS", "NORM_USE_SCALE", "SHARD_COLS", "SHARD_ROWS",
]
