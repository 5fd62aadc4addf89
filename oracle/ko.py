"""ctypes front end of the CPU oracle (test infrastructure only).

Only tests/, the smoke check and the CPU-baseline leg of the benchmark may import
this module; the shipped package never does.  Arrays are numpy: float32 for F32,
uint16 bit patterns for F16 / BF16.
"""
import ctypes
import os
import subprocess

import numpy as np

F32, F16, BF16, S32, S8, U8 = 1, 2, 3, 4, 5, 6
ACT_NONE, ACT_RELU, ACT_TANH, ACT_SIGMOID, ACT_GELU_TANH, ACT_SWISH, ACT_GELU_ERF = 0, 5, 9, 10, 20, 25, 27
RES_NONE, RES_EXT, RES_IDENTICAL, RES_ELTWISE_MUL = 0, 1, 2, 3
ACC_F32, ACC_F64 = 0, 1

_HERE = os.path.dirname(os.path.abspath(__file__))


class Desc(ctypes.Structure):
    """Mirror of ko_desc in kudnn_linear_oracle.c."""

    _fields_ = [
        ("m", ctypes.c_int64), ("n", ctypes.c_int64), ("k", ctypes.c_int64),
        ("batch", ctypes.c_int64 * 3),
        ("a_dtype", ctypes.c_int32), ("b_dtype", ctypes.c_int32), ("c_dtype", ctypes.c_int32),
        ("bias_dtype", ctypes.c_int32), ("res_dtype", ctypes.c_int32), ("out_dtype", ctypes.c_int32),
        ("has_bias", ctypes.c_int32), ("act", ctypes.c_int32), ("res_op", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("act_alpha", ctypes.c_float), ("act_beta", ctypes.c_float),
        ("a_sm", ctypes.c_int64), ("a_sk", ctypes.c_int64), ("a_sb", ctypes.c_int64 * 3),
        ("b_sk", ctypes.c_int64), ("b_sn", ctypes.c_int64), ("b_sb", ctypes.c_int64 * 3),
        ("c_sm", ctypes.c_int64), ("c_sn", ctypes.c_int64), ("c_sb", ctypes.c_int64 * 3),
        ("bias_sm", ctypes.c_int64), ("bias_sn", ctypes.c_int64), ("bias_sb", ctypes.c_int64 * 3),
        ("res_sm", ctypes.c_int64), ("res_sn", ctypes.c_int64), ("res_sb", ctypes.c_int64 * 3),
        ("out_sm", ctypes.c_int64), ("out_sn", ctypes.c_int64), ("out_sb", ctypes.c_int64 * 3),
    ]


def build(march=None, out=None, quiet=True):
    """Compile the oracle with gcc (make).  Returns the path of the shared library."""
    cmd = ["make", "-C", _HERE]
    if march:
        cmd.append("KO_MARCH=" + march)
    if out:
        cmd.append("KO_OUT=" + out)
    subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL if quiet else None)
    return out or os.path.join(_HERE, "libkudnn_oracle.so")


_lib_cache = {}


def load(path=None):
    path = path or os.path.join(_HERE, "libkudnn_oracle.so")
    if path in _lib_cache:
        return _lib_cache[path]
    if not os.path.exists(path):
        build()
    lib = ctypes.CDLL(path)
    lib.ko_linear.restype = ctypes.c_int
    lib.ko_linear.argtypes = [ctypes.POINTER(Desc)] + [ctypes.c_void_p] * 6 + [ctypes.c_float] * 3 + [ctypes.c_int] * 2
    lib.ko_num_threads.restype = ctypes.c_int
    lib.ko_activation.restype = ctypes.c_float
    lib.ko_activation.argtypes = [ctypes.c_float, ctypes.c_int, ctypes.c_float]
    lib.ko_linear_int.restype = ctypes.c_int
    lib.ko_linear_int.argtypes = [ctypes.POINTER(Desc)] + [ctypes.c_void_p] * 4 + [ctypes.c_float] * 2
    lib.ko_activation_run.restype = ctypes.c_int
    lib.ko_activation_run.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_int, ctypes.c_float]
    lib.ko_rmsnorm.restype = ctypes.c_int
    lib.ko_rmsnorm.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                                       ctypes.c_int, ctypes.c_float]
    for name in ("ko_convert_f32_to_bf16", "ko_convert_f32_to_f16", "ko_convert_bf16_to_f32", "ko_convert_f16_to_f32"):
        fn = getattr(lib, name)
        fn.restype = None
        fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
    _lib_cache[path] = lib
    return lib


def np_dtype(code):
    return {F32: np.float32, S32: np.int32, S8: np.int8, U8: np.uint8}.get(code, np.uint16)


def to_storage(x_f32, code, lib=None):
    """Round a float32 array to the storage type (RNE) and return its storage array."""
    lib = lib or load()
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    if code == F32:
        return x.copy()
    out = np.empty(x.shape, dtype=np.uint16)
    fn = lib.ko_convert_f32_to_bf16 if code == BF16 else lib.ko_convert_f32_to_f16
    fn(x.ctypes.data, out.ctypes.data, x.size)
    return out


def to_f32(x, code, lib=None):
    lib = lib or load()
    if code == F32:
        return np.asarray(x, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    fn = lib.ko_convert_bf16_to_f32 if code == BF16 else lib.ko_convert_f16_to_f32
    fn(x.ctypes.data, out.ctypes.data, x.size)
    return out


def _ptr(arr):
    return None if arr is None else ctypes.c_void_p(arr.ctypes.data)


def linear(desc, a, b, c=None, bias=None, res=None, out=None, alpha=1.0, beta=0.0, gamma=1.0, acc=ACC_F32,
           num_threads=0, lib=None):
    """Evaluate one Linear(+post-op) on the CPU.  Output arrays are written in place."""
    lib = lib or load()
    if desc.c_dtype == S32:
        rc = lib.ko_linear_int(ctypes.byref(desc), _ptr(a), _ptr(b), _ptr(c), _ptr(bias), alpha, beta)
        if rc != 0:
            raise RuntimeError("ko_linear_int failed with code %d" % rc)
        return
    rc = lib.ko_linear(ctypes.byref(desc), _ptr(a), _ptr(b), _ptr(c), _ptr(bias), _ptr(res), _ptr(out),
                       alpha, beta, gamma, acc, num_threads)
    if rc != 0:
        raise RuntimeError("ko_linear failed with code %d" % rc)


def activation(src, dst, src_dtype, dst_dtype, act, alpha=0.0, lib=None):
    """Stand-alone activation pass on the CPU; dst is written in place."""
    lib = lib or load()
    rc = lib.ko_activation_run(_ptr(src), _ptr(dst), src.size, src_dtype, dst_dtype, act, alpha)
    if rc != 0:
        raise RuntimeError("ko_activation_run failed with code %d" % rc)


def rmsnorm(src, dst, scale, variance, rows, axis, dtype, flags, save_stats, eps, lib=None):
    """RMS normalisation over the last axis on the CPU; dst (and variance when save_stats) are written in place."""
    lib = lib or load()
    rc = lib.ko_rmsnorm(_ptr(src), _ptr(dst), _ptr(scale), _ptr(variance), rows, axis, dtype, flags, 1 if save_stats else 0, eps)
    if rc != 0:
        raise RuntimeError("ko_rmsnorm failed with code %d" % rc)
