"""ctypes binding of include/kudnn_b200.h.

Pointers are passed as integers (``tensor.data_ptr()`` of a torch tensor, ``array.ctypes.data`` of a numpy array):
this module never touches the data itself.
"""
import ctypes
import os

F32, F16, BF16, S32, S8, U8 = 1, 2, 3, 4, 5, 6
ACT_NONE, ACT_RELU, ACT_TANH, ACT_SIGMOID, ACT_GELU_TANH, ACT_SWISH, ACT_GELU_ERF = 0, 5, 9, 10, 20, 25, 27
RES_NONE, RES_EXT, RES_IDENTICAL, RES_ELTWISE_MUL = 0, 1, 2, 3
KERNEL_AUTO, KERNEL_SIMT, KERNEL_GEMV_FMA, KERNEL_GEMV_MMA, KERNEL_TC = 0, 1, 2, 3, 4
KERNEL_NAMES = {0: "auto", 1: "simt", 2: "gemv_fma", 3: "gemv_mma", 4: "tc"}

SHARD_ROWS, SHARD_COLS = 0, 1

STATUS_NAMES = {0: "OK", 1: "UNSUPPORTED", 2: "BAD_ARGUMENTS", 3: "ALLOC_FAILED", 4: "CUDA_ERROR", 5: "TIMEOUT",
                6: "NO_DEVICE"}

_PKG = os.path.dirname(os.path.abspath(__file__))


class KudnnError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("kudnn_b200 status %d (%s): %s" % (status, STATUS_NAMES.get(status, "?"), message))
        self.status = status


class LinearDesc(ctypes.Structure):
    """kudnn_b200_linear_desc."""

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


class LinearArgs(ctypes.Structure):
    """kudnn_b200_linear_args."""

    _fields_ = [
        ("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("c", ctypes.c_void_p), ("bias", ctypes.c_void_p),
        ("res", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("alpha", ctypes.c_float), ("beta", ctypes.c_float), ("gamma", ctypes.c_float),
    ]


EXPORTS = [
    "kudnn_b200_linear_validate", "kudnn_b200_linear_create", "kudnn_b200_linear_clone", "kudnn_b200_linear_destroy",
    "kudnn_b200_linear_prepack", "kudnn_b200_linear_run", "kudnn_b200_linear_run_host", "kudnn_b200_linear_check",
    "kudnn_b200_linear_run_static_scratch", "kudnn_b200_linear_run_any",
    "kudnn_b200_linear_force_kernel", "kudnn_b200_linear_last_kernel", "kudnn_b200_linear_last_launches",
    "kudnn_b200_linear_workspace_bytes", "kudnn_b200_shard_range", "kudnn_b200_last_error", "kudnn_b200_version",
    "kudnn_b200_device_count", "kudnn_b200_linear_set_mirrors", "kudnn_b200_peer_buffer_create",
    "kudnn_b200_peer_buffer_open", "kudnn_b200_peer_buffer_close", "kudnn_b200_peer_buffer_destroy",
    "kudnn_b200_linear_unpack", "kudnn_b200_debug_set_wait", "kudnn_b200_debug_fail_allocation",
    "kudnn_b200_linear_run_sharded", "kudnn_b200_activation_validate", "kudnn_b200_activation_run", "kudnn_b200_rmsnorm_validate", "kudnn_b200_rmsnorm_run",
    "kudnn_b200_linear_set_multicast",
]

_lib = None


def library_path():
    return os.path.join(_PKG, "libkudnn_b200.so")


def library():
    """Loads libkudnn_b200.so; raises if it has not been built (there is no fallback path)."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise KudnnError(6, "%s is missing: build it with `python -m kudnn_b200.build` "
                            "(or __graft_entry__.build())" % path)
    lib = ctypes.CDLL(path)
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    lib.kudnn_b200_linear_validate.argtypes = [ctypes.POINTER(LinearDesc)]
    lib.kudnn_b200_linear_create.argtypes = [ctypes.POINTER(LinearDesc), ctypes.POINTER(vp)]
    lib.kudnn_b200_linear_clone.argtypes = [vp, ctypes.POINTER(vp)]
    lib.kudnn_b200_linear_destroy.argtypes = [vp]
    lib.kudnn_b200_linear_prepack.argtypes = [vp, vp, vp]
    lib.kudnn_b200_linear_run.argtypes = [vp, ctypes.POINTER(LinearArgs), vp]
    lib.kudnn_b200_linear_run_host.argtypes = [vp, ctypes.POINTER(LinearArgs)]
    lib.kudnn_b200_linear_check.argtypes = [vp, vp]
    lib.kudnn_b200_linear_run_any.argtypes = [vp, ctypes.POINTER(LinearArgs), vp]
    lib.kudnn_b200_linear_run_static_scratch.argtypes = [ctypes.POINTER(LinearDesc), ctypes.POINTER(LinearArgs), vp]
    lib.kudnn_b200_linear_set_mirrors.argtypes = [vp, i32, ctypes.POINTER(vp), ctypes.POINTER(vp)]
    lib.kudnn_b200_linear_set_multicast.argtypes = [vp, vp, vp]
    lib.kudnn_b200_peer_buffer_create.argtypes = [ctypes.c_size_t, ctypes.POINTER(vp), ctypes.c_char_p]
    lib.kudnn_b200_peer_buffer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    lib.kudnn_b200_peer_buffer_close.argtypes = [vp]
    lib.kudnn_b200_peer_buffer_destroy.argtypes = [vp]
    lib.kudnn_b200_activation_validate.argtypes = [i64, i32, i32, i32]
    lib.kudnn_b200_activation_run.argtypes = [vp, vp, i64, i32, i32, i32, ctypes.c_float, vp]
    lib.kudnn_b200_rmsnorm_validate.argtypes = [i64, i64, i32, i32]
    lib.kudnn_b200_rmsnorm_run.argtypes = [vp, vp, vp, vp, i64, i64, i32, i32, i32, ctypes.c_float, vp]
    lib.kudnn_b200_linear_run_sharded.argtypes = [vp, ctypes.POINTER(LinearArgs), i32, i32]
    lib.kudnn_b200_linear_unpack.argtypes = [vp]
    lib.kudnn_b200_debug_set_wait.argtypes = [vp, ctypes.c_longlong, i32]
    lib.kudnn_b200_debug_fail_allocation.argtypes = [i32]
    lib.kudnn_b200_linear_force_kernel.argtypes = [vp, i32]
    lib.kudnn_b200_linear_last_kernel.argtypes = [vp]
    lib.kudnn_b200_linear_last_launches.argtypes = [vp]
    lib.kudnn_b200_linear_workspace_bytes.argtypes = [vp]
    lib.kudnn_b200_linear_workspace_bytes.restype = i64
    lib.kudnn_b200_shard_range.argtypes = [i64, i32, i32, i64, ctypes.POINTER(i64), ctypes.POINTER(i64)]
    lib.kudnn_b200_last_error.restype = ctypes.c_char_p
    lib.kudnn_b200_version.restype = ctypes.c_char_p
    _lib = lib
    return lib


def _check(status):
    if status != 0:
        raise KudnnError(status, library().kudnn_b200_last_error().decode("utf-8", "replace"))


def make_desc(m, n, k, dtype, *, a_strides=None, b_strides=None, c_strides=None, has_bias=False, bias_strides=None,
              bias_dtype=None, c_dtype=None, b_dtype=None, act=ACT_NONE, act_alpha=1.0, act_beta=0.0, res_op=RES_NONE,
              res_strides=None, out_strides=None, res_dtype=None, out_dtype=None, batch=(0, 0, 0), a_sb=(0, 0, 0),
              b_sb=(0, 0, 0), c_sb=(0, 0, 0), bias_sb=(0, 0, 0), res_sb=(0, 0, 0), out_sb=(0, 0, 0)):
    """Descriptor for c[m,n] = act(a[m,k] . b[k,n] + bias), out = c (+) res.

    Strides are (row, column) element strides of the logical matrices: a_strides = (a_sm, a_sk), b_strides =
    (b_sk, b_sn).  Defaults: a, c, res, out row-major; b stored as W[n, k] with k contiguous (b_sk = 1, b_sn = k), the
    layout the reference calls Layout::BA; bias a row vector [n].
    """
    d = LinearDesc()
    d.m, d.n, d.k = m, n, k
    d.batch[:] = batch
    d.a_dtype = dtype
    d.b_dtype = b_dtype or dtype
    d.c_dtype = c_dtype or dtype
    d.bias_dtype = bias_dtype or dtype
    d.res_dtype = res_dtype or (c_dtype or dtype)
    d.out_dtype = out_dtype or (c_dtype or dtype)
    d.has_bias = 1 if has_bias else 0
    d.act, d.res_op = act, res_op
    d.act_alpha, d.act_beta = act_alpha, act_beta
    d.a_sm, d.a_sk = a_strides or (k, 1)
    d.b_sk, d.b_sn = b_strides or (1, k)
    d.c_sm, d.c_sn = c_strides or (n, 1)
    d.bias_sm, d.bias_sn = bias_strides or (0, 1)
    d.res_sm, d.res_sn = res_strides or (n, 1)
    d.out_sm, d.out_sn = out_strides or (n, 1)
    d.a_sb[:] = a_sb
    d.b_sb[:] = b_sb
    d.c_sb[:] = c_sb
    d.bias_sb[:] = bias_sb
    d.res_sb[:] = res_sb
    d.out_sb[:] = out_sb
    return d


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    raise TypeError("expected an address, a torch tensor or a numpy array")


def validate(desc):
    return library().kudnn_b200_linear_validate(ctypes.byref(desc))


def shard_range(total, nparts, part, align=1):
    b, c = ctypes.c_int64(), ctypes.c_int64()
    _check(library().kudnn_b200_shard_range(total, nparts, part, align, ctypes.byref(b), ctypes.byref(c)))
    return b.value, c.value


PEER_HANDLE_BYTES = 64


def peer_buffer_create(nbytes):
    """A device buffer other processes on this machine can map.  Returns (device pointer, 64-byte handle)."""
    ptr = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(PEER_HANDLE_BYTES)
    _check(library().kudnn_b200_peer_buffer_create(nbytes, ctypes.byref(ptr), handle))
    return ptr.value, handle.raw


def peer_buffer_open(handle):
    """Maps a buffer another process created with peer_buffer_create; returns its device pointer in this process."""
    ptr = ctypes.c_void_p()
    _check(library().kudnn_b200_peer_buffer_open(bytes(handle), ctypes.byref(ptr)))
    return ptr.value


def peer_buffer_close(ptr):
    _check(library().kudnn_b200_peer_buffer_close(ptr))


def peer_buffer_destroy(ptr):
    _check(library().kudnn_b200_peer_buffer_destroy(ptr))


NORM_USE_GLOBAL_STATS, NORM_USE_SCALE, NORM_USE_SHIFT, NORM_FUSE_RELU = 1, 2, 4, 8


def activation(src, dst, count, src_dtype, dst_dtype, act, alpha=0.0, stream=None):
    """Stand-alone activation pass; src and dst both device (asynchronous on `stream`) or both host memory."""
    _check(library().kudnn_b200_activation_run(_ptr(src), _ptr(dst), count, src_dtype, dst_dtype, act, alpha, stream))


def rmsnorm(src, dst, rows, axis, dtype, scale=None, variance=None, flags=0, save_stats=False, eps=1e-6, stream=None):
    """RMS normalisation over the last axis of a dense [rows, axis] tensor; device or host pointers."""
    _check(library().kudnn_b200_rmsnorm_run(_ptr(src), _ptr(dst), _ptr(scale), _ptr(variance), rows, axis, dtype, flags,
                                            1 if save_stats else 0, eps, stream))


def debug_fail_allocation(nth):
    """Test hook: the nth (0 = next) device allocation of the library fails; negative switches it off."""
    _check(library().kudnn_b200_debug_fail_allocation(nth))


def run_static_scratch(desc, a, b, c=None, bias=None, res=None, out=None, alpha=1.0, beta=0.0, gamma=1.0, stream=None):
    """Decode-shaped Linear (m <= 16) through the entry point that allocates no device memory.

    For callers that cannot call cudaMalloc when they need the result (all of HBM already given to their own pools, or
    an operator call in which the host framework forbids allocation).  Device pointers, asynchronous on `stream`.  The
    scratch is one fixed array per device, shared by all calls: keep the calls on one stream, because calls that
    overlap on the GPU race.  Problems that need more than the built-in 8 MiB raise KudnnError (UNSUPPORTED).
    """
    args = LinearArgs()
    args.a, args.b, args.c, args.bias, args.res, args.out = (_ptr(a), _ptr(b), _ptr(c), _ptr(bias), _ptr(res), _ptr(out))
    args.alpha, args.beta, args.gamma = alpha, beta, gamma
    _check(library().kudnn_b200_linear_run_static_scratch(ctypes.byref(desc), ctypes.byref(args), stream))


class Linear:
    """One created primitive (kudnn_b200_linear_t)."""

    def __init__(self, desc):
        self._lib = library()
        self.desc = desc
        h = ctypes.c_void_p()
        _check(self._lib.kudnn_b200_linear_create(ctypes.byref(desc), ctypes.byref(h)))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            self._lib.kudnn_b200_linear_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _args(self, a, b, c, bias, res, out, alpha, beta, gamma):
        args = LinearArgs()
        args.a, args.b, args.c, args.bias, args.res, args.out = (_ptr(a), _ptr(b), _ptr(c), _ptr(bias), _ptr(res),
                                                                  _ptr(out))
        args.alpha, args.beta, args.gamma = alpha, beta, gamma
        return args

    def prepack(self, b, stream=None):
        _check(self._lib.kudnn_b200_linear_prepack(self._h, _ptr(b), stream))

    def unpack(self):
        """Forgets the packed weights: later runs read the weight pointer they are given."""
        _check(self._lib.kudnn_b200_linear_unpack(self._h))

    def debug_set_wait(self, wait_limit_cycles, skip_kblock=-1):
        """Test hook: limit of the device-side waits in SM cycles, and the k-block whose loads CTA 0 leaves out."""
        _check(self._lib.kudnn_b200_debug_set_wait(self._h, wait_limit_cycles, skip_kblock))

    def run(self, a, b, c=None, bias=None, res=None, out=None, alpha=1.0, beta=0.0, gamma=1.0, stream=None):
        """Device pointers; asynchronous on `stream` (a cudaStream_t value, None = default stream)."""
        args = self._args(a, b, c, bias, res, out, alpha, beta, gamma)
        _check(self._lib.kudnn_b200_linear_run(self._h, ctypes.byref(args), stream))

    def run_host(self, a, b, c=None, bias=None, res=None, out=None, alpha=1.0, beta=0.0, gamma=1.0):
        """Host pointers, as the reference's callers pass them; returns when the outputs are in host memory."""
        args = self._args(a, b, c, bias, res, out, alpha, beta, gamma)
        _check(self._lib.kudnn_b200_linear_run_host(self._h, ctypes.byref(args)))

    def run_sharded(self, a, b, c=None, bias=None, res=None, out=None, alpha=1.0, beta=0.0, gamma=1.0, nshards=1,
                    mode=SHARD_ROWS):
        """Host pointers; the rows (SHARD_ROWS) or columns (SHARD_COLS) of the layer are split into `nshards` pieces
        that run on this machine's GPUs (shard i on device i modulo the device count) from this one process."""
        args = self._args(a, b, c, bias, res, out, alpha, beta, gamma)
        _check(self._lib.kudnn_b200_linear_run_sharded(self._h, ctypes.byref(args), nshards, mode))

    def check(self, stream=None):
        _check(self._lib.kudnn_b200_linear_check(self._h, stream))

    def force_kernel(self, kernel):
        _check(self._lib.kudnn_b200_linear_force_kernel(self._h, kernel))

    def set_mirrors(self, c_mirrors=None, out_mirrors=None):
        """Every later run also stores c / out through these device pointers (tensors or integers), same strides:
        the same output tensor in other GPUs' memory, for column-sharded layers.  Empty or None switches it off."""
        cm = [_ptr(p) for p in (c_mirrors or [])]
        om = [_ptr(p) for p in (out_mirrors or [])]
        count = max(len(cm), len(om))
        arr_t = ctypes.c_void_p * max(count, 1)
        ca = arr_t(*(cm + [None] * (count - len(cm))))
        oa = arr_t(*(om + [None] * (count - len(om))))
        _check(self._lib.kudnn_b200_linear_set_mirrors(self._h, count, ca, oa))

    def set_multicast(self, c_multicast=None, out_multicast=None):
        """Addresses of c / out in a multicast mapping over every rank's copy (with the mirrors still set): the
        tensor-core kernel then writes each row piece with one multimem.st.  None switches it off."""
        _check(self._lib.kudnn_b200_linear_set_multicast(self._h, _ptr(c_multicast), _ptr(out_multicast)))

    @property
    def last_kernel(self):
        return self._lib.kudnn_b200_linear_last_kernel(self._h)

    @property
    def last_launches(self):
        return self._lib.kudnn_b200_linear_last_launches(self._h)

    @property
    def workspace_bytes(self):
        return self._lib.kudnn_b200_linear_workspace_bytes(self._h)
