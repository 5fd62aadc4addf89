"""Host-only checks of the C ABI: the library loads, exports every declared symbol, validates descriptors,
creates and destroys handles without touching a device, and refuses to compute without one."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import kudnn_b200 as kb
from kudnn_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "kudnn_b200.h")).read()
    return re.findall(r"KUDNN_B200_API\s+[\w\s\*]+?\b(kudnn_b200_\w+)\s*\(", text)


def test_header_and_binding_agree():
    names = declared_symbols()
    assert len(names) >= 15
    assert sorted(names) == sorted(capi.EXPORTS)


def test_every_declared_symbol_is_exported():
    lib = ctypes.CDLL(kb.library_path())
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_version_and_error_strings():
    lib = kb.library()
    assert b"sm_100a" in lib.kudnn_b200_version()
    assert isinstance(lib.kudnn_b200_last_error(), bytes)


def test_validate_accepts_the_five_configurations():
    configs = [
        kb.make_desc(128, 1024, 1024, kb.F32, has_bias=True, act=kb.ACT_RELU, act_alpha=0.0),
        kb.make_desc(4096, 11008, 4096, kb.BF16, has_bias=True, act=kb.ACT_SWISH),
        kb.make_desc(8192, 4096, 4096, kb.F16, has_bias=True, act=kb.ACT_GELU_TANH, res_op=kb.RES_IDENTICAL),
        kb.make_desc(16, 28672, 8192, kb.BF16, res_op=kb.RES_ELTWISE_MUL),
        kb.make_desc(32768, 28672, 8192, kb.BF16, has_bias=True, act=kb.ACT_SWISH),
    ]
    for d in configs:
        assert capi.validate(d) == 0


@pytest.mark.parametrize("mutate,status", [
    (lambda d: setattr(d, "m", 0), 1),
    (lambda d: setattr(d, "a_dtype", 4), 1),        # S32 input: UNSUPPORTED, as kudnn_gemm.cpp:390-392
    (lambda d: setattr(d, "c_dtype", 5), 1),
    (lambda d: setattr(d, "act", 1), 1),            # ABS: valid in the reference, not implemented here
    (lambda d: setattr(d, "res_op", 9), 1),
    (lambda d: setattr(d, "a_sk", -1), 2),
    (lambda d: setattr(d, "c_sn", 0), 2),
])
def test_validate_rejects(mutate, status):
    d = kb.make_desc(8, 8, 8, kb.F32)
    mutate(d)
    assert capi.validate(d) == status
    assert kb.library().kudnn_b200_last_error() != b""


def test_create_is_host_only_and_clone_copies():
    lin = kb.Linear(kb.make_desc(8, 16, 32, kb.BF16, has_bias=True))
    other = ctypes.c_void_p()
    assert kb.library().kudnn_b200_linear_clone(lin._h, ctypes.byref(other)) == 0
    assert other.value and other.value != lin._h.value
    assert kb.library().kudnn_b200_linear_destroy(other) == 0
    assert lin.last_kernel == 0 and lin.workspace_bytes == 0
    lin.close()
    with pytest.raises(kb.KudnnError):
        kb.Linear(kb.make_desc(8, 16, 0, kb.BF16))


def test_null_pointers_are_bad_arguments():
    lin = kb.Linear(kb.make_desc(8, 16, 32, kb.F32))
    with pytest.raises(kb.KudnnError) as e:
        lin.run(None, None, None)
    assert e.value.status == 2


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-device behaviour")
def test_no_silent_cpu_fallback():
    lin = kb.Linear(kb.make_desc(4, 4, 4, kb.F32))
    a = np.ones((4, 4), np.float32)
    c = np.zeros((4, 4), np.float32)
    with pytest.raises(kb.KudnnError) as e:
        lin.run_host(a, a, c)
    assert e.value.status == 6
    assert not c.any()


def test_shard_range_partitions_exactly():
    for total, nparts, align in [(32768, 8, 128), (4096, 3, 128), (1000, 7, 16), (5, 8, 1), (28672, 8, 256)]:
        covered = 0
        for part in range(nparts):
            begin, count = kb.shard_range(total, nparts, part, align)
            assert begin == covered
            assert count >= 0
            if begin + count < total:
                assert count % align == 0
            covered += count
        assert covered == total
    with pytest.raises(kb.KudnnError):
        kb.shard_range(10, 0, 0)
