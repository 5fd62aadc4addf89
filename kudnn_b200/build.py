"""In-tree build of the CUDA library (libkudnn_b200.so) and the C++ host library (libkudnn.so).

nvcc cross-compiles for sm_100a without a GPU.  Objects land in kudnn_b200/_build/, the shared libraries in
kudnn_b200/ next to this file so that they travel with the source tree.
"""
import concurrent.futures
import os
import shutil
import subprocess
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_PKG)
_CSRC = os.path.join(_PKG, "csrc")
_HOST = os.path.join(_PKG, "host")
_BUILD = os.path.join(_PKG, "_build")

CUDA_LIB = os.path.join(_PKG, "libkudnn_b200.so")
HOST_LIB = os.path.join(_PKG, "libkudnn.so")
HOST_TEST_BIN = os.path.join(_PKG, "kudnn_host_tests")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    # products and sums are contracted only where the source says fmaf(), as in the CPU oracle
    "-fmad=false",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
    "-I", os.path.join(_ROOT, "include"),
]

CUDA_SOURCES = ["linear_api.cu", "simt_gemm.cu", "gemv.cu", "tc_gemm.cu", "pack.cu", "static_scratch.cu", "peer.cu", "eltwise.cu", "eltwise_api.cu"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _gxx():
    # the image exports CXX to a wrapper that cannot link OpenMP programs; use the plain compiler
    return shutil.which("g++") or "g++"


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("command failed: " + " ".join(cmd))
    if verbose and res.stdout.strip():
        print(res.stdout)
    return res.stdout


def build_cuda(verbose=False, force=False, ptxas_info=False):
    os.makedirs(_BUILD, exist_ok=True)
    headers = [os.path.join(_CSRC, f) for f in os.listdir(_CSRC) if f.endswith(".cuh")]
    headers.append(os.path.join(_ROOT, "include", "kudnn_b200.h"))
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in CUDA_SOURCES:
        s = os.path.join(_CSRC, src)
        o = os.path.join(_BUILD, src.replace(".cu", ".o"))
        objs.append(o)
        if force or not _newer(o, [s] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", s, "-o", o]
            jobs.append(cmd)
    outputs = []
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 2)) as pool:
            outputs = list(pool.map(lambda c: _run(c, verbose), jobs))
    if jobs or not os.path.exists(CUDA_LIB):
        _run([nvcc, "-shared", "-o", CUDA_LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                          "-Xcompiler", "-fPIC", "-lcudart_static", "-lpthread", "-ldl",
                                                          "-lrt"], verbose)
    return "\n".join(outputs)


def build_host(verbose=False, force=False):
    """C++ classes of the reference API over the C ABI, plus their self-checking test program."""
    if not os.path.isdir(_HOST):
        return
    srcs = [os.path.join(_HOST, f) for f in sorted(os.listdir(_HOST)) if f.endswith(".cpp") and not f.startswith("test_")]
    hdrs = [os.path.join(_HOST, f) for f in os.listdir(_HOST) if f.endswith(".hpp")]
    hdrs.append(os.path.join(_ROOT, "include", "kudnn_b200.h"))
    gxx = _gxx()
    common = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wextra", "-I", os.path.join(_ROOT, "include"), "-I", _HOST]
    if srcs and (force or not _newer(HOST_LIB, srcs + hdrs + [CUDA_LIB])):
        _run([gxx] + common + ["-shared", "-o", HOST_LIB] + srcs +
             ["-L", _PKG, "-lkudnn_b200", "-Wl,-rpath,$ORIGIN"], verbose)
    tests = [os.path.join(_HOST, f) for f in sorted(os.listdir(_HOST)) if f.endswith(".cpp") and f.startswith("test_")]
    if tests and (force or not _newer(HOST_TEST_BIN, tests + hdrs + [HOST_LIB])):
        _run([gxx] + common + ["-o", HOST_TEST_BIN] + tests +
             ["-L", _PKG, "-lkudnn", "-lkudnn_b200", "-Wl,-rpath,$ORIGIN"], verbose)


def build_all(verbose=False, force=False):
    build_cuda(verbose=verbose, force=force)
    build_host(verbose=verbose, force=force)


if __name__ == "__main__":
    info = build_cuda(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    build_host(verbose=True, force="--force" in sys.argv)
