#!/usr/bin/env python
"""Benchmark of the Linear(+post-op) hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c5m] [--impl ours|reference]

A step is one Linear+post-op call over one batch of synthetic input.  The default workload, at every N, is the large
sharded prefill layer (x[32768,8192] . W[28672,8192]^T + b, SiLU, bf16) with its rows split over the N ranks and the
weights replicated (`c5m`): no collective on the data path, strong scaling, and at N = 1 the whole layer on one GPU.
`--workload c5n` is the column-sharded form in which every rank ends with the full output; `c1` .. `c4` are the
other benchmark configurations (at N > 1 they run as replicas).

Rank 0 prints one JSON line.  `value` is device-timed throughput with inputs resident in HBM; `e2e` is the same
metric through the host-pointer entry point of the C ABI with the host<->device copies inside the timed region;
`roofline` relates the kernel to the measured peaks of this GPU pool; at N = 1 `configs` holds the other four
configurations (time, rate, fraction of the measured peak, kernel), `cublas_compare` a library GEMM of the same
shape timed the same way (a comparison leg only), and `cpu_baseline` the CPU restatement of the reference path timed
on this machine's cores.  `--impl reference` times that CPU path alone.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "Linear+postop TFLOP/s (% bf16 tensor peak); decode GEMV HBM GB/s (% peak)"

# name -> (m, n, k, dtype, has_bias, act, act_alpha, res_op)
WORKLOADS = {
    "c1": dict(m=128, n=1024, k=1024, dtype="f32", bias="normal", act="relu", res=None, x="uniform",
               label="Linear+ReLU fp32 M128 K1024 N1024"),
    "c2": dict(m=4096, n=11008, k=4096, dtype="bf16", bias="zeros", act="silu", res=None, x="normal",
               label="Linear+SiLU bf16 prefill FFN up-proj M4096 K4096 N11008"),
    "c3": dict(m=8192, n=4096, k=4096, dtype="f16", bias="normal", act="gelu_tanh", res="add", x="normal",
               label="Linear+GELU(tanh)+residual-add fp16 M8192 K4096 N4096"),
    "c4": dict(m=16, n=28672, k=8192, dtype="bf16", bias=None, act=None, res="mul", x="normal",
               label="decode Linear+gate-mul bf16 K8192 N28672"),
    "c5": dict(m=32768, n=28672, k=8192, dtype="bf16", bias="normal", act="silu", res=None, x="normal",
               label="Linear+SiLU bf16 M32768 K8192 N28672"),
}

# DRAM bytes per launch of the dominant kernel, from ncu captures (dram__bytes_read.sum + dram__bytes_write.sum) of
# reduced cases, scaled to the full launch by the rows processed (null where nothing was captured)
NCU_TRAFFIC_BYTES = {
    # ncu capture of a half-size case (m = 2048): 110.7 MB read + 29.1 MB written; x and y scale with the rows, W does
    # not, and the part of y still in L2 at kernel end is counted as written
    "c2": 127.5e6 + 90.2e6,
    # ncu capture of an n = 8192 case: traffic equals the algorithmic bytes within 0.1 % (+3 % for the m = 16 partial
    # sums); scaled to n = 28672 by the rows
    "c4": 471.9e6 + 11.5e6,
}


def c5m_traffic_bytes(rows):
    """DRAM bytes per launch of the tensor-core kernel on `rows` rows of the large prefill layer: ncu capture of an
    8192-row launch (dram__bytes_read.sum 6.47 GB + dram__bytes_write.sum 0.56 GB), scaled by the rows; the weights are
    streamed once per group of 4096 rows and rows of x are fetched again for later tile columns, so the traffic grows
    in proportion to the rows.  The full-size launch is too large to capture."""
    return 7.03e9 * rows / 8192.0


FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"]))}, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


def algorithmic_bytes(w, m=None):
    m = m or w["m"]
    es = 4 if w["dtype"] == "f32" else 2
    extra = 1 if w["res"] else 0
    return es * (m * w["k"] + w["n"] * w["k"] + (w["n"] if w["bias"] else 0) + m * w["n"] * (1 + extra))


def flops(w, m=None):
    return 2.0 * (m or w["m"]) * w["n"] * w["k"]


# ----------------------------------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while the benchmark runs."""

    REASONS = [(0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"),
               (0x80, "hw_power_brake"), (0x2, "applications_clocks_setting"), (0x100, "display_clock_setting")]

    def __init__(self, index):
        self.samples = []
        self.stop_flag = threading.Event()
        self.thread = None
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        while not self.stop_flag.is_set():
            try:
                mhz = self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)
                mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            except Exception:
                try:
                    mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                except Exception:
                    mask = 0
                    mhz = 0
            self.samples.append((time.perf_counter(), mhz, mask))
            time.sleep(0.004)

    def start(self):
        if self.nv is not None:
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()

    def stop(self):
        self.stop_flag.set()
        if self.thread is not None:
            self.thread.join(timeout=2.0)

    def summary(self, t0, t1):
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "NVML unavailable"}
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        note = "sampled during the timed region"
        if len(inside) < 3:
            inside = self.samples
            note = "timed region shorter than the sampling period; samples cover warm-up and timed region"
        clocks = sorted(s[1] for s in inside if s[1])
        mask = 0
        for s in inside:
            mask |= s[2]
        reasons = [name for bit, name in self.REASONS if mask & bit]
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "sm_mhz_min": clocks[0] if clocks else None, "samples": len(inside), "note": note}


# ----------------------------------------------------------------------------------------------------- inputs

def make_inputs(w, m, device, seed=0, n=None):
    """Synthetic inputs of the workload's shapes and distributions; draw order x -> W -> bias -> residual/gate."""
    import torch
    n = n or w["n"]
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[w["dtype"]]
    g = torch.Generator(device=device).manual_seed(seed)
    if w["x"] == "normal":
        x = torch.randn(m, w["k"], generator=g, device=device, dtype=torch.float32).to(tdt)
    else:
        x = (torch.rand(m, w["k"], generator=g, device=device, dtype=torch.float32) * 2 - 1).to(tdt)
    wt = torch.empty(n, w["k"], device=device, dtype=tdt)
    rows = max(1, (1 << 27) // w["k"])
    for r0 in range(0, n, rows):  # in slabs: a full fp32 copy of the largest weight matrix is not needed
        r1 = min(n, r0 + rows)
        wt[r0:r1] = (torch.randn(r1 - r0, w["k"], generator=g, device=device, dtype=torch.float32) * 0.02).to(tdt)
    bias = None
    if w["bias"] == "normal":
        bias = (torch.randn(n, generator=g, device=device, dtype=torch.float32) * 0.02).to(tdt)
    elif w["bias"] == "zeros":
        bias = torch.zeros(n, device=device, dtype=tdt)
    res = None
    if w["res"]:
        res = torch.randn(m, n, generator=g, device=device, dtype=torch.float32).to(tdt)
    return x, wt, bias, res


def make_desc(kb, w, m, n=None, ldc=None):
    n = n or w["n"]
    code = {"f32": kb.F32, "f16": kb.F16, "bf16": kb.BF16}[w["dtype"]]
    act = {None: kb.ACT_NONE, "relu": kb.ACT_RELU, "silu": kb.ACT_SWISH, "gelu_tanh": kb.ACT_GELU_TANH}[w["act"]]
    res = {None: kb.RES_NONE, "add": kb.RES_IDENTICAL, "mul": kb.RES_ELTWISE_MUL}[w["res"]]
    ldc = ldc or n
    return kb.make_desc(m, n, w["k"], code, has_bias=w["bias"] is not None, act=act,
                        act_alpha=0.0 if w["act"] == "relu" else 1.0, res_op=res, c_strides=(ldc, 1),
                        out_strides=(ldc, 1), res_strides=(n, 1))


# ----------------------------------------------------------------------------------------------------- CPU arm

class CpuArm:
    """The CPU restatement of the reference path (oracle/), timed on an m-slice of the workload.  The weight matrix
    is built once; every timed call converts it again, as the reference's BLAS packs its operands on every call."""

    def __init__(self, w, threads=0):
        import tempfile
        import numpy as np
        from oracle import ko
        self.np, self.ko, self.w = np, ko, w
        lib = None
        try:  # a build tuned to this host's cores, kept out of the source tree
            path = os.path.join(tempfile.gettempdir(), "kudnn_oracle_native_%d.so" % os.getuid())
            ko.build(march="native", out=path)
            lib = ko.load(path)
            self.build = "-march=native"
        except Exception:
            lib = ko.load()
            self.build = "-march=x86-64-v3 (prebuilt)"
        self.lib = lib
        if threads <= 0:
            # all cores this process may use; launchers such as torch.distributed.run export OMP_NUM_THREADS=1
            try:
                threads = len(os.sched_getaffinity(0))
            except AttributeError:
                threads = os.cpu_count() or 1
        self.threads = threads
        self.cores = threads
        self.code = {"f32": ko.F32, "f16": ko.F16, "bf16": ko.BF16}[w["dtype"]]
        self.act = {None: ko.ACT_NONE, "relu": ko.ACT_RELU, "silu": ko.ACT_SWISH, "gelu_tanh": ko.ACT_GELU_TANH}[w["act"]]
        self.res_op = {None: ko.RES_NONE, "add": ko.RES_IDENTICAL, "mul": ko.RES_ELTWISE_MUL}[w["res"]]
        n, k = w["n"], w["k"]
        self.rng = np.random.default_rng(0)
        self.wt = ko.to_storage(self.rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02), self.code, lib)
        self.bias = ko.to_storage(self.rng.standard_normal((n,), dtype=np.float32) * np.float32(0.02), self.code,
                                  lib) if w["bias"] else None
        self.per_row = None
        self.fixed = 0.0

    def run(self, rows):
        np, ko, w = self.np, self.ko, self.w
        n, k, code = w["n"], w["k"], self.code
        d = ko.Desc()
        d.m, d.n, d.k = rows, n, k
        d.a_dtype = d.b_dtype = d.c_dtype = d.bias_dtype = d.res_dtype = d.out_dtype = code
        d.has_bias = 1 if self.bias is not None else 0
        d.act, d.res_op = self.act, self.res_op
        d.act_alpha = 0.0 if w["act"] == "relu" else 1.0
        d.a_sm, d.a_sk, d.b_sk, d.b_sn, d.c_sm, d.c_sn = k, 1, 1, k, n, 1
        d.bias_sm, d.bias_sn, d.res_sm, d.res_sn, d.out_sm, d.out_sn = 0, 1, n, 1, n, 1
        x = ko.to_storage(self.rng.standard_normal((rows, k), dtype=np.float32), code, self.lib)
        r = ko.to_storage(self.rng.standard_normal((rows, n), dtype=np.float32), code, self.lib) if self.res_op else None
        c = np.zeros((rows, n), dtype=ko.np_dtype(code))
        o = np.zeros((rows, n), dtype=ko.np_dtype(code)) if self.res_op else None
        t0 = time.perf_counter()
        ko.linear(d, x, self.wt, c, self.bias, r, o, num_threads=self.threads, lib=self.lib)
        return time.perf_counter() - t0

    def rows_for(self, budget_s):
        if self.per_row is None:
            t8 = min(self.run(8), self.run(8))
            t40 = self.run(40)
            self.per_row = max((t40 - t8) / 32.0, 1e-9)
            self.fixed = max(t8 - 8 * self.per_row, 0.0)
        rows = int(max(4, min(self.w["m"], (budget_s - self.fixed) / self.per_row)))
        return max(4, rows // 4 * 4)

    def sample(self, budget_s):
        """Returns (tflops, rows, seconds)."""
        rows = self.rows_for(budget_s)
        t = self.run(rows)
        return 2.0 * rows * self.w["n"] * self.w["k"] / t / 1e12, rows, t


def config_block(w, wname, world):
    """What the run is about; identical in both arms.  How each arm ran it is in the line's `details`."""
    if wname == "c5m":
        par = "rows of x split over %d rank(s), weights replicated, no collective" % world
    elif wname == "c5n":
        par = "columns of W split over %d rank(s), every rank ends with the full y" % world
    else:
        par = "single GPU" if world == 1 else "%d replicas of the full batch" % world
    return {"workload": wname + ": " + w["label"], "m": w["m"], "n": w["n"], "k": w["k"], "dtype": w["dtype"],
            "parallelism": par}


def run_reference_arm(args, w, wname, rank):
    """--impl reference: the CPU path alone, all host threads, bounded sample per step."""
    if rank != 0:
        return
    arm = CpuArm(w)
    total_budget = 150.0
    per_step = max(0.5, min(3.0, total_budget / max(1, args.steps + args.warmup)))
    times = []
    for i in range(args.warmup + args.steps):
        sample = arm.sample(per_step)
        if i >= args.warmup:
            times.append(sample)
    best = (None, None, None, arm.cores)
    tfs = sorted(x[0] for x in times)
    value = tfs[len(tfs) // 2]
    rows = times[-1][1]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(x[2] for x in times) / len(times),
        "higher_is_better": True, "scaling": "strong" if wname.startswith("c5") else "weak", "vs_baseline": None,
        "dtype": w["dtype"], "data": "synthetic",
        "config": config_block(w, wname, args.gpus),
        "details": {"note": "KuDNN itself needs aarch64 SVE/SME and the closed KML BLAS; this arm times the scalar-"
                            "semantics C restatement of its Linear path (oracle/kudnn_linear_oracle.c) on rank 0's "
                            "host cores"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": best[3], "kind": "port",
                         "sample": "%d of %d rows of x per step, full W (weight conversion included), built %s"
                                   % (rows, w["m"], arm.build)},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------------- GPU arm

def timed_steps(torch, fn, steps, warmup, flush):
    """Runs warmup + steps calls of fn; every timed call sits between its own event pair, the L2 flush between calls
    is outside the pairs.  Returns the list of per-step milliseconds."""
    for _ in range(warmup):
        flush()
        fn()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    # Head start for the host: with a few flushes queued first, the launches of a step are already in the stream when
    # the device reaches its start event, so short kernels are not timed together with host launch latency.
    for _ in range(16):
        flush()
    for i in range(steps):
        flush()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    return [s.elapsed_time(e) for s, e in zip(starts, ends)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c5m", choices=["c1", "c2", "c3", "c4", "c5m", "c5n"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=0, help="override the row count (c4: 1, 4 or 16)")
    ap.add_argument("--n", type=int, default=0, help="override the column count (smaller cases for profiler captures)")
    ap.add_argument("--k", type=int, default=0, help="override the contraction length")
    ap.add_argument("--no-extras", action="store_true", help="skip the decode-GEMV, e2e and CPU legs")
    ap.add_argument("--leg", default="", choices=["", "configs", "decode", "eltwise", "int8"],
                    help="run only this side leg of the single-GPU line and print its object (small commands for "
                         "profiler captures)")
    ap.add_argument("--c5n-gather", default="fused", choices=["fused", "multimem", "nccl"],
                    help="column-sharded workload: every rank's kernel writes its slab of y into all ranks' copies "
                         "with plain peer stores (fused) or with one multimem.st per row piece through an NVLink "
                         "multicast mapping of y (multimem; falls back to fused where no multicast object can be made), "
                         "or NCCL all-gather plus a re-stride copy after the kernel (nccl)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    wname = args.workload
    w = dict(WORKLOADS["c5" if wname.startswith("c5") else wname])
    if args.m:
        w["m"] = args.m
    if args.n:
        w["n"] = args.n
    if args.k:
        w["k"] = args.k
    if args.m or args.n or args.k:
        w["label"] += " [overridden: m=%d n=%d k=%d]" % (w["m"], w["n"], w["k"])

    if args.impl == "reference":
        run_reference_arm(args, w, wname, rank)
        return 0

    import torch
    import kudnn_b200 as kb

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    peaks, peak_kind = load_peaks()

    if args.leg:
        fbuf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
        dbuf = torch.zeros(256 << 18, dtype=torch.float32, device=device)

        def leg_flush():
            fbuf.zero_()
            dbuf.sum()
        leg = {"configs": lambda: other_configs_leg(torch, kb, device, peaks, leg_flush),
               "decode": lambda: gemv_leg(torch, kb, device, peaks, leg_flush),
               "eltwise": lambda: eltwise_leg(torch, kb, device, peaks, leg_flush),
               "int8": lambda: int8_leg(torch, kb, device, peaks, leg_flush)}[args.leg]()
        if rank == 0:
            print(json.dumps({args.leg: leg}), flush=True)
        return 0

    # ---- per-rank problem
    n_total = w["n"]
    if wname == "c5m":
        begin, m_local = kb.shard_range(w["m"], world, rank, 128)
        n_local, scaling, par = n_total, "strong", "m-sharded x%d, replicated W, no collective" % world
    elif wname == "c5n":
        m_local = w["m"] if not args.m else args.m
        nb, n_local = kb.shard_range(n_total, world, rank, 256)
        scaling = "strong"
        par = "n-sharded x%d, " % world + {
            "fused": "the epilogue stores each slab of y into every rank's copy over NVLink (one store per peer)",
            "multimem": "the epilogue stores each slab of y into every rank's copy with multimem.st through NVSwitch",
            "nccl": "NCCL all-gather of y + re-stride copy"}[args.c5n_gather]
    else:
        m_local, n_local = w["m"], n_total
        scaling, par = "weak", ("replicas x%d: each GPU runs the full batch against replicated W" % world) if world > 1 \
            else "single GPU"
    x, wt, bias, res = make_inputs(w, m_local, device, seed=rank, n=n_local)
    tdt = x.dtype
    fused_gather = wname == "c5n" and world > 1 and args.c5n_gather in ("fused", "multimem")
    peer_ptrs, y_full_ptr, y_sym, mc_ptr, multicast_note = [], None, None, 0, None
    if fused_gather and args.c5n_gather == "multimem":
        # y lives in symmetric memory: torch allocates it, exchanges the handles and, where the machine can, binds every
        # rank's copy to one NVLink multicast object.  Plumbing only: the stores are issued by this library's kernel.
        import torch.distributed._symmetric_memory as symm_mem
        esize = x.element_size()
        y_sym = symm_mem.empty((m_local, n_total), dtype=tdt, device=device)
        sym = symm_mem.rendezvous(y_sym, dist.group.WORLD)
        y_full_ptr = y_sym.data_ptr()
        peer_ptrs = [int(p) for r, p in enumerate(sym.buffer_ptrs) if r != rank]
        mc_ptr = int(sym.multicast_ptr or 0)  # 0 where the machine cannot make a multicast object
        flag = torch.tensor([1 if mc_ptr else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            mc_ptr, multicast_note = 0, "no multicast object on this machine: plain peer stores"
        y = y_full_ptr + nb * esize
        desc = make_desc(kb, w, m_local, n=n_local, ldc=n_total)
    elif fused_gather:
        # every rank holds the full [m, n_total] y in a buffer the others map; this rank's kernel writes columns
        # [nb, nb + n_local) of all of them
        esize = x.element_size()
        y_full_ptr, handle = kb.peer_buffer_create(m_local * n_total * esize)
        handles = [None] * world
        dist.all_gather_object(handles, handle)
        peer_ptrs = [kb.peer_buffer_open(h) for r, h in enumerate(handles) if r != rank]
        y = y_full_ptr + nb * esize
        desc = make_desc(kb, w, m_local, n=n_local, ldc=n_total)
    else:
        y = torch.empty(m_local, n_local, device=device, dtype=tdt)
        desc = make_desc(kb, w, m_local, n=n_local)
    lin = kb.Linear(desc)
    stream = torch.cuda.current_stream().cuda_stream
    lin.prepack(wt, stream=stream)  # weights are packed once, at set-up
    if fused_gather:
        mirrors = [p + nb * x.element_size() for p in peer_ptrs]
        lin.set_mirrors(None if w["res"] else mirrors, mirrors if w["res"] else None)
        if mc_ptr:
            mc = mc_ptr + nb * x.element_size()
            lin.set_multicast(None if w["res"] else mc, mc if w["res"] else None)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    drain_buf = torch.zeros(256 << 18, dtype=torch.float32, device=device)  # 256 MiB

    def flush():
        # 256 MiB written: nothing of the previous step is left in the 126 MB L2.  256 MiB of another buffer read:
        # the written lines are back in DRAM, so the timed kernel is not charged for writing the flush buffer back.
        flush_buf.zero_()
        drain_buf.sum()

    # The other configurations and the decode shapes are short kernels: they are measured first, on a GPU that has
    # not yet been driven into its power cap by the long steps of the main workload.
    early = {}
    if world == 1 and not args.no_extras and wname == "c5m":
        early["configs"] = other_configs_leg(torch, kb, device, peaks, flush)
        early["decode_gemv"] = gemv_leg(torch, kb, device, peaks, flush)
        early["eltwise"] = eltwise_leg(torch, kb, device, peaks, flush)
        early["int8"] = int8_leg(torch, kb, device, peaks, flush)
        torch.cuda.synchronize()
        time.sleep(1.0)

    gathered = None
    if wname == "c5n" and world > 1 and not fused_gather:
        gathered = torch.empty(world * m_local, n_local, device=device, dtype=tdt)
        y_full = torch.empty(m_local, n_total, device=device, dtype=tdt)

    launches = [0]

    def step():
        if w["res"]:
            lin.run(x, wt, None, bias, res, y, stream=stream)
        else:
            lin.run(x, wt, y, bias, stream=stream)
        launches[0] += lin.last_launches
        if gathered is not None:
            dist.all_gather_into_tensor(gathered, y)
            y_full.view(m_local, world, n_local).copy_(gathered.view(world, m_local, n_local).permute(1, 0, 2))

    sampler = ClockSampler(local_rank)
    sampler.start()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    for _ in range(args.warmup):
        flush()
        step()
    torch.cuda.synchronize()
    launches[0] = 0
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ms = timed_steps(torch, step, args.steps, 0, flush)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    lin.check(stream=stream)
    sampler.stop()
    total_ms = sum(ms)
    if dist is not None:
        t = torch.tensor([total_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps

    if wname in ("c5m", "c5n"):
        job_flops = flops(w, w["m"] if wname == "c5m" else m_local)
    else:
        job_flops = flops(w, m_local) * world
    tflops = job_flops / (ms_per_step * 1e-3) / 1e12

    kernel_name = kb.KERNEL_NAMES.get(lin.last_kernel)
    my_ms = sum(ms) / len(ms)
    if wname == "c4":
        abytes = algorithmic_bytes(w, m_local)
        achieved = abytes / (my_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES.get(wname),
                    "peak_source": peak_kind + " (copy bandwidth)", "kernel": kernel_name,
                    "algorithmic_bytes": abytes}
        value, unit = achieved * (world if world > 1 else 1), "GB/s"
    else:
        kflops = flops(w, m_local) * (n_local / float(n_total))
        achieved = kflops / (my_ms * 1e-3) / 1e12
        # a step of several milliseconds runs under the power cap: the sustained cuBLAS figure is its denominator
        long_step = my_ms >= 5.0
        tensor_peak = peaks["bf16_tflops_sustained"] if long_step else peaks["bf16_tflops"]
        roofline = {"bound": "tensor", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s",
                    "frac": achieved / tensor_peak,
                    "traffic": c5m_traffic_bytes(m_local) if wname == "c5m" else NCU_TRAFFIC_BYTES.get(wname),
                    "peak_source": peak_kind + (" (cuBLAS bf16 sustained: a %.1f ms step runs under the power cap; burst %.1f)"
                                                % (my_ms, peaks["bf16_tflops"]) if long_step else
                                                " (cuBLAS bf16 burst; sustained %.1f)" % peaks["bf16_tflops_sustained"]),
                    "kernel": kernel_name, "algorithmic_flops": kflops,
                    "algorithmic_bytes": algorithmic_bytes(w, m_local)}
        value, unit = tflops, "TFLOP/s"

    line = {
        "metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
        "dtype": w["dtype"], "data": "synthetic (seeded; shapes and distributions of the named configuration)",
        "config": config_block(w, wname, world),
        "details": {"rows_per_gpu": m_local, "cols_per_gpu": n_local, "parallelism": par,
                    "l2": "256 MiB written, then 256 MiB of another buffer read (L2 left clean), between steps and "
                          "outside the timed event pairs",
                    "timing": "CUDA events around every step on the launching stream, summed; max over ranks",
                    "weights": "pre-packed once at set-up (for K-major 16-bit weights the caller's buffer is used as "
                               "is)"},
        "roofline": roofline,
        "gpu_launches": launches[0],
        "clocks": sampler.summary(t0, t1),
    }

    # ---- extras on a single GPU: e2e through host pointers, decode GEMV, CPU baseline
    if world == 1 and not args.no_extras:
        line["e2e"] = e2e_leg(torch, kb, w, wname, m_local, device, min(args.steps, 10))
        if wname == "c5m":
            mhz = line["clocks"].get("sm_mhz")
            line["roofline"]["ms_x_mhz"] = my_ms * mhz if mhz else None
            line["cublas_compare"] = cublas_leg(torch, x, wt, peaks, flush, local_rank, min(args.steps, 20))
            line.update(early)
        try:
            arm = CpuArm(w)
            tf, rows, t = arm.sample(12.0)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": arm.cores, "kind": "port",
                                    "sample": "%d of %d rows of x, full W, one pass of %.1f s (weight conversion "
                                              "included), built %s" % (rows, w["m"], t, arm.build)}
        except Exception as exc:  # the oracle is optional test infrastructure
            line["cpu_baseline"] = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "port",
                                    "sample": "unavailable: %s" % exc}
    elif world > 1 and not args.no_extras and wname != "c5n":
        # every rank pushes its own rows through the host-pointer call at the same time (they share the host's PCIe
        # and memory system); the job's rate is all rows over the slowest rank's time
        e = e2e_leg(torch, kb, w, wname, m_local, device, min(args.steps, 10), sync=dist.barrier)
        tmax = torch.tensor([e["ms_per_step"]], device=device, dtype=torch.float64)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        worst_ms = float(tmax.item())
        if wname == "c4":
            e["value"] = algorithmic_bytes(w, m_local) * world / (worst_ms * 1e-3) / 1e9
        else:
            e["value"] = job_flops / (worst_ms * 1e-3) / 1e12
        e["ms_per_step"] = worst_ms
        e["h2d_bytes_per_step"] *= world
        e["d2h_bytes_per_step"] *= world
        e["timing"] = "host clock around run_host calls on every rank at once; slowest rank; bytes summed over ranks"
        line["e2e"] = e
    elif world > 1:
        line["e2e"] = {"value": None, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                       "note": "not measured in this mode (--no-extras, or the column-sharded workload whose output "
                               "lives in peer-mapped device buffers)"}
    if y_sym is not None:
        # every rank must hold the same bytes: checksums of each rank's slab, compared across the copies
        torch.cuda.synchronize()
        dist.barrier()
        sums = torch.stack([y_sym[:, kb.shard_range(n_total, world, r, 256)[0]:][:, :kb.shard_range(n_total, world, r, 256)[1]]
                            .to(torch.float64).abs().sum() for r in range(world)])
        all_sums = [torch.empty_like(sums) for _ in range(world)]
        dist.all_gather(all_sums, sums)
        same = all(bool(torch.equal(all_sums[0], t)) for t in all_sums) and bool((sums > 0).all())
        line["details"]["multicast"] = {"used": bool(mc_ptr), "note": multicast_note, "copies_identical": same}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        # no rank frees its buffers or leaves while another may still store into them
        torch.cuda.synchronize()
        dist.barrier()
        if y_sym is not None:
            lin.set_multicast(None, None)
            lin.set_mirrors(None, None)
        dist.barrier()
        dist.destroy_process_group()
    return 0


def e2e_leg(torch, kb, w, wname, m, device, steps, sync=None):
    """The same step through kudnn_b200_linear_run_host: pinned host buffers in, pinned host buffers out."""
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[w["dtype"]]
    x, wt, bias, res = make_inputs(w, m, torch.device("cpu"), seed=0)
    x, wt = x.pin_memory(), wt.pin_memory()
    bias = bias.pin_memory() if bias is not None else None
    res = res.pin_memory() if res is not None else None
    y = torch.empty(m, w["n"], dtype=tdt).pin_memory()
    desc = make_desc(kb, w, m)
    lin = kb.Linear(desc)
    lin.prepack(wt)  # the weight matrix goes to the device once; every step moves x (and residual) in and y out

    def step():
        if w["res"]:
            lin.run_host(x, wt, None, bias, res, y)
        else:
            lin.run_host(x, wt, y, bias)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    if sync is not None:
        sync()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()  # returns after the device-to-host copy has completed
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / steps
    h2d = x.numel() * x.element_size() + (bias.numel() * bias.element_size() if bias is not None else 0) + \
        (res.numel() * res.element_size() if res is not None else 0)
    d2h = y.numel() * y.element_size()
    if wname == "c4":
        return {"value": algorithmic_bytes(w, m) / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": dt * 1e3}
    return {"value": flops(w, m) / dt / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "ms_per_step": dt * 1e3, "timing": "host clock around run_host calls, which return after the D2H copy"}


def cublas_leg(torch, x, wt, peaks, flush, gpu_index, steps):
    """Comparison only, never on the product path: torch.matmul (a library GEMM, no bias, no activation) on the same
    x and W, timed like the product step, with the SM clock sampled meanwhile.  time x clock says whether a gap
    between the two is cycles or power."""
    y = torch.empty(x.shape[0], wt.shape[0], device=x.device, dtype=x.dtype)
    wt_t = wt.t()
    sampler = ClockSampler(gpu_index)
    sampler.start()
    for _ in range(3):
        flush()
        torch.matmul(x, wt_t, out=y)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ms = timed_steps(torch, lambda: torch.matmul(x, wt_t, out=y), steps, 0, flush)
    t1 = time.perf_counter()
    sampler.stop()
    clocks = sampler.summary(t0, t1)
    my_ms = sum(ms) / len(ms)
    tf = 2.0 * x.shape[0] * wt.shape[0] * x.shape[1] / (my_ms * 1e-3) / 1e12
    return {"what": "torch.matmul(x, W^T), bf16, no bias or activation (cuBLAS); comparison leg", "ms_per_step": my_ms,
            "tflops": tf, "frac_of_sustained_peak": tf / peaks["bf16_tflops_sustained"], "sm_mhz": clocks.get("sm_mhz"),
            "sm_mhz_min": clocks.get("sm_mhz_min"), "clock_samples": clocks.get("samples"), "reasons": clocks.get("reasons"),
            "ms_x_mhz": my_ms * clocks["sm_mhz"] if clocks.get("sm_mhz") else None}


def other_configs_leg(torch, kb, device, peaks, flush):
    """Configurations 1, 2 and 3 on one GPU: time, rate, fraction of the measured burst peak, kernel."""
    out = {}
    stream = torch.cuda.current_stream().cuda_stream
    for name in ("c1", "c2", "c3"):
        w = dict(WORKLOADS[name])
        x, wt, bias, res = make_inputs(w, w["m"], device, seed=0)
        y = torch.empty(w["m"], w["n"], device=device, dtype=x.dtype)
        lin = kb.Linear(make_desc(kb, w, w["m"]))
        lin.prepack(wt, stream=stream)
        if w["res"]:
            fn = lambda: lin.run(x, wt, None, bias, res, y, stream=stream)
        else:
            fn = lambda: lin.run(x, wt, y, bias, stream=stream)
        ms = timed_steps(torch, fn, 30, 5, flush)
        lin.check(stream=stream)
        ms.sort()
        med = ms[len(ms) // 2]
        tf = flops(w) / (med * 1e-3) / 1e12
        out[name] = {"workload": w["label"], "us": med * 1e3, "tflops": tf,
                     "frac_of_measured_bf16_burst": tf / peaks["bf16_tflops"],
                     "kernel": kb.KERNEL_NAMES.get(lin.last_kernel), "launches_per_call": lin.last_launches,
                     "algorithmic_flops": flops(w), "algorithmic_bytes": algorithmic_bytes(w)}
        if name == "c1":
            out[name]["note"] = "latency-bound: 0.27 GFLOP and 5.2 MB per call"
        del x, wt, bias, res, y, lin
        torch.cuda.empty_cache()
    return out


def eltwise_leg(torch, kb, device, peaks, flush):
    """The operators either side of Linear, stand-alone: SiLU over the output of configuration 2 and RMS normalisation
    (with scale) over the input of configuration 3.  Algorithmic bytes = every element read once and written once."""
    out = {}
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=device).manual_seed(0)
    m, n = 4096, 11008
    x = torch.randn(m, n, generator=g, device=device).to(torch.bfloat16)
    y = torch.empty_like(x)
    ms = timed_steps(torch, lambda: kb.activation(x, y, m * n, kb.BF16, kb.BF16, kb.ACT_SWISH, 1.0, stream=stream), 30, 5, flush)
    ms.sort()
    gbs = 2.0 * m * n * 2 / (ms[len(ms) // 2] * 1e-3) / 1e9
    out["activation_silu_bf16_4096x11008"] = {"us": ms[len(ms) // 2] * 1e3, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                                              "algorithmic_bytes": 2 * m * n * 2}
    rows, axis = 8192, 4096
    x = torch.randn(rows, axis, generator=g, device=device).to(torch.float16)
    scale = torch.randn(axis, generator=g, device=device).to(torch.float16)
    y = torch.empty_like(x)
    ms = timed_steps(torch, lambda: kb.rmsnorm(x, y, rows, axis, kb.F16, scale=scale, flags=kb.NORM_USE_SCALE, eps=1e-5,
                                               stream=stream), 30, 5, flush)
    ms.sort()
    gbs = (2.0 * rows * axis + axis) * 2 / (ms[len(ms) // 2] * 1e-3) / 1e9
    out["rmsnorm_f16_8192x4096"] = {"us": ms[len(ms) // 2] * 1e3, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                                    "algorithmic_bytes": (2 * rows * axis + axis) * 2}
    return out


def int8_leg(torch, kb, device, peaks, flush):
    """s8 x s8 -> s32 (exact sums) on configuration 2's shape through tcgen05 kind::i8: TOP/s.  No measured integer peak
    exists for this pool, so no fraction is given (nominal dense 8-bit rate of the part: 4500 TOP/s)."""
    m, n, k = 4096, 11008, 4096
    g = torch.Generator(device=device).manual_seed(0)
    a = torch.randint(-128, 128, (m, k), generator=g, device=device, dtype=torch.int8)
    w = torch.randint(-128, 128, (n, k), generator=g, device=device, dtype=torch.int8)
    c = torch.empty(m, n, device=device, dtype=torch.int32)
    stream = torch.cuda.current_stream().cuda_stream
    lin = kb.Linear(kb.make_desc(m, n, k, kb.S8, b_dtype=kb.S8, c_dtype=kb.S32, b_strides=(1, k)))
    lin.prepack(w, stream=stream)
    ms = timed_steps(torch, lambda: lin.run(a, w, c, stream=stream), 20, 5, flush)
    lin.check(stream=stream)
    ms.sort()
    med = ms[len(ms) // 2]
    out = {"s8s8s32_4096x11008x4096": {"us": med * 1e3, "tops": 2.0 * m * n * k / (med * 1e-3) / 1e12,
                                       "kernel": kb.KERNEL_NAMES.get(lin.last_kernel), "launches_per_call": lin.last_launches}}
    del a, w, c, lin
    # decode with 8-bit weights (fp16 activations, fp16 result) on configuration 4's matrix: a single row streams the
    # weights as they are, one byte per element; more rows read their fp16 form (the bytes counted here are the 8-bit ones)
    n, k = 28672, 8192
    w8 = torch.randint(-128, 128, (n, k), generator=g, device=device, dtype=torch.int8)
    for rows in (1, 4):
        x = torch.randn(rows, k, generator=g, device=device).to(torch.float16)
        y = torch.empty(rows, n, device=device, dtype=torch.float16)
        lin = kb.Linear(kb.make_desc(rows, n, k, kb.F16, b_dtype=kb.S8, b_strides=(1, k)))
        lin.prepack(w8, stream=stream)
        ms = timed_steps(torch, lambda: lin.run(x, w8, y, stream=stream), 30, 5, flush)
        lin.check(stream=stream)
        ms.sort()
        med = ms[len(ms) // 2]
        abytes = n * k + rows * k * 2 + rows * n * 2
        out["w8a16_decode_m%d" % rows] = {"us": med * 1e3, "gbs": abytes / (med * 1e-3) / 1e9,
                                           "frac_of_measured_hbm": abytes / (med * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                           "kernel": kb.KERNEL_NAMES.get(lin.last_kernel), "algorithmic_bytes": abytes}
        del lin
    return out


def gemv_leg(torch, kb, device, peaks, flush):
    """Decode-shaped Linear + gate product (m = 1, 4, 16) on the streaming kernels: achieved HBM GB/s."""
    w = dict(WORKLOADS["c4"])
    out = {}
    x16, wt, _, gate16 = make_inputs(w, 16, device, seed=0)
    stream = torch.cuda.current_stream().cuda_stream
    for m in (1, 4, 16):
        x, gate = x16[:m].contiguous(), gate16[:m].contiguous()
        y = torch.empty(m, w["n"], device=device, dtype=x.dtype)
        lin = kb.Linear(make_desc(kb, w, m))
        lin.prepack(wt, stream=stream)  # at set-up: for 2 <= m <= 16 this stores the weights once more in 8 x 64 blocks
        ms = timed_steps(torch, lambda: lin.run(x, wt, None, None, gate, y, stream=stream), 30, 5, flush)
        lin.check(stream=stream)
        ms.sort()
        med = ms[len(ms) // 2]
        gbs = algorithmic_bytes(w, m) / (med * 1e-3) / 1e9
        out["m%d" % m] = {"us": med * 1e3, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                          "kernel": kb.KERNEL_NAMES.get(lin.last_kernel), "algorithmic_bytes": algorithmic_bytes(w, m)}
    return out


if __name__ == "__main__":
    sys.exit(main())
