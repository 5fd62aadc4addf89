"""Output mirrors (kudnn_b200_linear_set_mirrors): the kernels store c / out through extra pointers as well.

On one GPU the mirrors are further buffers of the same device, which exercises every kernel family's mirrored store.
With two GPUs, two processes open each other's buffers through the CUDA IPC handles of the C ABI and a column-sharded
layer writes its slab into both copies of y from the epilogue (no gather step).
"""
import os
import subprocess
import sys

import numpy as np
import pytest

import kudnn_b200 as kb
from oracle import ko
from tests import helpers

torch = pytest.importorskip("torch")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
@pytest.mark.parametrize("kernel,m,n,k,dtype", [
    (kb.KERNEL_SIMT, 23, 40, 24, "f32"),
    (kb.KERNEL_GEMV_FMA, 1, 1000, 1032, "bf16"),
    (kb.KERNEL_GEMV_MMA, 4, 1003, 1048, "bf16"),
    (kb.KERNEL_GEMV_MMA, 16, 520, 4096, "f16"),
    (kb.KERNEL_TC, 300, 520, 264, "bf16"),       # single CTA tiles, vector and generic epilogue rows
    (kb.KERNEL_TC, 128, 1024, 1024, "f32"),      # cluster split-K
    (kb.KERNEL_TC, 512, 9000, 128, "bf16"),      # CTA pairs
])
def test_mirrors_on_one_device(cuda_device, kernel, m, n, k, dtype):
    case = dict(m=m, n=n, k=k, dtype=dtype, bias="row", act=kb.ACT_SWISH, res_op=kb.RES_EXT, gamma=0.5, x_dist="normal",
                w_std=0.03, seed=71)
    desc, arrays, c = helpers.build_case(case)
    ref_c, ref_o = helpers.run_oracle(desc, arrays, c, acc=ko.ACC_F64)
    d = {key: helpers._to_torch(v, cuda_device) for key, v in arrays.items()}
    np_t = ko.np_dtype(desc.c_dtype)
    fill = 0x7fc0 if np_t == np.uint16 else np.nan

    def blank():
        return helpers._to_torch(np.full((1, m, n), fill, dtype=np_t), cuda_device)

    t_c, t_o = blank(), blank()
    mir_c, mir_o = [blank(), blank()], [blank(), blank()]
    lin = kb.Linear(desc)
    lin.force_kernel(kernel)
    lin.set_mirrors(mir_c, mir_o)
    stream = torch.cuda.current_stream().cuda_stream
    lin.run(d["a"], d["b"], t_c, d.get("bias"), d["res"], t_o, gamma=0.5, stream=stream)
    lin.check(stream=stream)
    assert lin.last_kernel == kernel
    got_c, got_o = helpers._from_torch(t_c), helpers._from_torch(t_o)
    helpers.compare(got_c, ref_c, desc.c_dtype)
    helpers.compare(got_o, ref_o, desc.out_dtype)
    for t in mir_c:
        assert np.array_equal(helpers._from_torch(t).view(np.uint8), got_c.view(np.uint8))
    for t in mir_o:
        assert np.array_equal(helpers._from_torch(t).view(np.uint8), got_o.view(np.uint8))
    # switching mirroring off again leaves other buffers alone
    lin.set_mirrors()
    probe = blank()
    before = helpers._from_torch(mir_c[0]).copy()
    lin.run(d["a"], d["b"], probe, d.get("bias"), d["res"], t_o, gamma=0.5, stream=stream)
    lin.check(stream=stream)
    assert np.array_equal(helpers._from_torch(mir_c[0]).view(np.uint8), before.view(np.uint8))
    lin.close()


@pytest.mark.gpu
def test_mirror_argument_checks(cuda_device):
    desc = kb.make_desc(32, 64, 64, kb.BF16)
    lin = kb.Linear(desc)
    with pytest.raises(kb.KudnnError):
        lin.set_mirrors([1 << 20] * 8)            # more than 7
    a = torch.zeros(32, 64, dtype=torch.bfloat16, device=cuda_device)
    w = torch.zeros(64, 64, dtype=torch.bfloat16, device=cuda_device)
    y = torch.zeros(32, 64, dtype=torch.bfloat16, device=cuda_device)
    other = torch.zeros(32 * 64 + 8, dtype=torch.bfloat16, device=cuda_device)
    lin.set_mirrors([other.data_ptr() + 2])       # not 16-byte congruent with y
    with pytest.raises(kb.KudnnError):
        lin.run(a, w, y, stream=torch.cuda.current_stream().cuda_stream)
    lin.close()


_PEER_WORKER = r"""
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["KUDNN_ROOT"])
import kudnn_b200 as kb
from oracle import ko
from tests import helpers

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("gloo", rank=rank, world_size=world)
m, n_total, k = 384, 1024, 512
case = dict(m=m, n=n_total, k=k, dtype="bf16", bias="row", act=kb.ACT_SWISH, x_dist="normal", w_std=0.03, seed=72)
desc_full, arrays, c = helpers.build_case(case)
ref_c, _ = helpers.run_oracle(desc_full, arrays, c, acc=ko.ACC_F64)
n0, cnt = kb.shard_range(n_total, world, rank, 128)
# every rank holds a full [m, n_total] y that the other ranks can map
nbytes = m * n_total * 2
y_ptr, handle = kb.peer_buffer_create(nbytes)
handles = [None] * world
dist.all_gather_object(handles, handle)
peers = [kb.peer_buffer_open(h) if r != rank else None for r, h in enumerate(handles)]
# this rank's slab: columns [n0, n0 + cnt) of y, rows of W [n0, n0 + cnt)
desc = kb.make_desc(m, cnt, k, kb.BF16, has_bias=True, act=kb.ACT_SWISH, c_strides=(n_total, 1))
x = helpers._to_torch(arrays["a"], dev)
w = helpers._to_torch(np.ascontiguousarray(arrays["b"][0, n0:n0 + cnt]), dev)
b = helpers._to_torch(np.ascontiguousarray(arrays["bias"].reshape(-1)[n0:n0 + cnt]), dev)
lin = kb.Linear(desc)
lin.set_mirrors([p + n0 * 2 for p in peers if p is not None])
stream = torch.cuda.current_stream().cuda_stream
lin.run(x, w, y_ptr + n0 * 2, b, stream=stream)
lin.check(stream=stream)
dist.barrier()          # every rank's slab is complete in every copy
host = torch.empty(m * n_total, dtype=torch.int16)
import ctypes
cudart = ctypes.CDLL("libcudart.so")
assert cudart.cudaMemcpy(ctypes.c_void_p(host.data_ptr()), ctypes.c_void_p(y_ptr), ctypes.c_size_t(nbytes), 2) == 0
got = host.numpy().view(np.uint16).reshape(1, m, n_total)
helpers.compare(got, ref_c, desc_full.c_dtype)
dist.barrier()          # nobody unmaps while another rank may still be writing or reading
for p in peers:
    if p is not None:
        kb.peer_buffer_close(p)
dist.barrier()
kb.peer_buffer_destroy(y_ptr)
lin.close()
print("rank %d ok" % rank)
dist.destroy_process_group()
"""


@pytest.mark.gpu
def test_column_sharded_layer_writes_every_copy(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "peer_worker.py"
    script.write_text(_PEER_WORKER)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29533",
                   KUDNN_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, "rank %d failed:\n%s" % (rank, out[-3000:])


_MULTICAST_WORKER = r"""
import os, sys
import numpy as np
import torch
import torch.distributed as dist
import torch.distributed._symmetric_memory as symm_mem
sys.path.insert(0, os.environ["KUDNN_ROOT"])
import kudnn_b200 as kb
from oracle import ko
from tests import helpers

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
m, n_total, k = 384, 1024, 512
case = dict(m=m, n=n_total, k=k, dtype="bf16", bias="row", act=kb.ACT_SWISH, x_dist="normal", w_std=0.03, seed=73)
desc_full, arrays, c = helpers.build_case(case)
ref_c, _ = helpers.run_oracle(desc_full, arrays, c, acc=ko.ACC_F64)
n0, cnt = kb.shard_range(n_total, world, rank, 128)
# every rank's full [m, n_total] y in symmetric memory: peer addresses and, where the machine has it, one multicast address
y = symm_mem.empty((m, n_total), dtype=torch.bfloat16, device=dev)
y.zero_()
sym = symm_mem.rendezvous(y, dist.group.WORLD)
mc = int(sym.multicast_ptr or 0)
flag = torch.tensor([1 if mc else 0], device=dev)
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
status = "multicast"
if int(flag.item()) == 0:
    status = "no multicast object on this machine"
else:
    desc = kb.make_desc(m, cnt, k, kb.BF16, has_bias=True, act=kb.ACT_SWISH, c_strides=(n_total, 1))
    x = helpers._to_torch(arrays["a"], dev)
    w = helpers._to_torch(np.ascontiguousarray(arrays["b"][0, n0:n0 + cnt]), dev)
    b = helpers._to_torch(np.ascontiguousarray(arrays["bias"].reshape(-1)[n0:n0 + cnt]), dev)
    lin = kb.Linear(desc)
    lin.set_mirrors([int(p) + n0 * 2 for r, p in enumerate(sym.buffer_ptrs) if r != rank])
    lin.set_multicast(mc + n0 * 2)
    stream = torch.cuda.current_stream().cuda_stream
    lin.run(x, w, y.data_ptr() + n0 * 2, b, stream=stream)
    lin.check(stream=stream)
    assert lin.last_kernel == kb.KERNEL_TC
    torch.cuda.synchronize()
    dist.barrier()          # every rank's slab is complete in every copy
    got = y.cpu().view(torch.int16).numpy().view(np.uint16).reshape(1, m, n_total)
    helpers.compare(got, ref_c, desc_full.c_dtype)
    torch.cuda.synchronize()
    dist.barrier()          # no rank goes on to free anything while another may still store or read
    lin.set_multicast(None)
    lin.set_mirrors(None)
    lin.close()
print("rank %d ok: %s" % (rank, status))
torch.cuda.synchronize()
dist.barrier()
dist.destroy_process_group()
"""


@pytest.mark.gpu
def test_column_sharded_layer_through_a_multicast_mapping(tmp_path):
    """Two ranks, y bound to one NVLink multicast object: each slab is written once with multimem.st and must arrive in
    both copies.  Both ranks run to the end and leave together (no rank ends while its memory is bound and in use)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "multicast_worker.py"
    script.write_text(_MULTICAST_WORKER)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29534", KUDNN_ROOT=ROOT)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, "rank %d failed:\n%s" % (rank, out[-3000:])
