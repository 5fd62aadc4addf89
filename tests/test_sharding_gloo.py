"""Host logic of the multi-GPU launchers on CPU ranks (gloo, world size 2): the shard arithmetic every rank derives
independently must tile the problem exactly, the m-sharded run needs no exchange, and the column-sharded run's
all-gather plus re-stride (the same calls bench.py issues over NCCL) rebuilds y[m, n] in row-major order.  The
per-shard products are taken from the CPU oracle here; on the GPU box the same shards go through the CUDA library."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import kudnn_b200 as kb
from oracle import ko
from tests import helpers


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _oracle_product(x, w, bias, code):
    m, k = x.shape
    n = w.shape[0]
    desc = kb.make_desc(m, n, k, code, has_bias=True, act=kb.ACT_SWISH)
    y = np.zeros((m, n), dtype=ko.np_dtype(code))
    ko.linear(helpers.oracle_desc(desc), np.ascontiguousarray(x), np.ascontiguousarray(w), y, np.ascontiguousarray(bias))
    return y


def _worker(rank, world, port, m, n, k, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)  # every rank builds the same replicated tensors
    code = kb.BF16
    x = ko.to_storage(rng.standard_normal((m, k), dtype=np.float32), code)
    w = ko.to_storage(rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05), code)
    bias = ko.to_storage(rng.standard_normal((n,), dtype=np.float32) * np.float32(0.05), code)
    whole = _oracle_product(x, w, bias, code)

    # m-sharded: own rows, replicated weights, nothing exchanged
    begin, count = kb.shard_range(m, world, rank, 16)
    mine = _oracle_product(x[begin:begin + count], w, bias, code)
    assert np.array_equal(mine, whole[begin:begin + count])
    covered = torch.tensor([count], dtype=torch.int64)
    dist.all_reduce(covered)  # control-plane check only
    assert int(covered.item()) == m

    # column-sharded: own weight rows, all-gather of y[:, slab], re-stride to [m, n]
    nb, ncount = kb.shard_range(n, world, rank, 8)
    assert ncount == n // world  # equal slabs are what all_gather_into_tensor needs
    slab = _oracle_product(x, w[nb:nb + ncount], bias[nb:nb + ncount], code)
    # gloo moves bytes here (it has no 16-bit integer type); NCCL on the GPU box moves the bf16 tensors themselves
    gathered = torch.empty(world * m, ncount * 2, dtype=torch.uint8)
    dist.all_gather_into_tensor(gathered, torch.from_numpy(slab.view(np.uint8)).contiguous())
    full = torch.empty(m, n * 2, dtype=torch.uint8)
    full.view(m, world, ncount * 2).copy_(gathered.view(world, m, ncount * 2).permute(1, 0, 2))
    assert np.array_equal(full.numpy().view(np.uint16), whole)
    np.save(os.path.join(out_dir, "rank%d.npy" % rank), full.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_shard_ranges_match_the_benchmark_layout():
    # config 5 over 8 ranks: 4096 rows each, 3584 columns each (a multiple of the 256-wide tile)
    assert [kb.shard_range(32768, 8, r, 128) for r in range(8)] == [(4096 * r, 4096) for r in range(8)]
    assert [kb.shard_range(28672, 8, r, 256) for r in range(8)] == [(3584 * r, 3584) for r in range(8)]
    assert kb.shard_range(100, 3, 2, 16) == (80, 20)


@pytest.mark.timeout(300)
def test_two_rank_sharded_linear_on_cpu(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, 64, 48, 96, str(tmp_path)), nprocs=world, join=True)
    a = np.load(tmp_path / "rank0.npy")
    b = np.load(tmp_path / "rank1.npy")
    assert np.array_equal(a, b)
