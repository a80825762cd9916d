"""CPU test of the multi-GPU partition, world_size 2 over gloo: every rank takes its contiguous
slab of the flattened (batch, head) axis, computes it alone (here with the CPU oracle standing in
for the kernel), and the gathered result equals the unsharded computation. There is no exchange
step on the data path; the gather exists only to verify."""
import os
import socket
import sys

import numpy as np
import pytest

from conftest import ROOT, make_inputs


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, total_heads, N, d, result_path):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    import bench

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ob = entry.load_oracle()
    q, k, v = make_inputs(31, 1, total_heads, N, d)
    h0, h1 = bench.shard(rank, world, total_heads)
    mine = ob.attention(q[:, h0:h1], k[:, h0:h1], v[:, h0:h1], causal=True, nthreads=1)
    gathered = [None] * world
    dist.all_gather_object(gathered, mine.view(np.uint16).ravel())
    if rank == 0:
        np.save(result_path, np.concatenate(gathered))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,total_heads", [(2, 6), (2, 5)])
def test_head_shards_gather_to_full_result(ob, tmp_path, world, total_heads):
    import torch.multiprocessing as mp

    N, d = 160, 64
    path = str(tmp_path / "gathered.npy")
    mp.spawn(_worker, args=(world, _free_port(), total_heads, N, d, path), nprocs=world, join=True)
    q, k, v = make_inputs(31, 1, total_heads, N, d)
    full = ob.attention(q, k, v, causal=True, nthreads=1)
    got = np.load(path)
    assert np.array_equal(got.view(np.uint16), full.view(np.uint16).ravel())


def test_shard_covers_axis_without_overlap():
    sys.path.insert(0, ROOT)
    import bench

    for total in (1, 5, 64, 512, 513):
        for world in (1, 2, 4, 8):
            spans = [bench.shard(r, world, total) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for (a, b), (c, e) in zip(spans, spans[1:]):
                assert b == c and a <= b
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    assert bench.shard(3, 8, 512) == (192, 256)
