"""Multi-rank host logic on CPU: two gloo ranks shard a batch, each computes its slice (with the
oracle standing in for the GPU here) and the gather reassembles the whole batch in order."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from n2d2_b200 import netdesc
from n2d2_b200.sharding import gather_outputs, shard_bounds, shard_sizes


def test_shard_bounds_cover_the_batch_without_overlap():
    for total in (0, 1, 7, 64, 1024, 1025):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_bounds(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for a, b in zip(spans, spans[1:]):
                assert a[1] == b[0]
            sizes = shard_sizes(total, world)
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, total, out_path):
    from oracle import oracle
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    net = netdesc.mnist24()
    x = netdesc.make_input(net, total)
    b, e = shard_bounds(total, world, rank)
    local = oracle.run_net(net, x[b:e], 'i64')[-1].reshape(e - b, -1)
    full = gather_outputs(torch.from_numpy(local.astype(np.int8)), total)
    if rank == 0:
        np.save(out_path, full.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize('total', [7, 16])
def test_two_ranks_reassemble_the_batch(tmp_path, total):
    from oracle import oracle
    out = str(tmp_path / 'full.npy')
    mp.spawn(_worker, args=(2, _free_port(), total, out), nprocs=2, join=True)
    net = netdesc.mnist24()
    want = oracle.run_net(net, netdesc.make_input(net, total), 'i64')[-1].reshape(total, -1)
    assert np.array_equal(np.load(out).astype(np.int64), want)
