"""World-size-2 gloo run of the multi-rank host logic: sharding by batch needs no exchange
(the gathered shard results equal the unsharded result) and the timing reduction is a max."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mixlab_b200 import sharding


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import gdn, inputs
        torch.set_num_threads(1)
        B = 3  # odd on purpose: ranks get 2 and 1 sequences
        full = inputs.gdn_inputs(B, 40, 2, 8, 8, seed=5)
        lo, hi = sharding.shard_range(B, world, rank)
        mine = {k: v[lo:hi] for k, v in full.items()}
        out, st = gdn.scan_chunked(mine["q"].double(), mine["k"].double(), mine["v"].double(), mine["beta"].double(),
                                   torch.exp(mine["g"].double()), 16)
        bufs = [None] * world  # shards have different sizes (2 and 1 sequences)
        dist.all_gather_object(bufs, out)
        got = torch.cat(bufs)
        want, _ = gdn.scan_chunked(full["q"].double(), full["k"].double(), full["v"].double(), full["beta"].double(),
                                   torch.exp(full["g"].double()), 16)
        t = sharding.max_over_ranks(10.0 + rank)
        ok = torch.equal(got, want) and t == 10.0 + world - 1
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_sharding():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}


def test_shard_range_partitions():
    for total in (0, 1, 7, 8, 256):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)
    assert sharding.whole_job_rate(100, 8, 0.5) == 1600.0
    assert len({sharding.rank_seed(1, r, i) for r in range(8) for i in range(8)}) == 64
