"""World-size-2 gloo run of the multi-rank host logic: sharding by batch needs no exchange
(the gathered shard results equal the unsharded result) and the timing reduction is a max."""
import math
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


# ---------------------------------------------------------------- data-parallel gradient exchange
def test_gradient_bucket_plan_follows_reference_rule():
    """gpu/distributed_step.cpp:61-100: weight order, a bucket closes before the entry that would pass the target,
    an oversized entry stands alone; the digest changes with any layout change."""
    from mixlab_b200 import dp
    shapes = [(256, 256), (256,), (1024, 256), (3000, 1000), (8,), (8, 8)]   # 256 KiB, 1 KiB, 1 MiB, 11.4 MiB, ...
    plan = dp.build_gradient_bucket_plan(shapes, target_bytes=1 << 20)
    layout = [[e.weight_index for e in b.entries] for b in plan.buckets]
    assert layout == [[0, 1], [2], [3], [4, 5]]
    assert plan.total_bytes == 4 * sum(int(torch.tensor(s).prod()) for s in shapes)
    for b in plan.buckets:
        off = 0
        for e in b.entries:
            assert e.offset == off
            off += e.elements
        assert b.elements == off and b.bytes == 4 * off
    assert dp.build_gradient_bucket_plan(shapes, 1 << 20).digest == plan.digest
    assert dp.build_gradient_bucket_plan(shapes, 1 << 21).digest != plan.digest
    assert dp.build_gradient_bucket_plan(shapes[:-1] + [(64,)], 1 << 20).digest != plan.digest
    big = dp.build_gradient_bucket_plan(dp.hybrid_lm_weight_shapes())            # the end-to-end training config
    assert 0.9e9 < big.total_bytes < 1.3e9 and all(b.bytes <= 32 << 20 or len(b.entries) == 1 for b in big.buckets)
    with pytest.raises(ValueError):
        dp.build_gradient_bucket_plan(shapes, 0)


def _dp_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mixlab_b200 import dp
        torch.set_num_threads(1)
        shapes = [(40, 30), (30,), (300, 20), (7,)]
        plan = dp.build_gradient_bucket_plan(shapes, target_bytes=6000)
        digests = [None] * world
        dist.all_gather_object(digests, plan.digest)
        ok = len(set(digests)) == 1 and len(plan.buckets) >= 2
        g = torch.Generator().manual_seed(100)
        per_rank = [[torch.randn(*s, generator=g) for s in shapes] for _ in range(world)]   # every rank knows all
        norm = [3.0, 5.0][:world] if world == 2 else [float(r + 1) for r in range(world)]

        # 1. ordinary step: mean gradients, global denominator = sum of the tokens, weighted average, no clipping
        grads = [t.clone() for t in per_rank[rank]]
        res = dp.staged_gradient_allreduce(grads, torch.tensor(1.0), norm[rank], False, 0.0, plan)
        want = [sum(per_rank[r][i] * norm[r] for r in range(world)) / sum(norm) for i in range(len(shapes))]
        ok &= (not res.globally_bad) and (not res.zero_denominator) and res.denominator == sum(norm)
        ok &= all(torch.allclose(a, b, atol=1e-6) for a, b in zip(grads, want)) and res.gradient_nonfinite == 0.0

        # 2. clipping to a global norm
        grads = [t.clone() for t in per_rank[rank]]
        dp.staged_gradient_allreduce(grads, torch.tensor(1.0), norm[rank], False, 0.5, plan)
        total = math.sqrt(sum(float(w.pow(2).sum()) for w in want))
        ok &= all(torch.allclose(a, b * min(1.0, 0.5 / (total + 1e-6)), atol=1e-6) for a, b in zip(grads, want))

        # 3. one rank sees a NaN in a gradient: every rank learns that the step is bad
        grads = [t.clone() for t in per_rank[rank]]
        if rank == world - 1:
            grads[2][5, 3] = float("nan")
        res = dp.staged_gradient_allreduce(grads, torch.tensor(1.0), norm[rank], False, 0.0, plan)
        ok &= res.globally_bad and all(torch.isfinite(t).all() for t in grads)

        # 4. a non-finite loss on one rank, and an invalid normaliser on one rank, are bad steps too
        res = dp.staged_gradient_allreduce([t.clone() for t in per_rank[rank]],
                                           torch.tensor(float("inf") if rank == 0 else 1.0), norm[rank], False, 0.0, plan)
        ok &= res.globally_bad
        res = dp.staged_gradient_allreduce([t.clone() for t in per_rank[rank]], torch.tensor(1.0),
                                           float("nan") if rank == 0 else 1.0, False, 0.0, plan)
        ok &= res.globally_bad

        # 5. all normalisers zero: reported, not divided by
        res = dp.staged_gradient_allreduce([t.clone() for t in per_rank[rank]], torch.tensor(1.0), 0.0, False, 0.0, plan)
        ok &= res.zero_denominator and not res.globally_bad

        # 6. gradients written straight into the bucket storage (no packing copy), numerators already
        store = dp.BucketStorage(plan, "cpu")
        for v, t in zip(store.views, per_rank[rank]):
            v.copy_(t)
        grads = list(store.views)
        res = dp.staged_gradient_allreduce(grads, torch.tensor(1.0), norm[rank], True, 0.0, plan, storage=store)
        want_num = [sum(per_rank[r][i] for r in range(world)) / sum(norm) for i in range(len(shapes))]
        ok &= all(torch.allclose(a, b, atol=1e-6) for a, b in zip(grads, want_num))
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_staged_gradient_allreduce():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_dp_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}
