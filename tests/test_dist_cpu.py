"""World-size-2 tests of the data-parallel bucket scheduler (nc_bucket_plan in the C host library, the logic nc_dist runs
over NCCL) with gloo on CPU as the transport: the buckets cover the arena exactly once; the first step, which learns which
entries report, sends everything after the sweep; from the second step on a bucket is sent as soon as its last reporting
entry is final, in backward order, although one of its entries never reports (a parameter no backward reaches) and another
reports twice (a shared weight); and the arena ends up holding the sum over ranks.  A rank that leaves between steps makes
the others' next exchange fail with an error instead of hanging."""
import os
import socket
from datetime import timedelta

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

SIZES = [7, 64, 3, 1000, 129, 5000, 17]
NEVER = {1}        # entries that never report ready
TWICE = {5}        # entries that report twice per step


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entries():
    entries, off = [], 0
    for n in SIZES:
        entries.append((off, n))
        off += (n + 63) // 64 * 64
    return entries, off


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nocta_b200.dist_native import BucketPlan, load_host_library
    entries, total = _entries()
    rng = np.random.default_rng(100 + rank)
    arena = torch.from_numpy(rng.standard_normal(total).astype(np.float32))
    mine = arena.clone()
    plan = BucketPlan(load_host_library(), entries, total, bucket_floats=2048)
    ranges = [plan.range(b) for b in range(plan.count())]
    cover = sorted(ranges)
    assert cover[0][0] == 0 and cover[-1][1] == total
    for (a0, b0), (a1, b1) in zip(cover, cover[1:]):
        assert b0 == a1
    early = []          # (step, bucket) sent from inside the sweep
    for step in range(3):
        works = []

        def send(b):
            s, e = plan.range(b)
            works.append(dist.all_reduce(arena[s:e], async_op=True))

        for i in reversed(range(len(entries))):      # backward order: last parameter first
            if i in NEVER:
                continue
            for _ in range(2 if i in TWICE else 1):
                b = plan.on_ready(i)
                if b >= 0:
                    early.append((step, b))
                    send(b)
        while True:
            b = plan.next_unfired()
            if b < 0:
                break
            send(b)
        for w in works:
            w.wait()
        assert plan.end_step() == 0
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    expect = (gathered[0] + gathered[1]) * world * world    # three steps: the sum, summed again twice
    ok = torch.allclose(arena, expect, rtol=0, atol=1e-4)
    results[rank] = (bool(ok), plan.count(), early)
    plan.close()
    dist.destroy_process_group()


def test_bucket_plan_world2():
    world, port = 2, _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert len(results) == 2
    for r in range(world):
        ok, nb, early = results[r]
        assert ok and nb >= 2
        assert not any(step == 0 for step, _ in early)          # the learning step sends nothing early
        per_step = [[b for s, b in early if s == k] for k in (1, 2)]
        for fired in per_step:
            # every bucket with a reporting entry is sent from inside the sweep, the one at the end of the arena first;
            # the never-reporting entry does not hold its bucket back and the twice-reporting one is waited for twice
            assert fired and fired[0] == 0 and fired == sorted(fired)
            assert len(fired) == nb


def _leaver(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=5))
    t = torch.ones(16)
    dist.all_reduce(t)                    # step 1: everyone is here
    if rank == 1:
        results[rank] = "left"
        os._exit(0)                       # leaves between steps, nothing of its own in flight
    try:
        dist.all_reduce(t)                # step 2: the peer is gone
        results[rank] = "no error"
    except Exception as ex:               # the exchange fails instead of waiting forever
        results[rank] = "error: " + type(ex).__name__


def test_rank_leaving_between_steps_gives_an_error_not_a_hang():
    world, port = 2, _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    ctx = mp.spawn(_leaver, args=(world, port, results), nprocs=world, join=False)
    for p in ctx.processes:
        p.join(60)
        assert not p.is_alive(), "a rank is still waiting for the one that left"
    assert results.get(1) == "left"
    assert str(results.get(0, "")).startswith("error")
