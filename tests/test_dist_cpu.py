"""World-size-2 test of the data-parallel gradient exchange over gloo on CPU: buckets cover the arena
exactly once, fire when their last gradient is ready (in backward order), and the arena ends up
holding the sum over ranks."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nocta_b200.dist import BucketedAllReduce
    sizes = [7, 64, 3, 1000, 129, 5000, 17]
    entries, off = [], 0
    for i, n in enumerate(sizes):
        entries.append((f"p{i}", off, n))
        off += (n + 63) // 64 * 64
    rng = np.random.default_rng(100 + rank)
    arena = torch.from_numpy(rng.standard_normal(off).astype(np.float32))
    mine = arena.clone()
    sync = BucketedAllReduce(arena, entries, bucket_floats=2048)
    ranges = sync.ranges()
    # contiguous cover of the whole arena
    cover = sorted((a, b) for a, b, _ in ranges)
    assert cover[0][0] == 0 and cover[-1][1] == off
    for (a0, b0), (a1, b1) in zip(cover, cover[1:]):
        assert b0 == a1
    fired = []
    for step in range(2):
        for key, _, _ in reversed(entries):       # backward order: last parameter first
            before = sum(b.work is not None for b in sync.buckets)
            sync.on_ready(key)
            if sum(b.work is not None for b in sync.buckets) > before:
                fired.append(key)
        sync.finish()
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    expect = gathered[0] + gathered[1]
    # two steps: the arena was reduced twice (sum of sums)
    expect2 = expect * world
    ok = torch.allclose(arena, expect2, rtol=0, atol=1e-5)
    results[rank] = (bool(ok), len(ranges), fired[:3])
    dist.destroy_process_group()


def test_bucketed_allreduce_world2():
    world, port = 2, _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert len(results) == 2
    for r in range(world):
        ok, nb, fired = results[r]
        assert ok and nb >= 2
        assert fired[0] in ("p6", "p5")  # the bucket holding the last parameters fires first
