"""Data-parallel gradient exchange: one process per GPU, a flat gradient arena cut into buckets, one
NCCL all-reduce per bucket started as soon as the backward sweep has produced every gradient in it,
so the exchange of the late layers overlaps the backward of the early ones.

The class is engine-agnostic: it works on any 1-D torch tensor (the arena) and a list of
(key, offset, numel) entries, and is told through `on_ready(key)` when an entry is final.  On the GPU
the arena is the device range returned by nc_optimizer_flatten_grads and `on_ready` is driven by the
nc_set_grad_ready_hook callback; the CPU tests drive it by hand over gloo.
The 1/world scale is NOT applied here: it is folded into the optimizer kernel (nc_optimizer_set_grad_scale).
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class Bucket:
    start: int
    stop: int
    keys: list = field(default_factory=list)
    pending: int = 0
    work: object = None


class BucketedAllReduce:
    def __init__(self, arena, entries, bucket_floats: int = 1 << 20, group=None):
        """entries: [(key, offset, numel)] in arena order (offsets ascending).  Buckets are contiguous
        arena ranges of about `bucket_floats` elements; the backward sweep fills the arena from the end
        (last layer first), so the last bucket completes first."""
        import torch.distributed as dist
        self.dist = dist
        self.arena = arena
        self.group = group
        self.buckets: list[Bucket] = []
        self.key_to_bucket = {}
        entries = sorted(entries, key=lambda e: e[1])
        cur = None
        for key, off, n in reversed(entries):  # build from the end so the first-ready bucket is tight
            if cur is None or (cur.stop - off) > bucket_floats and cur.keys:
                cur = Bucket(start=off, stop=off + n if cur is None else cur.start)
                if len(self.buckets) == 0:
                    cur.stop = arena.numel()
                self.buckets.append(cur)
            cur.start = off
            cur.keys.append(key)
            self.key_to_bucket[key] = cur
        if self.buckets:
            self.buckets[-1].start = 0
        self.reset()

    def reset(self):
        for b in self.buckets:
            b.pending = len(b.keys)
            b.work = None

    def on_ready(self, key):
        b = self.key_to_bucket.get(key)
        if b is None or b.work is not None:
            return
        b.pending -= 1
        if b.pending <= 0:
            b.work = self.dist.all_reduce(self.arena[b.start:b.stop], group=self.group, async_op=True)

    def finish(self):
        """Start whatever was not triggered (e.g. parameters without a gradient this step) and wait."""
        for b in self.buckets:
            if b.work is None:
                b.work = self.dist.all_reduce(self.arena[b.start:b.stop], group=self.group, async_op=True)
        for b in self.buckets:
            b.work.wait()
        self.reset()

    def ranges(self):
        return [(b.start, b.stop, len(b.keys)) for b in self.buckets]
