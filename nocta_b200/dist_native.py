"""Harness-side bindings of the host library's data-parallel layer (nocta_b200/host/dist.c).

  BucketPlan           ctypes view of nc_bucket_plan, the host-only bucket scheduler; the CPU tests drive it over gloo.
  NativeDataParallel   nc_dist: the plan + NCCL inside the C library.  Python only carries rank 0's 128-byte NCCL id to
                       the other ranks (over the torch.distributed group the benchmark already has for its barriers).
  check_data_parallel_step   one checked training step on a small network: the all-reduced gradient arena equals the
                       float64 sum of the ranks' own gradients, the updated parameters are bit-identical on every rank,
                       and on rank 0 they equal the compiled reference applying the mean of the per-shard gradients.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import capi

_sz = C.c_size_t


def _bind_plan(lib):
    if getattr(lib, "_plan_bound", False):
        return
    lib.nc_bucket_plan_create.restype = C.c_void_p
    lib.nc_bucket_plan_create.argtypes = [_sz, C.POINTER(_sz), C.POINTER(_sz), _sz, _sz]
    lib.nc_bucket_plan_free.argtypes = [C.c_void_p]
    lib.nc_bucket_plan_free.restype = None
    lib.nc_bucket_plan_count.restype = _sz
    lib.nc_bucket_plan_count.argtypes = [C.c_void_p]
    lib.nc_bucket_plan_range.argtypes = [C.c_void_p, _sz, C.POINTER(_sz), C.POINTER(_sz)]
    lib.nc_bucket_plan_range.restype = None
    lib.nc_bucket_plan_begin_step.argtypes = [C.c_void_p]
    lib.nc_bucket_plan_begin_step.restype = None
    lib.nc_bucket_plan_on_ready.argtypes = [C.c_void_p, _sz]
    lib.nc_bucket_plan_next_unfired.argtypes = [C.c_void_p]
    lib.nc_bucket_plan_end_step.argtypes = [C.c_void_p]
    lib._plan_bound = True


class BucketPlan:
    """nc_bucket_plan over entries [(offset, numel)] in arena order."""

    def __init__(self, lib, entries, arena_floats: int, bucket_floats: int):
        _bind_plan(lib)
        self.lib = lib
        n = len(entries)
        offs = (_sz * n)(*[int(o) for o, _ in entries])
        nums = (_sz * n)(*[int(m) for _, m in entries])
        self.p = lib.nc_bucket_plan_create(n, offs, nums, arena_floats, bucket_floats)
        if not self.p:
            raise RuntimeError("nc_bucket_plan_create failed")

    def count(self) -> int:
        return int(self.lib.nc_bucket_plan_count(self.p))

    def range(self, b: int):
        s, e = _sz(0), _sz(0)
        self.lib.nc_bucket_plan_range(self.p, b, C.byref(s), C.byref(e))
        return s.value, e.value

    def on_ready(self, entry: int) -> int:
        return int(self.lib.nc_bucket_plan_on_ready(self.p, entry))

    def next_unfired(self) -> int:
        return int(self.lib.nc_bucket_plan_next_unfired(self.p))

    def end_step(self) -> int:
        return int(self.lib.nc_bucket_plan_end_step(self.p))

    def close(self):
        if self.p:
            self.lib.nc_bucket_plan_free(self.p)
            self.p = None


def load_host_library():
    """libnocta.so as a plain CDLL (no device needed for the bucket plan)."""
    path = Path(__file__).resolve().parent / "lib" / "libnocta.so"
    if not path.exists():
        raise RuntimeError(f"{path} is missing: run `python -m nocta_b200.build`")
    return C.CDLL(str(path))


def _bind_dist(lib):
    if getattr(lib, "_dist_bound", False):
        return
    lib.nc_dist_unique_id.argtypes = [C.c_void_p]
    lib.nc_dist_init.restype = C.c_void_p
    lib.nc_dist_init.argtypes = [C.c_int, C.c_int, C.c_void_p, capi.OptimizerP, _sz]
    lib.nc_dist_allreduce_grads.argtypes = [C.c_void_p]
    lib.nc_dist_num_buckets.restype = _sz
    lib.nc_dist_num_buckets.argtypes = [C.c_void_p]
    lib.nc_dist_arena.restype = C.c_void_p
    lib.nc_dist_arena.argtypes = [C.c_void_p, C.POINTER(_sz)]
    lib.nc_dist_exposed_ms.restype = C.c_double
    lib.nc_dist_exposed_ms.argtypes = [C.c_void_p]
    lib.nc_dist_free.argtypes = [C.c_void_p]
    lib.nc_dist_free.restype = None
    lib._dist_bound = True


class NativeDataParallel:
    def __init__(self, api, optimizer, rank: int, world: int, bucket_floats: int = 1 << 21):
        import torch
        import torch.distributed as dist
        lib = api.lib
        _bind_dist(lib)
        self.lib = lib
        ident = (C.c_ubyte * 128)()
        if rank == 0 and lib.nc_dist_unique_id(ident) != 0:
            raise RuntimeError("nc_dist_unique_id failed")
        t = torch.tensor(list(ident), dtype=torch.uint8, device="cuda")
        dist.broadcast(t, src=0)
        ident = (C.c_ubyte * 128)(*t.cpu().tolist())
        self.d = lib.nc_dist_init(rank, world, ident, optimizer, bucket_floats)
        if not self.d:
            raise RuntimeError("nc_dist_init failed")
        self.buckets = int(lib.nc_dist_num_buckets(self.d))
        n = _sz(0)
        self.arena_ptr = lib.nc_dist_arena(self.d, C.byref(n))
        self.arena_floats = int(n.value)

    def allreduce(self):
        rc = self.lib.nc_dist_allreduce_grads(self.d)
        if rc != 0:
            raise RuntimeError(f"nc_dist_allreduce_grads failed with {rc}")

    def exposed_ms(self) -> float:
        return float(self.lib.nc_dist_exposed_ms(self.d))

    def arena_tensor(self):
        import torch

        class _Dev:
            pass
        o = _Dev()
        o.__cuda_array_interface__ = {"shape": (self.arena_floats,), "typestr": "<f4", "data": (self.arena_ptr, False), "version": 2}
        return torch.as_tensor(o, device="cuda")

    def close(self):
        if self.d:
            self.lib.nc_dist_free(self.d)
            self.d = None


SMALL_NET = dict(batch=8, size=16, widths=(32, 64, 128), classes=10)


def check_data_parallel_step(api, runner, rank: int, world: int, local_rank: int) -> dict:
    """Two checked steps of the small VGG-style network in 3xTF32 mode (the first sends every bucket after the sweep, the
    second uses the learned plan and sends buckets from inside the sweep).  Returns a dict for the benchmark's JSON line."""
    import torch
    import torch.distributed as dist
    from . import configs
    lib = api.lib
    prev_mode = lib.nc_cuda_get_math_mode()
    lib.nc_cuda_set_math_mode(2)
    out = {"ok": False, "steps": 2}
    try:
        net, forward, kind, data = configs.build_vgg(runner, rank=rank, **SMALL_NET)
        tensors = configs.upload(runner, kind, data)
        dp = NativeDataParallel(api, net.optimizer, rank, world, bucket_floats=1 << 15)
        arena = dp.arena_tensor()
        worst_sum = 0.0
        identical = True
        first_params = None
        for step in range(2):
            pre = {}

            def after_backward():
                torch.cuda.synchronize()
                if step == 0:   # nothing has been sent yet: the arena holds this rank's own gradients
                    pre["mine"] = arena.clone()
                dp.allreduce()

            configs.train_step(runner, net, forward, kind, tensors, after_backward=after_backward if step == 0 else dp.allreduce)
            net.free_step_tensors()
            torch.cuda.synchronize()
            if step == 0:
                shards = [torch.zeros_like(pre["mine"]) for _ in range(world)]
                dist.all_gather(shards, pre["mine"])
                want = torch.stack([s.double() for s in shards]).sum(0)
                got = arena.double()
                scale = float(want.abs().max()) or 1.0
                worst_sum = float((got - want).abs().max()) / scale
                first_params = {n: api.to_numpy(p) for n, p in net.named_params()}
            # parameters bit-identical on every rank
            flat = torch.cat([torch.from_numpy(api.to_numpy(p).ravel()) for _, p in net.named_params()]).cuda()
            ref0 = flat.clone()
            dist.broadcast(ref0, src=0)
            same = torch.tensor([1 if torch.equal(flat, ref0) else 0], device="cuda")
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            identical = identical and bool(int(same[0]))
        out.update({"allreduce_vs_float64_sum_max_rel_err": worst_sum, "params_bit_identical_across_ranks": identical,
                    "buckets": dp.buckets})
        # rank 0: the compiled reference applying the mean of the per-shard gradients (first SGD-momentum step: v = g)
        vs_ref = None
        if rank == 0:
            from oracle import ref_lib
            if ref_lib.available():
                ref = configs.Runner(ref_lib.load(), on_device=False)
                gsum, p0 = None, None
                for w in range(world):
                    rnet, rfwd, rkind, rdata = configs.build_vgg(ref, rank=w, **SMALL_NET)
                    rt = configs.upload(ref, rkind, rdata)
                    ref.api.nc_optimizer_zero_grad(rnet.optimizer)
                    o = rfwd(rnet, rt[0])
                    loss = ref.api.nc_cross_entropy_loss(o, rt[1])
                    rnet.keep.append(loss)
                    assert ref.api.nc_backward_scalar(loss) == 0
                    g = {n: ref.api.grad_numpy(p) for n, p in rnet.named_params()}
                    if p0 is None:
                        p0 = {n: ref.api.to_numpy(p) for n, p in rnet.named_params()}
                        gsum = {n: (v.astype(np.float64) if v is not None else None) for n, v in g.items()}
                    else:
                        for n, v in g.items():
                            if v is not None:
                                gsum[n] += v
                    rnet.free_step_tensors()
                vs_ref = 0.0
                for n, g in gsum.items():
                    if g is None or n.endswith("running_mean") or n.endswith("running_var"):
                        continue
                    want = p0[n].astype(np.float64) - 0.01 * g / world
                    scale = float(np.abs(want).max()) or 1.0
                    vs_ref = max(vs_ref, float(np.abs(first_params[n] - want).max()) / scale)
        out["updated_weights_vs_reference_mean_gradient_max_rel_err"] = vs_ref
        out["ok"] = bool(worst_sum <= 1e-6 and identical and (vs_ref is None or vs_ref <= 2e-5))
        dp.close()
        configs.free_inputs(runner, kind, tensors)
    finally:
        lib.nc_cuda_set_math_mode(prev_mode)
    return out
