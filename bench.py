#!/usr/bin/env python
"""Benchmark of the training hot path: images/s for one full forward + backward + optimizer step.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...        # the reference's own CPU path, bounded sample

Workload: the data-parallel VGG-style CNN (per-GPU batch 256 of 3x64x64, six conv3x3+BN+ReLU layers,
three max-pools, linear 16384->100, cross-entropy, SGD momentum 0.9) — weak scaling, one process per
GPU, gradients summed with one NCCL all-reduce over a flat gradient arena.  Synthetic inputs.
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "train_images_per_sec"
UNIT = "images/s"
WORKLOADS = {
    "vgg": dict(builder="vgg", batch=256, name="config5_dp_vgg_cnn_b256_per_gpu_3x64x64"),
    "convbn": dict(builder="convbn", batch=128, name="config2_conv_bn_cnn_b128_3x32x32"),
    "lenet": dict(builder="lenet", batch=64, name="config1_lenet_b64_1x28x28"),
    "mlp": dict(builder="mlp", batch=4096, name="config4_mlp_b4096_1024x4096"),
}
# algorithmic multiply-adds of one forward pass per image (conv + linear contractions); a training step
# costs 3x that minus the input gradient of the first layer, which is never needed
VGG_FWD_MACS_PER_IMAGE = 156.85e9 / 256
VGG_FIRST_LAYER_MACS_PER_IMAGE = 1.81e9 / 256


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="vgg", choices=sorted(WORKLOADS))
    ap.add_argument("--math", default="tf32", choices=["tf32", "3xtf32", "simt"])
    ap.add_argument("--cpu-sample-batch", type=int, default=2)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


# ----------------------------------------------------------------------------------------------
# clocks during the timed region
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit())
        mx = [float(s[2]) for s in self.samples if s[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            for name, v in zip(names, s[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------
# the reference arm / CPU baseline: the compiled reference on the host cores, bounded sample
# ----------------------------------------------------------------------------------------------
def reference_throughput(workload: str, sample_batch: int, steps: int, warmup: int):
    cores = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(cores)
    from nocta_b200 import configs
    from oracle import ref_lib
    path_fast = ref_lib.REF_FAST_SO
    if not path_fast.exists() and not ref_lib.REF_SO.exists():
        return None
    api = ref_lib.load(fast=path_fast.exists())
    r = configs.Runner(api, on_device=False)
    kw = dict(batch=sample_batch) if workload in ("vgg", "convbn") else {}
    if workload == "mlp":
        kw = dict(batch=max(sample_batch * 16, 32))
    net, forward, kind, data = configs.BUILDERS[workload](r, **kw)
    tensors = configs.upload(r, kind, data)
    images = data[0].shape[0]
    for _ in range(warmup):
        configs.train_step(r, net, forward, kind, tensors)
        net.free_step_tensors()
    t0 = time.perf_counter()
    for _ in range(steps):
        configs.train_step(r, net, forward, kind, tensors)
        net.free_step_tensors()
    dt = time.perf_counter() - t0
    return {"value": images * steps / dt, "ms_per_step": 1e3 * dt / steps, "cores": cores, "images": images,
            "kind": "reference",
            "sample": f"{steps} step(s) of the same network at batch {images} (reference Release flags, OpenMP, "
                      f"{cores} threads); images/s does not depend on the batch for the reference's per-image loops"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    steps = max(1, min(args.steps, 3))
    res = reference_throughput(args.workload, args.cpu_sample_batch, steps, min(args.warmup, 1))
    if res is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref was not built (reference sources absent at build time)"}))
        return
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": min(args.warmup, 1), "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["name"], "note": "reference CPU path on the host cores; bounded sample, see cpu_baseline.sample"},
        "cpu_baseline": {"value": res["value"], "unit": UNIT, "cores": res["cores"], "kind": res["kind"], "sample": res["sample"]},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------------
class _DevMem:
    """Exposes a raw device range to torch (zero-copy) through the CUDA array interface."""

    def __init__(self, ptr: int, n_floats: int):
        self.__cuda_array_interface__ = {"shape": (n_floats,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def run_ours(args):
    import numpy as np
    import torch

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus or world == 1, (world, args.gpus)
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from nocta_b200 import capi, configs
    api = configs.load_library()
    lib = api.lib
    lib.nc_cuda_set_device.argtypes = [C.c_int]
    lib.nc_cuda_set_device(local_rank)
    r = configs.Runner(api, on_device=True)
    lib.nc_cuda_set_math_mode.argtypes = [C.c_int]
    lib.nc_cuda_set_math_mode({"tf32": 0, "3xtf32": 2, "simt": 3}[args.math])
    lib.nc_cuda_launch_count.restype = C.c_ulonglong
    lib.nc_cuda_tc_profile_end.argtypes = [C.POINTER(C.c_double), C.POINTER(C.c_ulonglong), C.POINTER(C.c_double)]
    lib.nc_cuda_host_alloc.restype = C.c_void_p
    lib.nc_cuda_host_alloc.argtypes = [C.c_size_t]
    lib.nc_cuda_device_error_word.restype = C.c_uint

    w = WORKLOADS[args.workload]
    kw = dict(rank=rank) if args.workload == "vgg" else {}
    net, forward, kind, data = configs.BUILDERS[w["builder"]](r, **kw)
    images = data[0].shape[0]
    tensors = configs.upload(r, kind, data)

    # data parallel: one flat gradient arena, one all-reduce, 1/world folded into the update
    sync = None
    hook_keepalive = None
    if world > 1:
        from nocta_b200.dist import BucketedAllReduce
        lib.nc_optimizer_flatten_grads.restype = C.c_void_p
        lib.nc_optimizer_flatten_grads.argtypes = [capi.OptimizerP, C.POINTER(C.c_size_t)]
        n = C.c_size_t(0)
        ptr = lib.nc_optimizer_flatten_grads(net.optimizer, C.byref(n))
        assert ptr, "gradient arena allocation failed"
        arena = torch.as_tensor(_DevMem(ptr, n.value), device=f"cuda:{local_rank}")
        opt = net.optimizer.contents
        entries, off = [], 0
        for i in range(opt.n_params):
            pt = opt.params[i]
            entries.append((C.addressof(pt.contents), off, pt.contents.numel))
            off += (pt.contents.numel + 63) // 64 * 64
        assert off == n.value
        sync = BucketedAllReduce(arena, entries, bucket_floats=int(os.environ.get("NOCTA_BUCKET_FLOATS", 1 << 21)))  # 2 buckets for config 5: measured faster than 4 or 7
        HOOK = C.CFUNCTYPE(None, capi.TensorP, C.c_void_p)
        hook_keepalive = HOOK(lambda leaf, ctx: sync.on_ready(C.addressof(leaf.contents)))
        lib.nc_set_grad_ready_hook.argtypes = [HOOK, C.c_void_p]
        lib.nc_set_grad_ready_hook(hook_keepalive, None)
        lib.nc_optimizer_set_grad_scale.argtypes = [capi.OptimizerP, C.c_double]
        lib.nc_optimizer_set_grad_scale(net.optimizer, 1.0 / world)

    def allreduce():
        if sync is not None:
            sync.finish()

    def step(ts):
        loss = configs.train_step(r, net, forward, kind, ts, after_backward=allreduce)
        return loss

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step(tensors)
        net.free_step_tensors()
    barrier()

    # ---- timed region: inputs resident in HBM ----
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    lib.nc_cuda_reset_launch_count()
    lib.nc_cuda_tc_profile_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step(tensors)
        net.free_step_tensors()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = int(lib.nc_cuda_launch_count())
    tc_ms, tc_n, tc_flops = C.c_double(0), C.c_ulonglong(0), C.c_double(0)
    lib.nc_cuda_tc_profile_end(C.byref(tc_ms), C.byref(tc_n), C.byref(tc_flops))
    # ---- end-to-end: host batch in pinned memory -> device every step, loss read back every step ----
    pinned = []
    for a in (data[0], data[1]) if kind == "ce" else (data[0], data[1]):
        a = np.ascontiguousarray(a)
        p = lib.nc_cuda_host_alloc(a.nbytes)
        C.memmove(p, a.ctypes.data, a.nbytes)
        pinned.append((p, a.shape, a.dtype))
    h2d = sum(int(np.prod(s)) * np.dtype(d).itemsize for _, s, d in pinned)

    # The batch of step i+1 is uploaded by the library's double-buffered feeder (copy stream) while step i
    # runs; every step still copies its own inputs host -> device inside the timed region.
    TP = C.POINTER(capi.Tensor)
    lib.nc_feeder_create.restype = C.c_void_p
    lib.nc_feeder_create.argtypes = [C.c_int, C.POINTER(C.c_size_t), C.c_size_t, C.c_int, C.POINTER(C.c_size_t), C.c_size_t, C.c_int]
    lib.nc_feeder_submit.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    lib.nc_feeder_acquire.argtypes = [C.c_void_p, C.c_int, C.POINTER(TP), C.POINTER(TP)]
    lib.nc_feeder_release.argtypes = [C.c_void_p, C.c_int]
    lib.nc_feeder_free.argtypes = [C.c_void_p]
    lib.nc_feeder_free.restype = None

    def nc_dt(dtype):
        return capi.NC_I64 if np.dtype(dtype) == np.int64 else capi.NC_F32

    (px, xshape, xdt), (py, yshape, ydt) = pinned
    feeder = lib.nc_feeder_create(2, capi.shape_arr(xshape), len(xshape), nc_dt(xdt), capi.shape_arr(yshape), len(yshape), nc_dt(ydt))
    if not feeder:
        raise RuntimeError("nc_feeder_create failed")

    def e2e_run(n):
        """n steps; returns the last loss.  Slot i%2 holds the batch of step i."""
        last = 0.0
        if lib.nc_feeder_submit(feeder, 0, px, py) != 0:
            raise RuntimeError("nc_feeder_submit failed")
        for i in range(n):
            slot = i & 1
            xt, yt = TP(), TP()
            if lib.nc_feeder_acquire(feeder, slot, C.byref(xt), C.byref(yt)) != 0:
                raise RuntimeError("nc_feeder_acquire failed")
            if i + 1 < n and lib.nc_feeder_submit(feeder, slot ^ 1, px, py) != 0:  # next batch: overlaps this step
                raise RuntimeError("nc_feeder_submit failed")
            full = (xt, yt) if kind == "ce" else (xt, yt, tensors[2])
            loss = step(full)
            last = float(api.nc_tensor_get_flat(loss, 0))  # device -> host read of the step's result
            net.free_step_tensors()
            lib.nc_feeder_release(feeder, slot)
        return last

    e2e_run(2)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    last = e2e_run(args.steps)
    f1.record()
    barrier()
    lib.nc_feeder_free(feeder)
    ms_e2e = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else None  # sampled across both timed regions
    errword = int(lib.nc_cuda_device_error_word())

    # max over ranks
    if world > 1:
        t = torch.tensor([ms, ms_e2e], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])

    if rank == 0:
        peaks = {}
        pk = ROOT / "MEASURED_PEAKS.json"
        if pk.exists():
            peaks = json.loads(pk.read_text())
        tf32_peak = (peaks.get("bf16_tflops_sustained", 1400.0)) / 2.0
        achieved = tc_flops.value / (tc_ms.value * 1e9) if tc_ms.value > 0 else None
        roofline = {
            "bound": "tensor", "kernel": "convh_kernel + tc_kernel (tcgen05 kind::tf32 convolutions, weight gradients, GEMM)",
            "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s",
            "frac": (achieved / tf32_peak) if achieved else None,
            "peak_source": ("MEASURED_PEAKS.json bf16_tflops_sustained / 2 (TF32 issues at half the bf16 rate); of measured"
                            if pk.exists() else "fallback 1400/2; of fallback"),
            "launches_timed": int(tc_n.value), "kernel_ms_per_step": tc_ms.value / args.steps,
            "share_of_step": tc_ms.value / ms if ms > 0 else None,
            # dram__bytes_read.sum + dram__bytes_write.sum of ONE launch, from the ncu capture summarised in
            # profiles/convh_and_dw_kernel_conv128x128_32x32_b256.md (128->128 channel 32x32 layer, batch 256):
            # it equals that launch's algorithmic bytes (134.2 MB in, 134.2 MB out, 0.6 MB weights; 50 MB of the
            # output were still in L2 when the kernel ended)
            "traffic": 219.0e6, "traffic_unit": "bytes per launch (convh_kernel, 77.3 GFLOP launch)",
        }
        line = {
            "metric": METRIC, "value": images * world * args.steps / (ms / 1e3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": {"tf32": "tf32", "3xtf32": "3xtf32", "simt": "f32"}[args.math],
            "data": "synthetic",
            "config": {"workload": w["name"], "per_gpu_batch": images, "global_batch": images * world,
                       "parallelism": f"dp{world}", "grad_buckets": (len(sync.buckets) if sync else 0), "optimizer": "sgd_momentum_0.9" if args.workload in ("vgg", "lenet") else "adam",
                       "l2": "per-step working set (~3 GB of activations) exceeds the 126 MB L2; no explicit flush"},
            "clocks": clocks,
            "e2e": {"value": images * world * args.steps / (ms_e2e / 1e3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4, "last_loss": last},
            "gpu_launches": launches,
            "roofline": roofline,
            "device_error_word": errword,
        }
        if world == 1 and not args.no_cpu_baseline:
            cb = reference_throughput(args.workload, args.cpu_sample_batch, 1, 0)
            if cb:
                line["cpu_baseline"] = {"value": cb["value"], "unit": UNIT, "cores": cb["cores"], "kind": cb["kind"], "sample": cb["sample"]}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
