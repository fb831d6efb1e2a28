#!/usr/bin/env python
"""Benchmark of the training hot path: one full forward + backward + optimizer step per "step".

    python bench.py --gpus 1 --steps 20 --warmup 5                 # config 5 (the data-parallel VGG-style CNN)
    python bench.py --workload lenet|convbn|mlp|conv3              # configs 1, 2, 4 and the isolated conv backward (3)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...                           # the reference's own CPU path, bounded sample

Default workload: per-GPU batch 256 of 3x64x64, six conv3x3+BN+ReLU layers, three max-pools, linear 16384->100,
cross-entropy, SGD momentum 0.9 — weak scaling, one process per GPU, gradients summed by the library's own bucketed NCCL
all-reduce over a flat gradient arena (nc_dist_*).  Synthetic inputs.  Prints ONE JSON line on rank 0.

Timing: `--repeats` regions of exactly `--steps` steps each, every region bracketed by a barrier + device synchronize on
both sides and timed with CUDA events on the library's stream; per region the maximum over ranks; `value` is the median
region.  Kernel-family times (the roofline objects) come from a separate pass of `--steps` steps with the library's
per-call event timing switched on, so the event records do not sit in the throughput measurement.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

UNIT = "images/s"
WORKLOADS = {
    "vgg": dict(builder="vgg", name="config5_dp_vgg_cnn_b256_per_gpu_3x64x64", metric="train_images_per_sec", optimizer="sgd_momentum_0.9"),
    "convbn": dict(builder="convbn", name="config2_conv_bn_cnn_b128_3x32x32", metric="train_images_per_sec", optimizer="adamw"),
    "lenet": dict(builder="lenet", name="config1_lenet_b64_1x28x28", metric="train_images_per_sec", optimizer="sgd_momentum_0.9"),
    "mlp": dict(builder="mlp", name="config4_mlp_b4096_1024x4096", metric="train_images_per_sec", optimizer="adam"),
    "conv3": dict(builder=None, name="config3_isolated_conv2d_backward_n256_c64_56x56_k64_3x3", metric="conv2d_backward_images_per_sec", optimizer=None),
}
CONV3 = dict(N=256, C=64, H=56, K=64)
TENSOR_FAMILIES = ("conv_fwd", "conv_dx", "conv_dw", "gemm_nt", "gemm_nn", "gemm_tn", "gemm_tt")
BACKWARD_FAMILIES = ("conv_dx", "conv_dw", "gemm_nn", "gemm_tn")
# ncu captures summarised under profiles/ (dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the family's main kernel)
NCU_TRAFFIC = {
    "vgg": (215.2e6, "convh_kernel, 128->128 channel 32x32 layer at batch 256 (77.3 GFLOP launch; algorithmic 269 MB, the output tail was still in L2)"),
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="vgg", choices=sorted(WORKLOADS))
    ap.add_argument("--math", default="tf32", choices=["tf32", "3xtf32", "simt"])
    ap.add_argument("--cpu-sample-batch", type=int, default=0, help="images per reference sample step (default: the host core count, at least 8)")
    ap.add_argument("--cpu-samples", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-dp-check", action="store_true")
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
        pw = [float(s[3]) for s in self.samples if s[3].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            for name, v in zip(names, s[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------
# the reference arm / CPU baseline: the compiled reference on the host cores, bounded sample
# ----------------------------------------------------------------------------------------------
def reference_throughput(workload: str, sample_batch: int, samples: int):
    """Median images/s of `samples` timed steps of the compiled reference (Release flags, OpenMP, all host cores).

    Every sample is ONE training step of a freshly built network (fresh weights, same seeded batch) after one untimed
    step of another fresh network that warms the code and the allocator.  Rebuilding matters: a network trained for a
    few steps on a batch this small memorises it, its loss and gradients underflow into denormal floats, and the
    reference's scalar loops then run an order of magnitude slower (measured: 5.2, 5.1, 5.1, 54.9, 33.2 s for five
    consecutive steps at batch 2), so consecutive steps of one network are not a stationary sample.  The sample batch is
    at least the core count because the reference parallelises its input-gradient loop over the batch
    (src/nn/conv.c:231-233): a smaller batch would leave cores idle there.
    """
    cores = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(cores)
    import numpy as np
    from nocta_b200 import configs
    from oracle import ref_lib
    path_fast = ref_lib.REF_FAST_SO
    if not path_fast.exists() and not ref_lib.REF_SO.exists():
        return None
    api = ref_lib.load(fast=path_fast.exists())
    r = configs.Runner(api, on_device=False)
    batch = sample_batch if sample_batch > 0 else max(cores, 8)

    def one_step():
        if workload == "conv3":
            g = CONV3
            rng = np.random.default_rng(3)
            x = api.from_numpy(rng.standard_normal((batch, g["C"], g["H"], g["H"])).astype(np.float32), requires_grad=True)
            w = api.from_numpy(rng.standard_normal((g["K"], g["C"], 3, 3)).astype(np.float32), requires_grad=True)
            b = api.from_numpy(rng.standard_normal(g["K"]).astype(np.float32), requires_grad=True)
            go = api.from_numpy(rng.standard_normal((batch, g["K"], g["H"], g["H"])).astype(np.float32))
            y = api.nc_conv2d_forward(x, w, b, 1, 1)
            t0 = time.perf_counter()
            rc = api.nc_backward(y, go)           # only the backward is the workload
            dt = time.perf_counter() - t0
            assert rc == 0
            for t in (y, go, x, w, b):
                api.nc_tensor_free(t)
            return batch, dt
        kw = {}
        if workload in ("vgg", "convbn"):
            kw = dict(batch=batch)
        elif workload == "mlp":
            kw = dict(batch=max(batch * 8, 128))
        net, forward, kind, data = configs.BUILDERS[workload](r, **kw)
        tensors = configs.upload(r, kind, data)
        t0 = time.perf_counter()
        configs.train_step(r, net, forward, kind, tensors)
        dt = time.perf_counter() - t0
        net.free_step_tensors()
        configs.free_inputs(r, kind, tensors)
        for m in net.modules.values():
            api.nc_module_free(m)
        return data[0].shape[0], dt

    one_step()  # untimed warm-up
    rates, images = [], 0
    for _ in range(max(1, samples)):
        images, dt = one_step()
        rates.append(images / dt)
    med = statistics.median(rates)
    what = "nc_backward of the isolated convolution" if workload == "conv3" else "training step"
    return {"value": med, "min": min(rates), "max": max(rates), "ms_per_step": 1e3 * images / med, "cores": cores, "images": images,
            "kind": "reference", "samples": len(rates),
            "sample": f"median of {len(rates)} single {what}s (fresh weights each) of the same network at batch {images}; compiled "
                      f"reference, Release flags, OpenMP, {cores} threads; spread {min(rates):.3g}-{max(rates):.3g} images/s"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    samples = max(1, min(args.steps, args.cpu_samples))
    res = reference_throughput(args.workload, args.cpu_sample_batch, samples)
    if res is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref was not built (reference sources absent at build time)"}))
        return
    line = {
        "impl": "reference", "metric": w["metric"], "value": res["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": samples,
        "warmup": 1, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["name"], "note": "reference CPU path on the host cores; bounded sample, see cpu_baseline.sample"},
        "cpu_baseline": {"value": res["value"], "unit": UNIT, "cores": res["cores"], "kind": res["kind"], "sample": res["sample"],
                         "min": res["min"], "max": res["max"]},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------------
def read_families(lib, steps):
    """Per kernel family: device ms per step, calls per step, algorithmic work per step (FLOPs or bytes)."""
    lib.nc_cuda_profile_category_name.restype = C.c_char_p
    lib.nc_cuda_profile_read.argtypes = [C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_ulonglong), C.POINTER(C.c_double)]
    out = {}
    for cat in range(lib.nc_cuda_profile_categories()):
        ms, n, work = C.c_double(0), C.c_ulonglong(0), C.c_double(0)
        lib.nc_cuda_profile_read(cat, C.byref(ms), C.byref(n), C.byref(work))
        if n.value:
            out[lib.nc_cuda_profile_category_name(cat).decode()] = {"ms": ms.value / steps, "calls": n.value / steps, "work": work.value / steps}
    return out


def roofline_objects(fam, peaks, step_ms, workload):
    have = bool(peaks)
    burst = peaks.get("bf16_tflops", 1590.0) / 2.0
    sustained = peaks.get("bf16_tflops_sustained", 1400.0) / 2.0
    hbm = peaks.get("hbm_gbs", 6650.0)
    src = "of measured" if have else "of fallback"

    def tensor(names, label):
        ms = sum(fam[n]["ms"] for n in names if n in fam)
        fl = sum(fam[n]["work"] for n in names if n in fam)
        calls = sum(fam[n]["calls"] for n in names if n in fam)
        if ms <= 0:
            return None
        ach = fl / (ms * 1e9)
        o = {"bound": "tensor", "kernel": label, "achieved": ach, "peak": burst, "unit": "TFLOP/s", "frac": ach / burst,
             "frac_sustained": ach / sustained, "peak_sustained": sustained,
             "peak_source": f"MEASURED_PEAKS.json bf16_tflops / 2 (burst; a TF32 MMA issues at half the bf16 rate); {src}",
             "launches_per_step": calls, "kernel_ms_per_step": ms, "share_of_step": ms / step_ms,
             "algorithmic_gflop_per_step": fl / 1e9,
             "per_family_tflops": {n: fam[n]["work"] / (fam[n]["ms"] * 1e9) for n in names if n in fam and fam[n]["ms"] > 0}}
        return o

    def memory(names, label):
        ms = sum(fam[n]["ms"] for n in names if n in fam)
        by = sum(fam[n]["work"] for n in names if n in fam)
        calls = sum(fam[n]["calls"] for n in names if n in fam)
        if ms <= 0:
            return None
        ach = by / (ms * 1e6)
        return {"bound": "hbm", "kernel": label, "achieved": ach, "peak": hbm, "unit": "GB/s", "frac": ach / hbm,
                "peak_source": f"MEASURED_PEAKS.json hbm_gbs; {src}", "calls_per_step": calls, "kernel_ms_per_step": ms,
                "share_of_step": ms / step_ms, "algorithmic_mb_per_step": by / 1e6, "traffic": None,
                "per_family_gbs": {n: fam[n]["work"] / (fam[n]["ms"] * 1e6) for n in names if n in fam and fam[n]["ms"] > 0}}

    res = {}
    res["roofline"] = tensor(TENSOR_FAMILIES, "tcgen05 kind::tf32 kernels: halo-resident convolutions and weight gradients, per-tap convolutions, GEMM")
    res["roofline_bwd"] = tensor(BACKWARD_FAMILIES, "the backward contractions only (input-gradient and weight-gradient launches)")
    if workload in ("mlp", "convbn"):
        res["roofline_hbm"] = memory(("adam", "layernorm", "activation", "elementwise", "batchnorm", "maxpool"),
                                     "optimizer, normalisation and activation kernels")
    else:
        res["roofline_hbm"] = memory(("batchnorm", "maxpool", "sgd", "conv_first"),
                                     "BatchNorm(+ReLU, +max-pool) forward / backward, the SGD update and the first-layer convolution (3 input channels: bound by its 268 MB output / gradient)")
    if res["roofline"] is not None and workload in NCU_TRAFFIC:
        res["roofline"]["traffic"], note = NCU_TRAFFIC[workload]
        res["roofline"]["traffic_source"] = "ncu capture summarised under profiles/, not measured by this run: " + note
    elif res["roofline"] is not None:
        res["roofline"]["traffic"] = None
    if res["roofline"] is None:   # no tensor-core launches (LeNet's shapes are below the tile sizes): the memory-bound families lead
        res["roofline"] = res["roofline_hbm"]
    return res


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
    lib.nc_cuda_host_alloc.restype = C.c_void_p
    lib.nc_cuda_host_alloc.argtypes = [C.c_size_t]
    lib.nc_cuda_device_error_word.restype = C.c_uint
    lib.nc_cuda_get_stream.restype = C.c_void_p
    stream_ptr = lib.nc_cuda_get_stream()
    stream = torch.cuda.ExternalStream(stream_ptr) if stream_ptr else torch.cuda.default_stream()

    w = WORKLOADS[args.workload]
    if args.workload == "conv3":
        return run_conv3(args, api, r, rank, local_rank, world, stream)
    kw = dict(rank=rank) if args.workload == "vgg" else {}
    net, forward, kind, data = configs.BUILDERS[w["builder"]](r, **kw)
    images = data[0].shape[0]
    tensors = configs.upload(r, kind, data)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- data parallel: the library's own NCCL exchange (bucketed, overlapped with the backward sweep) ----
    dp = None
    dp_check = None
    if world > 1:
        from nocta_b200 import dist_native
        if not args.no_dp_check:
            dp_check = dist_native.check_data_parallel_step(api, r, rank, world, local_rank)
        dp = dist_native.NativeDataParallel(api, net.optimizer, rank, world, bucket_floats=int(os.environ.get("NOCTA_BUCKET_FLOATS", 1 << 21)))

    def step(ts):
        return configs.train_step(r, net, forward, kind, ts, after_backward=(dp.allreduce if dp else None))

    for _ in range(max(args.warmup, 3)):
        step(tensors)
        net.free_step_tensors()
    barrier()

    # ---- timed regions: inputs resident in HBM ----
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    region_ms, launches = [], 0
    for _ in range(max(1, args.repeats)):
        lib.nc_cuda_reset_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            step(tensors)
            net.free_step_tensors()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        launches = int(lib.nc_cuda_launch_count())
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        region_ms.append(ms)
    ms = statistics.median(region_ms)

    # ---- kernel families: a separate pass with per-call event timing ----
    lib.nc_cuda_profile_begin()
    exposed = []
    for _ in range(args.steps):
        step(tensors)
        net.free_step_tensors()
        if dp:
            exposed.append(dp.exposed_ms())
    lib.nc_cuda_profile_end()
    fam = read_families(lib, args.steps)

    # ---- end-to-end: host batch in pinned memory -> device every step, loss read back every step ----
    pinned = []
    for a in (data[0], data[1]):
        a = np.ascontiguousarray(a)
        p = lib.nc_cuda_host_alloc(a.nbytes)
        C.memmove(p, a.ctypes.data, a.nbytes)
        pinned.append((p, a.shape, a.dtype))
    h2d = sum(int(np.prod(s)) * np.dtype(d).itemsize for _, s, d in pinned)
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
        """n steps; returns the losses.  Slot i%2 holds the batch of step i; the upload of step i+1 overlaps step i."""
        losses = []
        if lib.nc_feeder_submit(feeder, 0, px, py) != 0:
            raise RuntimeError("nc_feeder_submit failed")
        for i in range(n):
            slot = i & 1
            xt, yt = TP(), TP()
            if lib.nc_feeder_acquire(feeder, slot, C.byref(xt), C.byref(yt)) != 0:
                raise RuntimeError("nc_feeder_acquire failed")
            if i + 1 < n and lib.nc_feeder_submit(feeder, slot ^ 1, px, py) != 0:
                raise RuntimeError("nc_feeder_submit failed")
            full = (xt, yt) if kind == "ce" else (xt, yt, tensors[2])
            loss = step(full)
            losses.append(float(api.nc_tensor_get_flat(loss, 0)))  # device -> host read of the step's result
            net.free_step_tensors()
            lib.nc_feeder_release(feeder, slot)
        return losses

    e2e_run(2)
    e2e_ms, losses = [], []
    for _ in range(3):
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        losses = e2e_run(args.steps)
        f1.record(stream)
        barrier()
        t_ms = f0.elapsed_time(f1)
        if world > 1:
            t = torch.tensor([t_ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_ms = float(t[0])
        e2e_ms.append(t_ms)
    lib.nc_feeder_free(feeder)
    ms_e2e = statistics.median(e2e_ms)
    clocks = sampler.stop() if rank == 0 else None  # sampled across all timed regions
    errword = int(lib.nc_cuda_device_error_word())

    if rank == 0:
        peaks = {}
        pk = ROOT / "MEASURED_PEAKS.json"
        if pk.exists():
            peaks = json.loads(pk.read_text())
        step_ms = ms / args.steps
        rate = lambda region: images * world * args.steps / (region / 1e3)
        line = {
            "metric": w["metric"], "value": rate(ms), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": {"tf32": "tf32", "3xtf32": "3xtf32", "simt": "f32"}[args.math],
            "data": "synthetic",
            "config": {"workload": w["name"], "per_gpu_batch": images, "global_batch": images * world,
                       "parallelism": f"dp{world}", "grad_buckets": (dp.buckets if dp else 0), "optimizer": w["optimizer"],
                       "l2": "per-step working set (activations and gradients, GBs for the CNN configs, >600 MB for the MLP) exceeds the 126 MB L2; "
                             "no explicit flush" if args.workload != "lenet" else
                             "LeNet's whole working set fits in L2 (launch-bound configuration); no flush: every step rewrites its activations"},
            "repeats": {"n": len(region_ms), "value_is": "median region", "min": rate(max(region_ms)), "max": rate(min(region_ms)),
                        "region_ms": [round(v, 3) for v in region_ms]},
            "clocks": clocks,
            "e2e": {"value": images * world * args.steps / (ms_e2e / 1e3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4, "last_loss": losses[-1], "first_loss": losses[0], "regions": len(e2e_ms)},
            "gpu_launches": launches,
            "device_error_word": errword,
            "kernel_families": {k: {"ms_per_step": round(v["ms"], 4), "calls_per_step": v["calls"],
                                    ("tflops" if k in TENSOR_FAMILIES else "gb_per_s"): (v["work"] / (v["ms"] * (1e9 if k in TENSOR_FAMILIES else 1e6)) if v["ms"] > 0 else None)}
                                for k, v in fam.items()},
        }
        line.update(roofline_objects(fam, peaks, step_ms, args.workload))
        if dp:
            line["dp"] = {"exposed_allreduce_ms_per_step": statistics.median(exposed) if exposed else None,
                          "note": "device time between the end of the backward sweep and the end of the last bucket's all-reduce on rank 0 (profiling pass)",
                          "buckets": dp.buckets, "arena_floats": dp.arena_floats}
        if dp_check is not None:
            line["dp_check"] = dp_check
        if world == 1 and not args.no_cpu_baseline:
            cb = reference_throughput(args.workload, args.cpu_sample_batch, args.cpu_samples)
            if cb:
                line["cpu_baseline"] = {"value": cb["value"], "unit": UNIT, "cores": cb["cores"], "kind": cb["kind"], "sample": cb["sample"],
                                        "min": cb["min"], "max": cb["max"]}
        print(json.dumps(line))
    if dp:
        dp.close()
    if world > 1:
        dist.destroy_process_group()


def run_conv3(args, api, r, rank, local_rank, world, stream):
    """Config 3: dX, dW and db of one 3x3 convolution (N=256, C=64, 56x56, K=64).  A step = the three backward entry
    points on resident channels-last tensors; e2e = nc_conv2d_forward + nc_backward through the nc_* API with x and
    grad_output uploaded from pinned host memory every step and db read back."""
    import numpy as np
    import torch
    from nocta_b200 import capi, cuda_abi
    lib = api.lib
    abi = cuda_abi.load()
    g = CONV3
    N, Ci, H, Co = g["N"], g["C"], g["H"], g["K"]
    rng = np.random.default_rng(3 + rank)
    gen = torch.Generator(device="cuda").manual_seed(3 + rank)
    x = torch.randn(N, H, H, Ci, device="cuda", generator=gen)
    go = torch.randn(N, H, H, Co, device="cuda", generator=gen)
    wt = torch.randn(Co, Ci, 3, 3, device="cuda", generator=gen)
    dx, dw, db = torch.empty_like(x), torch.empty_like(wt), torch.empty(Co, device="cuda")
    xs = cuda_abi.size4([H * H * Ci, 1, H * Ci, Ci])
    ys = cuda_abi.size4([H * H * Co, 1, H * Co, Co])
    P = lambda t: C.c_void_p(t.data_ptr())
    sp = C.c_void_p(lib.nc_cuda_get_stream())

    def step():
        assert abi.nc_cuda_conv2d_backward_input_f32_ex(P(dx), xs, P(go), ys, P(wt), N, Ci, H, H, Co, 3, 3, 1, 1, sp) == 0
        assert abi.nc_cuda_conv2d_backward_weight_f32_ex(P(dw), P(db), P(go), ys, P(x), xs, N, Ci, H, H, Co, 3, 3, 1, 1, sp) == 0

    warm = max(args.warmup, 10)
    for _ in range(warm):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    steps = max(args.steps, 50) if args.steps == 20 else args.steps   # default: 50 timed launches of each entry point
    region_ms = []
    for _ in range(max(1, args.repeats)):
        lib.nc_cuda_reset_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(steps):
            step()
        e1.record(stream)
        torch.cuda.synchronize()
        region_ms.append(e0.elapsed_time(e1))
    launches = int(lib.nc_cuda_launch_count())
    ms = statistics.median(region_ms)
    lib.nc_cuda_profile_begin()
    for _ in range(steps):
        step()
    lib.nc_cuda_profile_end()
    fam = read_families(lib, steps)

    # e2e through the nc_* API: upload x and grad_output (pinned host memory), forward, backward, read db back
    lib.nc_cuda_host_alloc.restype = C.c_void_p
    xh = rng.standard_normal((N, Ci, H, H)).astype(np.float32)
    gh = rng.standard_normal((N, Co, H, H)).astype(np.float32)
    px, pg = lib.nc_cuda_host_alloc(xh.nbytes), lib.nc_cuda_host_alloc(gh.nbytes)
    C.memmove(px, xh.ctypes.data, xh.nbytes)
    C.memmove(pg, gh.ctypes.data, gh.nbytes)
    TP = C.POINTER(capi.Tensor)
    lib.nc_feeder_create.restype = C.c_void_p
    lib.nc_feeder_create.argtypes = [C.c_int, C.POINTER(C.c_size_t), C.c_size_t, C.c_int, C.POINTER(C.c_size_t), C.c_size_t, C.c_int]
    lib.nc_feeder_submit.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    lib.nc_feeder_acquire.argtypes = [C.c_void_p, C.c_int, C.POINTER(TP), C.POINTER(TP)]
    lib.nc_feeder_release.argtypes = [C.c_void_p, C.c_int]
    lib.nc_feeder_free.argtypes = [C.c_void_p]
    feeder = lib.nc_feeder_create(2, capi.shape_arr(xh.shape), 4, capi.NC_F32, capi.shape_arr(gh.shape), 4, capi.NC_F32)
    wn = r.tensor(rng.standard_normal((Co, Ci, 3, 3)).astype(np.float32), requires_grad=True)
    bn = r.tensor(rng.standard_normal(Co).astype(np.float32), requires_grad=True)

    def e2e_run(n):
        last = 0.0
        assert lib.nc_feeder_submit(feeder, 0, px, pg) == 0
        for i in range(n):
            slot = i & 1
            xt, gt = TP(), TP()
            assert lib.nc_feeder_acquire(feeder, slot, C.byref(xt), C.byref(gt)) == 0
            if i + 1 < n:
                assert lib.nc_feeder_submit(feeder, slot ^ 1, px, pg) == 0
            api.nc_tensor_requires_grad_(xt, True)
            api.nc_tensor_zero_grad_(xt); api.nc_tensor_zero_grad_(wn); api.nc_tensor_zero_grad_(bn)
            y = api.nc_conv2d_forward(xt, wn, bn, 1, 1)
            assert y and api.nc_backward(y, gt) == 0
            last = float(api.nc_tensor_get_flat(bn.contents.grad, 0))   # device -> host read of a result
            api.nc_tensor_free(y)
            lib.nc_feeder_release(feeder, slot)
        return last

    e2e_steps = min(steps, 10)
    e2e_run(2)
    torch.cuda.synchronize()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    e2e_run(e2e_steps)
    f1.record(stream)
    torch.cuda.synchronize()
    ms_e2e = f0.elapsed_time(f1)
    lib.nc_feeder_free(feeder)
    clocks = sampler.stop()
    errword = int(lib.nc_cuda_device_error_word())
    peaks = {}
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    step_ms = ms / steps
    w = WORKLOADS["conv3"]
    rate = lambda region: N * steps / (region / 1e3)
    line = {
        "metric": w["metric"], "value": rate(ms), "unit": UNIT, "n_gpus": 1, "steps": steps, "warmup": warm,
        "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": {"tf32": "tf32", "3xtf32": "3xtf32", "simt": "f32"}[args.math], "data": "synthetic",
        "config": {"workload": w["name"], "per_gpu_batch": N, "step": "dX + dW + db of the layer on resident channels-last tensors",
                   "l2": "x, grad_output and dX are 205 MB each: larger than the 126 MB L2, no explicit flush"},
        "repeats": {"n": len(region_ms), "value_is": "median region", "min": rate(max(region_ms)), "max": rate(min(region_ms))},
        "clocks": clocks,
        "e2e": {"value": N * e2e_steps / (ms_e2e / 1e3), "unit": UNIT, "h2d_bytes_per_step": int(xh.nbytes + gh.nbytes), "d2h_bytes_per_step": 8,
                "path": "nc_conv2d_forward + nc_backward with x and grad_output uploaded every step (the forward is inside this number)"},
        "gpu_launches": launches, "device_error_word": errword,
        "kernel_families": {k: {"ms_per_step": round(v["ms"], 4), "calls_per_step": v["calls"],
                                ("tflops" if k in TENSOR_FAMILIES else "gb_per_s"): (v["work"] / (v["ms"] * (1e9 if k in TENSOR_FAMILIES else 1e6)) if v["ms"] > 0 else None)}
                            for k, v in fam.items()},
    }
    line.update(roofline_objects(fam, peaks, step_ms, "conv3"))
    line["roofline_hbm"] = None
    if rank == 0:
        if not args.no_cpu_baseline:
            cb = reference_throughput("conv3", args.cpu_sample_batch, args.cpu_samples)
            if cb:
                line["cpu_baseline"] = {"value": cb["value"], "unit": UNIT, "cores": cb["cores"], "kind": cb["kind"], "sample": cb["sample"],
                                        "min": cb["min"], "max": cb["max"]}
        print(json.dumps(line))


def main():
    args = parse()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
