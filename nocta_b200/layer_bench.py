"""Per-layer timing of the convolution kernels through the nc_cuda_* C ABI.

    python -m nocta_b200.layer_bench --layers 256,128,32,128 [--iters 5] [--warmup 2] [--mode 0]

--norm N,C,H times the BatchNorm kernels the same way.  Each --layers entry is N,Cin,H,Cout (square images, 3x3 filters, stride 1, padding 1, channels-last
activations as the training path uses them).  Prints the CUDA-event time and the algorithmic TFLOP/s of the
forward, input-gradient and weight-gradient launches.  With --iters 1 --warmup 1 it is a small, bounded
workload suitable for a profiler capture of single launches.
"""
from __future__ import annotations

import argparse
import ctypes as C


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", nargs="*", default=["256,128,32,128"])
    ap.add_argument("--norm", nargs="*", default=[], help="N,C,H entries: time BatchNorm(+ReLU) forward / backward and the fused "
                    "BatchNorm+ReLU+max-pool pair on a channels-last (N, H, H, C) tensor")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--mode", type=int, default=0, help="0 TF32, 1 TF32 with in-kernel rounding, 2 3xTF32, 3 FP32 SIMT")
    args = ap.parse_args()

    import torch

    from nocta_b200 import cuda_abi

    if not torch.cuda.is_available():
        raise SystemExit("layer_bench needs a CUDA device")
    abi = cuda_abi.load()
    abi.nc_cuda_set_math_mode(args.mode)
    dev = "cuda"

    def P(t):
        return C.c_void_p(t.data_ptr())

    def timed(fn):
        for _ in range(args.warmup):
            assert fn() == 0
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.iters):
            assert fn() == 0
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / args.iters

    for spec in args.layers:
        N, Cin, H, Cout = (int(v) for v in spec.split(","))
        g = torch.Generator(device=dev).manual_seed(1)
        x = torch.randn(N, H, H, Cin, device=dev, generator=g)
        w = torch.randn(Cout, Cin, 3, 3, device=dev, generator=g)
        dy = torch.randn(N, H, H, Cout, device=dev, generator=g)
        y, dx, dw = torch.empty_like(dy), torch.empty_like(x), torch.empty_like(w)
        xs = cuda_abi.size4([H * H * Cin, 1, H * Cin, Cin])    # NCHW shape, channels-last memory
        ys = cuda_abi.size4([H * H * Cout, 1, H * Cout, Cout])
        gflop = 2.0 * N * H * H * Cout * Cin * 9 / 1e9
        t_f = timed(lambda: abi.nc_cuda_conv2d_forward_f32_ex(P(y), ys, P(x), xs, P(w), None, N, Cin, H, H, Cout, 3, 3, 1, 1, None))
        t_x = timed(lambda: abi.nc_cuda_conv2d_backward_input_f32_ex(P(dx), xs, P(dy), ys, P(w), N, Cin, H, H, Cout, 3, 3, 1, 1, None))
        t_w = timed(lambda: abi.nc_cuda_conv2d_backward_weight_f32_ex(P(dw), None, P(dy), ys, P(x), xs, N, Cin, H, H, Cout, 3, 3, 1, 1, None))
        print(f"layer N={N} Cin={Cin} H=W={H} Cout={Cout} ({gflop:.1f} GFLOP per pass): "
              f"forward {t_f * 1e3:.1f} us {gflop / t_f:.0f} TFLOP/s | input grad {t_x * 1e3:.1f} us {gflop / t_x:.0f} TFLOP/s | "
              f"weight grad {t_w * 1e3:.1f} us {gflop / t_w:.0f} TFLOP/s", flush=True)
    for spec in args.norm:
        N, Cc, H = (int(v) for v in spec.split(","))
        g = torch.Generator(device=dev).manual_seed(2)
        x = torch.randn(N, H, H, Cc, device=dev, generator=g)
        dy = torch.randn(N, H, H, Cc, device=dev, generator=g)
        gamma, beta = torch.rand(Cc, device=dev, generator=g) + 0.5, torch.randn(Cc, device=dev, generator=g)
        y, dx = torch.empty_like(x), torch.empty_like(x)
        sm, sv, dg, db = (torch.empty(Cc, device=dev) for _ in range(4))
        pooled = torch.empty(N, H // 2, H // 2, Cc, device=dev)
        dp = torch.randn(N, H // 2, H // 2, Cc, device=dev, generator=g)
        idx = torch.empty(N, H // 2, H // 2, Cc, dtype=torch.uint8, device=dev)
        mb = x.numel() * 4 / 1e6
        t1 = timed(lambda: abi.nc_cuda_batchnorm_forward_f32_ex(P(y), P(x), P(gamma), P(beta), None, None, P(sm), P(sv), N, Cc, H * H, 0.1, 1e-5, 1, 1, 1, None))
        t2 = timed(lambda: abi.nc_cuda_batchnorm_backward_f32_ex(P(dx), P(dg), P(db), P(dy), P(x), P(gamma), P(sm), P(sv), None, P(beta), 1, N, Cc, H * H, 1e-5, 1, None))
        t3 = timed(lambda: abi.nc_cuda_batchnorm_relu_maxpool2_forward_f32_ex(P(pooled), P(idx), P(x), P(gamma), P(beta), None, None, P(sm), P(sv), N, Cc, H, H, 0.1, 1e-5, 1, None))
        t4 = timed(lambda: abi.nc_cuda_batchnorm_relu_maxpool2_backward_f32_ex(P(dx), P(dg), P(db), P(dp), P(idx), P(x), P(gamma), P(beta), P(sm), P(sv), N, Cc, H, H, 1e-5, None))
        # algorithmic bytes per element of x: forward 12 (read twice, write once), backward 20; fused pool 9.25 / 14.5
        print(f"norm N={N} C={Cc} H=W={H} ({mb:.0f} MB tensor): BN+ReLU forward {t1 * 1e3:.1f} us {3 * mb / t1 / 1e3:.2f} TB/s | backward {t2 * 1e3:.1f} us "
              f"{5 * mb / t2 / 1e3:.2f} TB/s | BN+ReLU+pool forward {t3 * 1e3:.1f} us {2.3125 * mb / t3 / 1e3:.2f} TB/s | backward {t4 * 1e3:.1f} us "
              f"{3.625 * mb / t4 / 1e3:.2f} TB/s", flush=True)
    word = abi.nc_cuda_device_error_word()
    if word:
        raise SystemExit(f"device error word {word:#x}")


if __name__ == "__main__":
    main()
