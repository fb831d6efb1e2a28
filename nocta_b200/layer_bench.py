"""Per-layer timing of the convolution kernels through the nc_cuda_* C ABI.

    python -m nocta_b200.layer_bench --layers 256,128,32,128 [--iters 5] [--warmup 2] [--mode 0]

--norm N,C,H times the BatchNorm kernels the same way; --kernels times the remaining families of the training path
(LayerNorm, GELU, stand-alone max-pool, softmax + cross-entropy, MSE, the multi-tensor SGD and Adam updates, the
first-layer convolution, and the Linear GEMMs of config 4 in each operand layout and math mode).  Each --layers entry is N,Cin,H,Cout (square images, 3x3 filters, stride 1, padding 1, channels-last
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
    ap.add_argument("--kernels", action="store_true", help="time the memory-bound families and the Linear GEMMs at the sizes of the "
                    "benchmarked configurations (and, where those fit in L2, at a size that does not)")
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
    if args.kernels:
        g = torch.Generator(device=dev).manual_seed(3)
        R = lambda *shape: torch.randn(*shape, device=dev, generator=g)

        def report(name, ms, bytes_=None, flops=None):
            if flops is not None:
                print(f"{name}: {ms * 1e3:.1f} us {flops / ms / 1e9:.0f} TFLOP/s", flush=True)
            else:
                print(f"{name}: {ms * 1e3:.1f} us {bytes_ / ms / 1e6:.0f} GB/s ({bytes_ / 1e6:.1f} MB algorithmic)", flush=True)

        # LayerNorm (config 4: 4096 x 1024; 65536 x 1024 does not fit in L2)
        for rows in (4096, 65536):
            cols = 1024
            x, dy = R(rows, cols), R(rows, cols)
            y, dx = torch.empty_like(x), torch.empty_like(x)
            gam, bet, dg, db = torch.rand(cols, device=dev) + 0.5, R(cols), torch.empty(cols, device=dev), torch.empty(cols, device=dev)
            n = rows * cols
            report(f"layernorm forward {rows}x{cols}", timed(lambda: abi.nc_cuda_layernorm_forward_f32_ex(P(y), P(x), P(gam), P(bet), rows, cols, 1e-5, None)), 8.0 * n)
            report(f"layernorm backward {rows}x{cols}", timed(lambda: abi.nc_cuda_layernorm_backward_f32_ex(P(dx), P(dg), P(db), P(dy), P(x), P(gam), rows, cols, 1e-5, None)), 20.0 * n)
        # GELU (config 4: 4096 x 4096)
        n = 4096 * 4096
        x, dy = R(n), R(n)
        y = torch.empty_like(x)
        report("gelu forward 4096x4096", timed(lambda: abi.nc_cuda_gelu_f32_ex(P(y), P(x), n, None)), 8.0 * n)
        report("gelu backward 4096x4096", timed(lambda: abi.nc_cuda_gelu_backward_f32_ex(P(y), P(dy), P(x), n, None)), 12.0 * n)
        # stand-alone max-pool 2x2, channels-last (config 2's first pool at batch 128 and a 268 MB tensor)
        for (N, Cc, H) in ((128, 64, 32), (256, 64, 64)):
            x = R(N, H, H, Cc)
            out, idx = torch.empty(N, H // 2, H // 2, Cc, device=dev), torch.empty(N, H // 2, H // 2, Cc, dtype=torch.uint8, device=dev)
            gout, gin = R(N, H // 2, H // 2, Cc), torch.empty_like(x)
            nin = x.numel()
            report(f"maxpool forward {N}x{Cc}x{H}x{H}", timed(lambda: abi.nc_cuda_maxpool2d_forward_idx_f32_ex(P(out), P(idx), P(x), N, Cc, H, H, 2, 2, 1, None)), 4.0 * nin + 1.25 * nin)
            report(f"maxpool backward {N}x{Cc}x{H}x{H}", timed(lambda: abi.nc_cuda_maxpool2d_backward_idx_f32_ex(P(gin), P(gout), P(idx), N, Cc, H, H, 2, 2, 1, None)), 4.0 * nin + 1.25 * nin)
        # softmax + cross-entropy (config 5: 256 x 100) and MSE (config 4: 4096 x 1024)
        logits, labels = R(256, 100), torch.randint(0, 100, (256,), device=dev)
        loss, grad = torch.zeros(1, device=dev), torch.empty(256, 100, device=dev)
        report("cross-entropy 256x100", timed(lambda: abi.nc_cuda_cross_entropy_fused_f32_ex(P(loss), P(grad), P(logits), P(labels), 256, 100, 1.0, None)), 8.0 * 25600)
        pred, tgt = R(4096 * 1024), R(4096 * 1024)
        gp = torch.empty_like(pred)
        report("mse 4096x1024", timed(lambda: abi.nc_cuda_mse_fused_f32_ex(P(loss), P(gp), None, P(pred), P(tgt), 4096 * 1024, 1.0, None)), 12.0 * 4096 * 1024)
        # multi-tensor optimizers at config 4's parameter count (8 matrices of 4096 x 1024 and their small vectors)
        sizes = [4096 * 1024] * 8 + [4096, 1024, 1024, 1024] * 4
        ps, ms_, vs, gs = ([R(s) for s in sizes] for _ in range(4))
        vs = [v.abs() for v in vs]
        tab = lambda ts: (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
        numel = (C.c_size_t * len(sizes))(*sizes)
        tot = float(sum(sizes))
        report("adam multi-tensor 33.6M parameters", timed(lambda: abi.nc_cuda_adam_update_multi_f32_ex(len(sizes), tab(ps), tab(ms_), tab(vs), None, tab(gs), numel, 1e-4, 0.9, 0.999, 1e-8, 0.0, 0.1, 0.001, 1.0, None)), 28.0 * tot)
        report("sgd-momentum multi-tensor 33.6M parameters", timed(lambda: abi.nc_cuda_sgd_update_multi_f32_ex(len(sizes), tab(ps), tab(ms_), tab(gs), numel, 0.01, 0.9, 0.0, 0.0, 0, 0, 1.0, None)), 20.0 * tot)
        # first-layer convolution (3 -> 64 channels, 64 x 64, batch 256; NCHW input as the network receives it)
        N, H, Co = 256, 64, 64
        x = R(N, 3, H, H)
        w3, dy = R(Co, 3, 3, 3), R(N, H, H, Co)
        y, dw3 = torch.empty(N, H, H, Co, device=dev), torch.empty_like(w3)
        xs = cuda_abi.size4([3 * H * H, H * H, H, 1])
        ys = cuda_abi.size4([H * H * Co, 1, H * Co, Co])
        by = 4.0 * N * H * H * (Co + 3)
        report("first-layer convolution forward 256x3x64x64 -> 64", timed(lambda: abi.nc_cuda_conv2d_forward_f32_ex(P(y), ys, P(x), xs, P(w3), None, N, 3, H, H, Co, 3, 3, 1, 1, None)), by)
        report("first-layer convolution weight gradient", timed(lambda: abi.nc_cuda_conv2d_backward_weight_f32_ex(P(dw3), None, P(dy), ys, P(x), xs, N, 3, H, H, Co, 3, 3, 1, 1, None)), by)
        # Linear GEMMs of config 4: batch 4096, 1024 <-> 4096, each operand layout; TF32 and 3xTF32
        B, I, O = 4096, 1024, 4096
        x, W, dy = R(B, I), R(O, I) * 0.03, R(B, O)
        y, dx, dW = torch.empty(B, O, device=dev), torch.empty(B, I, device=dev), torch.empty(O, I, device=dev)
        fl = 2.0 * B * I * O
        for mode in (0, 2):
            abi.nc_cuda_set_math_mode(mode)
            tag = "TF32" if mode == 0 else "3xTF32"
            report(f"linear forward y = x W^T (both K-major) 4096x1024x4096 {tag}", timed(lambda: abi.nc_cuda_linear_forward_f32_ex(P(y), P(x), P(W), None, B, I, O, None)), flops=fl)
            report(f"linear input gradient dx = dy W (B MN-major) {tag}", timed(lambda: abi.nc_cuda_linear_backward_f32_ex(P(dx), None, None, P(dy), P(x), P(W), B, I, O, None)), flops=fl)
            report(f"linear weight gradient dW = dy^T x (both MN-major) {tag}", timed(lambda: abi.nc_cuda_linear_backward_f32_ex(None, P(dW), None, P(dy), P(x), P(W), B, I, O, None)), flops=fl)
        abi.nc_cuda_set_math_mode(args.mode)
    word = abi.nc_cuda_device_error_word()
    if word:
        raise SystemExit(f"device error word {word:#x}")


if __name__ == "__main__":
    main()
