// Fused softmax + cross-entropy that never allocates.
//
// nc_cuda_cross_entropy_fused_f32_ex keeps its per-CTA partial losses and its ticket counter in a
// library scratch block that is obtained with cudaMalloc on first use and regrown (synchronise,
// free, allocate) when a larger batch arrives.  Some callers cannot tolerate that: a training
// loop that has handed all device memory to its own arena and must not see the driver allocator
// fail or fragment it; a host thread that issues the loss while a collective of another stream is
// in flight, where an implicit device-wide synchronisation inside an allocation stalls (or, with
// communication kernels that wait on peers, can deadlock) the whole step; and latency-critical
// loops that budget for kernel launches only.  For them this file offers the same computation
// with the scratch in a fixed array that is part of the loaded module.
//
// Rules of the entry point below:
//   * the scratch is one file-scope __device__ array per device (kScratchBytes, see below); its
//     device address is looked up once per device with cudaGetSymbolAddress while that device is
//     current, and only that pointer is handed to the kernel;
//   * the FIRST call on a device performs that look-up (which may make the runtime load this
//     module); make it before starting any stream capture;
//   * batches of more than NC_CUDA_CE_STATIC_MAX_ROWS rows are rejected with NC_CUDA_ERR_ARG;
//   * nothing here calls an allocating routine of the runtime, the driver or any library;
//   * every call on a device shares the one array: the ticket word is cleared in stream order at
//     the start of each call, the partials are fully rewritten before they are read.  Two calls
//     that may execute at the same time (different streams, different host threads) race on it
//     and give undefined results; serialise them.
// The arithmetic, the grid and the order in which the partial sums are combined are those of
// nc_cuda_cross_entropy_fused_f32_ex, so both entry points return identical bits.
// Semantics: src/ops/loss.c:176-351 of the reference (mean loss, labels read through (int),
// out-of-range labels contribute nothing).
#include "nc_common.cuh"
#include "../../include/nocta_cuda.h"

using namespace ncc;

namespace {

constexpr int kThreads = 256;                              // 8 warps, one row per warp per pass
constexpr int kMaxRows = NC_CUDA_CE_STATIC_MAX_ROWS;       // 4096
constexpr int kMaxBlocks = kMaxRows / (kThreads / 32);     // 512 CTAs at most
constexpr int kHeaderBytes = 256;                          // ticket word, padded
constexpr int kScratchBytes = kHeaderBytes + kMaxBlocks * (int)sizeof(double);  // 4352 B

// [ticket (4 B, padded to 256)] [kMaxBlocks partial losses (double)]
static __device__ __align__(256) unsigned char g_ce_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
static unsigned char* g_scratch_ptr[kMaxDevices] = {nullptr};  // per device, filled on first use

__global__ void __launch_bounds__(kThreads) ce_static_kernel(float* __restrict__ loss, float* __restrict__ grad,
                                                             const float* __restrict__ logits,
                                                             const int64_t* __restrict__ targets, int N, int C,
                                                             float gscale, double* __restrict__ partial,
                                                             unsigned int* __restrict__ ticket, int rnd) {
    __shared__ double sh[32];
    __shared__ bool last;
    const int lane = threadIdx.x & 31;
    const int warps_per_block = blockDim.x >> 5;
    const int nw = gridDim.x * warps_per_block;
    double acc = 0.0;
    for (int r = blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < N; r += nw) {
        const float* x = logits + (size_t)r * C;
        float m = -INFINITY;
        for (int c = lane; c < C; c += 32) m = fmaxf(m, x[c]);
        m = warp_max(m);
        float s = 0.f;
        for (int c = lane; c < C; c += 32) s += expf(x[c] - m);
        s = warp_sum(s);
        const int lab = (int)targets[r];
        const bool valid = lab >= 0 && lab < C;
        if (lane == 0 && valid) acc += (double)logf(s) + (double)m - (double)x[lab];
        if (grad) {
            const float inv = 1.f / s;
            float* g = grad + (size_t)r * C;
            for (int c = lane; c < C; c += 32) {
                float p = expf(x[c] - m) * inv;
                if (valid && c == lab) p -= 1.f;
                const float o = p * gscale;
                g[c] = rnd ? round_tf32(o) : o;
            }
        }
    }
    const double b = block_sum(acc, sh);
    if (threadIdx.x == 0) {
        partial[blockIdx.x] = b;
        __threadfence();
        last = (atomicAdd(ticket, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (last && threadIdx.x == 0) {
        __threadfence();
        double tot = 0.0;
        for (unsigned int i = 0; i < gridDim.x; i++) tot += ((volatile double*)partial)[i];
        if (loss) *loss = (float)(tot / (double)N);
        *ticket = 0;
    }
}

// Device address of the scratch array for the CURRENT device (resolved once per device).
int scratch_for_current_device(unsigned char** out) {
    int dev = -1;
    NCC_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return set_status(NC_CUDA_ERR_UNSUPPORTED, "cross_entropy_static: device index %d not supported", dev);
    if (!g_scratch_ptr[dev]) {
        unsigned char* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, g_ce_scratch);
        if (e != cudaSuccess || !p)
            return set_status(NC_CUDA_ERR_RUNTIME, "cross_entropy_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return NC_CUDA_OK;
}

}  // namespace

extern "C" int nc_cuda_cross_entropy_fused_static_f32_ex(float* loss, float* grad, const float* logits,
                                                          const int64_t* targets, int N, int C, float grad_scale,
                                                          void* stream) {
    NCC_REQUIRE(logits && targets && N > 0 && C > 0, "cross_entropy_static: bad argument");
    if (N > kMaxRows)
        return set_status(NC_CUDA_ERR_LIMIT, "cross_entropy_static: %d rows exceed the fixed scratch (at most %d rows per call)", N, kMaxRows);
    cudaStream_t st = (cudaStream_t)stream;
    unsigned char* base = nullptr;
    int rc = scratch_for_current_device(&base);
    if (rc) return rc;
    const int blocks = grid_for((long long)N * 32, kThreads, 4);  // same grid as the allocating entry point
    if (blocks > kMaxBlocks) return set_status(NC_CUDA_ERR_LIMIT, "cross_entropy_static: %d CTAs exceed the fixed scratch", blocks);
    // the ticket must start at zero whatever an earlier, possibly failed, call left behind
    NCC_TRY(cudaMemsetAsync(base, 0, 16, st));
    ce_static_kernel<<<blocks, kThreads, 0, st>>>(loss, grad, logits, targets, N, C, grad_scale / (float)N,
                                                  reinterpret_cast<double*>(base + kHeaderBytes),
                                                  reinterpret_cast<unsigned int*>(base), round_outputs() ? 1 : 0);
    NCC_COUNT_LAUNCH();
    return launch_status("cross_entropy_static");
}
