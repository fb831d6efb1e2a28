// Fused softmax + cross-entropy (loss and gradient in one pass), fused MSE, the optimizer updates
// (SGD / momentum / Nesterov with the CPU path's first-step rule; Adam / AdamW / AMSGrad) and the
// few reductions the training path needs (sum over an axis, row argmax).
// Semantics follow the reference CPU code: src/ops/loss.c:33-137,176-351, src/optim/sgd.c:13-115,
// src/optim/adam.c:11-75, src/ops/reduction.c:158-198,473-513.
#include "nc_common.cuh"
#include <string.h>
#include "../../include/nocta_cuda.h"

using namespace ncc;

namespace {

constexpr int kThreads = 256;

// ---------------------------------------------------------------------------------------------
// Cross entropy.  One warp per row: row max, sum of exponentials (f32 exp, double accumulation of
// the per-row loss), optional gradient (softmax - onehot) * scale.  Per-block partial losses go to
// `partial`; the last block (ticket counter) adds them in index order, so the loss is bit-stable
// from run to run.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) ce_fused_kernel(float* __restrict__ loss, float* __restrict__ grad,
                                                            const float* __restrict__ logits,
                                                            const int64_t* __restrict__ targets, int N, int C,
                                                            float gscale, double* __restrict__ partial,
                                                            unsigned int* __restrict__ ticket, int rnd) {
    __shared__ double sh[32];
    __shared__ bool last;
    const int lane = threadIdx.x & 31;
    const int warps_per_block = blockDim.x >> 5;
    const int gw = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int nw = gridDim.x * warps_per_block;
    double acc = 0.0;
    for (int r = gw; r < N; r += nw) {
        const float* x = logits + (size_t)r * C;
        float m = -INFINITY;
        for (int c = lane; c < C; c += 32) m = fmaxf(m, x[c]);
        m = warp_max(m);
        float s = 0.f;
        for (int c = lane; c < C; c += 32) s += expf(x[c] - m);
        s = warp_sum(s);
        const int64_t lab64 = targets[r];
        const int lab = (int)lab64;  // the CPU path reads labels through (int) (loss.c:278)
        const bool valid = lab >= 0 && lab < C;
        if (lane == 0 && valid) acc += (double)logf(s) + (double)m - (double)x[lab];
        if (grad) {
            float inv = 1.f / s;
            float* g = grad + (size_t)r * C;
            for (int c = lane; c < C; c += 32) {
                float p = expf(x[c] - m) * inv;
                if (valid && c == lab) p -= 1.f;
                float o = p * gscale;
                g[c] = rnd ? round_tf32(o) : o;
            }
        }
    }
    double b = block_sum(acc, sh);
    if (threadIdx.x == 0) {
        partial[blockIdx.x] = b;
        __threadfence();
        unsigned int t = atomicAdd(ticket, 1u);
        last = (t == gridDim.x - 1);
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

__global__ void __launch_bounds__(kThreads) mse_fused_kernel(float* __restrict__ loss, float* __restrict__ gp,
                                                             float* __restrict__ gt, const float* __restrict__ p,
                                                             const float* __restrict__ t, size_t n, double gscale,
                                                             double* __restrict__ partial,
                                                             unsigned int* __restrict__ ticket, int rnd) {
    __shared__ double sh[32];
    __shared__ bool last;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    double acc = 0.0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float d = p[i] - t[i];
        acc += (double)d * (double)d;
        float g = (float)(gscale * (double)d);
        if (rnd) g = round_tf32(g);
        if (gp) gp[i] = g;
        if (gt) gt[i] = -g;
    }
    double b = block_sum(acc, sh);
    if (threadIdx.x == 0) {
        partial[blockIdx.x] = b;
        __threadfence();
        unsigned int k = atomicAdd(ticket, 1u);
        last = (k == gridDim.x - 1);
    }
    __syncthreads();
    if (last && threadIdx.x == 0) {
        __threadfence();
        double tot = 0.0;
        for (unsigned int i = 0; i < gridDim.x; i++) tot += ((volatile double*)partial)[i];
        if (loss) *loss = (float)(tot / (double)n);
        *ticket = 0;
    }
}

// ---------------------------------------------------------------------------------------------
// Optimizers.  The CPU path computes in double and stores f32; so do these.
// 20 B/param (SGD momentum: p, v, g read; p, v written), 28 B/param (Adam).
// ---------------------------------------------------------------------------------------------
struct SgdArgs {
    double lr, momentum, dampening, wd, gscale;
    int nesterov, first, write_grad;
};

__device__ __forceinline__ void sgd_element(float* __restrict__ p, float* __restrict__ v, float* __restrict__ g, const SgdArgs& a, size_t i) {
    double gi = (double)g[i] * a.gscale;
    double pi = (double)p[i];
    if (a.wd != 0.0) {
        // the CPU path stores the decayed gradient as f32 before using it (sgd.c:24-30)
        float gf = (float)(gi + a.wd * pi);
        if (a.write_grad) g[i] = gf;
        gi = (double)gf;
    }
    double upd = gi;
    if (v) {
        double vi = (double)v[i];
        vi = a.first ? gi : a.momentum * vi + (1.0 - a.dampening) * gi;
        float vf = (float)vi;
        v[i] = vf;
        vi = (double)vf;
        upd = a.nesterov ? gi + a.momentum * vi : vi;
    }
    p[i] = (float)(pi - a.lr * upd);
}

__global__ void __launch_bounds__(kThreads) sgd_kernel(float* __restrict__ p, float* __restrict__ v,
                                                       float* __restrict__ g, SgdArgs a, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) sgd_element(p, v, g, a, i);
}

// Several parameter tensors in one launch: the table travels as a kernel argument; a block owns a run of
// kMultiChunk elements of one tensor (first_block[t] = index of tensor t's first block).
constexpr int kMultiMax = 48;
constexpr int kMultiChunk = 4096;
struct MultiTable {
    float* p[kMultiMax];
    float* s1[kMultiMax];   // SGD: velocity; Adam: m
    float* s2[kMultiMax];   // Adam: v
    float* s3[kMultiMax];   // Adam: v_max (may be null)
    float* g[kMultiMax];
    unsigned int n[kMultiMax];
    unsigned int first_block[kMultiMax + 1];
    int count;
};
__device__ __forceinline__ int multi_find(const MultiTable& t, unsigned int block) {
    int lo = 0, hi = t.count - 1;
    while (lo < hi) {  // last tensor whose first block is <= block
        const int mid = (lo + hi + 1) >> 1;
        if (t.first_block[mid] <= block) lo = mid; else hi = mid - 1;
    }
    return lo;
}
__global__ void __launch_bounds__(kThreads) sgd_multi_kernel(const __grid_constant__ MultiTable t, SgdArgs a) {
    const int k = multi_find(t, blockIdx.x);
    const size_t begin = (size_t)(blockIdx.x - t.first_block[k]) * kMultiChunk;
    size_t end = begin + kMultiChunk;
    if (end > t.n[k]) end = t.n[k];
    for (size_t i = begin + threadIdx.x; i < end; i += kThreads) sgd_element(t.p[k], t.s1[k], t.g[k], a, i);
}

struct AdamArgs {
    double lr, b1, b2, eps, wd, inv_bc1, inv_bc2, gscale;
};

// One element, following src/optim/adam.c:39-73: the moments are updated in double and stored as f32 like the CPU path.
// The two bias-correction divisions are multiplications by reciprocals formed on the host, and the square root and the
// final quotient are f32: their rounding (6e-8 relative) acts on an update of size lr, far below the f32 spacing of the
// parameter it is added to, and keeps the kernel off the double-precision divide / square-root sequences.
__device__ __forceinline__ void adam_math(float& p, float& m, float& v, float* vmax, float g, const AdamArgs& a) {
    const double gi = (double)g * a.gscale;
    double pi = (double)p;
    if (a.wd != 0.0) pi = pi - a.lr * a.wd * pi;
    const double mi = a.b1 * (double)m + (1.0 - a.b1) * gi;
    const double vi = a.b2 * (double)v + (1.0 - a.b2) * gi * gi;
    m = (float)mi;
    v = (float)vi;
    const double mh = mi * a.inv_bc1;
    double vh = vi * a.inv_bc2;
    if (vmax) {
        const float vmf = (float)fmax((double)*vmax, vh);
        *vmax = vmf;
        vh = (double)vmf;
    }
    const float step = (float)mh / (sqrtf((float)vh) + (float)a.eps);
    p = (float)(pi - a.lr * (double)step);
}
__device__ __forceinline__ void adam_element(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, float* __restrict__ vmax,
                                             const float* __restrict__ g, const AdamArgs& a, size_t i) {
    adam_math(p[i], m[i], v[i], vmax ? vmax + i : nullptr, g[i], a);
}
// Elements [begin, end) of one tensor by one block: float4 accesses when the four arrays allow it.
__device__ __forceinline__ void adam_range(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, float* __restrict__ vmax,
                                           const float* __restrict__ g, const AdamArgs& a, size_t begin, size_t end, size_t first,
                                           size_t stride) {
    const bool vec = ((begin & 3) == 0) && !vmax &&
                     (((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                        reinterpret_cast<uintptr_t>(g)) & 15u) == 0);
    if (!vec) {
        for (size_t i = begin + first; i < end; i += stride) adam_element(p, m, v, vmax, g, a, i);
        return;
    }
    const size_t n4 = (end - begin) >> 2;
    for (size_t q = first; q < n4; q += stride) {
        const size_t i = begin + 4 * q;
        float4 p4 = *reinterpret_cast<float4*>(p + i), m4 = *reinterpret_cast<float4*>(m + i), v4 = *reinterpret_cast<float4*>(v + i);
        const float4 g4 = *reinterpret_cast<const float4*>(g + i);
        adam_math(p4.x, m4.x, v4.x, nullptr, g4.x, a);
        adam_math(p4.y, m4.y, v4.y, nullptr, g4.y, a);
        adam_math(p4.z, m4.z, v4.z, nullptr, g4.z, a);
        adam_math(p4.w, m4.w, v4.w, nullptr, g4.w, a);
        *reinterpret_cast<float4*>(p + i) = p4;
        *reinterpret_cast<float4*>(m + i) = m4;
        *reinterpret_cast<float4*>(v + i) = v4;
    }
    for (size_t i = begin + 4 * n4 + first; i < end; i += stride) adam_element(p, m, v, vmax, g, a, i);
}

__global__ void __launch_bounds__(kThreads) adam_kernel(float* __restrict__ p, float* __restrict__ m,
                                                        float* __restrict__ v, float* __restrict__ vmax,
                                                        const float* __restrict__ g, AdamArgs a, size_t n) {
    adam_range(p, m, v, vmax, g, a, 0, n, (size_t)blockIdx.x * blockDim.x + threadIdx.x, (size_t)gridDim.x * blockDim.x);
}

__global__ void __launch_bounds__(kThreads) adam_multi_kernel(const __grid_constant__ MultiTable t, AdamArgs a) {
    const int k = multi_find(t, blockIdx.x);
    const size_t begin = (size_t)(blockIdx.x - t.first_block[k]) * kMultiChunk;
    size_t end = begin + kMultiChunk;
    if (end > t.n[k]) end = t.n[k];
    adam_range(t.p[k], t.s1[k], t.s2[k], t.s3[k], t.g[k], a, begin, end, threadIdx.x, kThreads);
}

// ---------------------------------------------------------------------------------------------
// out[o][i] = sum_r in[o][r][i]  (double accumulation, as src/ops/reduction.c:158-198).
// A block owns 32 consecutive `i` for one `o`; 8 row-groups stride over r; coalesced along i.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) sum_axis_kernel(float* __restrict__ out, const float* __restrict__ in,
                                                       size_t reduce_dim, size_t inner) {
    __shared__ double sh[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const size_t o = blockIdx.y;
    const size_t i = (size_t)blockIdx.x * 32 + tx;
    double acc = 0.0;
    if (i < inner) {
        const float* base = in + o * reduce_dim * inner + i;
        for (size_t r = ty; r < reduce_dim; r += 8) acc += (double)base[r * inner];
    }
    sh[ty][tx] = acc;
    __syncthreads();
    if (ty == 0 && i < inner) {
        double t = 0.0;
#pragma unroll
        for (int k = 0; k < 8; k++) t += sh[k][tx];
        out[o * inner + i] = (float)t;
    }
}

// inner == 1: one warp per output, lanes stride over the reduced axis
__global__ void __launch_bounds__(kThreads) sum_rows_kernel(float* __restrict__ out, const float* __restrict__ in,
                                                            size_t outer, size_t reduce_dim) {
    const int lane = threadIdx.x & 31;
    const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t o = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; o < outer; o += warps) {
        double acc = 0.0;
        for (size_t r = lane; r < reduce_dim; r += 32) acc += (double)in[o * reduce_dim + r];
        acc = warp_sum(acc);
        if (lane == 0) out[o] = (float)acc;
    }
}

// First maximum per row (strict >), int64 result (src/ops/reduction.c:473-513).
__global__ void __launch_bounds__(kThreads) argmax_rows_kernel(int64_t* __restrict__ out, const float* __restrict__ in,
                                                               size_t rows, size_t cols) {
    const int lane = threadIdx.x & 31;
    const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const float* x = in + r * cols;
        float best = -INFINITY;
        long long bi = -1;
        for (size_t c = lane; c < cols; c += 32) {
            float v = x[c];
            if (bi < 0 || v > best) { best = v; bi = (long long)c; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
        }
        if (lane == 0) out[r] = bi < 0 ? 0 : bi;
    }
}

struct LossScratch { double* partial; unsigned int* ticket; int blocks; };

int loss_scratch(LossScratch* ls, long long work, cudaStream_t st) {
    int blocks = grid_for(work, kThreads, 4);
    // layout: [ticket (16 B)] [partials]
    char* base = (char*)scratch(0, 16 + sizeof(double) * (size_t)blocks, st);
    if (!base) return NC_CUDA_ERR_RUNTIME;
    // The ticket must start at zero.  A kernel resets it when it ends, but not after a failed or aborted launch, and a
    // regrown block starts with arbitrary contents: clear it in stream order on every call (calls on different streams
    // share this one block and must not overlap).
    cudaError_t e = cudaMemsetAsync(base, 0, 16, st);
    if (e != cudaSuccess) return set_status(NC_CUDA_ERR_RUNTIME, "loss scratch memset failed");
    ++g_epoch;
    ls->ticket = (unsigned int*)base;
    ls->partial = (double*)(base + 16);
    ls->blocks = blocks;
    return NC_CUDA_OK;
}

// Fills launch tables of at most kMultiMax tensors from the caller's host arrays and launches `launch` for each.
template <class L>
static int multi_launch(int count, float* const* params, float* const* s1, float* const* s2, float* const* s3, float* const* grads,
                        const size_t* numel, const char* what, L launch) {
    int done = 0;
    while (done < count) {
        MultiTable t;
        memset(&t, 0, sizeof(t));
        unsigned int blocks = 0;
        while (done < count && t.count < kMultiMax) {
            const size_t n = numel[done];
            if (n == 0) { done++; continue; }
            if (n > 0xffffffffull) return set_status(NC_CUDA_ERR_ARG, "%s: tensor %d has more than 2^32 elements", what, done);
            const int k = t.count++;
            t.p[k] = params[done];
            t.s1[k] = s1 ? s1[done] : nullptr;
            t.s2[k] = s2 ? s2[done] : nullptr;
            t.s3[k] = s3 ? s3[done] : nullptr;
            t.g[k] = grads[done];
            t.n[k] = (unsigned int)n;
            t.first_block[k] = blocks;
            blocks += (unsigned int)((n + kMultiChunk - 1) / kMultiChunk);
            done++;
        }
        t.first_block[t.count] = blocks;
        if (t.count == 0) break;
        launch(t, blocks);
        NCC_COUNT_LAUNCH();
        int rc = launch_status(what);
        if (rc) return rc;
    }
    return NC_CUDA_OK;
}

}  // namespace

extern "C" {

int nc_cuda_cross_entropy_fused_f32_ex(float* loss, float* grad, const float* logits, const int64_t* targets,
                                       int N, int C, float grad_scale, void* stream) {
    NCC_REQUIRE(logits && targets && N > 0 && C > 0, "cross_entropy: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    ProfScope prof(PROF_LOSS, (grad ? 8.0 : 4.0) * (double)N * C + 8.0 * N, st);
    LossScratch ls;
    int rc = loss_scratch(&ls, (long long)N * 32, st);
    if (rc) return rc;
    ce_fused_kernel<<<ls.blocks, kThreads, 0, st>>>(loss, grad, logits, targets, N, C, grad_scale / (float)N,
                                                    ls.partial, ls.ticket, round_outputs() ? 1 : 0);
    NCC_COUNT_LAUNCH();
    return launch_status("cross_entropy");
}

int nc_cuda_mse_fused_f32_ex(float* loss, float* gp, float* gt, const float* pred, const float* target, size_t n,
                             float grad_scale, void* stream) {
    NCC_REQUIRE(pred && target && n > 0, "mse: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    ProfScope prof(PROF_LOSS, (8.0 + (gp ? 4.0 : 0.0) + (gt ? 4.0 : 0.0)) * (double)n, st);
    LossScratch ls;
    int rc = loss_scratch(&ls, (long long)n, st);
    if (rc) return rc;
    mse_fused_kernel<<<ls.blocks, kThreads, 0, st>>>(loss, gp, gt, pred, target, n,
                                                     2.0 * (double)grad_scale / (double)n, ls.partial, ls.ticket, round_outputs() ? 1 : 0);
    NCC_COUNT_LAUNCH();
    return launch_status("mse");
}

void nc_cuda_cross_entropy_forward_f32(float* loss, const float* logits, const int64_t* targets, int N, int C) {
    nc_cuda_cross_entropy_fused_f32_ex(loss, nullptr, logits, targets, N, C, 1.f, current_stream());
}
void nc_cuda_cross_entropy_backward_f32(float* grad, const float* logits, const int64_t* targets, int N, int C) {
    nc_cuda_cross_entropy_fused_f32_ex(nullptr, grad, logits, targets, N, C, 1.f, current_stream());
}

int nc_cuda_sgd_update_f32_ex(float* param, float* velocity, float* grad, double lr, double momentum,
                              double dampening, double weight_decay, int nesterov, int first_step,
                              double grad_scale, size_t n, void* stream) {
    if (n == 0) return NC_CUDA_OK;
    NCC_REQUIRE(param && grad, "sgd: null pointer");
    SgdArgs a{lr, momentum, dampening, weight_decay, grad_scale, nesterov, first_step, 1};
    float* v = (momentum != 0.0) ? velocity : nullptr;
    NCC_REQUIRE(momentum == 0.0 || v, "sgd: momentum without a velocity buffer");
    ProfScope prof(PROF_SGD, (v ? 20.0 : 12.0) * (double)n, (cudaStream_t)stream);
    sgd_kernel<<<grid_for((long long)n, kThreads), kThreads, 0, (cudaStream_t)stream>>>(param, v, grad, a, n);
    NCC_COUNT_LAUNCH();
    return launch_status("sgd");
}

int nc_cuda_adam_update_f32_ex(float* param, float* m, float* v, float* v_max, const float* grad, double lr,
                               double beta1, double beta2, double eps, double weight_decay, double bias_corr1,
                               double bias_corr2, double grad_scale, size_t n, void* stream) {
    if (n == 0) return NC_CUDA_OK;
    NCC_REQUIRE(param && m && v && grad, "adam: null pointer");
    AdamArgs a{lr, beta1, beta2, eps, weight_decay, 1.0 / bias_corr1, 1.0 / bias_corr2, grad_scale};
    ProfScope prof(PROF_ADAM, (v_max ? 36.0 : 28.0) * (double)n, (cudaStream_t)stream);
    adam_kernel<<<grid_for((long long)n, kThreads), kThreads, 0, (cudaStream_t)stream>>>(param, m, v, v_max, grad, a, n);
    NCC_COUNT_LAUNCH();
    return launch_status("adam");
}

int nc_cuda_sgd_update_multi_f32_ex(int count, float* const* params, float* const* velocities, float* const* grads,
                                    const size_t* numel, double lr, double momentum, double dampening, double weight_decay,
                                    int nesterov, int first_step, double grad_scale, void* stream) {
    if (count <= 0) return NC_CUDA_OK;
    NCC_REQUIRE(params && grads && numel && (momentum == 0.0 || velocities), "sgd_multi: null table");
    for (int i = 0; i < count; i++)
        NCC_REQUIRE(numel[i] == 0 || (params[i] && grads[i] && (momentum == 0.0 || velocities[i])), "sgd_multi: null pointer in entry %d", i);
    SgdArgs a{lr, momentum, dampening, weight_decay, grad_scale, nesterov, first_step, 1};
    cudaStream_t st = (cudaStream_t)stream;
    double total = 0.0;
    for (int i = 0; i < count; i++) total += (double)numel[i];
    ProfScope prof(PROF_SGD, (momentum != 0.0 ? 20.0 : 12.0) * total, st);
    return multi_launch(count, params, momentum != 0.0 ? velocities : nullptr, nullptr, nullptr, grads, numel, "sgd_multi",
                        [&](const MultiTable& t, unsigned int blocks) { sgd_multi_kernel<<<blocks, kThreads, 0, st>>>(t, a); });
}

int nc_cuda_adam_update_multi_f32_ex(int count, float* const* params, float* const* m, float* const* v, float* const* v_max,
                                     float* const* grads, const size_t* numel, double lr, double beta1, double beta2, double eps,
                                     double weight_decay, double bias_corr1, double bias_corr2, double grad_scale, void* stream) {
    if (count <= 0) return NC_CUDA_OK;
    NCC_REQUIRE(params && m && v && grads && numel, "adam_multi: null table");
    for (int i = 0; i < count; i++)
        NCC_REQUIRE(numel[i] == 0 || (params[i] && m[i] && v[i] && grads[i]), "adam_multi: null pointer in entry %d", i);
    AdamArgs a{lr, beta1, beta2, eps, weight_decay, 1.0 / bias_corr1, 1.0 / bias_corr2, grad_scale};
    cudaStream_t st = (cudaStream_t)stream;
    double total = 0.0;
    bool amsgrad = false;
    for (int i = 0; i < count; i++) { total += (double)numel[i]; amsgrad = amsgrad || (v_max && v_max[i]); }
    ProfScope prof(PROF_ADAM, (amsgrad ? 36.0 : 28.0) * total, st);
    return multi_launch(count, params, m, v, v_max, grads, numel, "adam_multi",
                        [&](const MultiTable& t, unsigned int blocks) { adam_multi_kernel<<<blocks, kThreads, 0, st>>>(t, a); });
}

void nc_cuda_sgd_step_f32(float* param, const float* grad, float lr, size_t n) {
    nc_cuda_sgd_update_f32_ex(param, nullptr, const_cast<float*>(grad), lr, 0.0, 0.0, 0.0, 0, 0, 1.0, n, current_stream());
}
// Legacy entry: no first-step flag in the signature, so v = mu*v + (1-d)*g always
// (equal to the CPU rule when the velocity starts at zero and dampening is 0).
void nc_cuda_sgd_momentum_f32(float* param, float* velocity, const float* grad, float lr, float momentum,
                              float dampening, int nesterov, size_t n) {
    nc_cuda_sgd_update_f32_ex(param, velocity, const_cast<float*>(grad), lr, momentum, dampening, 0.0, nesterov, 0,
                              1.0, n, current_stream());
}

int nc_cuda_sum_axis_f32_ex(float* out, const float* in, size_t outer, size_t reduce_dim, size_t inner, void* stream) {
    if (outer == 0 || inner == 0) return NC_CUDA_OK;
    NCC_REQUIRE(out && in, "sum_axis: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    ProfScope prof(PROF_REDUCE, 4.0 * (double)outer * reduce_dim * inner, st);
    if (inner == 1) {
        sum_rows_kernel<<<grid_for((long long)outer * 32, kThreads), kThreads, 0, st>>>(out, in, outer, reduce_dim);
    } else {
        NCC_REQUIRE(outer <= 65535, "sum_axis: outer too large");
        dim3 grid(ceil_div((long long)inner, 32), (unsigned)outer);
        sum_axis_kernel<<<grid, 256, 0, st>>>(out, in, reduce_dim, inner);
    }
    NCC_COUNT_LAUNCH();
    return launch_status("sum_axis");
}
void nc_cuda_sum_axis_f32(float* out, const float* in, size_t outer, size_t reduce_dim, size_t inner) {
    nc_cuda_sum_axis_f32_ex(out, in, outer, reduce_dim, inner, current_stream());
}
int nc_cuda_argmax_rows_f32_ex(int64_t* out, const float* in, size_t rows, size_t cols, void* stream) {
    if (rows == 0) return NC_CUDA_OK;
    NCC_REQUIRE(out && in && cols > 0, "argmax_rows: bad argument");
    argmax_rows_kernel<<<grid_for((long long)rows * 32, kThreads), kThreads, 0, (cudaStream_t)stream>>>(out, in, rows, cols);
    NCC_COUNT_LAUNCH();
    return launch_status("argmax_rows");
}
float nc_cuda_sum_f32(const float* data, size_t n) {
    cudaStream_t st = current_stream();
    float* d = (float*)scratch(1, 16, st);
    if (!d) return 0.f;
    if (nc_cuda_sum_axis_f32_ex(d, data, 1, n, 1, st)) return 0.f;
    float h = 0.f;
    cudaMemcpyAsync(&h, d, sizeof(float), cudaMemcpyDeviceToHost, st);
    cudaStreamSynchronize(st);
    return h;
}
size_t nc_cuda_argmax_f32(const float* data, size_t n) {
    cudaStream_t st = current_stream();
    int64_t* d = (int64_t*)scratch(1, 16, st);
    if (!d) return 0;
    if (nc_cuda_argmax_rows_f32_ex(d, data, 1, n, st)) return 0;
    int64_t h = 0;
    cudaMemcpyAsync(&h, d, sizeof(h), cudaMemcpyDeviceToHost, st);
    cudaStreamSynchronize(st);
    return (size_t)h;
}

}  // extern "C"
