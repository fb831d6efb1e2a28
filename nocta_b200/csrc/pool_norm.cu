// MaxPool2d (forward with saved argmax, backward scatter), BatchNorm2d and LayerNorm forward/backward.
// Every reduction is two-stage and ordered (no float atomics): partial sums per CTA in double, then a
// fixed-order combine, so results are bit-stable from run to run.
// Semantics follow the reference CPU path: src/nn/conv.c:672-849 (max pool: start -1e30, strict >,
// first maximum wins), src/nn/batchnorm.c:43-165,171-371 (BatchNorm2d) and :600-702,946-1026 (LayerNorm).
#include "nc_common.cuh"
#include "../../include/nocta_cuda.h"

using namespace ncc;

namespace {

constexpr int kThreads = 256;
// tensors above this size cannot stay in the 126 MB L2 between two kernels: passes that read or write them exactly once use
// streaming (evict-first) accesses in the two plain apply kernels, which measured 2 - 3 % faster on the BatchNorm family of the
// 268 MB layers (the fused pooling kernels got slower with the same hints: their four window positions share lines)
constexpr size_t kStreamBytes = 100ull << 20;

// =============================================================================================
// Max pooling
// =============================================================================================
// NCHW: one thread per output element.  NHWC: one thread per output pixel x 4-channel vector when
// C % 4 == 0 (VEC = 4), else per single channel.
template <int LAYOUT, int VEC>
__global__ void __launch_bounds__(kThreads) maxpool_fwd_kernel(float* __restrict__ out, uint8_t* __restrict__ idx,
                                                               const float* __restrict__ in, int N, int C, int H,
                                                               int W, int Ho, int Wo, int k, int stride) {
    const size_t total = (size_t)N * (C / VEC) * Ho * Wo;
    const size_t gstride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gstride) {
        size_t r = i;
        int n, c, ho, wo;
        if (LAYOUT == 0) {
            wo = r % Wo; r /= Wo; ho = r % Ho; r /= Ho; c = r % C; n = (int)(r / C);
        } else {
            c = (int)(r % (C / VEC)) * VEC; r /= (C / VEC); wo = r % Wo; r /= Wo; ho = r % Ho; n = (int)(r / Ho);
        }
        float best[VEC];
        int bidx[VEC];
#pragma unroll
        for (int v = 0; v < VEC; v++) { best[v] = -1e30f; bidx[v] = 0; }
        for (int kh = 0; kh < k; kh++) {
            for (int kw = 0; kw < k; kw++) {
                const int h = ho * stride + kh, w = wo * stride + kw;
                float val[VEC];
                if (LAYOUT == 0) {
                    val[0] = in[(((size_t)n * C + c) * H + h) * W + w];
                } else if (VEC == 4) {
                    float4 t = *reinterpret_cast<const float4*>(in + (((size_t)n * H + h) * W + w) * C + c);
                    val[0] = t.x; val[1 % VEC] = t.y; val[2 % VEC] = t.z; val[3 % VEC] = t.w;
                } else {
                    val[0] = in[(((size_t)n * H + h) * W + w) * C + c];
                }
#pragma unroll
                for (int v = 0; v < VEC; v++)
                    if (val[v] > best[v]) { best[v] = val[v]; bidx[v] = kh * k + kw; }
            }
        }
        size_t o;
        if (LAYOUT == 0) o = (((size_t)n * C + c) * Ho + ho) * Wo + wo;
        else o = (((size_t)n * Ho + ho) * Wo + wo) * C + c;
        if (VEC == 4) {
            *reinterpret_cast<float4*>(out + o) = make_float4(best[0], best[1 % VEC], best[2 % VEC], best[3 % VEC]);
            if (idx) *reinterpret_cast<uchar4*>(idx + o) =
                make_uchar4((uint8_t)bidx[0], (uint8_t)bidx[1 % VEC], (uint8_t)bidx[2 % VEC], (uint8_t)bidx[3 % VEC]);
        } else {
            out[o] = best[0];
            if (idx) idx[o] = (uint8_t)bidx[0];
        }
    }
}

// Non-overlapping windows (stride >= k): every input pixel is owned by at most one output, so the
// thread of that output writes the whole window (gradient at the saved offset, zero elsewhere).
template <int LAYOUT, int VEC>
__global__ void __launch_bounds__(kThreads) maxpool_bwd_own_kernel(float* __restrict__ gin, const float* __restrict__ gout,
                                                                   const uint8_t* __restrict__ idx, int N, int C, int H,
                                                                   int W, int Ho, int Wo, int k, int stride) {
    const size_t total = (size_t)N * (C / VEC) * Ho * Wo;
    const size_t gstride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gstride) {
        size_t r = i;
        int n, c, ho, wo;
        if (LAYOUT == 0) {
            wo = r % Wo; r /= Wo; ho = r % Ho; r /= Ho; c = r % C; n = (int)(r / C);
        } else {
            c = (int)(r % (C / VEC)) * VEC; r /= (C / VEC); wo = r % Wo; r /= Wo; ho = r % Ho; n = (int)(r / Ho);
        }
        size_t o;
        if (LAYOUT == 0) o = (((size_t)n * C + c) * Ho + ho) * Wo + wo;
        else o = (((size_t)n * Ho + ho) * Wo + wo) * C + c;
        float g[VEC];
        int bi[VEC];
        if (VEC == 4) {
            float4 t = *reinterpret_cast<const float4*>(gout + o);
            uchar4 u = *reinterpret_cast<const uchar4*>(idx + o);
            g[0] = t.x; g[1 % VEC] = t.y; g[2 % VEC] = t.z; g[3 % VEC] = t.w;
            bi[0] = u.x; bi[1 % VEC] = u.y; bi[2 % VEC] = u.z; bi[3 % VEC] = u.w;
        } else {
            g[0] = gout[o];
            bi[0] = idx[o];
        }
        for (int kh = 0; kh < k; kh++) {
            for (int kw = 0; kw < k; kw++) {
                const int h = ho * stride + kh, w = wo * stride + kw, off = kh * k + kw;
                if (LAYOUT == 0) {
                    gin[(((size_t)n * C + c) * H + h) * W + w] = (bi[0] == off) ? g[0] : 0.f;
                } else if (VEC == 4) {
                    float4 t = make_float4(bi[0] == off ? g[0] : 0.f, bi[1 % VEC] == off ? g[1 % VEC] : 0.f,
                                           bi[2 % VEC] == off ? g[2 % VEC] : 0.f, bi[3 % VEC] == off ? g[3 % VEC] : 0.f);
                    *reinterpret_cast<float4*>(gin + (((size_t)n * H + h) * W + w) * C + c) = t;
                } else {
                    gin[(((size_t)n * H + h) * W + w) * C + c] = (bi[0] == off) ? g[0] : 0.f;
                }
            }
        }
    }
}

// Overlapping windows (stride < k): gather form — each input pixel sums the outputs whose saved
// offset points at it (fixed (ho, wo) order, no atomics).
template <int LAYOUT>
__global__ void __launch_bounds__(kThreads) maxpool_bwd_gather_kernel(float* __restrict__ gin, const float* __restrict__ gout,
                                                                      const uint8_t* __restrict__ idx, int N, int C, int H,
                                                                      int W, int Ho, int Wo, int k, int stride) {
    const size_t total = (size_t)N * C * H * W;
    const size_t gstride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gstride) {
        size_t r = i;
        int n, c, h, w;
        if (LAYOUT == 0) { w = r % W; r /= W; h = r % H; r /= H; c = r % C; n = (int)(r / C); }
        else { c = r % C; r /= C; w = r % W; r /= W; h = r % H; n = (int)(r / H); }
        float acc = 0.f;
        for (int kh = 0; kh < k; kh++) {
            int hh = h - kh;
            if (hh < 0 || hh % stride) continue;
            int ho = hh / stride;
            if (ho >= Ho) continue;
            for (int kw = 0; kw < k; kw++) {
                int ww = w - kw;
                if (ww < 0 || ww % stride) continue;
                int wo = ww / stride;
                if (wo >= Wo) continue;
                size_t o = LAYOUT == 0 ? (((size_t)n * C + c) * Ho + ho) * Wo + wo
                                       : (((size_t)n * Ho + ho) * Wo + wo) * C + c;
                if (idx[o] == kh * k + kw) acc += gout[o];
            }
        }
        gin[i] = acc;
    }
}

template <int LAYOUT>
int maxpool_fwd(float* out, uint8_t* idx, const float* in, int N, int C, int H, int W, int k, int s, cudaStream_t st) {
    const int Ho = (H - k) / s + 1, Wo = (W - k) / s + 1;
    const bool vec = LAYOUT == 1 && (C % 4 == 0) && ((uintptr_t)out % 16 == 0) && ((uintptr_t)in % 16 == 0) &&
                     (!idx || (uintptr_t)idx % 4 == 0);
    const size_t total = (size_t)N * C * Ho * Wo / (vec ? 4 : 1);
    if (total == 0) return NC_CUDA_OK;
    int grid = grid_for((long long)total, kThreads);
    if (vec) maxpool_fwd_kernel<1, 4><<<grid, kThreads, 0, st>>>(out, idx, in, N, C, H, W, Ho, Wo, k, s);
    else maxpool_fwd_kernel<LAYOUT, 1><<<grid, kThreads, 0, st>>>(out, idx, in, N, C, H, W, Ho, Wo, k, s);
    NCC_COUNT_LAUNCH();
    return launch_status("maxpool_forward");
}

template <int LAYOUT>
int maxpool_bwd(float* gin, const float* gout, const uint8_t* idx, int N, int C, int H, int W, int k, int s,
                cudaStream_t st) {
    const int Ho = (H - k) / s + 1, Wo = (W - k) / s + 1;
    if ((size_t)N * C * H * W == 0) return NC_CUDA_OK;
    if (s < k) {
        maxpool_bwd_gather_kernel<LAYOUT><<<grid_for((long long)N * C * H * W, kThreads), kThreads, 0, st>>>(
            gin, gout, idx, N, C, H, W, Ho, Wo, k, s);
        NCC_COUNT_LAUNCH();
        return launch_status("maxpool_backward(gather)");
    }
    const bool covers = (s == k) && (Ho * s == H) && (Wo * s == W);
    if (!covers) NCC_TRY(cudaMemsetAsync(gin, 0, sizeof(float) * (size_t)N * C * H * W, st));
    const bool vec = LAYOUT == 1 && (C % 4 == 0) && ((uintptr_t)gin % 16 == 0) && ((uintptr_t)gout % 16 == 0) &&
                     ((uintptr_t)idx % 4 == 0);
    const size_t total = (size_t)N * C * Ho * Wo / (vec ? 4 : 1);
    if (total == 0) return NC_CUDA_OK;
    int grid = grid_for((long long)total, kThreads);
    if (vec) maxpool_bwd_own_kernel<1, 4><<<grid, kThreads, 0, st>>>(gin, gout, idx, N, C, H, W, Ho, Wo, k, s);
    else maxpool_bwd_own_kernel<LAYOUT, 1><<<grid, kThreads, 0, st>>>(gin, gout, idx, N, C, H, W, Ho, Wo, k, s);
    NCC_COUNT_LAUNCH();
    return launch_status("maxpool_backward");
}

// =============================================================================================
// Per-channel / per-column two-value reductions (stage 1), shared by BatchNorm and LayerNorm.
// A functor maps an element to the two summands; partial[slab][col][2] (double) is the output.
// =============================================================================================

// Column reduce over a row-major (rows x cols) matrix: NHWC BatchNorm (cols = C) and LayerNorm
// dgamma/dbeta.  Block = 32 column lanes x 8 row lanes; grid.x = column tiles, grid.y = row slabs.
template <class F>
__global__ void __launch_bounds__(256) colreduce_kernel(double* __restrict__ partial, size_t rows, int cols,
                                                        size_t rows_per_slab, F f) {
    __shared__ double sh[2][8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + tx;
    const size_t r0 = (size_t)blockIdx.y * rows_per_slab;
    size_t r1 = r0 + rows_per_slab;
    if (r1 > rows) r1 = rows;
    double a = 0.0, b = 0.0;
    if (c < cols) {
        for (size_t r = r0 + ty; r < r1; r += 8) {
            float v1, v2;
            f(r, c, v1, v2);
            a += (double)v1;
            b += (double)v2;
        }
    }
    sh[0][ty][tx] = a;
    sh[1][ty][tx] = b;
    __syncthreads();
    if (ty == 0 && c < cols) {
        double s1 = 0.0, s2 = 0.0;
#pragma unroll
        for (int k = 0; k < 8; k++) { s1 += sh[0][k][tx]; s2 += sh[1][k][tx]; }
        double* p = partial + ((size_t)blockIdx.y * cols + c) * 2;
        p[0] = s1;
        p[1] = s2;
    }
}

// Same reduction for cols % 4 == 0: each thread owns FOUR consecutive columns (one float4 per row and
// operand), TX threads span the columns of the block and 256 / TX thread rows walk the slab two rows
// at a time, so a warp issues full 128-byte (or wider) requests and several are in flight.
template <class F>
__global__ void __launch_bounds__(256) colreduce4_kernel(double* __restrict__ partial, size_t rows, int cols, size_t rows_per_slab,
                                                         int TX, F f) {
    __shared__ double sh[256][9];
    const int tx = threadIdx.x % TX, ty = threadIdx.x / TX, TY = 256 / TX;
    const int c = (blockIdx.x * TX + tx) * 4;
    const size_t r0 = (size_t)blockIdx.y * rows_per_slab;
    size_t r1 = r0 + rows_per_slab;
    if (r1 > rows) r1 = rows;
    double a[4] = {0, 0, 0, 0}, b[4] = {0, 0, 0, 0};
    if (c < cols) {
        const typename F::Ctx ctx = f.prepare(c);  // per-column constants, read once
        // four rows per step: four independent loads in flight, their values added in f32 (4 terms)
        // before the running sums continue in double (the f32 -> f64 conversions would otherwise
        // limit the kernel, not the memory system)
        size_t r = r0 + ty;
        for (; r + 3 * (size_t)TY < r1; r += 4 * (size_t)TY) {
            float4 u1, u2, w1, w2, p1, p2, q1, q2;
            f.vec(ctx, r, c, u1, u2);
            f.vec(ctx, r + TY, c, w1, w2);
            f.vec(ctx, r + 2 * (size_t)TY, c, p1, p2);
            f.vec(ctx, r + 3 * (size_t)TY, c, q1, q2);
            a[0] += (double)((u1.x + w1.x) + (p1.x + q1.x)); a[1] += (double)((u1.y + w1.y) + (p1.y + q1.y));
            a[2] += (double)((u1.z + w1.z) + (p1.z + q1.z)); a[3] += (double)((u1.w + w1.w) + (p1.w + q1.w));
            b[0] += (double)((u2.x + w2.x) + (p2.x + q2.x)); b[1] += (double)((u2.y + w2.y) + (p2.y + q2.y));
            b[2] += (double)((u2.z + w2.z) + (p2.z + q2.z)); b[3] += (double)((u2.w + w2.w) + (p2.w + q2.w));
        }
        for (; r < r1; r += TY) {
            float4 u1, u2;
            f.vec(ctx, r, c, u1, u2);
            a[0] += u1.x; a[1] += u1.y; a[2] += u1.z; a[3] += u1.w;
            b[0] += u2.x; b[1] += u2.y; b[2] += u2.z; b[3] += u2.w;
        }
    }
#pragma unroll
    for (int j = 0; j < 4; j++) { sh[threadIdx.x][j] = a[j]; sh[threadIdx.x][4 + j] = b[j]; }
    __syncthreads();
    if (ty == 0 && c < cols) {
        double s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int k = 0; k < TY; k++)
#pragma unroll
            for (int j = 0; j < 8; j++) s[j] += sh[k * TX + tx][j];
        double* p = partial + ((size_t)blockIdx.y * cols + c) * 2;
#pragma unroll
        for (int j = 0; j < 4; j++) { p[2 * j] = s[j]; p[2 * j + 1] = s[4 + j]; }
    }
}

// NCHW channel reduce: block (c, j) walks images n = j, j+J, ... of channel c, each a contiguous run
// of `spatial` floats.
template <class F>
__global__ void __launch_bounds__(256) chanreduce_nchw_kernel(double* __restrict__ partial, int N, int C, int spatial, F f) {
    __shared__ double sh[32];
    const int c = blockIdx.x, j = blockIdx.y, J = gridDim.y;
    double a = 0.0, b = 0.0;
    for (int n = j; n < N; n += J) {
        const size_t base = ((size_t)n * C + c) * spatial;
        for (int s = threadIdx.x; s < spatial; s += blockDim.x) {
            float v1, v2;
            f(base + s, c, v1, v2);
            a += (double)v1;
            b += (double)v2;
        }
    }
    a = block_sum(a, sh);
    b = block_sum(b, sh);
    if (threadIdx.x == 0) {
        double* p = partial + ((size_t)j * C + c) * 2;
        p[0] = a;
        p[1] = b;
    }
}

struct BnFwdSum {  // (x, x^2)
    const float* x; int cols;
    __device__ void operator()(size_t r, int c, float& v1, float& v2) const {
        float t = x[r * cols + c]; v1 = t; v2 = t * t;
    }
    struct Ctx {};
    __device__ Ctx prepare(int) const { return Ctx{}; }
    __device__ void vec(const Ctx&, size_t r, int c, float4& v1, float4& v2) const {
        v1 = *reinterpret_cast<const float4*>(x + r * cols + c);
        v2 = make_float4(v1.x * v1.x, v1.y * v1.y, v1.z * v1.z, v1.w * v1.w);
    }
};
struct BnFwdSumFlat {  // NCHW flavour: flat index supplied
    const float* x;
    __device__ void operator()(size_t i, int, float& v1, float& v2) const { float t = x[i]; v1 = t; v2 = t * t; }
};
// (dy, dy * xhat) with optional ReLU mask taken from the forward output
// ReLU mask of a fused BatchNorm+ReLU: either read from the saved forward output y, or recomputed from x with
// exactly the forward expression gamma * ((x - mean) * inv_std) + beta (saves reading y at all)
struct ReluMask {
    const float* y; const float* gamma; const float* beta; int recompute;
    __device__ bool dead(size_t i, float xh, int c) const {
        if (y) return !(y[i] > 0.f);
        if (recompute) return !(((gamma ? gamma[c] : 1.f) * xh + (beta ? beta[c] : 0.f)) > 0.f);
        return false;
    }
};
struct BnBwdSum {
    const float* dy; const float* x; ReluMask m; const float* mean; const float* var; float eps; int cols;
    __device__ void operator()(size_t r, int c, float& v1, float& v2) const {
        size_t i = r * cols + c;
        float g = dy[i];
        float xh = (x[i] - mean[c]) * rsqrtf(var[c] + eps);
        if (m.dead(i, xh, c)) g = 0.f;
        v1 = g; v2 = g * xh;
    }
    struct Ctx { float mu[4], is[4], g[4], b[4]; };
    __device__ Ctx prepare(int c) const {
        Ctx k;
#pragma unroll
        for (int v = 0; v < 4; v++) {
            k.mu[v] = mean[c + v];
            k.is[v] = rsqrtf(var[c + v] + eps);
            k.g[v] = m.gamma ? m.gamma[c + v] : 1.f;
            k.b[v] = m.beta ? m.beta[c + v] : 0.f;
        }
        return k;
    }
    __device__ void vec(const Ctx& k, size_t r, int c, float4& v1, float4& v2) const {
        const size_t i = r * cols + c;
        const float4 gq = *reinterpret_cast<const float4*>(dy + i);
        const float4 xq = *reinterpret_cast<const float4*>(x + i);
        float4 yq = make_float4(1.f, 1.f, 1.f, 1.f);
        if (m.y) yq = *reinterpret_cast<const float4*>(m.y + i);
        const float xv[4] = {xq.x, xq.y, xq.z, xq.w}, yv[4] = {yq.x, yq.y, yq.z, yq.w};
        float g[4] = {gq.x, gq.y, gq.z, gq.w}, gx[4];
#pragma unroll
        for (int v = 0; v < 4; v++) {
            const float xh = (xv[v] - k.mu[v]) * k.is[v];
            if (m.y) { if (!(yv[v] > 0.f)) g[v] = 0.f; }
            else if (m.recompute && !((k.g[v] * xh + k.b[v]) > 0.f)) g[v] = 0.f;
            gx[v] = g[v] * xh;
        }
        v1 = make_float4(g[0], g[1], g[2], g[3]);
        v2 = make_float4(gx[0], gx[1], gx[2], gx[3]);
    }
};
struct BnBwdSumFlat {
    const float* dy; const float* x; ReluMask m; const float* mean; const float* var; float eps;
    __device__ void operator()(size_t i, int c, float& v1, float& v2) const {
        float g = dy[i];
        float xh = (x[i] - mean[c]) * rsqrtf(var[c] + eps);
        if (m.dead(i, xh, c)) g = 0.f;
        v1 = g; v2 = g * xh;
    }
};
// LayerNorm dgamma/dbeta: (g * xhat, g) with per-row statistics
struct LnParamSum {
    const float* g; const float* x; const float2* stats; int cols;
    __device__ void operator()(size_t r, int c, float& v1, float& v2) const {
        size_t i = r * cols + c;
        float2 s = stats[r];
        float gv = g[i];
        v1 = gv * ((x[i] - s.x) * s.y); v2 = gv;
    }
    struct Ctx {};
    __device__ Ctx prepare(int) const { return Ctx{}; }
    __device__ void vec(const Ctx&, size_t r, int c, float4& v1, float4& v2) const {
        const size_t i = r * cols + c;
        const float2 s = stats[r];
        const float4 gv = *reinterpret_cast<const float4*>(g + i);
        const float4 xv = *reinterpret_cast<const float4*>(x + i);
        v1 = make_float4(gv.x * ((xv.x - s.x) * s.y), gv.y * ((xv.y - s.x) * s.y), gv.z * ((xv.z - s.x) * s.y), gv.w * ((xv.w - s.x) * s.y));
        v2 = gv;
    }
};

// Launch the column reduction of a dense (rows x cols) problem; picks the float4 kernel when the
// columns and every operand pointer allow it.  Returns the slab count through *slabs_out.
template <class F>
int launch_colreduce(double** partial_out, int* slabs_out, size_t rows, int cols, bool vec_ok, F f, cudaStream_t st) {
    const bool vec = vec_ok && (cols % 4 == 0);
    int TX = 32, col_tiles;
    if (vec) {
        int c4 = cols / 4;
        TX = c4 >= 32 ? 32 : (c4 >= 16 ? 16 : (c4 >= 8 ? 8 : (c4 >= 4 ? 4 : (c4 >= 2 ? 2 : 1))));
        col_tiles = ceil_div(c4, TX);
    } else {
        col_tiles = ceil_div(cols, 32);
    }
    const size_t min_rows = vec ? (size_t)(256 / TX) * 4 : 64;
    // one wave: as many CTAs as are resident at once for this functor's register use
    static int occ4 = 0, occ1 = 0;  // per template instance
    int& occ = vec ? occ4 : occ1;
    if (occ == 0) {
        cudaError_t e = vec ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, colreduce4_kernel<F>, 256, 0)
                            : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, colreduce_kernel<F>, 256, 0);
        if (e != cudaSuccess || occ < 1) { occ = 2; (void)cudaGetLastError(); }
        if (occ > 4) occ = 4;
    }
    int want = (sm_count() * occ + col_tiles - 1) / col_tiles;
    size_t rps = (rows + want - 1) / want;
    if (rps < min_rows) rps = min_rows;
    int slabs = (int)((rows + rps - 1) / rps);
    if (slabs > 65535) { slabs = 65535; rps = (rows + slabs - 1) / slabs; slabs = (int)((rows + rps - 1) / rps); }
    double* partial = (double*)scratch(7, sizeof(double) * 2 * (size_t)slabs * cols, st);
    if (!partial) return NC_CUDA_ERR_RUNTIME;
    if (vec) colreduce4_kernel<<<dim3(col_tiles, slabs), 256, 0, st>>>(partial, rows, cols, rps, TX, f);
    else colreduce_kernel<<<dim3(col_tiles, slabs), 256, 0, st>>>(partial, rows, cols, rps, f);
    NCC_COUNT_LAUNCH();
    *partial_out = partial;
    *slabs_out = slabs;
    return launch_status("column reduce");
}
inline bool al16(const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Stage 2: a block of 256 threads combines the slabs of 4 neighbouring columns; thread (tx, ty) adds slabs
// ty, ty + 64, ... of column c0 + tx (a slab row of 4 columns is one 64-byte request), then a pairwise tree of
// fixed shape adds the 64 lane sums: the same partials always give the same bits.
constexpr int kFinCols = 4, kFinLanes = 64;
__device__ __forceinline__ bool combine_slabs(const double* __restrict__ partial, int slabs, int C, int* c_out, double* s1, double* s2) {
    __shared__ double sh1[kFinLanes][kFinCols], sh2[kFinLanes][kFinCols];
    const int tx = threadIdx.x & (kFinCols - 1), ty = threadIdx.x / kFinCols;
    const int c = blockIdx.x * kFinCols + tx;
    double a = 0.0, b = 0.0;
    if (c < C) {
#pragma unroll 8
        for (int s = ty; s < slabs; s += kFinLanes) {
            const double2 v = *reinterpret_cast<const double2*>(partial + ((size_t)s * C + c) * 2);
            a += v.x;
            b += v.y;
        }
    }
    sh1[ty][tx] = a;
    sh2[ty][tx] = b;
    __syncthreads();
    // fixed-shape pairwise tree over the lanes (the same order whatever the data)
#pragma unroll
    for (int half = kFinLanes / 2; half >= 1; half >>= 1) {
        if (ty < half) {
            sh1[ty][tx] += sh1[ty + half][tx];
            sh2[ty][tx] += sh2[ty + half][tx];
        }
        __syncthreads();
    }
    if (ty != 0 || c >= C) return false;
    *c_out = c; *s1 = sh1[0][tx]; *s2 = sh2[0][tx];
    return true;
}
inline int fin_grid(int C) { return (C + kFinCols - 1) / kFinCols; }

// Stage 2 for BatchNorm forward: mean / biased variance, running statistics (unbiased variance,
// src/nn/batchnorm.c:307-314).
__global__ void __launch_bounds__(kFinCols * kFinLanes) bn_fwd_finalize_kernel(const double* __restrict__ partial, int slabs, int C, double M,
                                       float* __restrict__ save_mean, float* __restrict__ save_var,
                                       float* __restrict__ run_mean, float* __restrict__ run_var, double momentum) {
    int c;
    double s1, s2;
    if (!combine_slabs(partial, slabs, C, &c, &s1, &s2)) return;
    double mean = s1 / M;
    double var_sum = s2 - s1 * mean;  // sum (x - mean)^2
    if (var_sum < 0.0) var_sum = 0.0;
    double var = var_sum / M;
    save_mean[c] = (float)mean;
    save_var[c] = (float)var;
    if (run_mean && run_var) {
        double unbiased = (M > 1.0) ? var_sum / (M - 1.0) : var;
        run_mean[c] = (float)((1.0 - momentum) * (double)run_mean[c] + momentum * mean);
        run_var[c] = (float)((1.0 - momentum) * (double)run_var[c] + momentum * unbiased);
    }
}

// eval mode: statistics come from the running buffers (or 0 / 1 when absent)
__global__ void bn_eval_stats_kernel(int C, float* __restrict__ save_mean, float* __restrict__ save_var,
                                     const float* __restrict__ run_mean, const float* __restrict__ run_var) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    save_mean[c] = run_mean ? run_mean[c] : 0.f;
    save_var[c] = run_var ? run_var[c] : 1.f;
}

// y = gamma * (x - mean) * inv_std + beta (optionally ReLU).  Flat, float4 when 4 neighbours share
// a channel (NCHW, spatial % 4 == 0) or are 4 consecutive channels (NHWC, C % 4 == 0).
template <int LAYOUT, int VEC>
__global__ void __launch_bounds__(kThreads) bn_apply_kernel(float* __restrict__ y, const float* __restrict__ x,
                                                            const float* __restrict__ gamma, const float* __restrict__ beta,
                                                            const float* __restrict__ mean, const float* __restrict__ var,
                                                            float eps, int C, int spatial, size_t nvec, int relu, int rnd) {
    const size_t gstride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += gstride) {
        const size_t e = i * VEC;
        float xv[VEC], out[VEC];
        if (VEC == 4) {
            float4 t = *reinterpret_cast<const float4*>(x + e);
            xv[0] = t.x; xv[1 % VEC] = t.y; xv[2 % VEC] = t.z; xv[3 % VEC] = t.w;
        } else xv[0] = x[e];
#pragma unroll
        for (int v = 0; v < VEC; v++) {
            int c = LAYOUT == 0 ? (int)((e / spatial) % C) : (int)((e + v) % C);
            float is = rsqrtf(var[c] + eps);
            float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
            float o = g * ((xv[v] - mean[c]) * is) + b;
            o = (relu && !(o > 0.f)) ? 0.f : o;
            out[v] = rnd ? round_tf32(o) : o;
        }
        if (VEC == 4) *reinterpret_cast<float4*>(y + e) = make_float4(out[0], out[1 % VEC], out[2 % VEC], out[3 % VEC]);
        else y[e] = out[0];
    }
}

// Channels-last fast path (C % 4 == 0, 16-byte aligned operands).  The launch makes the total thread
// count times 4 a multiple of C, so a thread meets the same four channels on every grid-stride step:
// their statistics and affine parameters are read once into registers and the loop body is three
// flops per element around one float4 load and one float4 store.  The expression is the one of
// bn_apply_kernel, term by term.
template <int RELU>
__global__ void __launch_bounds__(kThreads) bn_apply_nhwc4_kernel(float4* __restrict__ y, const float4* __restrict__ x,
                                                                  const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                  const float* __restrict__ mean, const float* __restrict__ var,
                                                                  float eps, int C, size_t nvec, int rnd) {
    const unsigned tid = blockIdx.x * kThreads + threadIdx.x, total = gridDim.x * kThreads;
    const int c = (int)((tid * 4ull) % (unsigned)C);
    float mu[4], is[4], g[4], b[4];
#pragma unroll
    for (int v = 0; v < 4; v++) {
        mu[v] = mean[c + v];
        is[v] = rsqrtf(var[c + v] + eps);
        g[v] = gamma ? gamma[c + v] : 1.f;
        b[v] = beta ? beta[c + v] : 0.f;
    }
#pragma unroll 4
    for (size_t i = tid; i < nvec; i += total) {
        const float4 t = (rnd & 2) ? __ldcs(&x[i]) : x[i];   // bit 1: tensors larger than L2, read and written once: streaming hints
        float o[4] = {g[0] * ((t.x - mu[0]) * is[0]) + b[0], g[1] * ((t.y - mu[1]) * is[1]) + b[1],
                      g[2] * ((t.z - mu[2]) * is[2]) + b[2], g[3] * ((t.w - mu[3]) * is[3]) + b[3]};
#pragma unroll
        for (int v = 0; v < 4; v++) {
            if (RELU && !(o[v] > 0.f)) o[v] = 0.f;
            if (rnd & 1) o[v] = round_tf32(o[v]);
        }
        if (rnd & 2) __stcs(&y[i], make_float4(o[0], o[1], o[2], o[3]));
        else y[i] = make_float4(o[0], o[1], o[2], o[3]);
    }
}

// MASK: 0 none, 1 read the forward output, 2 recompute the fused ReLU's sign from x.
template <int MASK>
__global__ void __launch_bounds__(kThreads) bn_bwd_apply_nhwc4_kernel(float4* __restrict__ dx, const float4* __restrict__ dy,
                                                                      const float4* __restrict__ x, const float4* __restrict__ yfwd,
                                                                      const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                      const float* __restrict__ mean, const float* __restrict__ var,
                                                                      const float* __restrict__ sums, float eps, float Mf, int C,
                                                                      size_t nvec, int rnd) {
    const unsigned tid = blockIdx.x * kThreads + threadIdx.x, total = gridDim.x * kThreads;
    const int c = (int)((tid * 4ull) % (unsigned)C);
    float mu[4], is[4], g[4], b[4], coeff[4], s1[4], s2[4];
#pragma unroll
    for (int v = 0; v < 4; v++) {
        mu[v] = mean[c + v];
        is[v] = rsqrtf(var[c + v] + eps);
        g[v] = gamma ? gamma[c + v] : 1.f;
        b[v] = beta ? beta[c + v] : 0.f;
        coeff[v] = g[v] * is[v] / Mf;
        s1[v] = sums[2 * (c + v)];
        s2[v] = sums[2 * (c + v) + 1];
    }
#pragma unroll 2
    for (size_t i = tid; i < nvec; i += total) {
        const float4 t = (rnd & 2) ? __ldcs(&x[i]) : x[i];
        const float4 u = (rnd & 2) ? __ldcs(&dy[i]) : dy[i];
        float4 yv = make_float4(1.f, 1.f, 1.f, 1.f);
        if (MASK == 1) yv = yfwd[i];
        const float xv[4] = {t.x, t.y, t.z, t.w}, yy[4] = {yv.x, yv.y, yv.z, yv.w};
        float gv[4] = {u.x, u.y, u.z, u.w}, o[4];
#pragma unroll
        for (int v = 0; v < 4; v++) {
            const float xh = (xv[v] - mu[v]) * is[v];
            if (MASK == 1 && !(yy[v] > 0.f)) gv[v] = 0.f;
            if (MASK == 2 && !((g[v] * xh + b[v]) > 0.f)) gv[v] = 0.f;
            o[v] = coeff[v] * (Mf * gv[v] - s1[v] - xh * s2[v]);
            if (rnd & 1) o[v] = round_tf32(o[v]);
        }
        if (rnd & 2) __stcs(&dx[i], make_float4(o[0], o[1], o[2], o[3]));
        else dx[i] = make_float4(o[0], o[1], o[2], o[3]);
    }
}

// ---------------------------------------------------------------------------------------------
// BatchNorm + ReLU + 2x2 / stride-2 max-pool in one pass each way (channels-last, C % 4 == 0, H and W even).
// Forward reads x once and writes only the pooled tensor and the window offsets: the full-resolution
// activation is never materialised (its backward needs x, the statistics and the offsets only).
// Same arithmetic, same order, same tie rule (first maximum in (kh, kw) order wins) as bn_apply followed
// by maxpool_fwd_kernel.  A thread keeps its four channels for the whole grid-stride walk.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) bn_relu_pool2_fwd_kernel(float4* __restrict__ pooled, uchar4* __restrict__ idx,
                                                                     const float4* __restrict__ x, const float* __restrict__ gamma,
                                                                     const float* __restrict__ beta, const float* __restrict__ mean,
                                                                     const float* __restrict__ var, float eps, int C, int H, int W,
                                                                     size_t nvec_out, int rnd) {
    const unsigned tid = blockIdx.x * kThreads + threadIdx.x, total = gridDim.x * kThreads;
    const int C4 = C >> 2, Ho = H >> 1, Wo = W >> 1;
    const int c = (int)((tid * 4ull) % (unsigned)C);
    float mu[4], is[4], g[4], b[4];
#pragma unroll
    for (int v = 0; v < 4; v++) {
        mu[v] = mean[c + v];
        is[v] = rsqrtf(var[c + v] + eps);
        g[v] = gamma ? gamma[c + v] : 1.f;
        b[v] = beta ? beta[c + v] : 0.f;
    }
    for (size_t i = tid; i < nvec_out; i += total) {
        const unsigned pix = (unsigned)(i / (unsigned)C4);  // pooled pixel (n, ho, wo)
        const unsigned wo = pix % (unsigned)Wo, t = pix / (unsigned)Wo, ho = t % (unsigned)Ho, n = t / (unsigned)Ho;
        const size_t base = (((size_t)n * H + 2 * ho) * W + 2 * wo) * C4 + (c >> 2);
        float best[4] = {-1e30f, -1e30f, -1e30f, -1e30f};
        int bi[4] = {0, 0, 0, 0};
#pragma unroll
        for (int pos = 0; pos < 4; pos++) {
            const float4 q = x[base + ((size_t)(pos >> 1) * W + (pos & 1)) * C4];
            const float xv[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int v = 0; v < 4; v++) {
                float o = g[v] * ((xv[v] - mu[v]) * is[v]) + b[v];
                if (!(o > 0.f)) o = 0.f;
                // the window offset is decided on the unrounded value, as the reference decides it: two candidates
                // closer than a TF32 step must not turn into a tie that the scan order breaks
                if (o > best[v]) { best[v] = o; bi[v] = pos; }
            }
        }
        if (rnd & 1) {   // rounding is monotonic: the rounded maximum is the maximum of the rounded values
#pragma unroll
            for (int v = 0; v < 4; v++) best[v] = round_tf32(best[v]);
        }
        pooled[i] = make_float4(best[0], best[1], best[2], best[3]);
        if (idx) idx[i] = make_uchar4((uint8_t)bi[0], (uint8_t)bi[1], (uint8_t)bi[2], (uint8_t)bi[3]);
    }
}

// Stage-1 functor of the fused backward: rows are POOLED pixels; the gradient lives only at each window's saved offset.
struct BnPoolBwdSum {
    const float* dp; const uint8_t* idx; const float* x; const float* gamma; const float* beta; const float* mean; const float* var;
    float eps; int cols, H, W;
    struct Ctx { float mu[4], is[4], g[4], b[4]; };
    __device__ Ctx prepare(int c) const {
        Ctx k;
#pragma unroll
        for (int v = 0; v < 4; v++) {
            k.mu[v] = mean[c + v];
            k.is[v] = rsqrtf(var[c + v] + eps);
            k.g[v] = gamma ? gamma[c + v] : 1.f;
            k.b[v] = beta ? beta[c + v] : 0.f;
        }
        return k;
    }
    __device__ void vec(const Ctx& k, size_t r, int c, float4& v1, float4& v2) const {
        const unsigned Wo = (unsigned)(W >> 1), Ho = (unsigned)(H >> 1);
        const unsigned pix = (unsigned)r, wo = pix % Wo, t = pix / Wo, ho = t % Ho, n = t / Ho;
        const float4 gq = *reinterpret_cast<const float4*>(dp + r * cols + c);
        const uchar4 iq = *reinterpret_cast<const uchar4*>(idx + r * cols + c);
        const size_t base = (((size_t)n * H + 2 * ho) * W + 2 * wo) * cols + c;
        const int pos[4] = {iq.x, iq.y, iq.z, iq.w};
        float g[4] = {gq.x, gq.y, gq.z, gq.w}, gx[4];
#pragma unroll
        for (int v = 0; v < 4; v++) {
            const float xv = x[base + ((size_t)(pos[v] >> 1) * W + (pos[v] & 1)) * cols + v];
            const float xh = (xv - k.mu[v]) * k.is[v];
            if (!((k.g[v] * xh + k.b[v]) > 0.f)) g[v] = 0.f;
            gx[v] = g[v] * xh;
        }
        v1 = make_float4(g[0], g[1], g[2], g[3]);
        v2 = make_float4(gx[0], gx[1], gx[2], gx[3]);
    }
    __device__ void operator()(size_t, int, float& v1, float& v2) const { v1 = 0.f; v2 = 0.f; }  // scalar path unused (C % 4 == 0 required)
};

// dx for all four positions of each window: the pooled gradient at the saved offset, zero elsewhere, both under
// the recomputed ReLU mask, through dx = gamma * inv_std / M * (M * g - sum_g - xhat * sum_gx).
__global__ void __launch_bounds__(kThreads) bn_relu_pool2_bwd_apply_kernel(float4* __restrict__ dx, const float4* __restrict__ dp,
                                                                           const uchar4* __restrict__ idx, const float4* __restrict__ x,
                                                                           const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                           const float* __restrict__ mean, const float* __restrict__ var,
                                                                           const float* __restrict__ sums, float eps, float Mf, int C, int H,
                                                                           int W, size_t nvec_out, int rnd) {
    const unsigned tid = blockIdx.x * kThreads + threadIdx.x, total = gridDim.x * kThreads;
    const int C4 = C >> 2, Ho = H >> 1, Wo = W >> 1;
    const int c = (int)((tid * 4ull) % (unsigned)C);
    float mu[4], is[4], g[4], b[4], coeff[4], s1[4], s2[4];
#pragma unroll
    for (int v = 0; v < 4; v++) {
        mu[v] = mean[c + v];
        is[v] = rsqrtf(var[c + v] + eps);
        g[v] = gamma ? gamma[c + v] : 1.f;
        b[v] = beta ? beta[c + v] : 0.f;
        coeff[v] = g[v] * is[v] / Mf;
        s1[v] = sums[2 * (c + v)];
        s2[v] = sums[2 * (c + v) + 1];
    }
    for (size_t i = tid; i < nvec_out; i += total) {
        const unsigned pix = (unsigned)(i / (unsigned)C4);
        const unsigned wo = pix % (unsigned)Wo, t = pix / (unsigned)Wo, ho = t % (unsigned)Ho, n = t / (unsigned)Ho;
        const size_t base = (((size_t)n * H + 2 * ho) * W + 2 * wo) * C4 + (c >> 2);
        const float4 gq = dp[i];
        const uchar4 iq = idx[i];
        const float gp[4] = {gq.x, gq.y, gq.z, gq.w};
        const int sel[4] = {iq.x, iq.y, iq.z, iq.w};
#pragma unroll
        for (int pos = 0; pos < 4; pos++) {
            const size_t at = base + ((size_t)(pos >> 1) * W + (pos & 1)) * C4;
            const float4 q = x[at];
            const float xv[4] = {q.x, q.y, q.z, q.w};
            float o[4];
#pragma unroll
            for (int v = 0; v < 4; v++) {
                const float xh = (xv[v] - mu[v]) * is[v];
                float gv = sel[v] == pos ? gp[v] : 0.f;
                if (!((g[v] * xh + b[v]) > 0.f)) gv = 0.f;
                o[v] = coeff[v] * (Mf * gv - s1[v] - xh * s2[v]);
                if (rnd & 1) o[v] = round_tf32(o[v]);
            }
            dx[at] = make_float4(o[0], o[1], o[2], o[3]);
        }
    }
}

// Grid for the channels-last fast path: blocks * kThreads * 4 must be a multiple of C.
inline int nhwc4_grid(size_t nvec, int C) {
    int a = C, b = kThreads * 4;
    while (b) { int t = a % b; a = b; b = t; }
    const int unit = C / a;  // C / gcd(C, 1024)
    long long want = grid_for((long long)nvec, kThreads);
    long long g = (want / unit) * unit;
    if (g < unit) g = unit;
    return (int)g;
}

__global__ void __launch_bounds__(kFinCols * kFinLanes) bn_bwd_finalize_kernel(const double* __restrict__ partial, int slabs, int C,
                                       float* __restrict__ dgamma, float* __restrict__ dbeta, float* __restrict__ sums) {
    int c;
    double s1, s2;
    if (!combine_slabs(partial, slabs, C, &c, &s1, &s2)) return;
    if (dbeta) dbeta[c] = (float)s1;
    if (dgamma) dgamma[c] = (float)s2;
    sums[2 * c] = (float)s1;
    sums[2 * c + 1] = (float)s2;
}

// dx = gamma * inv_std / M * (M * g - sum_g - xhat * sum_gx)   (src/nn/batchnorm.c:145-158)
template <int LAYOUT, int VEC>
__global__ void __launch_bounds__(kThreads) bn_bwd_apply_kernel(float* __restrict__ dx, const float* __restrict__ dy,
                                                                const float* __restrict__ x, ReluMask mask,
                                                                const float* __restrict__ gamma, const float* __restrict__ mean,
                                                                const float* __restrict__ var, const float* __restrict__ sums,
                                                                float eps, float Mf, int C, int spatial, size_t nvec, int rnd) {
    const size_t gstride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += gstride) {
        const size_t e = i * VEC;
        float xv[VEC], gv[VEC], out[VEC];
        if (VEC == 4) {
            float4 t = *reinterpret_cast<const float4*>(x + e);
            float4 u = *reinterpret_cast<const float4*>(dy + e);
            xv[0] = t.x; xv[1 % VEC] = t.y; xv[2 % VEC] = t.z; xv[3 % VEC] = t.w;
            gv[0] = u.x; gv[1 % VEC] = u.y; gv[2 % VEC] = u.z; gv[3 % VEC] = u.w;
        } else {
            xv[0] = x[e]; gv[0] = dy[e];
        }
#pragma unroll
        for (int v = 0; v < VEC; v++) {
            int c = LAYOUT == 0 ? (int)((e / spatial) % C) : (int)((e + v) % C);
            float is = rsqrtf(var[c] + eps);
            float g = gv[v];
            float xh = (xv[v] - mean[c]) * is;
            if (mask.dead(e + v, xh, c)) g = 0.f;
            float coeff = (gamma ? gamma[c] : 1.f) * is / Mf;
            float o = coeff * (Mf * g - sums[2 * c] - xh * sums[2 * c + 1]);
            out[v] = rnd ? round_tf32(o) : o;
        }
        if (VEC == 4) *reinterpret_cast<float4*>(dx + e) = make_float4(out[0], out[1 % VEC], out[2 % VEC], out[3 % VEC]);
        else dx[e] = out[0];
    }
}

// Launch stage 1 for a (N, C, spatial) tensor in either layout; returns the slab count.
template <class FR, class FF>
int channel_reduce(double** partial_out, int* slabs_out, int N, int C, int spatial, int layout, FR frows, FF fflat,
                   bool vec_ok, cudaStream_t st) {
    if (layout == 1) {
        int rc = launch_colreduce(partial_out, slabs_out, (size_t)N * spatial, C, vec_ok, frows, st);
        if (rc) return rc;
    } else {
        int J = (sm_count() * 4 + C - 1) / C;
        if (J > N) J = N;
        if (J < 1) J = 1;
        if (J > 65535) J = 65535;
        double* partial = (double*)scratch(7, sizeof(double) * 2 * (size_t)J * C, st);
        if (!partial) return NC_CUDA_ERR_RUNTIME;
        chanreduce_nchw_kernel<<<dim3(C, J), 256, 0, st>>>(partial, N, C, spatial, fflat);
        NCC_COUNT_LAUNCH();
        *partial_out = partial;
        *slabs_out = J;
    }
    return launch_status("channel_reduce");
}

// =============================================================================================
// LayerNorm: one warp per row.
// =============================================================================================
__global__ void __launch_bounds__(kThreads) ln_fwd_kernel(float* __restrict__ y, const float* __restrict__ x,
                                                          const float* __restrict__ gamma, const float* __restrict__ beta,
                                                          size_t rows, int cols, float eps, int rnd) {
    const int lane = threadIdx.x & 31;
    const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const float* xr = x + r * cols;
        float* yr = y + r * cols;
        double s = 0.0;
        for (int c = lane; c < cols; c += 32) s += (double)xr[c];
        s = warp_sum(s);
        const float mean = (float)(s / cols);
        double q = 0.0;
        for (int c = lane; c < cols; c += 32) { float d = xr[c] - mean; q += (double)d * d; }
        q = warp_sum(q);
        const float inv = (float)(1.0 / sqrt(q / cols + (double)eps));
        for (int c = lane; c < cols; c += 32) {
            float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
            float o = g * ((xr[c] - mean) * inv) + b;
            yr[c] = rnd ? round_tf32(o) : o;
        }
    }
}

// dx and per-row (mean, inv_std) for the parameter-gradient pass.
__global__ void __launch_bounds__(kThreads) ln_bwd_rows_kernel(float* __restrict__ dx, float2* __restrict__ stats,
                                                               const float* __restrict__ dy, const float* __restrict__ x,
                                                               const float* __restrict__ gamma, size_t rows, int cols,
                                                               float eps, int rnd) {
    const int lane = threadIdx.x & 31;
    const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const float* xr = x + r * cols;
        const float* gr = dy + r * cols;
        double s = 0.0;
        for (int c = lane; c < cols; c += 32) s += (double)xr[c];
        s = warp_sum(s);
        const float mean = (float)(s / cols);
        double q = 0.0;
        for (int c = lane; c < cols; c += 32) { float d = xr[c] - mean; q += (double)d * d; }
        q = warp_sum(q);
        const float inv = (float)(1.0 / sqrt(q / cols + (double)eps));
        double sg = 0.0, sgx = 0.0;
        for (int c = lane; c < cols; c += 32) {
            float gg = gr[c] * (gamma ? gamma[c] : 1.f);
            float xh = (xr[c] - mean) * inv;
            sg += (double)gg;
            sgx += (double)gg * (double)xh;
        }
        sg = warp_sum(sg);
        sgx = warp_sum(sgx);
        const float fsg = (float)sg, fsgx = (float)sgx, D = (float)cols, coeff = inv / D;
        for (int c = lane; c < cols; c += 32) {
            float gg = gr[c] * (gamma ? gamma[c] : 1.f);
            float xh = (xr[c] - mean) * inv;
            float o = coeff * (D * gg - fsg - xh * fsgx);
            dx[r * cols + c] = rnd ? round_tf32(o) : o;
        }
        if (lane == 0 && stats) stats[r] = make_float2(mean, inv);
    }
}

__global__ void __launch_bounds__(kFinCols * kFinLanes) ln_param_finalize_kernel(const double* __restrict__ partial, int slabs, int cols,
                                         float* __restrict__ dgamma, float* __restrict__ dbeta) {
    int c;
    double s1, s2;
    if (!combine_slabs(partial, slabs, cols, &c, &s1, &s2)) return;
    if (dgamma) dgamma[c] = (float)s1;
    if (dbeta) dbeta[c] = (float)s2;
}

struct ColSum {  // (x, 0)
    const float* x; int cols;
    __device__ void operator()(size_t r, int c, float& v1, float& v2) const { v1 = x[r * cols + c]; v2 = 0.f; }
    struct Ctx {};
    __device__ Ctx prepare(int) const { return Ctx{}; }
    __device__ void vec(const Ctx&, size_t r, int c, float4& v1, float4& v2) const {
        v1 = *reinterpret_cast<const float4*>(x + r * cols + c);
        v2 = make_float4(0.f, 0.f, 0.f, 0.f);
    }
};

}  // namespace

int ncc::column_sums(float* out, const float* in, size_t rows, int cols, cudaStream_t st) {
    if (cols <= 0) return NC_CUDA_OK;
    NCC_REQUIRE(out && (in || rows == 0), "column_sums: null pointer");
    ProfScope prof(PROF_REDUCE, 4.0 * (double)rows * cols, st);
    if (rows == 0) { NCC_TRY(cudaMemsetAsync(out, 0, sizeof(float) * cols, st)); return NC_CUDA_OK; }
    double* partial = nullptr;
    int slabs = 0;
    int rc = launch_colreduce(&partial, &slabs, rows, cols, al16(in), ColSum{in, cols}, st);
    if (rc) return rc;
    ln_param_finalize_kernel<<<fin_grid(cols), kFinCols * kFinLanes, 0, st>>>(partial, slabs, cols, out, nullptr);
    NCC_COUNT_LAUNCH();
    return launch_status("column_sums");
}

extern "C" {

int nc_cuda_maxpool2d_forward_idx_f32_ex(float* out, uint8_t* argmax, const float* in, int N, int C, int H, int W,
                                         int k, int stride, int layout, void* stream) {
    NCC_REQUIRE(out && in && N >= 0 && C > 0 && k > 0 && stride > 0 && H >= k && W >= k && k * k <= 255,
                "maxpool_forward: bad argument");
    // algorithmic bytes: the input once, the pooled output, one byte of window offset per output
    const double n_out = (double)N * C * ((H - k) / stride + 1) * ((W - k) / stride + 1);
    ProfScope prof(PROF_MAXPOOL, 4.0 * N * C * (double)H * W + n_out * (4.0 + (argmax ? 1.0 : 0.0)), (cudaStream_t)stream);
    if (layout == 0) return maxpool_fwd<0>(out, argmax, in, N, C, H, W, k, stride, (cudaStream_t)stream);
    return maxpool_fwd<1>(out, argmax, in, N, C, H, W, k, stride, (cudaStream_t)stream);
}
int nc_cuda_maxpool2d_backward_idx_f32_ex(float* gin, const float* gout, const uint8_t* argmax, int N, int C, int H,
                                          int W, int k, int stride, int layout, void* stream) {
    NCC_REQUIRE(gin && gout && argmax && C > 0 && k > 0 && stride > 0 && H >= k && W >= k,
                "maxpool_backward: bad argument");
    const double n_out = (double)N * C * ((H - k) / stride + 1) * ((W - k) / stride + 1);
    ProfScope prof(PROF_MAXPOOL, 4.0 * N * C * (double)H * W + n_out * 5.0, (cudaStream_t)stream);
    if (layout == 0) return maxpool_bwd<0>(gin, gout, argmax, N, C, H, W, k, stride, (cudaStream_t)stream);
    return maxpool_bwd<1>(gin, gout, argmax, N, C, H, W, k, stride, (cudaStream_t)stream);
}
void nc_cuda_maxpool2d_forward_f32(float* out, const float* in, int N, int C, int H, int W, int kH, int kW, int stride) {
    if (kH != kW) { set_status(NC_CUDA_ERR_UNSUPPORTED, "maxpool: only square windows"); return; }
    nc_cuda_maxpool2d_forward_idx_f32_ex(out, nullptr, in, N, C, H, W, kH, stride, 0, current_stream());
}
// The legacy backward has no saved argmax: recompute it from the saved input (as the CPU path does).
void nc_cuda_maxpool2d_backward_f32(float* gin, const float* gout, const float* input, const float* output, int N,
                                    int C, int H, int W, int kH, int kW, int stride) {
    (void)output;
    if (kH != kW) { set_status(NC_CUDA_ERR_UNSUPPORTED, "maxpool: only square windows"); return; }
    cudaStream_t st = current_stream();
    const int Ho = (H - kH) / stride + 1, Wo = (W - kW) / stride + 1;
    const size_t no = (size_t)N * C * Ho * Wo;
    char* buf = (char*)scratch(4, no * sizeof(float) + no + 64, st);
    if (!buf) return;
    float* tmp = (float*)buf;
    uint8_t* idx = (uint8_t*)(buf + no * sizeof(float));
    if (nc_cuda_maxpool2d_forward_idx_f32_ex(tmp, idx, input, N, C, H, W, kH, stride, 0, st)) return;
    nc_cuda_maxpool2d_backward_idx_f32_ex(gin, gout, idx, N, C, H, W, kH, stride, 0, st);
}

int nc_cuda_batchnorm_forward_f32_ex(float* y, const float* x, const float* gamma, const float* beta, float* run_mean,
                                     float* run_var, float* save_mean, float* save_var, int N, int C, int spatial,
                                     double momentum, double eps, int training, int layout, int relu, void* stream) {
    NCC_REQUIRE(y && x && save_mean && save_var && N > 0 && C > 0 && spatial > 0, "batchnorm_forward: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t total = (size_t)N * C * spatial;
    ProfScope prof(PROF_BATCHNORM, 8.0 * (double)total, st);   // read x, write y (+ read x for the statistics, below)
    if (training) {
        double* partial = nullptr;
        int slabs = 0;
        // the convolution that produced x may have left its per-channel sums behind (see nc_cuda_set_conv_stats)
        if (!(layout == 1 && conv_stats_take(x, C, (long long)N * spatial, &partial, &slabs))) {
            prof.add_work(4.0 * (double)total);
            int rc = channel_reduce(&partial, &slabs, N, C, spatial, layout, BnFwdSum{x, C}, BnFwdSumFlat{x}, al16(x), st);
            if (rc) return rc;
        }
        bn_fwd_finalize_kernel<<<fin_grid(C), kFinCols * kFinLanes, 0, st>>>(partial, slabs, C, (double)N * spatial, save_mean,
                                                                save_var, run_mean, run_var, momentum);
    } else {
        bn_eval_stats_kernel<<<ceil_div(C, 128), 128, 0, st>>>(C, save_mean, save_var, run_mean, run_var);
    }
    NCC_COUNT_LAUNCH();
    const bool al = ((uintptr_t)y % 16 == 0) && ((uintptr_t)x % 16 == 0);
    const bool vec = al && (layout == 0 ? spatial % 4 == 0 : C % 4 == 0);
    const size_t nvec = vec ? total / 4 : total;
    const int grid = grid_for((long long)nvec, kThreads);
    const float fe = (float)eps;
    if (layout == 0) {
        if (vec) bn_apply_kernel<0, 4><<<grid, kThreads, 0, st>>>(y, x, gamma, beta, save_mean, save_var, fe, C, spatial, nvec, relu, round_outputs() ? 1 : 0);
        else bn_apply_kernel<0, 1><<<grid, kThreads, 0, st>>>(y, x, gamma, beta, save_mean, save_var, fe, C, spatial, nvec, relu, round_outputs() ? 1 : 0);
    } else {
        if (vec) {
            const int g4 = nhwc4_grid(nvec, C);
            const int flags = (round_outputs() ? 1 : 0) | (total * 4 > kStreamBytes ? 2 : 0);
            if (relu) bn_apply_nhwc4_kernel<1><<<g4, kThreads, 0, st>>>((float4*)y, (const float4*)x, gamma, beta, save_mean, save_var, fe, C, nvec, flags);
            else bn_apply_nhwc4_kernel<0><<<g4, kThreads, 0, st>>>((float4*)y, (const float4*)x, gamma, beta, save_mean, save_var, fe, C, nvec, flags);
        } else bn_apply_kernel<1, 1><<<grid, kThreads, 0, st>>>(y, x, gamma, beta, save_mean, save_var, fe, C, spatial, nvec, relu, round_outputs() ? 1 : 0);
    }
    NCC_COUNT_LAUNCH();
    return launch_status("batchnorm_forward");
}

int nc_cuda_batchnorm_backward_f32_ex(float* dx, float* dgamma, float* dbeta, const float* dy, const float* x,
                                      const float* gamma, const float* save_mean, const float* save_var,
                                      const float* relu_out, const float* relu_beta, int relu_recompute, int N, int C,
                                      int spatial, double eps, int layout, void* stream) {
    NCC_REQUIRE(dx && dy && x && save_mean && save_var && N > 0 && C > 0 && spatial > 0, "batchnorm_backward: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t total = (size_t)N * C * spatial;
    const float fe = (float)eps;
    double* partial = nullptr;
    int slabs = 0;
    // sums pass reads dy and x (and the saved ReLU output when there is one), apply pass reads them again and writes dx
    // ... unless the convolution that wrote dy summed on its way out (nc_cuda_offer_batchnorm_backward_sums_f32)
    const bool folded = layout == 1 && relu_recompute && !relu_out &&
                        bn_fold_take(dy, BnFold{x, save_mean, save_var, gamma, relu_beta, fe, C, (long long)N * spatial}, &partial, &slabs);
    ProfScope prof(PROF_BATCHNORM, (folded ? 12.0 : (relu_out ? 28.0 : 20.0)) * (double)total, st);
    const ReluMask mask{relu_out, gamma, relu_beta, relu_out ? 0 : (relu_recompute ? 1 : 0)};
    if (!folded) {
        int rc = channel_reduce(&partial, &slabs, N, C, spatial, layout,
                                BnBwdSum{dy, x, mask, save_mean, save_var, fe, C},
                                BnBwdSumFlat{dy, x, mask, save_mean, save_var, fe},
                                al16(dy) && al16(x) && al16(relu_out) && al16(save_mean) && al16(save_var), st);
        if (rc) return rc;
    }
    float* sums = (float*)scratch(6, sizeof(float) * 2 * (size_t)C, st);
    if (!sums) return NC_CUDA_ERR_RUNTIME;
    bn_bwd_finalize_kernel<<<fin_grid(C), kFinCols * kFinLanes, 0, st>>>(partial, slabs, C, dgamma, dbeta, sums);
    NCC_COUNT_LAUNCH();
    const bool al = ((uintptr_t)dx % 16 == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)dy % 16 == 0) &&
                    (!relu_out || (uintptr_t)relu_out % 16 == 0);
    const bool vec = al && (layout == 0 ? spatial % 4 == 0 : C % 4 == 0);
    const size_t nvec = vec ? total / 4 : total;
    const int grid = grid_for((long long)nvec, kThreads);
    const float Mf = (float)((double)N * spatial);
    if (layout == 0) {
        if (vec) bn_bwd_apply_kernel<0, 4><<<grid, kThreads, 0, st>>>(dx, dy, x, mask, gamma, save_mean, save_var, sums, fe, Mf, C, spatial, nvec, round_outputs() ? 1 : 0);
        else bn_bwd_apply_kernel<0, 1><<<grid, kThreads, 0, st>>>(dx, dy, x, mask, gamma, save_mean, save_var, sums, fe, Mf, C, spatial, nvec, round_outputs() ? 1 : 0);
    } else {
        if (vec) {
            const int g4 = nhwc4_grid(nvec, C);
            const int rnd = (round_outputs() ? 1 : 0) | (total * 4 > kStreamBytes ? 2 : 0);
            if (relu_out) bn_bwd_apply_nhwc4_kernel<1><<<g4, kThreads, 0, st>>>((float4*)dx, (const float4*)dy, (const float4*)x, (const float4*)relu_out, gamma, relu_beta, save_mean, save_var, sums, fe, Mf, C, nvec, rnd);
            else if (relu_recompute) bn_bwd_apply_nhwc4_kernel<2><<<g4, kThreads, 0, st>>>((float4*)dx, (const float4*)dy, (const float4*)x, nullptr, gamma, relu_beta, save_mean, save_var, sums, fe, Mf, C, nvec, rnd);
            else bn_bwd_apply_nhwc4_kernel<0><<<g4, kThreads, 0, st>>>((float4*)dx, (const float4*)dy, (const float4*)x, nullptr, gamma, relu_beta, save_mean, save_var, sums, fe, Mf, C, nvec, rnd);
        } else bn_bwd_apply_kernel<1, 1><<<grid, kThreads, 0, st>>>(dx, dy, x, mask, gamma, save_mean, save_var, sums, fe, Mf, C, spatial, nvec, round_outputs() ? 1 : 0);
    }
    NCC_COUNT_LAUNCH();
    return launch_status("batchnorm_backward");
}

int nc_cuda_batchnorm_relu_maxpool2_forward_f32_ex(float* pooled, uint8_t* argmax, const float* x, const float* gamma,
                                                   const float* beta, float* run_mean, float* run_var, float* save_mean,
                                                   float* save_var, int N, int C, int H, int W, double momentum, double eps,
                                                   int training, void* stream) {
    NCC_REQUIRE(pooled && x && save_mean && save_var && N > 0 && C > 0 && H > 0 && W > 0, "batchnorm_relu_maxpool2_forward: bad argument");
    NCC_REQUIRE((C % 4 == 0) && (H % 2 == 0) && (W % 2 == 0), "batchnorm_relu_maxpool2_forward: needs C %% 4 == 0 and even H, W");
    NCC_REQUIRE(al16(pooled) && al16(x) && ((uintptr_t)argmax % 4 == 0), "batchnorm_relu_maxpool2_forward: misaligned operand");
    NCC_REQUIRE((size_t)N * (H / 2) * (W / 2) < 0xffffffffull, "batchnorm_relu_maxpool2_forward: too many pixels");
    cudaStream_t st = (cudaStream_t)stream;
    // read x, write the pooled quarter and one byte of window offset per pooled element (+ x again for the statistics)
    ProfScope prof(PROF_BATCHNORM, (4.0 + 1.0 + 0.25) * (double)N * C * H * W, st);
    if (training) {
        double* partial = nullptr;
        int slabs = 0;
        if (!conv_stats_take(x, C, (long long)N * H * W, &partial, &slabs)) {
            prof.add_work(4.0 * (double)N * C * H * W);
            int rc = channel_reduce(&partial, &slabs, N, C, H * W, 1, BnFwdSum{x, C}, BnFwdSumFlat{x}, true, st);
            if (rc) return rc;
        }
        bn_fwd_finalize_kernel<<<fin_grid(C), kFinCols * kFinLanes, 0, st>>>(partial, slabs, C, (double)N * H * W, save_mean, save_var, run_mean,
                                                                run_var, momentum);
    } else {
        bn_eval_stats_kernel<<<ceil_div(C, 128), 128, 0, st>>>(C, save_mean, save_var, run_mean, run_var);
    }
    NCC_COUNT_LAUNCH();
    const size_t nvec = (size_t)N * (H / 2) * (W / 2) * (C / 4);
    bn_relu_pool2_fwd_kernel<<<nhwc4_grid(nvec, C), kThreads, 0, st>>>((float4*)pooled, (uchar4*)argmax, (const float4*)x, gamma, beta,
                                                                     save_mean, save_var, (float)eps, C, H, W, nvec,
                                                                     round_outputs() ? 1 : 0);
    NCC_COUNT_LAUNCH();
    return launch_status("batchnorm_relu_maxpool2_forward");
}

int nc_cuda_batchnorm_relu_maxpool2_backward_f32_ex(float* dx, float* dgamma, float* dbeta, const float* dpooled,
                                                    const uint8_t* argmax, const float* x, const float* gamma, const float* beta,
                                                    const float* save_mean, const float* save_var, int N, int C, int H, int W,
                                                    double eps, void* stream) {
    NCC_REQUIRE(dx && dpooled && argmax && x && save_mean && save_var && N > 0 && C > 0 && H > 0 && W > 0,
                "batchnorm_relu_maxpool2_backward: bad argument");
    NCC_REQUIRE((C % 4 == 0) && (H % 2 == 0) && (W % 2 == 0), "batchnorm_relu_maxpool2_backward: needs C %% 4 == 0 and even H, W");
    NCC_REQUIRE(al16(dx) && al16(dpooled) && al16(x) && ((uintptr_t)argmax % 4 == 0), "batchnorm_relu_maxpool2_backward: misaligned operand");
    NCC_REQUIRE((size_t)N * (H / 2) * (W / 2) < 0xffffffffull, "batchnorm_relu_maxpool2_backward: too many pixels");
    cudaStream_t st = (cudaStream_t)stream;
    const float fe = (float)eps;
    double* partial = nullptr;
    int slabs = 0;
    const size_t prow = (size_t)N * (H / 2) * (W / 2);
    // both passes read x, the pooled gradient and the window offsets; the second writes dx
    ProfScope prof(PROF_BATCHNORM, (2.0 * (4.0 + 1.0 + 0.25) + 4.0) * (double)N * C * H * W, st);
    int rc = launch_colreduce(&partial, &slabs, prow, C, true, BnPoolBwdSum{dpooled, argmax, x, gamma, beta, save_mean, save_var, fe, C, H, W}, st);
    if (rc) return rc;
    float* sums = (float*)scratch(6, sizeof(float) * 2 * (size_t)C, st);
    if (!sums) return NC_CUDA_ERR_RUNTIME;
    bn_bwd_finalize_kernel<<<fin_grid(C), kFinCols * kFinLanes, 0, st>>>(partial, slabs, C, dgamma, dbeta, sums);
    NCC_COUNT_LAUNCH();
    const size_t nvec = prow * (C / 4);
    bn_relu_pool2_bwd_apply_kernel<<<nhwc4_grid(nvec, C), kThreads, 0, st>>>((float4*)dx, (const float4*)dpooled, (const uchar4*)argmax,
                                                                           (const float4*)x, gamma, beta, save_mean, save_var, sums, fe,
                                                                           (float)((double)N * H * W), C, H, W, nvec,
                                                                           round_outputs() ? 1 : 0);
    NCC_COUNT_LAUNCH();
    return launch_status("batchnorm_relu_maxpool2_backward");
}

void nc_cuda_batchnorm_forward_f32(float* y, const float* x, const float* gamma, const float* beta, float* rm, float* rv,
                                   float* save_mean, float* save_var, int N, int C, int spatial, float momentum,
                                   float eps, bool training) {
    nc_cuda_batchnorm_forward_f32_ex(y, x, gamma, beta, rm, rv, save_mean, save_var, N, C, spatial, momentum, eps,
                                     training ? 1 : 0, 0, 0, current_stream());
}
void nc_cuda_batchnorm_backward_f32(float* dx, float* dgamma, float* dbeta, const float* dy, const float* x,
                                    const float* gamma, const float* save_mean, const float* save_var, int N, int C,
                                    int spatial, float eps) {
    nc_cuda_batchnorm_backward_f32_ex(dx, dgamma, dbeta, dy, x, gamma, save_mean, save_var, nullptr, nullptr, 0, N, C, spatial,
                                      eps, 0, current_stream());
}

int nc_cuda_layernorm_forward_f32_ex(float* y, const float* x, const float* gamma, const float* beta, size_t rows,
                                     size_t cols, double eps, void* stream) {
    if (rows == 0 || cols == 0) return NC_CUDA_OK;
    NCC_REQUIRE(y && x && cols <= 0x7fffffff, "layernorm_forward: bad argument");
    ProfScope prof(PROF_LAYERNORM, 8.0 * (double)rows * cols, (cudaStream_t)stream);
    ln_fwd_kernel<<<grid_for((long long)rows * 32, kThreads), kThreads, 0, (cudaStream_t)stream>>>(y, x, gamma, beta, rows, (int)cols, (float)eps, round_outputs() ? 1 : 0);
    NCC_COUNT_LAUNCH();
    return launch_status("layernorm_forward");
}

int nc_cuda_layernorm_backward_f32_ex(float* dx, float* dgamma, float* dbeta, const float* dy, const float* x,
                                      const float* gamma, size_t rows, size_t cols, double eps, void* stream) {
    if (rows == 0 || cols == 0) return NC_CUDA_OK;
    NCC_REQUIRE(dx && dy && x && cols <= 0x7fffffff, "layernorm_backward: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const bool params = dgamma || dbeta;
    // rows pass: read dy, x, write dx; parameter pass: read dy, x again
    ProfScope prof(PROF_LAYERNORM, (params ? 20.0 : 12.0) * (double)rows * cols, st);
    float2* stats = nullptr;
    if (params) {
        stats = (float2*)scratch(6, sizeof(float2) * rows, st);
        if (!stats) return NC_CUDA_ERR_RUNTIME;
    }
    ln_bwd_rows_kernel<<<grid_for((long long)rows * 32, kThreads), kThreads, 0, st>>>(dx, stats, dy, x, gamma, rows, (int)cols, (float)eps, round_outputs() ? 1 : 0);
    NCC_COUNT_LAUNCH();
    if (params) {
        int C = (int)cols;
        double* partial = nullptr;
        int slabs = 0;
        int rc = launch_colreduce(&partial, &slabs, rows, C, al16(dy) && al16(x), LnParamSum{dy, x, stats, C}, st);
        if (rc) return rc;
        ln_param_finalize_kernel<<<fin_grid(C), kFinCols * kFinLanes, 0, st>>>(partial, slabs, C, dgamma, dbeta);
        NCC_COUNT_LAUNCH();
    }
    return launch_status("layernorm_backward");
}

}  // extern "C"
