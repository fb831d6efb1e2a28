// First-layer convolution (3 input channels, 3x3, stride 1) with a channels-last output: reduction length 27, bound by writing
// the output (forward) or reading the output gradient (weight gradient), not by arithmetic.
// TF32 mode with 64 output channels: tensor-core kernels (namespaces tcf and tcw below) whose operand rows are the 27-wide
// patches padded to 32 floats, built in shared memory by the threads themselves.
// Other modes and channel counts: CUDA-core kernels.  Forward: a shared-memory tiled kernel for the common channel counts,
// else 4..16 threads per output pixel, 16 output channels each, the 27 patch values in registers.  Weight gradient: the
// reduction over all pixels is split over CTAs; each CTA stages 64-pixel tiles of dY and of the 27-wide patches in shared
// memory (see dw_tile_kernel); per-CTA partial sums are combined in a fixed order.  No input gradient: the network input
// needs none.
// Semantics: src/nn/conv.c:269-299 (dW), :381-586 (forward) of the reference.
#include "nc_common.cuh"
#include "tc_ptx.cuh"
#include "../../include/nocta_cuda.h"

namespace convfirst {

constexpr int K = 27;   // 3 channels x 3 x 3, ordered (ci, kh, kw) like the reference weight layout
constexpr int KP = 32;  // padded patch width

struct Geo {
    int N, H, W, Cout, pad, Ho, Wo;
    int xs[4];  // input strides (n, c, h, w) in elements (the whole input is < 2^31 elements)
};

__device__ __forceinline__ void load_patch(float (&x)[K], const float* __restrict__ in, const Geo& g, int n, int ho, int wo) {
    // one base offset per pixel; the 27 tap offsets are small loop-invariant integers
    const int h0 = ho - g.pad, w0 = wo - g.pad;
    const float* base = in + (n * g.xs[0] + h0 * g.xs[2] + w0 * g.xs[3]);
    bool hok[3], wok[3];
#pragma unroll
    for (int t = 0; t < 3; t++) { hok[t] = (unsigned)(h0 + t) < (unsigned)g.H; wok[t] = (unsigned)(w0 + t) < (unsigned)g.W; }
#pragma unroll
    for (int ci = 0; ci < 3; ci++)
#pragma unroll
        for (int kh = 0; kh < 3; kh++)
#pragma unroll
            for (int kw = 0; kw < 3; kw++)
                x[(ci * 3 + kh) * 3 + kw] = (hok[kh] && wok[kw]) ? base[ci * g.xs[1] + kh * g.xs[2] + kw * g.xs[3]] : 0.f;
}

// y (N,Ho,Wo,Cout) channels-last; weights (Cout, 27)
__global__ void __launch_bounds__(256) fwd_kernel(float* __restrict__ y, const float* __restrict__ in, const float* __restrict__ w,
                                                  const float* __restrict__ bias, Geo g, int pixels) {
    extern __shared__ float ws[];  // [K][Cout] then bias [Cout]
    float* bs = ws + K * g.Cout;
    for (int i = threadIdx.x; i < K * g.Cout; i += blockDim.x) {
        const int co = i % g.Cout, k = i / g.Cout;
        ws[i] = w[co * K + k];
    }
    for (int i = threadIdx.x; i < g.Cout; i += blockDim.x) bs[i] = bias ? bias[i] : 0.f;
    __syncthreads();
    const int tpp = g.Cout / 16;  // threads per pixel
    const int ppb = blockDim.x / tpp;
    const int lp = threadIdx.x / tpp, cq = threadIdx.x % tpp;
    for (int p = blockIdx.x * ppb + lp; p < pixels; p += gridDim.x * ppb) {
        const int wo = p % g.Wo;
        const int t = p / g.Wo;
        const int ho = t % g.Ho, n = t / g.Ho;
        float x[K];
        load_patch(x, in, g, n, ho, wo);
        float acc[16];
#pragma unroll
        for (int j = 0; j < 16; j++) acc[j] = bs[cq * 16 + j];
#pragma unroll
        for (int k = 0; k < K; k++) {
            const float4* wr = reinterpret_cast<const float4*>(ws + k * g.Cout + cq * 16);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float4 wv = wr[q];
                acc[4 * q + 0] = fmaf(x[k], wv.x, acc[4 * q + 0]);
                acc[4 * q + 1] = fmaf(x[k], wv.y, acc[4 * q + 1]);
                acc[4 * q + 2] = fmaf(x[k], wv.z, acc[4 * q + 2]);
                acc[4 * q + 3] = fmaf(x[k], wv.w, acc[4 * q + 3]);
            }
        }
        float4* dst = reinterpret_cast<float4*>(y + (size_t)p * g.Cout + cq * 16);
#pragma unroll
        for (int q = 0; q < 4; q++) dst[q] = make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
    }
}

// Tiled forward for Cout in {16, 32, 64, 128}.  A CTA owns a strip of TR output rows x 64 output columns
// of one image: the 3 x (TR+2) x 66 input halo is staged in shared memory once (coalesced reads, zero
// fill = padding), every thread computes 4 consecutive pixels x 8 output channels (channels cg*4..+3 and
// Cout/2 + cg*4..+3, so that the lanes of a warp store whole 128-byte lines), reading its 6 input
// values per (ci, kh) with one float4 + one float2 and the weights with two float4: 8 shared loads per
// 96 FMAs.
constexpr int TW = 64, TWP = 68;
template <int COUT>
struct TileGeo {
    static constexpr int CG = COUT / 8;     // channel groups
    static constexpr int PG = 256 / CG;     // 4-pixel groups per CTA
    static constexpr int TR = PG / (TW / 4);  // output rows per CTA
};
template <int COUT, bool STAT>
__global__ void __launch_bounds__(256, 4) fwd_tile_kernel(float* __restrict__ y, const float* __restrict__ in,
                                                       const float* __restrict__ w, const float* __restrict__ bias, Geo g,
                                                       int tiles_h, int tiles_w, int ntiles, double* __restrict__ stat) {
    using T = TileGeo<COUT>;
    constexpr int CG = T::CG, TR = T::TR, ROWS = TR + 2;
    __shared__ __align__(16) float ws[K * COUT];
    __shared__ __align__(16) float bs[COUT];
    __shared__ __align__(16) float tile[3][ROWS][TWP];
    for (int i = threadIdx.x; i < K * COUT; i += 256) {
        const int co = i % COUT, k = i / COUT;
        ws[i] = w[co * K + k];
    }
    for (int i = threadIdx.x; i < COUT; i += 256) bs[i] = bias ? bias[i] : 0.f;
    // per-channel sum and sum of squares of this CTA's outputs, one private row per warp (no atomics: the result
    // does not depend on the order in which warps run)
    __shared__ float ssum[STAT ? 8 : 1][STAT ? 2 * COUT : 1];
    if (STAT)
        for (int i = threadIdx.x; i < 8 * 2 * COUT; i += 256) (&ssum[0][0])[i] = 0.f;
    const int cg = threadIdx.x % CG, pg = threadIdx.x / CG;
    const int prow = pg / (TW / 4), pcol = (pg % (TW / 4)) * 4;
    const float* wlo = ws + cg * 4;
    const float* whi = ws + COUT / 2 + cg * 4;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const int tw = t % tiles_w;
        const int t2 = t / tiles_w;
        const int th = t2 % tiles_h, n = t2 / tiles_h;
        const int ho0 = th * TR, wo0 = tw * TW;
        __syncthreads();  // the previous tile is no longer read (also orders the weight staging)
        for (int i = threadIdx.x; i < 3 * ROWS * 66; i += 256) {
            const int cc = i % 66;
            const int q = i / 66;
            const int r = q % ROWS, ci = q / ROWS;
            const int h = ho0 - g.pad + r, wc = wo0 - g.pad + cc;
            float v = 0.f;
            if ((unsigned)h < (unsigned)g.H && (unsigned)wc < (unsigned)g.W)
                v = in[n * g.xs[0] + ci * g.xs[1] + h * g.xs[2] + wc * g.xs[3]];
            tile[ci][r][cc] = v;
        }
        __syncthreads();
        float acc[4][8];
        {
            const float4 b0 = *reinterpret_cast<const float4*>(bs + cg * 4);
            const float4 b1 = *reinterpret_cast<const float4*>(bs + COUT / 2 + cg * 4);
#pragma unroll
            for (int p = 0; p < 4; p++) {
                acc[p][0] = b0.x; acc[p][1] = b0.y; acc[p][2] = b0.z; acc[p][3] = b0.w;
                acc[p][4] = b1.x; acc[p][5] = b1.y; acc[p][6] = b1.z; acc[p][7] = b1.w;
            }
        }
#pragma unroll
        for (int ci = 0; ci < 3; ci++)
#pragma unroll
            for (int kh = 0; kh < 3; kh++) {
                const float* row = &tile[ci][prow + kh][pcol];
                const float4 xa = *reinterpret_cast<const float4*>(row);
                const float2 xb = *reinterpret_cast<const float2*>(row + 4);
                const float xv[6] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y};
#pragma unroll
                for (int kw = 0; kw < 3; kw++) {
                    const int k = (ci * 3 + kh) * 3 + kw;
                    const float4 w0 = *reinterpret_cast<const float4*>(wlo + k * COUT);
                    const float4 w1 = *reinterpret_cast<const float4*>(whi + k * COUT);
#pragma unroll
                    for (int p = 0; p < 4; p++) {
                        const float xx = xv[p + kw];
                        acc[p][0] = fmaf(xx, w0.x, acc[p][0]); acc[p][1] = fmaf(xx, w0.y, acc[p][1]);
                        acc[p][2] = fmaf(xx, w0.z, acc[p][2]); acc[p][3] = fmaf(xx, w0.w, acc[p][3]);
                        acc[p][4] = fmaf(xx, w1.x, acc[p][4]); acc[p][5] = fmaf(xx, w1.y, acc[p][5]);
                        acc[p][6] = fmaf(xx, w1.z, acc[p][6]); acc[p][7] = fmaf(xx, w1.w, acc[p][7]);
                    }
                }
            }
        const int ho = ho0 + prow;
        if (ho < g.Ho) {
            float* dst = y + ((size_t)(n * g.Ho + ho) * g.Wo + wo0 + pcol) * COUT;
#pragma unroll
            for (int p = 0; p < 4; p++) {
                if (wo0 + pcol + p < g.Wo) {
                    *reinterpret_cast<float4*>(dst + (size_t)p * COUT + cg * 4) = make_float4(acc[p][0], acc[p][1], acc[p][2], acc[p][3]);
                    *reinterpret_cast<float4*>(dst + (size_t)p * COUT + COUT / 2 + cg * 4) = make_float4(acc[p][4], acc[p][5], acc[p][6], acc[p][7]);
                }
            }
        }
        if (STAT) {
            // The thread's 4 pixels, then the lanes of the warp that own the same channels (same lane % CG), then one
            // add per channel into the warp's row of shared memory.  Pixels outside the image count for nothing.
            static_assert(CG <= 16 && 32 % CG == 0, "lanes with equal lane % CG own the same channels");
#pragma unroll
            for (int c = 0; c < 8; c++) {
                float sv = 0.f, qv = 0.f;
#pragma unroll
                for (int p = 0; p < 4; p++) {
                    const bool in_img = ho < g.Ho && wo0 + pcol + p < g.Wo;
                    const float o = in_img ? acc[p][c] : 0.f;
                    sv += o;
                    qv = fmaf(o, o, qv);
                }
#pragma unroll
                for (int d = 16; d >= CG; d >>= 1) {
                    sv += __shfl_xor_sync(0xffffffffu, sv, d);
                    qv += __shfl_xor_sync(0xffffffffu, qv, d);
                }
                if ((threadIdx.x & 31) < CG) {
                    const int ch = (c < 4 ? 0 : COUT / 2) + cg * 4 + (c & 3);
                    float* mine = ssum[threadIdx.x >> 5];
                    mine[ch] += sv;
                    mine[COUT + ch] += qv;
                }
            }
        }
    }
    if (STAT) {
        __syncthreads();
        for (int i = threadIdx.x; i < COUT; i += 256) {
            double* sd = stat + ((size_t)blockIdx.x * COUT + i) * 2;
            double a = 0.0, b = 0.0;
#pragma unroll
            for (int wp = 0; wp < 8; wp++) {
                a += (double)ssum[wp][i];
                b += (double)ssum[wp][COUT + i];
            }
            sd[0] = a;
            sd[1] = b;
        }
    }
}

template <int COUT>
static int launch_fwd_tile(float* y, const float* x, const float* w, const float* bias, const Geo& g, cudaStream_t st, double** stat_out) {
    const int tiles_h = (g.Ho + TileGeo<COUT>::TR - 1) / TileGeo<COUT>::TR, tiles_w = (g.Wo + TW - 1) / TW;
    const long long ntiles = (long long)g.N * tiles_h * tiles_w;
    const long long cap = (long long)ncc::sm_count() * 4;  // 4 CTAs of 64 registers x 256 threads fit an SM
    const int grid = (int)(ntiles < cap ? ntiles : cap);
    // a BatchNorm that follows can take the per-channel sums from here instead of reading y again (one slab per CTA)
    double* stat = ncc::conv_stats_wanted() ? ncc::conv_stats_buffer((size_t)grid, COUT, st) : nullptr;
    if (stat) {
        fwd_tile_kernel<COUT, true><<<grid, 256, 0, st>>>(y, x, w, bias, g, tiles_h, tiles_w, (int)ntiles, stat);
    } else {
        fwd_tile_kernel<COUT, false><<<grid, 256, 0, st>>>(y, x, w, bias, g, tiles_h, tiles_w, (int)ntiles, nullptr);
    }
    *stat_out = stat;
    return grid;
}

// Tiled weight gradient for Cout in {32, 64}.  A CTA walks strips of 4 output rows x 64 columns; the
// input halo of a strip is staged in shared memory, dY is read straight from global memory (every
// element is needed by exactly one thread; a warp reads whole 128/256-byte pixel rows).  A warp takes
// groups of 4 consecutive pixels; lane l owns output channels l*CPT..+CPT-1 and ALL 27 taps, so the six
// input values of a (ci, kh) row (one float4 + one float2, broadcast) feed 12*CPT FMAs.  The 8 warps'
// sums are combined in warp order at the end, then the per-CTA partials by dw_reduce_kernel.
// partial[block][co][KP]
template <int COUT>
__global__ void __launch_bounds__(256) dw_tile_kernel(float* __restrict__ partial, const float* __restrict__ dy,
                                                      const float* __restrict__ in, Geo g, int tiles_h, int tiles_w, int ntiles) {
    constexpr int CPT = COUT / 32, TR = 4, ROWS = TR + 2, RS = (K * CPT) | 1;
    __shared__ __align__(16) float tile[3][ROWS][TWP];
    __shared__ float red[32][RS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float acc[CPT][K];
#pragma unroll
    for (int j = 0; j < CPT; j++)
#pragma unroll
        for (int k = 0; k < K; k++) acc[j][k] = 0.f;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const int tw = t % tiles_w;
        const int t2 = t / tiles_w;
        const int th = t2 % tiles_h, n = t2 / tiles_h;
        const int ho0 = th * TR, wo0 = tw * TW;
        __syncthreads();
        for (int i = threadIdx.x; i < 3 * ROWS * 66; i += 256) {
            const int cc = i % 66;
            const int q = i / 66;
            const int r = q % ROWS, ci = q / ROWS;
            const int h = ho0 - g.pad + r, wc = wo0 - g.pad + cc;
            float v = 0.f;
            if ((unsigned)h < (unsigned)g.H && (unsigned)wc < (unsigned)g.W)
                v = in[n * g.xs[0] + ci * g.xs[1] + h * g.xs[2] + wc * g.xs[3]];
            tile[ci][r][cc] = v;
        }
        __syncthreads();
#pragma unroll 1
        for (int grp = warp; grp < TR * (TW / 4); grp += 8) {
            const int prow = grp / (TW / 4), pcol = (grp % (TW / 4)) * 4;
            const int ho = ho0 + prow;
            if (ho >= g.Ho || wo0 + pcol >= g.Wo) continue;  // warp-uniform
            const float* src = dy + ((size_t)(n * g.Ho + ho) * g.Wo + wo0 + pcol) * COUT + lane * CPT;
            float d[4][CPT];
#pragma unroll
            for (int p = 0; p < 4; p++) {
                const bool ok = wo0 + pcol + p < g.Wo;
                if (CPT == 2) {
                    float2 v = ok ? *reinterpret_cast<const float2*>(src + (size_t)p * COUT) : make_float2(0.f, 0.f);
                    d[p][0] = v.x; d[p][CPT - 1] = v.y;
                } else {
                    d[p][0] = ok ? src[(size_t)p * COUT] : 0.f;
                }
            }
#pragma unroll
            for (int ci = 0; ci < 3; ci++)
#pragma unroll
                for (int kh = 0; kh < 3; kh++) {
                    const float* row = &tile[ci][prow + kh][pcol];
                    const float4 xa = *reinterpret_cast<const float4*>(row);
                    const float2 xb = *reinterpret_cast<const float2*>(row + 4);
                    const float xv[6] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y};
#pragma unroll
                    for (int kw = 0; kw < 3; kw++)
#pragma unroll
                        for (int p = 0; p < 4; p++)
#pragma unroll
                            for (int j = 0; j < CPT; j++)
                                acc[j][(ci * 3 + kh) * 3 + kw] = fmaf(d[p][j], xv[p + kw], acc[j][(ci * 3 + kh) * 3 + kw]);
                }
        }
    }
    // combine the 8 warps in warp order
    for (int wq = 0; wq < 8; wq++) {
        __syncthreads();
        if (warp == wq) {
#pragma unroll
            for (int j = 0; j < CPT; j++)
#pragma unroll
                for (int k = 0; k < K; k++) {
                    if (wq == 0) red[lane][j * K + k] = acc[j][k];
                    else red[lane][j * K + k] += acc[j][k];
                }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < COUT * K; i += 256) {
        const int co = i / K, k = i % K;
        partial[((size_t)blockIdx.x * COUT + co) * KP + k] = red[co / CPT][(co % CPT) * K + k];
    }
}

__global__ void __launch_bounds__(256) dw_reduce_kernel(float* __restrict__ dW, const float* __restrict__ partial, int blocks, int Cout) {
    // one warp per weight: lanes stride over the per-CTA partials, fixed-order shuffle tree
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (i >= Cout * K) return;
    const int co = i / K, k = i % K;
    double acc = 0.0;
    for (int b = lane; b < blocks; b += 32) acc += (double)partial[((long long)b * Cout + co) * KP + k];
    acc = ncc::warp_sum(acc);
    if (lane == 0) dW[i] = (float)acc;
}

// ------------------------------------------------------------------------------------------
// Tensor-core forward (TF32 mode, 64 output channels).  The 27-wide patch of an output pixel, padded to 32 floats, is
// exactly one 128-byte row of a K-major tcgen05 operand.  Weights (64 rows + 64 zero rows, x 32) are the A operand, a tile
// of 128 pixels' patches the B operand: four kind::tf32 MMAs (K = 8 each) leave channel co of pixel j in lane co, column j
// of tensor memory.  No TMA: eight builder warps gather the patches (the input is small and stays in L2) and write the rows
// with the 128-byte swizzle the MMA expects into a ring of four tiles; warp 16 issues the MMAs into a ring of four
// accumulators; eight epilogue warps read them (lane = channel), add the bias and store: for one pixel a warp writes 32
// consecutive floats, i.e. whole 128-byte lines (with the pixels on the lanes every store instruction would touch 32
// different lines, and the rate of such requests, not the bytes, bounds the kernel).  The rings let each role run ahead of
// the next by up to four tiles, which hides the load, tensor-memory and store latencies.
// ------------------------------------------------------------------------------------------
namespace tcf {
using namespace tc;
constexpr int G = 4;                 // ring depth: patch tiles and accumulators in flight per CTA
constexpr int COUT = 64;
constexpr int P_BYTES = 128 * 128;   // one patch tile: 128 pixels x 32 floats
constexpr int W_BYTES = 128 * 128;   // weights padded to 128 rows
constexpr int SMEM = G * P_BYTES + W_BYTES + 1024;

__device__ __forceinline__ uint32_t idesc_tf32_k(uint32_t M, uint32_t N) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);   // D f32, A = B = tf32, both K-major
}
// byte offset of 16-byte chunk c of row r in a K-major tile with 128-byte rows and the 128-byte swizzle
__device__ __forceinline__ uint32_t sw128(int r, int c) { return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)); }

__global__ void __launch_bounds__(544, 1) fwd_kernel(float* __restrict__ y, const float* __restrict__ in, const float* __restrict__ w,
                                                     const float* __restrict__ bias, Geo g, int pixels, int ntiles,
                                                     double* __restrict__ stat, unsigned int* err) {
    extern __shared__ uint8_t dyn[];
    __shared__ __align__(8) uint64_t bar_p_full[G], bar_p_empty[G], bar_acc_full[G], bar_acc_empty[G];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ double st_comb[8][32][2];
    const uint32_t base = (smem_u32(dyn) + 1023u) & ~1023u;
    uint8_t* gen = dyn + (base - smem_u32(dyn));
    const uint32_t w_base = base + G * P_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abortp = &abort_flag;

    if (threadIdx.x == 0) {
        for (int i = 0; i < G; i++) {
            mbar_init(smem_u32(&bar_p_full[i]), 128);
            mbar_init(smem_u32(&bar_p_empty[i]), 1);
            mbar_init(smem_u32(&bar_acc_full[i]), 1);
            mbar_init(smem_u32(&bar_acc_empty[i]), 256);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // weights = the A operand: row co, K index (ci, kh, kw) as the reference stores them, padded with zeros to 32, rounded to
    // TF32; rows 64..127 are zero (the MMA wants M = 128, those accumulator lanes are never read)
    for (int i = threadIdx.x; i < 128 * 8; i += blockDim.x) {
        const int co = i >> 3, c = i & 7;
        float4 q;
        float* qf = reinterpret_cast<float*>(&q);
#pragma unroll
        for (int e = 0; e < 4; e++) { const int k = c * 4 + e; qf[e] = (co < COUT && k < K) ? ncc::round_tf32(w[co * K + k]) : 0.f; }
        *reinterpret_cast<float4*>(gen + G * P_BYTES + sw128(co, c)) = q;
    }
    if (warp == 16) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the weight tile is read by the tensor core
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    // tiles of this CTA: local index i is tile blockIdx.x + i * gridDim.x, patch buffer and accumulator i % G
    const int nloc = ((int)blockIdx.x < ntiles) ? (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

    if (warp == 16) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = idesc_tf32_k(128u, 128u);
            const uint64_t dW = smem_desc(w_base, 16u, 1024u, 2u);
            for (int i = 0; i < nloc; i++) {
                const int b = i & (G - 1);
                const uint32_t ph = (uint32_t)((i / G) & 1);
                if (!mbar_wait(smem_u32(&bar_p_full[b]), ph, err, 0xC00u + b, abortp)) break;
                if (!mbar_wait(smem_u32(&bar_acc_empty[b]), ph ^ 1u, err, 0xC10u + b, abortp)) break;
                tc_fence_after();
                const uint64_t dP = smem_desc(base + (uint32_t)(b * P_BYTES), 16u, 1024u, 2u);
#pragma unroll
                for (int ks = 0; ks < 4; ks++) umma_tf32(tmem_base + (uint32_t)(b * 128), dW + (uint64_t)(ks * 2), dP + (uint64_t)(ks * 2), idesc, ks != 0);
                umma_commit(smem_u32(&bar_p_empty[b]));
                umma_commit(smem_u32(&bar_acc_full[b]));
            }
        }
    } else if ((warp & 3) >= 2) {
        // ---------------- builders (warps 2, 3, 6, 7, 10, 11, 14, 15): two sets of four warps, one set per tile; a thread
        // gathers one pixel's patch and writes its 128-byte row of the B operand ----------------
        const int bw = (warp >> 2) * 2 + (warp & 1);   // 0..7
        const int set = bw >> 2, r = (bw & 3) * 32 + lane;
        for (int i = set; i < nloc; i += 2) {
            const int b = i & (G - 1);
            const int p = ((int)blockIdx.x + i * (int)gridDim.x) * 128 + r;
            float x[K];
            if (p < pixels) {
                const int wo = p % g.Wo;
                const int t = p / g.Wo;
                load_patch(x, in, g, t / g.Ho, t % g.Ho, wo);
            } else {
#pragma unroll
                for (int k = 0; k < K; k++) x[k] = 0.f;
            }
            if (!mbar_wait(smem_u32(&bar_p_empty[b]), (uint32_t)(((i / G) & 1) ^ 1), err, 0xC20u + b, abortp)) break;
            uint8_t* prow = gen + b * P_BYTES;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                float4 qv;
                float* qf = reinterpret_cast<float*>(&qv);
#pragma unroll
                for (int e = 0; e < 4; e++) qf[e] = (c * 4 + e) < K ? ncc::round_tf32(x[(c * 4 + e) < K ? (c * 4 + e) : 0]) : 0.f;
                *reinterpret_cast<float4*>(prow + sw128(r, c)) = qv;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(smem_u32(&bar_p_full[b]));
        }
    } else {
        // ---------------- epilogue (warps 0, 1, 4, 5, 8, 9, 12, 13).  The accumulator holds channel co in lane co and pixel j
        // of the tile in column j; warp % 4 (0 or 1) is the quarter of the lanes a warp may read = its 32 channels, and the
        // four warps of a quarter take one 32-pixel chunk of every tile each.  For one pixel the 32 lanes store 32
        // consecutive floats: whole 128-byte lines.  A thread owns one channel, so the sums for the BatchNorm that
        // follows are plain running sums. ----------------
        const int q = warp & 1, chunk = warp >> 2, co = q * 32 + lane;
        const float bv = bias ? bias[co] : 0.f;
        double ssum = 0.0, ssq = 0.0;
        for (int i = 0; i < nloc; i++) {
            const int b = i & (G - 1);
            const int p0 = ((int)blockIdx.x + i * (int)gridDim.x) * 128 + chunk * 32;
            const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_acc_full[b]), (uint32_t)((i / G) & 1), err, 0xC30u + b, abortp));
            if (!ok) break;
            tc_fence_after();
            uint32_t v[32];
            tmem_ld32(tmem_base + (uint32_t)(b * 128 + chunk * 32) + ((uint32_t)(q * 32) << 16), v);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(smem_u32(&bar_acc_empty[b]));
            float* dst = y + (size_t)p0 * COUT + co;
            float fs = 0.f, fq = 0.f;
            if (p0 + 32 <= pixels) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const float o = __uint_as_float(v[j]) + bv;
                    dst[j * COUT] = o;
                    fs += o;
                    fq = fmaf(o, o, fq);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++)
                    if (p0 + j < pixels) {
                        const float o = __uint_as_float(v[j]) + bv;
                        dst[j * COUT] = o;
                        fs += o;
                        fq = fmaf(o, o, fq);
                    }
            }
            ssum += (double)fs;
            ssq += (double)fq;
        }
        const int ew = (warp >> 2) * 2 + (warp & 1);   // 0..7
        st_comb[ew][lane][0] = ssum;
        st_comb[ew][lane][1] = ssq;
    }
    tc_fence_before();
    __syncthreads();
    if (stat && threadIdx.x < COUT) {   // the four warps of a channel's quarter in a fixed order
        const int q = threadIdx.x >> 5, l = threadIdx.x & 31;
        double a = 0.0, b = 0.0;
        for (int c = 0; c < 4; c++) { a += st_comb[c * 2 + q][l][0]; b += st_comb[c * 2 + q][l][1]; }
        stat[((size_t)blockIdx.x * COUT + threadIdx.x) * 2] = a;
        stat[((size_t)blockIdx.x * COUT + threadIdx.x) * 2 + 1] = b;
    }
    if (warp == 16) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}
}  // namespace tcf

static int forward_tc(float* y, const float* x, const float* w, const float* bias, const Geo& g, cudaStream_t st) {
    static bool attr_set = false;
    if (!attr_set) {
        NCC_TRY(cudaFuncSetAttribute(tcf::fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tcf::SMEM));
        attr_set = true;
    }
    const int pixels = g.N * g.Ho * g.Wo;
    const int ntiles = (pixels + 127) / 128;
    const int sms = ncc::sm_count();
    const int grid = ntiles < sms ? ntiles : sms;
    double* stat = ncc::conv_stats_wanted() ? ncc::conv_stats_buffer((size_t)grid, tcf::COUT, st) : nullptr;
    tcf::fwd_kernel<<<grid, 544, tcf::SMEM, st>>>(y, x, w, bias, g, pixels, ntiles, stat, ncc::device_error_word());
    NCC_COUNT_LAUNCH();
    const int rc = ncc::launch_status("conv_first forward (tensor core)");
    if (rc == NC_CUDA_OK && stat) ncc::conv_stats_publish(y, tcf::COUT, (long long)pixels, grid, stat);
    return rc;
}

// ------------------------------------------------------------------------------------------
// Tensor-core weight gradient (TF32 mode, 64 output channels): dW[co][k] = sum over pixels of dY[pixel][co] * patch[pixel][k].
// The reduction runs over pixels, so both operands are MN-major: a pixel is a reduction row of 128 bytes per 32-value chunk.
// A stage holds TWO pixel tiles of 128: the A operand is dY of tile 0 (two 32-channel chunks) followed by dY of tile 1 (two
// more) = 128 "rows", the B operand the patch tile of tile 0 followed by that of tile 1 = 64 "columns".  One MMA
// (128 x 64 x 8 pixels) then accumulates tile 0's product in lanes 0-63 x columns 0-31 and tile 1's in lanes 64-127 x
// columns 32-63; the two off-diagonal blocks pair different pixels and are never read.  That gives the full M = 128 MMA
// shape from a 64-channel gradient without zero padding.  dY arrives by TMA (128-byte swizzle on 32-byte units, the
// layout MN-major 32-bit operands need), the patch tiles are written by the builder warps with the same swizzle.
// Every CTA leaves two partial 64 x 32 blocks; dw_reduce_kernel adds all of them in a fixed order.
// ------------------------------------------------------------------------------------------
namespace tcw {
using namespace tc;
constexpr int COUT = 64;
constexpr int CHUNK = 128 * 128;               // 128 pixels x 32 floats
constexpr int STAGE = 6 * CHUNK;               // dY: 4 chunks, patches: 2 chunks
constexpr int STAGES = 2;
constexpr int SMEM = STAGES * STAGE + 1024;

__device__ __forceinline__ uint32_t idesc_tf32_mn(uint32_t M, uint32_t N) {
    return (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (1u << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);   // both operands MN-major
}
// byte offset of 16-byte piece c (0..7) of reduction row r in an MN-major chunk: 128-byte swizzle on 32-byte units
__device__ __forceinline__ uint32_t sw32(int r, int c) { return (uint32_t)(r * 128 + ((((c >> 1) ^ (r & 3))) << 5) + ((c & 1) << 4)); }

__global__ void __launch_bounds__(320, 1) dw_kernel(const __grid_constant__ CUtensorMap tmDy, float* __restrict__ partial,
                                                    const float* __restrict__ in, Geo g, int pixels, int npairs, unsigned int* err) {
    extern __shared__ uint8_t dyn[];
    __shared__ __align__(8) uint64_t bar_full[STAGES], bar_empty[STAGES], bar_done;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const uint32_t base = (smem_u32(dyn) + 1023u) & ~1023u;
    uint8_t* gen = dyn + (base - smem_u32(dyn));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abortp = &abort_flag;
    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; i++) { mbar_init(smem_u32(&bar_full[i]), 257); mbar_init(smem_u32(&bar_empty[i]), 1); }
        mbar_init(smem_u32(&bar_done), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(64u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    // tile pairs of this CTA: local index i is pair blockIdx.x + i * gridDim.x, stage i % 2
    const int nloc = ((int)blockIdx.x < npairs) ? (npairs - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

    if (warp == 8) {
        // ---------------- dY by TMA: four boxes of 32 channels x 128 pixels (rows past the last pixel arrive as zeros) ----------------
        if (lane == 0) {
            for (int i = 0; i < nloc; i++) {
                const int s = i & 1;
                if (!mbar_wait(smem_u32(&bar_empty[s]), (uint32_t)(((i >> 1) & 1) ^ 1), err, 0xE00u + s, abortp)) break;
                const int pix0 = ((int)blockIdx.x + i * (int)gridDim.x) * 256;
                const uint32_t full = smem_u32(&bar_full[s]);
                mbar_expect_tx(full, 4u * CHUNK);
                const uint32_t a = base + (uint32_t)(s * STAGE);
                tma_2d(a, &tmDy, 0, pix0, full);
                tma_2d(a + CHUNK, &tmDy, 32, pix0, full);
                tma_2d(a + 2 * CHUNK, &tmDy, 0, pix0 + 128, full);
                tma_2d(a + 3 * CHUNK, &tmDy, 32, pix0 + 128, full);
            }
        }
    } else if (warp == 9) {
        // ---------------- MMA issuer: 16 k-steps of 8 pixels per stage, one accumulator for the whole kernel ----------------
        if (lane == 0) {
            const uint32_t idesc = idesc_tf32_mn(128u, 64u);
            bool ok = true;
            for (int i = 0; i < nloc && ok; i++) {
                const int s = i & 1;
                if (!mbar_wait(smem_u32(&bar_full[s]), (uint32_t)((i >> 1) & 1), err, 0xE10u + s, abortp)) { ok = false; break; }
                tc_fence_after();
                const uint64_t dA = smem_desc(base + (uint32_t)(s * STAGE), (uint32_t)CHUNK, 512u, 1u);
                const uint64_t dB = smem_desc(base + (uint32_t)(s * STAGE + 4 * CHUNK), (uint32_t)CHUNK, 512u, 1u);
#pragma unroll
                for (int k = 0; k < 16; k++) umma_tf32(tmem_base, dA + (uint64_t)(k * 64), dB + (uint64_t)(k * 64), idesc, (i | k) != 0);
                umma_commit(smem_u32(&bar_empty[s]));
            }
            if (ok) umma_commit(smem_u32(&bar_done));
        }
    } else {
        // ---------------- builders: warps 0-3 the first tile of a pair, warps 4-7 the second; a thread gathers one pixel's
        // patch and writes its 128-byte reduction row ----------------
        const int half = warp >> 2, r = (warp & 3) * 32 + lane;
        for (int i = 0; i < nloc; i++) {
            const int s = i & 1;
            const int p = ((int)blockIdx.x + i * (int)gridDim.x) * 256 + half * 128 + r;
            float x[K];
            if (p < pixels) {
                const int wo = p % g.Wo;
                const int t = p / g.Wo;
                load_patch(x, in, g, t / g.Ho, t % g.Ho, wo);
            } else {
#pragma unroll
                for (int k = 0; k < K; k++) x[k] = 0.f;
            }
            if (!mbar_wait(smem_u32(&bar_empty[s]), (uint32_t)(((i >> 1) & 1) ^ 1), err, 0xE20u + s, abortp)) break;
            uint8_t* prow = gen + s * STAGE + (4 + half) * CHUNK;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                float4 qv;
                float* qf = reinterpret_cast<float*>(&qv);
#pragma unroll
                for (int e = 0; e < 4; e++) qf[e] = (c * 4 + e) < K ? ncc::round_tf32(x[(c * 4 + e) < K ? (c * 4 + e) : 0]) : 0.f;
                *reinterpret_cast<float4*>(prow + sw32(r, c)) = qv;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(smem_u32(&bar_full[s]));
        }
        if (warp < 4) {
            // ---------------- the end: lanes 0-63 hold tile-0 sums in columns 0-31, lanes 64-127 tile-1 sums in columns 32-63 ----------------
            const bool ok = nloc == 0 || __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_done), 0u, err, 0xE30u, abortp));
            const int L = warp * 32 + lane, h = L >> 6, co = L & 63;
            float* dst = partial + ((size_t)(2 * blockIdx.x + h) * COUT + co) * KP;
            if (ok && nloc > 0) {
                tc_fence_after();
                uint32_t v[32];
                tmem_ld32(tmem_base + (uint32_t)(h * 32) + ((uint32_t)(warp * 32) << 16), v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
            } else {
#pragma unroll
                for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        // a wait expired somewhere: give copies still in flight time to land before the shared memory is released
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(64u) : "memory");
    }
}
}  // namespace tcw

static int weight_grad_tc(float* dW, const float* dy, const float* x, const Geo& g, cudaStream_t st) {
    static bool attr_set = false;
    if (!attr_set) {
        NCC_TRY(cudaFuncSetAttribute(tcw::dw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tcw::SMEM));
        attr_set = true;
    }
    const int pixels = g.N * g.Ho * g.Wo;
    const int npairs = (pixels + 255) / 256;
    const int sms = ncc::sm_count();
    const int grid = npairs < sms ? npairs : sms;
    CUtensorMap tm;
    unsigned long long dims[2] = {(unsigned long long)tcw::COUT, (unsigned long long)pixels};
    unsigned long long str[1] = {(unsigned long long)tcw::COUT};
    unsigned box[2] = {32, 128};
    if (!tc::make_map(&tm, dy, 2, dims, str, box, true)) return NC_CUDA_ERR_UNSUPPORTED;
    float* partial = (float*)ncc::scratch(2, sizeof(float) * (size_t)(2 * grid) * tcw::COUT * KP, st);
    if (!partial) return NC_CUDA_ERR_RUNTIME;
    tcw::dw_kernel<<<grid, 320, tcw::SMEM, st>>>(tm, partial, x, g, pixels, npairs, ncc::device_error_word());
    NCC_COUNT_LAUNCH();
    dw_reduce_kernel<<<ncc::ceil_div(tcw::COUT * K * 32, 256), 256, 0, st>>>(dW, partial, 2 * grid, tcw::COUT);
    NCC_COUNT_LAUNCH();
    return ncc::launch_status("conv_first weight_grad (tensor core)");
}

// 32-bit index arithmetic is used throughout: everything addressed must stay below 2^31 elements
static bool fits_int(int N, int H, int W, const long long xs[4], int Ho, int Wo) {
    long long span = 1 + (long long)(N - 1) * xs[0] + 2 * xs[1] + (long long)(H - 1) * xs[2] + (long long)(W - 1) * xs[3];
    for (int i = 0; i < 4; i++) if (xs[i] < 0 || xs[i] > 0x3fffffffLL) return false;
    return span < 0x7fffffffLL && (long long)N * Ho * Wo < 0x7fffffffLL / 256;
}

bool eligible(int Cin, int kH, int kW, int stride, int Cout) {
    return Cin == 3 && kH == 3 && kW == 3 && stride == 1 && Cout % 16 == 0 && Cout >= 16 && Cout <= 256;
}

int forward(float* y, const float* x, const long long xs[4], const float* w, const float* bias, int N, int H, int W, int Cout, int pad,
            cudaStream_t st) {
    Geo g{N, H, W, Cout, pad, H + 2 * pad - 2, W + 2 * pad - 2, {(int)xs[0], (int)xs[1], (int)xs[2], (int)xs[3]}};
    if (g.Ho <= 0 || g.Wo <= 0) return NC_CUDA_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(y) & 15u) != 0) return NC_CUDA_ERR_UNSUPPORTED;
    if (!fits_int(N, H, W, xs, g.Ho, g.Wo)) return NC_CUDA_ERR_UNSUPPORTED;
    const int pixels = N * g.Ho * g.Wo;
    if (Cout == tcf::COUT && ncc::math_mode() == NC_CUDA_MATH_TF32) return forward_tc(y, x, w, bias, g, st);
    if (Cout == 16 || Cout == 32 || Cout == 64 || Cout == 128) {
        double* stat = nullptr;
        int slabs;
        if (Cout == 16) slabs = launch_fwd_tile<16>(y, x, w, bias, g, st, &stat);
        else if (Cout == 32) slabs = launch_fwd_tile<32>(y, x, w, bias, g, st, &stat);
        else if (Cout == 64) slabs = launch_fwd_tile<64>(y, x, w, bias, g, st, &stat);
        else slabs = launch_fwd_tile<128>(y, x, w, bias, g, st, &stat);
        NCC_COUNT_LAUNCH();
        const int rc = ncc::launch_status("conv_first forward");
        if (rc == NC_CUDA_OK && stat) ncc::conv_stats_publish(y, Cout, (long long)pixels, slabs, stat);
        return rc;
    }
    const int ppb = 256 / (Cout / 16);
    long long need = ((long long)pixels + ppb - 1) / ppb;
    const long long cap = (long long)ncc::sm_count() * 8;
    const int grid = (int)(need < cap ? need : cap);
    const size_t smem = sizeof(float) * (size_t)(K + 1) * Cout;
    fwd_kernel<<<grid, 256, smem, st>>>(y, x, w, bias, g, pixels);
    NCC_COUNT_LAUNCH();
    return ncc::launch_status("conv_first forward");
}

int weight_grad(float* dW, const float* dy, const float* x, const long long xs[4], int N, int H, int W, int Cout, int pad, cudaStream_t st) {
    if (Cout != 64 && Cout != 32) return NC_CUDA_ERR_UNSUPPORTED;
    Geo g{N, H, W, Cout, pad, H + 2 * pad - 2, W + 2 * pad - 2, {(int)xs[0], (int)xs[1], (int)xs[2], (int)xs[3]}};
    if (g.Ho <= 0 || g.Wo <= 0) return NC_CUDA_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(dy) & 15u) != 0) return NC_CUDA_ERR_UNSUPPORTED;
    if (!fits_int(N, H, W, xs, g.Ho, g.Wo)) return NC_CUDA_ERR_UNSUPPORTED;
    if (Cout == tcw::COUT && ncc::math_mode() == NC_CUDA_MATH_TF32) {
        const int rc = weight_grad_tc(dW, dy, x, g, st);
        if (rc != NC_CUDA_ERR_UNSUPPORTED) return rc;
    }
    constexpr int TRW = 4;  // rows per strip of dw_tile_kernel
    const int tiles_h = (g.Ho + TRW - 1) / TRW, tiles_w = (g.Wo + TW - 1) / TW;
    const long long ntiles = (long long)N * tiles_h * tiles_w;
    long long blocks = (long long)ncc::sm_count() * 3;
    if (blocks > ntiles) blocks = ntiles;
    float* partial = (float*)ncc::scratch(2, sizeof(float) * (size_t)blocks * Cout * KP, st);
    if (!partial) return NC_CUDA_ERR_RUNTIME;
    if (Cout == 64) dw_tile_kernel<64><<<(int)blocks, 256, 0, st>>>(partial, dy, x, g, tiles_h, tiles_w, (int)ntiles);
    else dw_tile_kernel<32><<<(int)blocks, 256, 0, st>>>(partial, dy, x, g, tiles_h, tiles_w, (int)ntiles);
    NCC_COUNT_LAUNCH();
    dw_reduce_kernel<<<ncc::ceil_div(Cout * K * 32, 256), 256, 0, st>>>(dW, partial, (int)blocks, Cout);
    NCC_COUNT_LAUNCH();
    return ncc::launch_status("conv_first weight_grad");
}

}  // namespace convfirst
