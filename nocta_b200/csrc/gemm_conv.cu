// Entry points for the contractions of the training path — matmul, the three Linear GEMMs, conv2d
// forward / dX / dW / db — and their dispatch: the tcgen05 tensor-core kernels (tc_gemm.cu) when the
// operands can be described to TMA, else the FP32 SIMT tiled kernel (simt_gemm.cuh).  Both run on
// the device; there is no host fallback.
// Reference behaviour being replaced: src/cuda/cuda_matmul.cu:27-68 (cuBLAS), src/cuda/cuda_conv.cu:148-372
// (per-sample im2col + cuBLAS); arithmetic semantics from the CPU path src/nn/conv.c:118-375,381-586 and
// src/nn/linear.c:45-152.
#include "nc_common.cuh"
#include "simt_gemm.cuh"
#include "tc_gemm.cuh"
#include "../../include/nocta_cuda.h"

using namespace ncc;

namespace convfirst {
bool eligible(int Cin, int kH, int kW, int stride, int Cout);
int forward(float* y, const float* x, const long long xs[4], const float* w, const float* bias, int N, int H, int W, int Cout, int pad,
            cudaStream_t st);
int weight_grad(float* dW, const float* dy, const float* x, const long long xs[4], int N, int H, int W, int Cout, int pad, cudaStream_t st);
}  // namespace convfirst

namespace {

// ---------------- SIMT loaders / epilogues ----------------
struct MatLoad {  // element (i, k) of a strided matrix
    const float* p; long long s_outer, s_k;
    __device__ float operator()(int i, int k) const { return p[(long long)i * s_outer + (long long)k * s_k]; }
};

struct GemmStore {  // D = alpha*acc + beta*D + bias[n]   or raw partial[z][m][n]
    float* D; long long ldd; const float* bias; float alpha, beta; float* partial; int M, N;
    __device__ void operator()(int z, int m, int n, float acc) const {
        if (partial) { partial[((size_t)z * M + m) * N + n] = acc; return; }
        float* d = D + (long long)m * ldd + n;
        float o = alpha * acc;
        if (beta != 0.f) o += beta * *d;
        if (bias) o += bias[n];
        *d = o;
    }
};

__global__ void __launch_bounds__(256) partial_reduce_kernel(float* __restrict__ D, long long ldd, const float* __restrict__ partial,
                                                             int splits, int M, int N, const float* __restrict__ bias,
                                                             float alpha, float beta) {
    const size_t total = (size_t)M * N, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        float acc = 0.f;
        for (int z = 0; z < splits; z++) acc += partial[(size_t)z * total + i];
        const int m = (int)(i / N), n = (int)(i % N);
        float* d = D + (size_t)m * ldd + n;
        float o = alpha * acc;
        if (beta != 0.f) o += beta * *d;
        if (bias) o += bias[n];
        *d = o;
    }
}

struct ConvGeo {
    int N, Cin, H, W, Cout, kH, kW, stride, pad, Ho, Wo;
    long long xs[4], ys[4];  // element strides (n, c, h, w) of the input-side and output-side tensors
};

// forward: A(m = (n,ho,wo), k = (ci,kh,kw)) = x[n, ci, ho*s+kh-p, wo*s+kw-p]
struct ConvFwdA {
    const float* x; ConvGeo g;
    __device__ float operator()(int m, int k) const {
        int wo = m % g.Wo, t = m / g.Wo, ho = t % g.Ho, n = t / g.Ho;
        int kw = k % g.kW, t2 = k / g.kW, kh = t2 % g.kH, ci = t2 / g.kH;
        int h = ho * g.stride + kh - g.pad, w = wo * g.stride + kw - g.pad;
        if (h < 0 || h >= g.H || w < 0 || w >= g.W) return 0.f;
        return x[n * g.xs[0] + ci * g.xs[1] + h * g.xs[2] + w * g.xs[3]];
    }
};
struct ConvFwdStore {
    float* y; const float* bias; ConvGeo g;
    __device__ void operator()(int, int m, int co, float acc) const {
        int wo = m % g.Wo, t = m / g.Wo, ho = t % g.Ho, n = t / g.Ho;
        y[n * g.ys[0] + co * g.ys[1] + ho * g.ys[2] + wo * g.ys[3]] = acc + (bias ? bias[co] : 0.f);
    }
};
// dX (gather form, any stride): A(m = (n,h,w), k = (co,kh,kw)) = dy[n, co, (h+p-kh)/s, (w+p-kw)/s]
struct ConvDxA {
    const float* dy; ConvGeo g;
    __device__ float operator()(int m, int k) const {
        int w = m % g.W, t = m / g.W, h = t % g.H, n = t / g.H;
        int kw = k % g.kW, t2 = k / g.kW, kh = t2 % g.kH, co = t2 / g.kH;
        int hh = h + g.pad - kh, ww = w + g.pad - kw;
        if (hh < 0 || ww < 0 || hh % g.stride || ww % g.stride) return 0.f;
        int ho = hh / g.stride, wo = ww / g.stride;
        if (ho >= g.Ho || wo >= g.Wo) return 0.f;
        return dy[n * g.ys[0] + co * g.ys[1] + ho * g.ys[2] + wo * g.ys[3]];
    }
};
struct ConvDxB {  // B(ci, k = (co,kh,kw)) = w[co, ci, kh, kw]
    const float* w; ConvGeo g;
    __device__ float operator()(int ci, int k) const {
        int kw = k % g.kW, t2 = k / g.kW, kh = t2 % g.kH, co = t2 / g.kH;
        return w[(((long long)co * g.Cin + ci) * g.kH + kh) * g.kW + kw];
    }
};
struct ConvDxStore {
    float* dx; ConvGeo g;
    __device__ void operator()(int, int m, int ci, float acc) const {
        int w = m % g.W, t = m / g.W, h = t % g.H, n = t / g.H;
        dx[n * g.xs[0] + ci * g.xs[1] + h * g.xs[2] + w * g.xs[3]] = acc;
    }
};
// dW: A(co, k = (n,ho,wo)) = dy[n,co,ho,wo];  B(j = (ci,kh,kw), k) = x[n,ci,ho*s+kh-p,wo*s+kw-p]
struct ConvDwA {
    const float* dy; ConvGeo g;
    __device__ float operator()(int co, int k) const {
        int wo = k % g.Wo, t = k / g.Wo, ho = t % g.Ho, n = t / g.Ho;
        return dy[n * g.ys[0] + co * g.ys[1] + ho * g.ys[2] + wo * g.ys[3]];
    }
};
struct ConvDwB {
    const float* x; ConvGeo g;
    __device__ float operator()(int j, int k) const {
        int wo = k % g.Wo, t = k / g.Wo, ho = t % g.Ho, n = t / g.Ho;
        int kw = j % g.kW, t2 = j / g.kW, kh = t2 % g.kH, ci = t2 / g.kH;
        int h = ho * g.stride + kh - g.pad, w = wo * g.stride + kw - g.pad;
        if (h < 0 || h >= g.H || w < 0 || w >= g.W) return 0.f;
        return x[n * g.xs[0] + ci * g.xs[1] + h * g.xs[2] + w * g.xs[3]];
    }
};

// per-channel sum of a strided (N, C, Ho, Wo) tensor: fallback for layouts that are neither dense
// NCHW nor dense channels-last.  One block per channel, double accumulation, fixed order.
__global__ void __launch_bounds__(256) channel_sum_strided_kernel(float* __restrict__ out, const float* __restrict__ t, ConvGeo g) {
    __shared__ double sh[32];
    const int c = blockIdx.x;
    const long long per = (long long)g.Ho * g.Wo, total = per * g.N;
    double acc = 0.0;
    for (long long i = threadIdx.x; i < total; i += blockDim.x) {
        int wo = (int)(i % g.Wo);
        long long r = i / g.Wo;
        int ho = (int)(r % g.Ho), n = (int)(r / g.Ho);
        acc += (double)t[n * g.ys[0] + c * g.ys[1] + ho * g.ys[2] + wo * g.ys[3]];
    }
    acc = block_sum(acc, sh);
    if (threadIdx.x == 0) out[c] = (float)acc;
}

bool is_nchw(const long long s[4], int C, int H, int W) {
    return s[3] == 1 && s[2] == W && s[1] == (long long)H * W && s[0] == (long long)C * H * W;
}
bool is_nhwc(const long long s[4], int C, int H, int W) {
    return s[1] == 1 && s[3] == C && s[2] == (long long)W * C && s[0] == (long long)H * W * C;
}

int make_geo(ConvGeo* g, const size_t ys[4], const size_t xs[4], int N, int Cin, int H, int W, int Cout, int kH, int kW,
             int stride, int pad) {
    NCC_REQUIRE(N > 0 && Cin > 0 && Cout > 0 && kH > 0 && kW > 0 && stride > 0 && pad >= 0, "conv2d: bad dimensions");
    NCC_REQUIRE(H + 2 * pad >= kH && W + 2 * pad >= kW, "conv2d: kernel larger than padded input");
    g->N = N; g->Cin = Cin; g->H = H; g->W = W; g->Cout = Cout; g->kH = kH; g->kW = kW; g->stride = stride; g->pad = pad;
    g->Ho = (H + 2 * pad - kH) / stride + 1;
    g->Wo = (W + 2 * pad - kW) / stride + 1;
    for (int i = 0; i < 4; i++) { g->xs[i] = (long long)xs[i]; g->ys[i] = (long long)ys[i]; }
    NCC_REQUIRE((long long)N * g->Ho * g->Wo < 0x7fffffffLL && (long long)N * H * W < 0x7fffffffLL &&
                (long long)Cin * kH * kW < 0x7fffffffLL, "conv2d: index space exceeds 2^31");
    return NC_CUDA_OK;
}

int tc_mode() {
    int m = math_mode();
    return m;
}
bool tc_enabled() { return math_mode() != NC_CUDA_MATH_FP32_SIMT; }

// SIMT GEMM with automatic split over K when the output has too few tiles to fill the GPU.
int simt_matmul(float* C, long long ldc, MatLoad la, bool a_kfast, MatLoad lb, bool b_kfast, int M, int N, int K,
                const float* bias, float alpha, float beta, cudaStream_t st) {
    const int tiles = ceil_div(M, simt::TM) * ceil_div(N, simt::TN);
    int splits = 1;
    if (tiles * 2 <= sm_count() && K >= 256) {
        splits = sm_count() / tiles;
        if (splits > K / 64) splits = K / 64;
        if (splits < 1) splits = 1;
    }
    splits = simt::effective_splits(K, splits);
    float* partial = nullptr;
    if (splits > 1) {
        partial = (float*)scratch(2, sizeof(float) * (size_t)splits * M * N, st);
        if (!partial) return NC_CUDA_ERR_RUNTIME;
    }
    GemmStore ep{C, ldc, bias, alpha, beta, partial, M, N};
    int rc;
    if (a_kfast && b_kfast) rc = simt::launch<true, true>(M, N, K, splits, la, lb, ep, st, "simt_gemm");
    else if (a_kfast) rc = simt::launch<true, false>(M, N, K, splits, la, lb, ep, st, "simt_gemm");
    else if (b_kfast) rc = simt::launch<false, true>(M, N, K, splits, la, lb, ep, st, "simt_gemm");
    else rc = simt::launch<false, false>(M, N, K, splits, la, lb, ep, st, "simt_gemm");
    if (rc) return rc;
    if (splits > 1) {
        partial_reduce_kernel<<<grid_for((long long)M * N, 256), 256, 0, st>>>(C, ldc, partial, splits, M, N, bias, alpha, beta);
        NCC_COUNT_LAUNCH();
        return launch_status("partial_reduce");
    }
    return NC_CUDA_OK;
}

// C(M,N) = alpha * A' * B'^T + beta*C + bias, A' = (M,K) logical, B' = (N,K) logical.
//   a_mn: A stored (K,M);  b_mn: B stored (K,N).
int gemm_dispatch(float* C, int ldc, const float* A, int lda, bool a_mn, const float* B, int ldb, bool b_mn, int M, int N,
                  int K, const float* bias, float alpha, float beta, cudaStream_t st) {
    if (M <= 0 || N <= 0) return NC_CUDA_OK;
    NCC_REQUIRE(C && (K == 0 || (A && B)), "gemm: null pointer");
    if (tc_enabled() && K > 0) {
        prof_set_role(a_mn ? (b_mn ? PROF_GEMM_TN : PROF_GEMM_TT) : (b_mn ? PROF_GEMM_NN : PROF_GEMM_NT));
        int rc = tc::gemm(C, ldc, A, lda, a_mn, B, ldb, b_mn, M, N, K, bias, alpha, beta, tc_mode(), st);
        if (rc != NC_CUDA_ERR_UNSUPPORTED) return rc;
    }
    MatLoad la{A, a_mn ? 1 : lda, a_mn ? lda : 1};
    MatLoad lb{B, b_mn ? 1 : ldb, b_mn ? ldb : 1};
    return simt_matmul(C, ldc, la, !a_mn, lb, !b_mn, M, N, K, bias, alpha, beta, st);
}


// NCHW tensors can still use the tensor-core kernels: re-lay them out channels-last in library
// scratch (one coalesced transpose pass each way).  Worth it only when the channel counts tile.
bool relayout_ok(const ConvGeo& g) {
    return tc_enabled() && g.stride == 1 && (g.Cin % 32 == 0) && (g.Cout % 32 == 0) && g.kH == g.kW &&
           g.kH - 1 - g.pad >= 0 && (long long)g.N * g.Ho * g.Wo >= 128 && g.N <= 65535 &&
           is_nchw(g.xs, g.Cin, g.H, g.W) && is_nchw(g.ys, g.Cout, g.Ho, g.Wo);
}
// In plain TF32 mode the relayout pass also rounds to the nearest TF32 value, so the tensor core's
// dropping of low mantissa bits cannot bias the sums.
int round_in_relayout() { return math_mode() == NC_CUDA_MATH_TF32 ? 1 : 0; }

void nchw_strides(size_t s[4], int C, int H, int W) {
    s[0] = (size_t)C * H * W; s[1] = (size_t)H * W; s[2] = (size_t)W; s[3] = 1;
}
void nhwc_strides(size_t s[4], int C, int H, int W) {
    s[0] = (size_t)H * W * C; s[1] = 1; s[2] = (size_t)W * C; s[3] = (size_t)C;
}

// Parameters keep their full f32 value in memory; in plain TF32 mode the Linear GEMMs read a copy
// rounded to the nearest TF32 value (library scratch) so that the tensor core's truncation of its
// operands is exact.  Skipped when the GEMM will run on the FP32 SIMT kernel anyway (fewer than 128 rows).
const float* conditioned_weight(const float* W, size_t n, int rows, cudaStream_t st) {
    if (math_mode() != NC_CUDA_MATH_TF32 || rows < 128) return W;
    float* Wr = (float*)scratch(3, sizeof(float) * n, st);
    if (!Wr) return nullptr;
    if (nc_cuda_round_tf32_f32_ex(Wr, W, n, st)) return nullptr;
    return Wr;
}

}  // namespace

extern "C" {

int nc_cuda_matmul_f32_ex(float* C, int ldc, const float* A, int lda, const float* B, int ldb, int M, int N, int K,
                          float alpha, float beta, int transA, int transB, const float* bias, void* stream) {
    // op(A) is (M,K): stored (M,K) when !transA (K-major), stored (K,M) when transA (MN-major).
    // op(B) is (K,N): stored (K,N) when !transB (MN-major for the kernel), stored (N,K) when transB.
    return gemm_dispatch(C, ldc, A, lda, transA != 0, B, ldb, transB == 0, M, N, K, bias, alpha, beta, (cudaStream_t)stream);
}
void nc_cuda_matmul_f32(float* C, const float* A, const float* B, int M, int N, int K, float alpha, float beta,
                        int transA, int transB) {
    nc_cuda_matmul_f32_ex(C, N, A, transA ? M : K, B, transB ? K : N, M, N, K, alpha, beta, transA, transB, nullptr,
                          current_stream());
}

int nc_cuda_linear_forward_f32_ex(float* y, const float* x, const float* W, const float* bias, int batch, int in_f,
                                  int out_f, void* stream) {
    NCC_REQUIRE(y && x && W && batch > 0 && in_f > 0 && out_f > 0, "linear_forward: bad argument");
    const float* Wc = conditioned_weight(W, (size_t)out_f * in_f, batch, (cudaStream_t)stream);
    if (!Wc) return NC_CUDA_ERR_RUNTIME;
    // y(B,out) = x(B,in) * W(out,in)^T : both operands K-major
    return gemm_dispatch(y, out_f, x, in_f, false, Wc, in_f, false, batch, out_f, in_f, bias, 1.f, 0.f, (cudaStream_t)stream);
}

int nc_cuda_linear_backward_f32_ex(float* dx, float* dW, float* db, const float* dy, const float* x, const float* W,
                                   int batch, int in_f, int out_f, void* stream) {
    NCC_REQUIRE(dy && batch > 0 && in_f > 0 && out_f > 0, "linear_backward: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    int rc;
    if (dx) {
        NCC_REQUIRE(W, "linear_backward: dx needs W");
        const float* Wc = conditioned_weight(W, (size_t)out_f * in_f, batch, st);
        if (!Wc) return NC_CUDA_ERR_RUNTIME;
        // dx(B,in) = dy(B,out) * W(out,in): A K-major (k = out), B stored (K = out, N = in) -> MN-major
        rc = gemm_dispatch(dx, in_f, dy, out_f, false, Wc, in_f, true, batch, in_f, out_f, nullptr, 1.f, 0.f, st);
        if (rc) return rc;
    }
    if (dW) {
        NCC_REQUIRE(x, "linear_backward: dW needs x");
        // dW(out,in) = dy^T(out,B) * x(B,in): A stored (K = B, M = out), B stored (K = B, N = in): both MN-major
        rc = gemm_dispatch(dW, in_f, dy, out_f, true, x, in_f, true, out_f, in_f, batch, nullptr, 1.f, 0.f, st);
        if (rc) return rc;
    }
    if (db) {
        rc = column_sums(db, dy, (size_t)batch, out_f, st);
        if (rc) return rc;
    }
    return NC_CUDA_OK;
}

int nc_cuda_conv2d_forward_f32_ex(float* y, const size_t ys[4], const float* x, const size_t xs[4], const float* w,
                                  const float* bias, int N, int Cin, int H, int W, int Cout, int kH, int kW, int stride,
                                  int pad, void* stream) {
    NCC_REQUIRE(y && x && w && ys && xs, "conv2d_forward: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    ConvGeo g;
    int rc = make_geo(&g, ys, xs, N, Cin, H, W, Cout, kH, kW, stride, pad);
    if (rc) return rc;
    if (relayout_ok(g)) {
        float* xh = (float*)scratch(4, sizeof(float) * (size_t)N * Cin * H * W, st);
        float* yh = (float*)scratch(5, sizeof(float) * (size_t)N * Cout * g.Ho * g.Wo, st);
        if (!xh || !yh) return NC_CUDA_ERR_RUNTIME;
        rc = nc_cuda_nchw_to_nhwc_f32_ex(xh, x, N, Cin, H * W, round_in_relayout(), st);
        if (rc) return rc;
        size_t xs2[4], ys2[4];
        nhwc_strides(xs2, Cin, H, W);
        nhwc_strides(ys2, Cout, g.Ho, g.Wo);
        rc = nc_cuda_conv2d_forward_f32_ex(yh, ys2, xh, xs2, w, bias, N, Cin, H, W, Cout, kH, kW, stride, pad, stream);
        if (rc) return rc;
        return nc_cuda_nhwc_to_nchw_f32_ex(y, yh, N, Cout, g.Ho * g.Wo, st);
    }
    if (tc_enabled() && stride == 1 && is_nhwc(g.xs, Cin, H, W) && is_nhwc(g.ys, Cout, g.Ho, g.Wo)) {
        float* wp = (float*)scratch(3, sizeof(float) * (size_t)Cout * Cin * kH * kW, st);
        if (!wp) return NC_CUDA_ERR_RUNTIME;
        rc = tc::pack_weights_fwd(wp, w, Cout, Cin, kH, kW, round_in_relayout() != 0, st);
        if (rc) return rc;
        prof_set_role(PROF_CONV_FWD);
        rc = tc::conv_nhwc(y, x, wp, bias, N, H, W, Cin, Cout, kH, kW, pad, tc_mode(), st);
        if (rc != NC_CUDA_ERR_UNSUPPORTED) return rc;
    }
    if (convfirst::eligible(Cin, kH, kW, stride, Cout) && is_nhwc(g.ys, Cout, g.Ho, g.Wo)) {
        ProfScope prof(PROF_CONV_FIRST, 4.0 * ((double)N * g.Ho * g.Wo * Cout + (double)N * Cin * H * W), st);
        rc = convfirst::forward(y, x, g.xs, w, bias, N, H, W, Cout, pad, st);
        if (rc != NC_CUDA_ERR_UNSUPPORTED) return rc;
    }
    const int M = N * g.Ho * g.Wo, K = Cin * kH * kW;
    return simt::launch<false, true>(M, Cout, K, 1, ConvFwdA{x, g}, MatLoad{w, K, 1}, ConvFwdStore{y, bias, g}, st,
                                     "conv2d_forward(simt)");
}

int nc_cuda_conv2d_backward_input_f32_ex(float* dx, const size_t xs[4], const float* dy, const size_t ys[4], const float* w,
                                         int N, int Cin, int H, int W, int Cout, int kH, int kW, int stride, int pad,
                                         void* stream) {
    // an announced BatchNorm backward (nc_cuda_offer_batchnorm_backward_sums_f32) is served by this call or dropped
    struct FoldScope { FoldScope() { bn_fold_enter(); } ~FoldScope() { bn_fold_leave(); } } fold_scope;
    NCC_REQUIRE(dx && dy && w && ys && xs, "conv2d_backward_input: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    ConvGeo g;
    int rc = make_geo(&g, ys, xs, N, Cin, H, W, Cout, kH, kW, stride, pad);
    if (rc) return rc;
    if (tc_enabled() && stride == 1 && kH - 1 - pad >= 0 && kW == kH && is_nhwc(g.xs, Cin, H, W) &&
        is_nhwc(g.ys, Cout, g.Ho, g.Wo)) {
        float* wp = (float*)scratch(3, sizeof(float) * (size_t)Cout * Cin * kH * kW, st);
        if (!wp) return NC_CUDA_ERR_RUNTIME;
        rc = tc::pack_weights_dx(wp, w, Cout, Cin, kH, kW, round_in_relayout() != 0, st);
        if (rc) return rc;
        // dx = conv(dy, flipped weights) with padding k-1-pad; roles of Cin and Cout swap
        prof_set_role(PROF_CONV_DX);
        rc = tc::conv_nhwc(dx, dy, wp, nullptr, N, g.Ho, g.Wo, Cout, Cin, kH, kW, kH - 1 - pad, tc_mode(), st);
        if (rc != NC_CUDA_ERR_UNSUPPORTED) return rc;
    }
    const int M = N * H * W, K = Cout * kH * kW;
    return simt::launch<false, false>(M, Cin, K, 1, ConvDxA{dy, g}, ConvDxB{w, g}, ConvDxStore{dx, g}, st,
                                      "conv2d_backward_input(simt)");
}

int nc_cuda_conv2d_backward_weight_f32_ex(float* dW, float* db, const float* dy, const size_t ys[4], const float* x,
                                          const size_t xs[4], int N, int Cin, int H, int W, int Cout, int kH, int kW,
                                          int stride, int pad, void* stream) {
    NCC_REQUIRE(dy && ys && (dW == nullptr || (x && xs)), "conv2d_backward_weight: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    ConvGeo g;
    size_t dummy[4] = {0, 0, 0, 0};
    int rc = make_geo(&g, ys, xs ? xs : dummy, N, Cin, H, W, Cout, kH, kW, stride, pad);
    if (rc) return rc;
    if (db) {
        if (is_nhwc(g.ys, Cout, g.Ho, g.Wo)) {
            rc = column_sums(db, dy, (size_t)N * g.Ho * g.Wo, Cout, st);
        } else if (is_nchw(g.ys, Cout, g.Ho, g.Wo)) {
            float* tmp = (float*)scratch(4, sizeof(float) * (size_t)N * Cout, st);
            if (!tmp) return NC_CUDA_ERR_RUNTIME;
            rc = nc_cuda_sum_axis_f32_ex(tmp, dy, (size_t)N * Cout, (size_t)g.Ho * g.Wo, 1, st);
            if (!rc) rc = column_sums(db, tmp, (size_t)N, Cout, st);
        } else {
            channel_sum_strided_kernel<<<Cout, 256, 0, st>>>(db, dy, g);
            NCC_COUNT_LAUNCH();
            rc = launch_status("conv2d_backward_bias");
        }
        if (rc) return rc;
    }
    if (!dW) return NC_CUDA_OK;
    if (tc_enabled() && stride == 1 && is_nhwc(g.xs, Cin, H, W) && is_nhwc(g.ys, Cout, g.Ho, g.Wo)) {
        prof_set_role(PROF_CONV_DW);
        rc = tc::conv_dw_nhwc(dW, dy, x, N, H, W, Cin, Cout, kH, kW, pad, tc_mode(), st);
        if (rc != NC_CUDA_ERR_UNSUPPORTED) return rc;
    }
    if (convfirst::eligible(Cin, kH, kW, stride, Cout) && is_nhwc(g.ys, Cout, g.Ho, g.Wo)) {
        ProfScope prof(PROF_CONV_FIRST, 4.0 * ((double)N * g.Ho * g.Wo * Cout + (double)N * Cin * H * W), st);
        rc = convfirst::weight_grad(dW, dy, x, g.xs, N, H, W, Cout, pad, st);
        if (rc != NC_CUDA_ERR_UNSUPPORTED) return rc;
    }
    const int Kred = N * g.Ho * g.Wo, Ncols = Cin * kH * kW;
    const int tiles = ceil_div(Cout, simt::TM) * ceil_div(Ncols, simt::TN);
    int splits = (sm_count() * 2 + tiles - 1) / tiles;
    if (splits > Kred / 64) splits = Kred / 64;
    splits = simt::effective_splits(Kred, splits);
    float* partial = nullptr;
    if (splits > 1) {
        partial = (float*)scratch(2, sizeof(float) * (size_t)splits * Cout * Ncols, st);
        if (!partial) return NC_CUDA_ERR_RUNTIME;
    }
    GemmStore ep{dW, Ncols, nullptr, 1.f, 0.f, partial, Cout, Ncols};
    const bool nchw_in = is_nchw(g.xs, Cin, H, W);
    // dy is contiguous along the reduction index for NCHW (k-fast), along co for channels-last
    if (is_nchw(g.ys, Cout, g.Ho, g.Wo) && nchw_in)
        rc = simt::launch<true, true>(Cout, Ncols, Kred, splits, ConvDwA{dy, g}, ConvDwB{x, g}, ep, st, "conv2d_backward_weight(simt)");
    else
        rc = simt::launch<false, false>(Cout, Ncols, Kred, splits, ConvDwA{dy, g}, ConvDwB{x, g}, ep, st, "conv2d_backward_weight(simt)");
    if (rc) return rc;
    if (splits > 1) {
        partial_reduce_kernel<<<grid_for((long long)Cout * Ncols, 256), 256, 0, st>>>(dW, Ncols, partial, splits, Cout, Ncols, nullptr, 1.f, 0.f);
        NCC_COUNT_LAUNCH();
        return launch_status("partial_reduce");
    }
    return NC_CUDA_OK;
}

// ---- legacy NCHW names (reference: include/nocta/cuda/cuda_kernels.h:95-112) ----

int nc_cuda_conv2d_backward_f32_ex(float* dx, float* dW, float* db, const float* dy, const float* x, const float* w,
                                   int N, int Cin, int H, int W, int Cout, int kH, int kW, int stride, int pad,
                                   void* stream) {
    NCC_REQUIRE(dy && (!dx || w) && (!dW || x), "conv2d_backward: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    size_t xs[4], ys[4];
    nchw_strides(xs, Cin, H, W);
    ConvGeo g;
    {
        size_t t[4] = {0, 0, 0, 0};
        int rc0 = make_geo(&g, t, xs, N, Cin, H, W, Cout, kH, kW, stride, pad);
        if (rc0) return rc0;
    }
    nchw_strides(ys, Cout, g.Ho, g.Wo);
    for (int i = 0; i < 4; i++) g.ys[i] = (long long)ys[i];
    int rc;
    if (relayout_ok(g)) {
        size_t xs2[4], ys2[4];
        nhwc_strides(xs2, Cin, H, W);
        nhwc_strides(ys2, Cout, g.Ho, g.Wo);
        float* dyh = (float*)scratch(4, sizeof(float) * (size_t)N * Cout * g.Ho * g.Wo, st);
        if (!dyh) return NC_CUDA_ERR_RUNTIME;
        rc = nc_cuda_nchw_to_nhwc_f32_ex(dyh, dy, N, Cout, g.Ho * g.Wo, round_in_relayout(), st);
        if (rc) return rc;
        if (dW || db) {
            float* xh = nullptr;
            if (dW) {
                xh = (float*)scratch(5, sizeof(float) * (size_t)N * Cin * H * W, st);
                if (!xh) return NC_CUDA_ERR_RUNTIME;
                rc = nc_cuda_nchw_to_nhwc_f32_ex(xh, x, N, Cin, H * W, round_in_relayout(), st);
                if (rc) return rc;
            }
            rc = nc_cuda_conv2d_backward_weight_f32_ex(dW, db, dyh, ys2, xh, xs2, N, Cin, H, W, Cout, kH, kW, stride, pad, stream);
            if (rc) return rc;
        }
        if (dx) {
            float* dxh = (float*)scratch(6, sizeof(float) * (size_t)N * Cin * H * W, st);
            if (!dxh) return NC_CUDA_ERR_RUNTIME;
            rc = nc_cuda_conv2d_backward_input_f32_ex(dxh, xs2, dyh, ys2, w, N, Cin, H, W, Cout, kH, kW, stride, pad, stream);
            if (rc) return rc;
            rc = nc_cuda_nhwc_to_nchw_f32_ex(dx, dxh, N, Cin, H * W, st);
            if (rc) return rc;
        }
        return NC_CUDA_OK;
    }
    if (dW || db) {
        rc = nc_cuda_conv2d_backward_weight_f32_ex(dW, db, dy, ys, x, xs, N, Cin, H, W, Cout, kH, kW, stride, pad, stream);
        if (rc) return rc;
    }
    if (dx) {
        rc = nc_cuda_conv2d_backward_input_f32_ex(dx, xs, dy, ys, w, N, Cin, H, W, Cout, kH, kW, stride, pad, stream);
        if (rc) return rc;
    }
    return NC_CUDA_OK;
}

void nc_cuda_conv2d_forward_f32(float* y, const float* x, const float* w, const float* bias, int N, int Cin, int H, int W,
                                int Cout, int kH, int kW, int stride, int pad) {
    size_t xs[4], ys[4];
    nchw_strides(xs, Cin, H, W);
    nchw_strides(ys, Cout, (H + 2 * pad - kH) / stride + 1, (W + 2 * pad - kW) / stride + 1);
    nc_cuda_conv2d_forward_f32_ex(y, ys, x, xs, w, bias, N, Cin, H, W, Cout, kH, kW, stride, pad, current_stream());
}
void nc_cuda_conv2d_backward_input_f32(float* dx, const float* dy, const float* w, int N, int Cin, int H, int W, int Cout,
                                       int kH, int kW, int stride, int pad) {
    nc_cuda_conv2d_backward_f32_ex(dx, nullptr, nullptr, dy, nullptr, w, N, Cin, H, W, Cout, kH, kW, stride, pad, current_stream());
}
void nc_cuda_conv2d_backward_weight_f32(float* dW, const float* dy, const float* x, int N, int Cin, int H, int W, int Cout,
                                        int kH, int kW, int stride, int pad) {
    nc_cuda_conv2d_backward_f32_ex(nullptr, dW, nullptr, dy, x, nullptr, N, Cin, H, W, Cout, kH, kW, stride, pad, current_stream());
}
void nc_cuda_conv2d_backward_bias_f32(float* db, const float* dy, int N, int Cout, int Ho, int Wo) {
    size_t ys[4];
    nchw_strides(ys, Cout, Ho, Wo);
    // geometry with a 1x1 kernel, stride 1, no padding maps (H, W) onto (Ho, Wo)
    nc_cuda_conv2d_backward_weight_f32_ex(nullptr, db, dy, ys, nullptr, nullptr, N, 1, Ho, Wo, Cout, 1, 1, 1, 0, current_stream());
}

}  // extern "C"
