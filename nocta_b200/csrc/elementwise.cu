// Memory-bound elementwise kernels: fill/copy/arithmetic, ReLU and GELU (forward + mask-multiply
// backward), row softmax, strided gather copy, NCHW<->NHWC relayout, TF32 rounding.
// All are grid-stride, float4-vectorised when the pointers allow it, with a grid that is a
// multiple of the SM count.  Replaces src/cuda/cuda_elementwise.cu and src/cuda/cuda_activation.cu
// of the reference (one thread per element, scalar loads).
#include "nc_common.cuh"
#include "../../include/nocta_cuda.h"

using namespace ncc;

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float4 ld4(const float* p, size_t i) { return reinterpret_cast<const float4*>(p)[i]; }
__device__ __forceinline__ void st4(float* p, size_t i, float4 v) { reinterpret_cast<float4*>(p)[i] = v; }
__device__ __forceinline__ float4 rnd4(float4 v) { return make_float4(round_tf32(v.x), round_tf32(v.y), round_tf32(v.z), round_tf32(v.w)); }

// out[i] = f(a[i], b[i]); b may be null when NIN == 1; NIN == 0 means no input at all.
template <int NIN, bool RND, class F>
__global__ void __launch_bounds__(kThreads) ew_kernel(float* __restrict__ out, const float* __restrict__ a,
                                                      const float* __restrict__ b, size_t n4, size_t n, F f) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    // two vectors in flight per thread per trip
    size_t i = t0;
    for (; i + stride < n4; i += 2 * stride) {
        float4 a0 = make_float4(0, 0, 0, 0), a1 = a0, b0 = a0, b1 = a0;
        if (NIN >= 1) { a0 = ld4(a, i); a1 = ld4(a, i + stride); }
        if (NIN >= 2) { b0 = ld4(b, i); b1 = ld4(b, i + stride); }
        float4 r0, r1;
        r0.x = f(a0.x, b0.x); r0.y = f(a0.y, b0.y); r0.z = f(a0.z, b0.z); r0.w = f(a0.w, b0.w);
        r1.x = f(a1.x, b1.x); r1.y = f(a1.y, b1.y); r1.z = f(a1.z, b1.z); r1.w = f(a1.w, b1.w);
        if (RND) { r0 = rnd4(r0); r1 = rnd4(r1); }
        st4(out, i, r0);
        st4(out, i + stride, r1);
    }
    for (; i < n4; i += stride) {
        float4 a0 = make_float4(0, 0, 0, 0), b0 = a0;
        if (NIN >= 1) a0 = ld4(a, i);
        if (NIN >= 2) b0 = ld4(b, i);
        float4 r0;
        r0.x = f(a0.x, b0.x); r0.y = f(a0.y, b0.y); r0.z = f(a0.z, b0.z); r0.w = f(a0.w, b0.w);
        if (RND) r0 = rnd4(r0);
        st4(out, i, r0);
    }
    for (size_t j = n4 * 4 + t0; j < n; j += stride) {
        float av = NIN >= 1 ? a[j] : 0.f, bv = NIN >= 2 ? b[j] : 0.f;
        float r = f(av, bv);
        out[j] = RND ? round_tf32(r) : r;
    }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// rnd: round results to TF32 (activations / gradients in plain TF32 mode); never for fill / copy
template <int NIN, class F>
int launch_ew(float* out, const float* a, const float* b, size_t n, cudaStream_t st, F f, const char* what, bool rnd = false,
              int category = PROF_ELEMENTWISE) {
    if (n == 0) return NC_CUDA_OK;
    NCC_REQUIRE(out && (NIN < 1 || a) && (NIN < 2 || b), "%s: null pointer", what);
    ProfScope prof(category, 4.0 * (NIN + 1) * (double)n, st);
    bool vec = aligned16(out) && (NIN < 1 || aligned16(a)) && (NIN < 2 || aligned16(b));
    size_t n4 = vec ? n / 4 : 0;
    int grid = grid_for((long long)(vec ? (n + 3) / 4 : n), kThreads, 8);
    if (rnd) ew_kernel<NIN, true, F><<<grid, kThreads, 0, st>>>(out, a, b, n4, n, f);
    else ew_kernel<NIN, false, F><<<grid, kThreads, 0, st>>>(out, a, b, n4, n, f);
    NCC_COUNT_LAUNCH();
    return launch_status(what);
}

struct FillF { float v; __device__ float operator()(float, float) const { return v; } };
struct CopyF { __device__ float operator()(float a, float) const { return a; } };
struct AddF { __device__ float operator()(float a, float b) const { return a + b; } };
struct SubF { __device__ float operator()(float a, float b) const { return a - b; } };
struct MulF { __device__ float operator()(float a, float b) const { return a * b; } };
struct DivF { __device__ float operator()(float a, float b) const { return a / b; } };
struct AddSF { float s; __device__ float operator()(float a, float) const { return a + s; } };
struct SubSF { float s; __device__ float operator()(float a, float) const { return a - s; } };
struct MulSF { float s; __device__ float operator()(float a, float) const { return a * s; } };
struct DivSF { float s; __device__ float operator()(float a, float) const { return a / s; } };
struct ReluF { __device__ float operator()(float a, float) const { return a > 0.f ? a : 0.f; } };
// dx = x > 0 ? dy : 0, tested on the saved INPUT (src/ops/activation.c:63-67): a = dy, b = x
struct ReluBwdF { __device__ float operator()(float dy, float x) const { return x > 0.f ? dy : 0.f; } };
struct RoundF { __device__ float operator()(float a, float) const { return round_tf32(a); } };

// GELU, tanh approximation (src/ops/activation.c:295-306)
__device__ __forceinline__ float gelu_fwd(float x) {
    const float c = 0.7978845608028654f, a = 0.044715f;
    float u = c * (x + a * x * x * x);
    return 0.5f * x * (1.f + tanhf(u));
}
__device__ __forceinline__ float gelu_grad(float x) {
    const float c = 0.7978845608028654f, a = 0.044715f;
    float u = c * (x + a * x * x * x);
    float th = tanhf(u);
    return 0.5f * (1.f + th) + 0.5f * x * (1.f - th * th) * c * (1.f + 3.f * a * x * x);
}
// sigmoid and its derivative s * (1 - s) taken on the saved input (src/ops/activation.c:72-105, 312-340)
struct SigmoidF { __device__ float operator()(float a, float) const { return 1.f / (1.f + expf(-a)); } };
struct SigmoidBwdF {
    __device__ float operator()(float dy, float x) const { const float sg = 1.f / (1.f + expf(-x)); return dy * sg * (1.f - sg); }
};
struct GeluF { __device__ float operator()(float a, float) const { return gelu_fwd(a); } };
struct GeluBwdF { __device__ float operator()(float dy, float x) const { return dy * gelu_grad(x); } };

// out[i] = a[i] + b[i % inner]
__global__ void __launch_bounds__(kThreads) bias_rows_kernel(float* __restrict__ out, const float* __restrict__ a,
                                                             const float* __restrict__ b, size_t total, int inner, int rnd) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        float r = a[i] + b[i % (size_t)inner];
        out[i] = rnd ? round_tf32(r) : r;
    }
}

// One warp per row; columns strided over lanes.  Max-subtracted exponentials, f32.
__global__ void __launch_bounds__(kThreads) softmax_rows_kernel(float* __restrict__ out, const float* __restrict__ in,
                                                                size_t rows, size_t cols) {
    const int lane = threadIdx.x & 31;
    const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const float* x = in + r * cols;
        float* y = out + r * cols;
        float m = -INFINITY;
        for (size_t c = lane; c < cols; c += 32) m = fmaxf(m, x[c]);
        m = warp_max(m);
        float s = 0.f;
        for (size_t c = lane; c < cols; c += 32) s += expf(x[c] - m);
        s = warp_sum(s);
        float inv = 1.f / s;
        for (size_t c = lane; c < cols; c += 32) y[c] = expf(x[c] - m) * inv;
    }
}

struct Dims4 { size_t shape[4]; size_t stride[4]; };

__global__ void __launch_bounds__(kThreads) strided_copy_kernel(float* __restrict__ dst, const float* __restrict__ src,
                                                                Dims4 d, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        size_t r = i;
        size_t i3 = r % d.shape[3]; r /= d.shape[3];
        size_t i2 = r % d.shape[2]; r /= d.shape[2];
        size_t i1 = r % d.shape[1]; r /= d.shape[1];
        size_t i0 = r;
        dst[i] = src[i0 * d.stride[0] + i1 * d.stride[1] + i2 * d.stride[2] + i3 * d.stride[3]];
    }
}

// Batched transpose of a (R x Cc) row-major matrix per batch item into (Cc x R), 32x32 tiles
// through padded shared memory; both the read and the write are coalesced.
template <bool ROUND>
__global__ void __launch_bounds__(256) transpose_kernel(float* __restrict__ dst, const float* __restrict__ src,
                                                        int R, int Cc) {
    __shared__ float tile[32][33];
    const size_t base = (size_t)blockIdx.z * R * Cc;
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        int r = r0 + ty + j, c = c0 + tx;
        if (r < R && c < Cc) tile[ty + j][tx] = src[base + (size_t)r * Cc + c];
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        int c = c0 + ty + j, r = r0 + tx;
        if (r < R && c < Cc) {
            float v = tile[tx][ty + j];
            dst[base + (size_t)c * R + r] = ROUND ? round_tf32(v) : v;
        }
    }
}

int transpose_batched(float* dst, const float* src, int batch, int R, int Cc, bool round, cudaStream_t st) {
    if (batch <= 0 || R <= 0 || Cc <= 0) return NC_CUDA_OK;
    NCC_REQUIRE(dst && src, "transpose: null pointer");
    NCC_REQUIRE(batch <= 65535 && ceil_div(R, 32) <= 65535, "transpose: grid too large");
    ProfScope prof(PROF_RELAYOUT, 8.0 * (double)batch * R * Cc, st);
    dim3 grid(ceil_div(Cc, 32), ceil_div(R, 32), batch);
    if (round) transpose_kernel<true><<<grid, 256, 0, st>>>(dst, src, R, Cc);
    else transpose_kernel<false><<<grid, 256, 0, st>>>(dst, src, R, Cc);
    NCC_COUNT_LAUNCH();
    return launch_status("transpose");
}

}  // namespace

extern "C" {

int nc_cuda_fill_f32_ex(float* data, float value, size_t n, void* stream) {
    return launch_ew<0>(data, nullptr, nullptr, n, (cudaStream_t)stream, FillF{value}, "fill");
}
int nc_cuda_copy_f32_ex(float* dst, const float* src, size_t n, void* stream) {
    return launch_ew<1>(dst, src, nullptr, n, (cudaStream_t)stream, CopyF{}, "copy");
}
int nc_cuda_binary_f32_ex(int op, float* out, const float* a, const float* b, size_t n, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    switch (op) {
        case 0: return launch_ew<2>(out, a, b, n, st, AddF{}, "add", round_outputs());
        case 1: return launch_ew<2>(out, a, b, n, st, SubF{}, "sub", round_outputs());
        case 2: return launch_ew<2>(out, a, b, n, st, MulF{}, "mul", round_outputs());
        case 3: return launch_ew<2>(out, a, b, n, st, DivF{}, "div", round_outputs());
    }
    return set_status(NC_CUDA_ERR_ARG, "binary: unknown op %d", op);
}
int nc_cuda_scalar_f32_ex(int op, float* out, const float* a, float s, size_t n, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    switch (op) {
        case 0: return launch_ew<1>(out, a, nullptr, n, st, AddSF{s}, "add_scalar", round_outputs());
        case 1: return launch_ew<1>(out, a, nullptr, n, st, SubSF{s}, "sub_scalar", round_outputs());
        case 2: return launch_ew<1>(out, a, nullptr, n, st, MulSF{s}, "mul_scalar", round_outputs());
        case 3: return launch_ew<1>(out, a, nullptr, n, st, DivSF{s}, "div_scalar", round_outputs());
    }
    return set_status(NC_CUDA_ERR_ARG, "scalar: unknown op %d", op);
}
int nc_cuda_add_broadcast_batch_f32_ex(float* out, const float* a, const float* b, size_t total, int inner,
                                       void* stream) {
    if (total == 0) return NC_CUDA_OK;
    NCC_REQUIRE(out && a && b && inner > 0, "add_broadcast: bad argument");
    ProfScope prof(PROF_ELEMENTWISE, 8.0 * (double)total, (cudaStream_t)stream);
    bias_rows_kernel<<<grid_for((long long)total, kThreads), kThreads, 0, (cudaStream_t)stream>>>(out, a, b, total, inner, round_outputs() ? 1 : 0);
    NCC_COUNT_LAUNCH();
    return launch_status("add_broadcast");
}
int nc_cuda_strided_copy_f32_ex(float* dst, const float* src, const size_t shape[4], const size_t strides[4],
                                void* stream) {
    NCC_REQUIRE(dst && src && shape && strides, "strided_copy: null pointer");
    Dims4 d;
    size_t n = 1;
    for (int i = 0; i < 4; i++) {
        d.shape[i] = shape[i];
        d.stride[i] = strides[i];
        n *= shape[i];
    }
    if (n == 0) return NC_CUDA_OK;
    // channels-last storage viewed as NCHW: a batched 2-D transpose
    if (strides[1] == 1 && strides[3] == shape[1] && strides[2] == shape[3] * shape[1] &&
        strides[0] == shape[2] * shape[3] * shape[1] && shape[0] <= 65535)
        return transpose_batched(dst, src, (int)shape[0], (int)(shape[2] * shape[3]), (int)shape[1], false,
                                 (cudaStream_t)stream);
    strided_copy_kernel<<<grid_for((long long)n, kThreads), kThreads, 0, (cudaStream_t)stream>>>(dst, src, d, n);
    NCC_COUNT_LAUNCH();
    return launch_status("strided_copy");
}
int nc_cuda_nchw_to_nhwc_f32_ex(float* dst, const float* src, int N, int C, int HW, int round, void* stream) {
    return transpose_batched(dst, src, N, C, HW, round != 0, (cudaStream_t)stream);
}
int nc_cuda_nhwc_to_nchw_f32_ex(float* dst, const float* src, int N, int C, int HW, void* stream) {
    return transpose_batched(dst, src, N, HW, C, false, (cudaStream_t)stream);
}
int nc_cuda_round_tf32_f32_ex(float* dst, const float* src, size_t n, void* stream) {
    return launch_ew<1>(dst, src, nullptr, n, (cudaStream_t)stream, RoundF{}, "round_tf32");
}
int nc_cuda_relu_f32_ex(float* out, const float* in, size_t n, void* stream) {
    return launch_ew<1>(out, in, nullptr, n, (cudaStream_t)stream, ReluF{}, "relu", round_outputs(), PROF_ACTIVATION);
}
int nc_cuda_relu_backward_f32_ex(float* gi, const float* go, const float* input, size_t n, void* stream) {
    return launch_ew<2>(gi, go, input, n, (cudaStream_t)stream, ReluBwdF{}, "relu_backward", round_outputs(), PROF_ACTIVATION);
}
int nc_cuda_gelu_f32_ex(float* out, const float* in, size_t n, void* stream) {
    return launch_ew<1>(out, in, nullptr, n, (cudaStream_t)stream, GeluF{}, "gelu", round_outputs(), PROF_ACTIVATION);
}
int nc_cuda_gelu_backward_f32_ex(float* gi, const float* go, const float* input, size_t n, void* stream) {
    return launch_ew<2>(gi, go, input, n, (cudaStream_t)stream, GeluBwdF{}, "gelu_backward", round_outputs(), PROF_ACTIVATION);
}
int nc_cuda_softmax_f32_ex(float* out, const float* in, size_t batch, size_t dim, void* stream) {
    if (batch == 0 || dim == 0) return NC_CUDA_OK;
    NCC_REQUIRE(out && in, "softmax: null pointer");
    softmax_rows_kernel<<<grid_for((long long)batch * 32, kThreads), kThreads, 0, (cudaStream_t)stream>>>(out, in, batch, dim);
    NCC_COUNT_LAUNCH();
    return launch_status("softmax");
}

// ---- legacy void names (reference: include/nocta/cuda/cuda_kernels.h:26-58) ----
void nc_cuda_fill_f32(float* d, float v, size_t n) { nc_cuda_fill_f32_ex(d, v, n, current_stream()); }
void nc_cuda_copy_f32(float* d, const float* s, size_t n) { nc_cuda_copy_f32_ex(d, s, n, current_stream()); }
void nc_cuda_add_f32(float* o, const float* a, const float* b, size_t n) { nc_cuda_binary_f32_ex(0, o, a, b, n, current_stream()); }
void nc_cuda_sub_f32(float* o, const float* a, const float* b, size_t n) { nc_cuda_binary_f32_ex(1, o, a, b, n, current_stream()); }
void nc_cuda_mul_f32(float* o, const float* a, const float* b, size_t n) { nc_cuda_binary_f32_ex(2, o, a, b, n, current_stream()); }
void nc_cuda_div_f32(float* o, const float* a, const float* b, size_t n) { nc_cuda_binary_f32_ex(3, o, a, b, n, current_stream()); }
void nc_cuda_add_scalar_f32(float* o, const float* a, float s, size_t n) { nc_cuda_scalar_f32_ex(0, o, a, s, n, current_stream()); }
void nc_cuda_mul_scalar_f32(float* o, const float* a, float s, size_t n) { nc_cuda_scalar_f32_ex(2, o, a, s, n, current_stream()); }
void nc_cuda_add_broadcast_batch_f32(float* o, const float* a, const float* b, size_t t, int inner) {
    nc_cuda_add_broadcast_batch_f32_ex(o, a, b, t, inner, current_stream());
}
int nc_cuda_sigmoid_f32_ex(float* out, const float* in, size_t n, void* stream) {
    return launch_ew<1>(out, in, nullptr, n, (cudaStream_t)stream, SigmoidF{}, "sigmoid", round_outputs(), PROF_ACTIVATION);
}
int nc_cuda_sigmoid_backward_f32_ex(float* gi, const float* go, const float* input, size_t n, void* stream) {
    return launch_ew<2>(gi, go, input, n, (cudaStream_t)stream, SigmoidBwdF{}, "sigmoid_backward", round_outputs(), PROF_ACTIVATION);
}
void nc_cuda_sigmoid_f32(float* o, const float* in, size_t n) { nc_cuda_sigmoid_f32_ex(o, in, n, current_stream()); }
void nc_cuda_relu_f32(float* o, const float* in, size_t n) { nc_cuda_relu_f32_ex(o, in, n, current_stream()); }
void nc_cuda_relu_backward_f32(float* gi, const float* go, const float* in, size_t n) {
    nc_cuda_relu_backward_f32_ex(gi, go, in, n, current_stream());
}
void nc_cuda_softmax_f32(float* o, const float* in, size_t b, size_t d) { nc_cuda_softmax_f32_ex(o, in, b, d, current_stream()); }

}  // extern "C"
