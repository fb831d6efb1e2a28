// Shared helpers for the sm_100a kernel library behind the nc_cuda_* C ABI.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>
#include <stddef.h>
#include <stdio.h>

// Status codes returned by every *_ex entry point (0 = success).
enum {
    NC_CUDA_OK = 0,
    NC_CUDA_ERR_ARG = 1,        // bad pointer / size / unsupported shape
    NC_CUDA_ERR_RUNTIME = 2,    // a CUDA runtime call or launch failed
    NC_CUDA_ERR_UNSUPPORTED = 3,// shape not covered by this kernel family
    NC_CUDA_ERR_DEVICE_WAIT = 4,// a bounded in-kernel wait gave up (see nc_cuda_device_error_word)
    NC_CUDA_ERR_LIMIT = 5       // request exceeds a stated fixed capacity
};

namespace ncc {

// Last status + message seen by this process (single host thread drives one device).
int  set_status(int code, const char* fmt, ...);
int  last_status();
const char* last_message();

// The stream the legacy void entry points launch on (default: the legacy default stream).
cudaStream_t current_stream();

// Device-side scratch owned by the library (grown on demand, freed at nc_cuda_cleanup).
// `slot` separates users whose lifetimes overlap inside one entry point.
void* scratch(int slot, size_t bytes, cudaStream_t st);

// Per-channel output statistics offered by a forward convolution to the BatchNorm that follows (runtime.cu).
// partial[slab][C][2] doubles: (sum, sum of squares) of the slab's pixels.
int set_conv_stats(int on);
bool conv_stats_wanted();
double* conv_stats_buffer(size_t slabs, int C, cudaStream_t st);
void conv_stats_publish(const float* y, int C, long long rows, int slabs, double* partial);
bool conv_stats_take(const float* x, int C, long long rows, double** partial, int* slabs);

// Backward counterpart: the input-gradient convolution whose output is the upstream gradient of a BatchNorm(+ReLU)
// can sum, per channel, what that BatchNorm's backward pass needs (sum of g and of g * xhat, g zeroed where the ReLU
// was inactive) while it stores the gradient, so the BatchNorm backward does not read both tensors once more.
// The caller announces the BatchNorm (nc_cuda_offer_batchnorm_backward_sums_f32); the next input-gradient call consumes
// the announcement, and if its kernel could honour it publishes partial[slab][C][2]; a BatchNorm backward that is the
// very next launching call on exactly that gradient takes them.
struct BnFold {
    const float* x;      // the BatchNorm's input (channels-last, same shape as the gradient)
    const float* mean;   // batch mean and (biased) variance per channel
    const float* var;
    const float* gamma;  // may be null (1)
    const float* beta;   // may be null (0)
    float eps;
    int C;
    long long rows;      // N * H * W
};
void bn_fold_announce(const BnFold& f);
void bn_fold_enter();                 // input-gradient entry point: takes the pending announcement (if any) for this call
void bn_fold_leave();
const BnFold* bn_fold_active();       // non-null inside that entry point while an announcement is being served
double* bn_fold_buffer(size_t slabs, int C, cudaStream_t st);
void bn_fold_publish(const float* dy, int slabs, double* partial);
bool bn_fold_take(const float* dy, const BnFold& want, double** partial, int* slabs);
extern unsigned long long g_bn_fold_hits;

// Device-resident error word the tensor-core kernels set when a bounded wait expires.
unsigned int* device_error_word();

int sm_count();

// NC_CUDA_MATH_* mode selected with nc_cuda_set_math_mode.
int math_mode();

// When switched on (nc_cuda_set_round_outputs), the activation / gradient kernels round what they
// write to the nearest TF32 value, so a tensor-core contraction that consumes it (and drops the low
// 13 mantissa bits of its operands) reads exactly representable data and its error stays zero-mean.
// Costs one cvt per element in kernels that wait on memory.  Off by default: results are plain f32.
bool round_outputs();
int set_round_outputs(int on);

// Number of kernels launched by this library (bench bookkeeping).
extern unsigned long long g_launches;
// g_epoch also advances when device memory is written by a copy or a memset of this library: together they
// stamp "nothing this library does has touched device memory since".
extern unsigned long long g_epoch;
#define NCC_COUNT_LAUNCH() (++ncc::g_launches, ++ncc::g_epoch)

// ---- device timing per kernel family (nc_cuda_profile_begin / _read) ----
// While armed, every profiled call is bracketed by a pair of CUDA events on its launching stream and filed under one
// category together with its algorithmic work: FLOPs (2 * M * N * K of the logical contraction) for the tensor-core
// families, bytes that must cross HBM for the memory-bound ones.  Tensor-core kernels are timed per launch; the
// memory-bound families per entry point (all launches of one call), outermost call only.
enum {
    PROF_CONV_FWD = 0, PROF_CONV_DX, PROF_CONV_DW,         // tcgen05 convolutions: forward, input gradient, weight gradient
    PROF_GEMM_NT, PROF_GEMM_NN, PROF_GEMM_TN, PROF_GEMM_TT,  // tcgen05 GEMM by operand layout (Linear forward / dX / dW / other)
    PROF_CONV_FIRST,                                        // CUDA-core kernels of the 3-channel input layer
    PROF_BATCHNORM, PROF_LAYERNORM, PROF_ACTIVATION, PROF_ELEMENTWISE, PROF_MAXPOOL, PROF_LOSS, PROF_SGD, PROF_ADAM,
    PROF_REDUCE, PROF_RELAYOUT,
    PROF_CATEGORIES
};
bool prof_armed();
// Category the next tensor-core launch is filed under (set by the entry point that knows which pass it is).
void prof_set_role(int cat);
int prof_role();
struct ProfScope {
    int slot;
    cudaStream_t st;
    bool outer;
    // kernel_level: a single tensor-core launch (always recorded); otherwise an entry point (recorded when outermost)
    ProfScope(int cat, double work, cudaStream_t stream, bool kernel_level = false);
    ~ProfScope();
    void add_work(double more);   // for work only known after the scope opened
};

// out[c] = sum over rows of in[r][c] for a dense row-major (rows x cols) matrix; two-stage,
// double accumulation, fixed combine order (defined in pool_norm.cu).
int column_sums(float* out, const float* in, size_t rows, int cols, cudaStream_t st);

inline int launch_status(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_status(NC_CUDA_ERR_RUNTIME, "%s: %s", what, cudaGetErrorString(e));
    return NC_CUDA_OK;
}

#define NCC_TRY(expr)                                                                      \
    do {                                                                                   \
        cudaError_t _e = (expr);                                                           \
        if (_e != cudaSuccess)                                                             \
            return ncc::set_status(NC_CUDA_ERR_RUNTIME, "%s: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

#define NCC_REQUIRE(cond, ...)                                                             \
    do {                                                                                   \
        if (!(cond)) return ncc::set_status(NC_CUDA_ERR_ARG, __VA_ARGS__);                 \
    } while (0)

static inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Grid size for grid-stride kernels: a multiple of the SM count, capped by the work.
inline int grid_for(long long work_items, int threads, int ctas_per_sm = 8) {
    long long need = (work_items + threads - 1) / threads;
    long long cap = (long long)sm_count() * ctas_per_sm;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

// ---------------- device helpers ----------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum of a double; result valid in every thread. `sh` must hold 32 doubles.
__device__ __forceinline__ double block_sum(double v, double* sh) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    double r = (lane < nw) ? sh[lane] : 0.0;
    r = warp_sum(r);
    return r;
}

// Round an f32 to the nearest TF32 value (ties away), keeping it in an f32 container.
__device__ __forceinline__ float round_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

}  // namespace ncc
