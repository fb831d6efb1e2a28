/*
 * nocta_cuda.h — the extern "C" nc_cuda_* kernel ABI of the B200 (sm_100a) training backend.
 *
 * This is the inner drop-in boundary: plain pointers and sizes, no C++ or framework types.
 * It replaces the reference's include/nocta/cuda/cuda_kernels.h (and the memory functions of
 * include/nocta/core/device.h); every entry point below cites the reference declaration it
 * stands in for, or says that it is new.
 *
 * Conventions
 *   - All pointers are device pointers unless the comment says "host".
 *   - Every op has an `_ex` form returning an int status (0 = ok, see NC_CUDA_* below) and
 *     taking the CUDA stream as `void*` (a cudaStream_t; NULL = legacy default stream).
 *   - The legacy `void` names of the reference are thin wrappers that launch on the library's
 *     current stream (nc_cuda_set_stream) and record the status in nc_cuda_last_status().
 *   - Nothing here falls back to the CPU: an unsupported shape is an error status.
 *   - Activations are f32; 4-D tensors are NCHW for the legacy names and NHWC (channels-last)
 *     for the *_nhwc names used by the host library's own device layout.
 *   - Contractions run on tcgen05 tensor cores in TF32 (math mode 0), TF32 with
 *     round-to-nearest operand conditioning (mode 1) or 3xTF32 (mode 2) when the shape can be
 *     tiled for TMA, otherwise on an FP32 SIMT kernel; see nc_cuda_set_math_mode.
 */
#ifndef NOCTA_CUDA_ABI_H
#define NOCTA_CUDA_ABI_H

#include <stddef.h>
#include <stdint.h>
#include <stdbool.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NC_CUDA_OK 0
#define NC_CUDA_ERR_ARG 1
#define NC_CUDA_ERR_RUNTIME 2
#define NC_CUDA_ERR_UNSUPPORTED 3
#define NC_CUDA_ERR_DEVICE_WAIT 4
#define NC_CUDA_ERR_LIMIT 5

/* math modes for the tensor-core contractions */
#define NC_CUDA_MATH_TF32 0       /* operands fed as stored; the tensor core drops low mantissa bits */
#define NC_CUDA_MATH_TF32_RNA 1   /* operands rounded to nearest TF32 in shared memory first */
#define NC_CUDA_MATH_3XTF32 2     /* hi/lo split, three MMAs per k-step: near-FP32 accuracy */
#define NC_CUDA_MATH_FP32_SIMT 3  /* force the FP32 CUDA-core kernels (no tensor cores) */

/* ---------------- runtime / device (reference: include/nocta/core/device.h:41-69,
 *                  src/cuda/cuda_device.cu:22-136) ---------------- */
bool  nc_cuda_available(void);
int   nc_cuda_device_count(void);
void  nc_cuda_set_device(int index);
void  nc_cuda_synchronize(void);
void  nc_cuda_init(void);
void  nc_cuda_cleanup(void);
void* nc_cuda_malloc(size_t size);                                  /* cuda_kernels.h:16 */
void  nc_cuda_free(void* ptr);                                      /* cuda_kernels.h:17 */
void  nc_cuda_memcpy_h2d(void* dst, const void* src, size_t size);  /* cuda_kernels.h:18 */
void  nc_cuda_memcpy_d2h(void* dst, const void* src, size_t size);  /* cuda_kernels.h:19 */
void  nc_cuda_memcpy_d2d(void* dst, const void* src, size_t size);  /* cuda_kernels.h:20 */
void  nc_cuda_memset(void* ptr, int value, size_t size);            /* cuda_kernels.h:21 */
/* new: device name / memory without the reference's struct (device.h:18-24) */
int   nc_cuda_device_props(int index, char* name256, size_t* total_bytes, size_t* free_bytes, int* sm_count);
/* new: stream control for the legacy names, async copies, pinned host memory, status */
void  nc_cuda_set_stream(void* stream);
void* nc_cuda_get_stream(void);
int   nc_cuda_memcpy_h2d_async(void* dst, const void* src_host, size_t size, void* stream);
int   nc_cuda_memcpy_d2h_async(void* dst_host, const void* src, size_t size, void* stream);
int   nc_cuda_memset_async(void* ptr, int value, size_t size, void* stream);
void* nc_cuda_host_alloc(size_t size);
void  nc_cuda_host_free(void* ptr);
int   nc_cuda_stream_synchronize(void* stream);
/* new: a second stream and events, for copies that overlap the compute stream (input prefetch).
 * The stream does not synchronise implicitly with the legacy default stream. */
void* nc_cuda_stream_create(void);
void  nc_cuda_stream_destroy(void* stream);
void* nc_cuda_event_create(void);
void  nc_cuda_event_destroy(void* event);
int   nc_cuda_event_record(void* event, void* stream);
int   nc_cuda_stream_wait_event(void* stream, void* event);
int   nc_cuda_event_synchronize(void* event);
/* new: an event that records time, and the device time between two such events that have completed */
void* nc_cuda_event_create_timed(void);
int   nc_cuda_event_elapsed_ms(void* start, void* stop, float* ms);
int   nc_cuda_last_status(void);
const char* nc_cuda_last_message(void);
void  nc_cuda_clear_status(void);
/* new: math mode for contractions (NC_CUDA_MATH_*); returns the previous mode.  The initial mode is TF32, or the
 * digit in the environment variable NOCTA_CUDA_MATH_MODE when the library is loaded. */
int   nc_cuda_set_math_mode(int mode);
int   nc_cuda_get_math_mode(void);
/* new: operand conditioning for NC_CUDA_MATH_TF32.  While on, the activation / gradient kernels (relu, gelu,
 * add/sub/mul, bias add, batchnorm, layernorm, loss gradients and their backward forms) round each value
 * they store to the nearest TF32 number, which removes the truncation bias of a tensor-core contraction
 * that reads it next.  Off by default (plain f32 results).  Returns the previous setting. */
int   nc_cuda_set_round_outputs(int on);
/* new: while on, nc_cuda_conv2d_forward_f32_ex (channels-last output, tensor-core or first-layer kernels)
 * also sums its output per channel, and a training-mode BatchNorm forward that is the library's very next
 * kernel-launching call on exactly that output takes those sums instead of reading the tensor again.  Any other
 * launch, copy or memset of the library in between cancels the offer; switching off afterwards does not.  The library
 * only sees its own calls: a caller that lets ANYTHING ELSE write that tensor between the two calls (its own kernel,
 * another library, a peer copy, a collective) must leave the switch off, or stale sums are used.  Off by default.
 * Returns the previous setting. */
int   nc_cuda_set_conv_stats(int on);
/* new: the backward counterpart of the above.  Announces that the gradient the NEXT nc_cuda_conv2d_backward_input_f32_ex call
 * writes is the upstream gradient of a training-mode BatchNorm with fused ReLU whose input is x (channels-last, C channels,
 * rows = N*H*W pixels; batch mean / biased variance as saved by the forward pass; gamma / beta may be NULL).  That call
 * consumes the announcement; if its kernel can (the halo-resident tensor-core kernel with the channels on M: TF32 mode, 3x3
 * stride 1, images of 24 rows or more, more than 96 channels, dense channels-last gradient of the same shape), it also sums per channel g and g * xhat with g zeroed where gamma * xhat + beta <= 0, and a
 * nc_cuda_batchnorm_backward_f32_ex(relu_recompute = 1) that is the library's very next launching call on exactly that
 * gradient and that x takes the sums instead of reading both tensors again.  Same hazard as above: nothing outside the
 * library may write the gradient between the two calls.  Results are the same sums in another order of addition. */
int   nc_cuda_offer_batchnorm_backward_sums_f32(const float* x, const float* mean, const float* var, const float* gamma,
                                                const float* beta, double eps, int C, long long rows);
/* new: while off, announcements are ignored (every BatchNorm backward does its own reduction).  On by default.
 * Returns the previous setting. */
int   nc_cuda_set_batchnorm_backward_fold(int on);
/* new: how many BatchNorm backward calls have taken folded sums so far (bookkeeping for tests and benches) */
unsigned long long nc_cuda_batchnorm_backward_fold_count(void);
/* new: reads and clears the device-side error word set when a bounded in-kernel wait expires */
unsigned int nc_cuda_device_error_word(void);
/* new: number of kernels this library has launched since the last reset (bookkeeping for benches) */
unsigned long long nc_cuda_launch_count(void);
void  nc_cuda_reset_launch_count(void);

/* new: device timing per kernel family (CUDA events on the launching stream).  begin() arms it; every call of a profiled
 * entry point is then bracketed by an event pair and filed under one category with its algorithmic work: FLOPs
 * (2*M*N*K of the logical contraction) for the tensor-core families, which are timed per kernel launch (conv_fwd, conv_dx,
 * conv_dw, gemm_nt = Linear forward, gemm_nn = Linear dX, gemm_tn = Linear dW, gemm_tt), and bytes that must cross HBM for
 * the memory-bound ones, which are timed per outermost entry-point call (conv_first, batchnorm, layernorm, activation,
 * elementwise, maxpool, loss, sgd, adam, reduce, relayout).  end() disarms and waits for the last timed call; read()
 * then returns the summed device time, the number of timed calls and their summed work for one category.  The events cost
 * a few microseconds of host time per call: measure throughput with profiling off. */
int nc_cuda_profile_begin(void);
int nc_cuda_profile_end(void);
int nc_cuda_profile_categories(void);
const char* nc_cuda_profile_category_name(int category);
int nc_cuda_profile_read(int category, double* total_ms, unsigned long long* calls, double* work);

/* ---------------- elementwise (reference: cuda_kernels.h:26-49, src/cuda/cuda_elementwise.cu) ---- */
void nc_cuda_fill_f32(float* data, float value, size_t n);                        /* :26 */
void nc_cuda_copy_f32(float* dst, const float* src, size_t n);                    /* :28 */
void nc_cuda_add_f32(float* out, const float* a, const float* b, size_t n);       /* :32 */
void nc_cuda_sub_f32(float* out, const float* a, const float* b, size_t n);       /* :33 */
void nc_cuda_mul_f32(float* out, const float* a, const float* b, size_t n);       /* :34 */
void nc_cuda_div_f32(float* out, const float* a, const float* b, size_t n);       /* :35 */
void nc_cuda_add_scalar_f32(float* out, const float* a, float scalar, size_t n);  /* :37 */
void nc_cuda_mul_scalar_f32(float* out, const float* a, float scalar, size_t n);  /* :38 */
void nc_cuda_add_broadcast_batch_f32(float* out, const float* a, const float* b,
                                     size_t total_elements, int inner_dim);       /* :48-49 */
int nc_cuda_fill_f32_ex(float* data, float value, size_t n, void* stream);
int nc_cuda_copy_f32_ex(float* dst, const float* src, size_t n, void* stream);
/* op: 0 add, 1 sub, 2 mul, 3 div */
int nc_cuda_binary_f32_ex(int op, float* out, const float* a, const float* b, size_t n, void* stream);
int nc_cuda_scalar_f32_ex(int op, float* out, const float* a, float scalar, size_t n, void* stream);
int nc_cuda_add_broadcast_batch_f32_ex(float* out, const float* a, const float* b,
                                       size_t total_elements, int inner_dim, void* stream);
/* new: generic strided gather copy (up to 4 dims) — tensor_contiguous on device
 * (reference does this on the host: src/core/tensor.c:559-575).  dst is dense row-major. */
int nc_cuda_strided_copy_f32_ex(float* dst, const float* src, const size_t shape[4],
                                const size_t src_strides[4], void* stream);
/* new: NCHW <-> NHWC relayout (batched 2-D transpose through shared memory) */
int nc_cuda_nchw_to_nhwc_f32_ex(float* dst, const float* src, int N, int C, int HW, int round_tf32, void* stream);
int nc_cuda_nhwc_to_nchw_f32_ex(float* dst, const float* src, int N, int C, int HW, void* stream);
/* new: round every element to the nearest TF32 value (operand conditioning for math mode 0) */
int nc_cuda_round_tf32_f32_ex(float* dst, const float* src, size_t n, void* stream);

/* ---------------- activations (reference: cuda_kernels.h:54-58, src/cuda/cuda_activation.cu;
 *                  CPU semantics src/ops/activation.c:33-70,195-225,289-310) ---------------- */
void nc_cuda_relu_f32(float* out, const float* in, size_t n);                                            /* :54 */
void nc_cuda_relu_backward_f32(float* grad_in, const float* grad_out, const float* input, size_t n);     /* :55 */
void nc_cuda_softmax_f32(float* out, const float* in, size_t batch, size_t dim);                         /* :58 */
int nc_cuda_relu_f32_ex(float* out, const float* in, size_t n, void* stream);
int nc_cuda_relu_backward_f32_ex(float* grad_in, const float* grad_out, const float* input, size_t n, void* stream);
void nc_cuda_sigmoid_f32(float* out, const float* in, size_t n);                      /* :56 */
int nc_cuda_sigmoid_f32_ex(float* out, const float* in, size_t n, void* stream);
int nc_cuda_sigmoid_backward_f32_ex(float* grad_in, const float* grad_out, const float* input, size_t n, void* stream);
int nc_cuda_softmax_f32_ex(float* out, const float* in, size_t batch, size_t dim, void* stream);
/* new (the reference has GELU forward on the CPU only and no backward at all) */
int nc_cuda_gelu_f32_ex(float* out, const float* in, size_t n, void* stream);
int nc_cuda_gelu_backward_f32_ex(float* grad_in, const float* grad_out, const float* input, size_t n, void* stream);

/* ---------------- matmul (reference: cuda_kernels.h:63-66, src/cuda/cuda_matmul.cu:27-68) -------
 * Row-major C(M,N) = alpha * op(A) * op(B) + beta * C, op = transpose when the flag is set;
 * A is (M,K) or (K,M) when transposed, B is (K,N) or (N,K) when transposed. */
void nc_cuda_matmul_f32(float* C, const float* A, const float* B, int M, int N, int K,
                        float alpha, float beta, int transA, int transB);
/* new: explicit leading dimensions, optional bias (length N, added to every row) and
 * optional column sums of op(A)^T... see nc_cuda_linear_* for the fused training forms. */
int nc_cuda_matmul_f32_ex(float* C, int ldc, const float* A, int lda, const float* B, int ldb,
                          int M, int N, int K, float alpha, float beta, int transA, int transB,
                          const float* bias, void* stream);
/* new: the three GEMMs of a Linear layer (reference host code: src/nn/linear.c:45-152).
 *   forward : y(B,out) = x(B,in) * W(out,in)^T + bias
 *   backward: dx(B,in) = dy * W        (skipped when dx == NULL)
 *             dW(out,in) = dy^T * x
 *             db(out)    = column sums of dy (skipped when db == NULL) */
int nc_cuda_linear_forward_f32_ex(float* y, const float* x, const float* W, const float* bias,
                                  int batch, int in_f, int out_f, void* stream);
int nc_cuda_linear_backward_f32_ex(float* dx, float* dW, float* db, const float* dy, const float* x,
                                   const float* W, int batch, int in_f, int out_f, void* stream);

/* ---------------- reductions (reference: cuda_kernels.h:76-86, src/cuda/cuda_reduction.cu) ------- */
float  nc_cuda_sum_f32(const float* data, size_t n);        /* :76 */
size_t nc_cuda_argmax_f32(const float* data, size_t n);     /* :78 */
void   nc_cuda_sum_axis_f32(float* out, const float* in, size_t outer, size_t reduce_dim, size_t inner); /* :83-84 */
int nc_cuda_sum_axis_f32_ex(float* out, const float* in, size_t outer, size_t reduce_dim, size_t inner, void* stream);
/* new: per-row argmax (int64 out) for accuracy bookkeeping (CPU: src/ops/reduction.c:473-513) */
int nc_cuda_argmax_rows_f32_ex(int64_t* out, const float* in, size_t rows, size_t cols, void* stream);

/* ---------------- convolution (reference: cuda_kernels.h:91-112, src/cuda/cuda_conv.cu:148-372;
 *                  CPU semantics src/nn/conv.c:118-375,381-586).  NCHW, weight (C_out,C_in,kH,kW). */
void nc_cuda_conv2d_forward_f32(float* output, const float* input, const float* weight, const float* bias,
                                int N, int C_in, int H, int W, int C_out, int kH, int kW,
                                int stride, int padding);                                        /* :95-102 */
void nc_cuda_conv2d_backward_input_f32(float* grad_input, const float* grad_output, const float* weight,
                                       int N, int C_in, int H, int W, int C_out, int kH, int kW,
                                       int stride, int padding);                                 /* :105-106 */
/* unlike the reference (beta = 1, cuda_conv.cu:294-317) grad_weight is overwritten, not accumulated */
void nc_cuda_conv2d_backward_weight_f32(float* grad_weight, const float* grad_output, const float* input,
                                        int N, int C_in, int H, int W, int C_out, int kH, int kW,
                                        int stride, int padding);                                /* :108-109 */
void nc_cuda_conv2d_backward_bias_f32(float* grad_bias, const float* grad_output,
                                      int N, int C_out, int H_out, int W_out);                   /* :111-112 */
/* new: stream/status forms with explicit element strides for the activation tensors, so the same
 * entry serves NCHW (strides C*H*W, H*W, W, 1) and channels-last (H*W*C, 1, W*C, C) storage.
 * xs/ys = strides of input / output in elements, order (n, c, h, w).  Weight is always dense
 * (C_out, C_in, kH, kW). */
int nc_cuda_conv2d_forward_f32_ex(float* output, const size_t ys[4], const float* input, const size_t xs[4],
                                  const float* weight, const float* bias,
                                  int N, int C_in, int H, int W, int C_out, int kH, int kW,
                                  int stride, int padding, void* stream);
int nc_cuda_conv2d_backward_input_f32_ex(float* grad_input, const size_t xs[4],
                                         const float* grad_output, const size_t ys[4], const float* weight,
                                         int N, int C_in, int H, int W, int C_out, int kH, int kW,
                                         int stride, int padding, void* stream);
/* grad_bias may be NULL */
int nc_cuda_conv2d_backward_weight_f32_ex(float* grad_weight, float* grad_bias,
                                          const float* grad_output, const size_t ys[4],
                                          const float* input, const size_t xs[4],
                                          int N, int C_in, int H, int W, int C_out, int kH, int kW,
                                          int stride, int padding, void* stream);

/* new: all gradients of one NCHW convolution in one call (each of dx, dW, db may be NULL).  When the
 * shape tiles for the tensor-core kernels (stride 1, channel counts multiples of 32) the activations are
 * re-laid out channels-last ONCE in library scratch and shared by the dX and dW kernels; otherwise the
 * FP32 SIMT kernels read the NCHW data directly.  The three legacy backward names call this. */
int nc_cuda_conv2d_backward_f32_ex(float* grad_input, float* grad_weight, float* grad_bias,
                                   const float* grad_output, const float* input, const float* weight,
                                   int N, int C_in, int H, int W, int C_out, int kH, int kW,
                                   int stride, int padding, void* stream);

/* ---------------- max pooling (reference: cuda_kernels.h:114-119, src/cuda/cuda_conv.cu:378-500;
 *                  CPU semantics src/nn/conv.c:672-849: init -1e30, strict >, first maximum wins) --- */
void nc_cuda_maxpool2d_forward_f32(float* output, const float* input, int N, int C, int H, int W,
                                   int kH, int kW, int stride);                                   /* :114-116 */
void nc_cuda_maxpool2d_backward_f32(float* grad_input, const float* grad_output, const float* input,
                                    const float* output, int N, int C, int H, int W,
                                    int kH, int kW, int stride);                                  /* :118-119 */
/* new: forward that also records the window offset (kh*kW+kw) of the first maximum as uint8, and the
 * backward that scatters by it.  layout: 0 = NCHW, 1 = NHWC.  argmax may be NULL in the forward. */
int nc_cuda_maxpool2d_forward_idx_f32_ex(float* output, uint8_t* argmax, const float* input,
                                         int N, int C, int H, int W, int k, int stride, int layout, void* stream);
int nc_cuda_maxpool2d_backward_idx_f32_ex(float* grad_input, const float* grad_output, const uint8_t* argmax,
                                          int N, int C, int H, int W, int k, int stride, int layout, void* stream);

/* ---------------- batch norm (reference: cuda_kernels.h:124-147, src/cuda/cuda_batchnorm.cu;
 *                  CPU semantics src/nn/batchnorm.c:43-165,171-371: biased batch variance for the
 *                  normalisation, UNBIASED variance into running_var) ---------------------------- */
void nc_cuda_batchnorm_forward_f32(float* output, const float* input, const float* gamma, const float* beta,
                                   float* running_mean, float* running_var, float* save_mean, float* save_var,
                                   int N, int C, int spatial, float momentum, float eps, bool training); /* :124-135 */
void nc_cuda_batchnorm_backward_f32(float* grad_input, float* grad_gamma, float* grad_beta,
                                    const float* grad_output, const float* input, const float* gamma,
                                    const float* save_mean, const float* save_var,
                                    int N, int C, int spatial, float eps);                               /* :137-147 */
/* new: layout 0 = NCHW (N, C, spatial), 1 = NHWC (N*spatial, C).  save_var holds the biased batch
 * variance (as on the reference CPU path).  relu != 0 fuses max(0, .) into the forward output; the
 * backward then masks grad_output where that output was <= 0, either by reading it (`relu_out` = the
 * forward output y) or, with relu_out == NULL and relu_recompute != 0, by re-evaluating
 * gamma * x_hat + beta from x (`relu_beta` = the forward beta, may be NULL), which reads no extra tensor. */
int nc_cuda_batchnorm_forward_f32_ex(float* output, const float* input, const float* gamma, const float* beta,
                                     float* running_mean, float* running_var, float* save_mean, float* save_var,
                                     int N, int C, int spatial, double momentum, double eps, int training,
                                     int layout, int relu, void* stream);
int nc_cuda_batchnorm_backward_f32_ex(float* grad_input, float* grad_gamma, float* grad_beta,
                                      const float* grad_output, const float* input, const float* gamma,
                                      const float* save_mean, const float* save_var, const float* relu_out,
                                      const float* relu_beta, int relu_recompute,
                                      int N, int C, int spatial, double eps, int layout, void* stream);

/* new: BatchNorm + ReLU + 2x2 stride-2 max-pool as one pass each way, channels-last only (x is (N, H, W, C) in
 * memory, C % 4 == 0, H and W even).  Forward writes the pooled tensor (N, H/2, W/2, C) and one window offset
 * (kh * 2 + kw, first maximum wins) per pooled element; the full-resolution activation is never stored.
 * Backward takes the pooled gradient and those offsets and returns dx (N, H, W, C), dgamma, dbeta.
 * Results equal nc_cuda_batchnorm_forward_f32_ex(relu = 1) followed by nc_cuda_maxpool2d_forward_idx_f32_ex. */
int nc_cuda_batchnorm_relu_maxpool2_forward_f32_ex(float* pooled, uint8_t* argmax, const float* x, const float* gamma,
                                                   const float* beta, float* running_mean, float* running_var,
                                                   float* save_mean, float* save_var, int N, int C, int H, int W,
                                                   double momentum, double eps, int training, void* stream);
int nc_cuda_batchnorm_relu_maxpool2_backward_f32_ex(float* grad_input, float* grad_gamma, float* grad_beta,
                                                    const float* grad_pooled, const uint8_t* argmax, const float* x,
                                                    const float* gamma, const float* beta, const float* save_mean,
                                                    const float* save_var, int N, int C, int H, int W, double eps,
                                                    void* stream);

/* ---------------- layer norm (new; CPU semantics src/nn/batchnorm.c:600-702,946-1026) ---------- */
int nc_cuda_layernorm_forward_f32_ex(float* output, const float* input, const float* gamma, const float* beta,
                                     size_t rows, size_t cols, double eps, void* stream);
int nc_cuda_layernorm_backward_f32_ex(float* grad_input, float* grad_gamma, float* grad_beta,
                                      const float* grad_output, const float* input, const float* gamma,
                                      size_t rows, size_t cols, double eps, void* stream);

/* ---------------- losses (reference: cuda_kernels.h:152-162, src/cuda/cuda_loss.cu;
 *                  CPU semantics src/ops/loss.c:33-137,176-351) ---------------------------------- */
void nc_cuda_cross_entropy_forward_f32(float* loss, const float* logits, const int64_t* targets, int N, int C);         /* :152-156 */
void nc_cuda_cross_entropy_backward_f32(float* grad_logits, const float* logits, const int64_t* targets, int N, int C);  /* :158-162 */
/* new: one pass writes the mean loss and, when grad_logits != NULL, (softmax - onehot) * grad_scale / N.
 * Out-of-range labels contribute nothing, as on the CPU path (loss.c:278-281, 86-91). */
int nc_cuda_cross_entropy_fused_f32_ex(float* loss, float* grad_logits, const float* logits,
                                       const int64_t* targets, int N, int C, float grad_scale, void* stream);
/* No counterpart in the reference.  Same computation and same bits as nc_cuda_cross_entropy_fused_f32_ex,
 * for callers that must not trigger a device allocation (all memory already handed to their own arena;
 * a collective in flight on another stream that an allocation's device-wide synchronisation would stall):
 * the partial sums live in a fixed array inside the library, so no allocating routine is ever called.
 * At most NC_CUDA_CE_STATIC_MAX_ROWS rows per call (more: status 5, "exceeds a stated fixed capacity", nothing is
 * launched).  The first call on each device resolves the array's address; make that call before beginning a stream
 * capture.  All calls on a device share the array: calls that may run concurrently race and must be serialised by the
 * caller.  The resolved address is kept per device ordinal for the life of the process, so a process that resets a
 * device must reload the library before calling again; `stream` must belong to the device that is current at the
 * call (it is not checked). */
#define NC_CUDA_CE_STATIC_MAX_ROWS 4096
int nc_cuda_cross_entropy_fused_static_f32_ex(float* loss, float* grad_logits, const float* logits,
                                              const int64_t* targets, int N, int C, float grad_scale, void* stream);
/* new: mean squared error; grad_pred = 2*(p-t)*grad_scale/numel, grad_target = -grad_pred (either may be NULL) */
int nc_cuda_mse_fused_f32_ex(float* loss, float* grad_pred, float* grad_target, const float* pred,
                             const float* target, size_t n, float grad_scale, void* stream);

/* ---------------- optimizers (reference: cuda_kernels.h:41-45, src/cuda/cuda_elementwise.cu:195-240;
 *                  CPU semantics src/optim/sgd.c:13-115, src/optim/adam.c:11-75) ------------------ */
void nc_cuda_sgd_step_f32(float* param, const float* grad, float lr, size_t n);                     /* :41 */
void nc_cuda_sgd_momentum_f32(float* param, float* velocity, const float* grad, float lr, float momentum,
                              float dampening, int nesterov, size_t n);                             /* :43-45 */
/* new: full CPU-path semantics. first_step != 0 -> v = g (sgd.c:74-78). weight_decay folds g += wd*p and,
 * like the CPU path (sgd.c:24-30), writes the decayed gradient back into `grad`.
 * grad_scale multiplies the gradient first (1/world for data parallel). velocity may be NULL (momentum 0). */
int nc_cuda_sgd_update_f32_ex(float* param, float* velocity, float* grad, double lr, double momentum,
                              double dampening, double weight_decay, int nesterov, int first_step,
                              double grad_scale, size_t n, void* stream);
/* new: Adam / AdamW (decoupled decay) with bias corrections computed on the host in double:
 * bias_corr1 = 1 - beta1^t, bias_corr2 = 1 - beta2^t.  v_max may be NULL (no AMSGrad). */
int nc_cuda_adam_update_f32_ex(float* param, float* m, float* v, float* v_max, const float* grad,
                               double lr, double beta1, double beta2, double eps, double weight_decay,
                               double bias_corr1, double bias_corr2, double grad_scale, size_t n, void* stream);
/* new: the same updates for `count` parameter tensors in one launch (per 48 tensors).  The four tables are HOST
 * arrays of device pointers, read during the call; every tensor uses the same hyper-parameters. */
int nc_cuda_sgd_update_multi_f32_ex(int count, float* const* params, float* const* velocities, float* const* grads,
                                    const size_t* numel, double lr, double momentum, double dampening,
                                    double weight_decay, int nesterov, int first_step, double grad_scale, void* stream);
int nc_cuda_adam_update_multi_f32_ex(int count, float* const* params, float* const* m, float* const* v,
                                     float* const* v_max, float* const* grads, const size_t* numel, double lr,
                                     double beta1, double beta2, double eps, double weight_decay, double bias_corr1,
                                     double bias_corr2, double grad_scale, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NOCTA_CUDA_ABI_H */
