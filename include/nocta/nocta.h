/*
 * nocta/nocta.h — the nc_* C API of the B200 training backend (host side).
 *
 * Source-compatible with the reference library's public API for the training path: same type
 * names, struct field order (applications read t->shape, t->grad, m->params, opt->t directly),
 * function names, argument meaning and error behaviour (NULL + nc_last_error, never abort).
 * Reference declarations: include/nocta/core/{dtype,error,memory,device,tensor}.h,
 * autograd/{node,backward}.h, ops/{arithmetic,matmul,activation,reduction,loss}.h,
 * nn/{module,linear,conv,batchnorm,dropout}.h, optim/{optimizer,sgd,adam}.h.
 *
 * Differences a caller can observe:
 *   - Arithmetic runs on the CUDA device only.  nc_init() makes CUDA the default device, so
 *     tensors created afterwards live in device memory; an op given a CPU-resident tensor moves it
 *     to the device first (NC_ERR_DEVICE when there is no GPU): nothing is ever computed on the host.
 *   - Element accessors (the nc_tensor_get / nc_tensor_set family) work on device tensors by copying the one element.
 *   - 4-D activations produced by conv / batchnorm / relu / maxpool on the device are stored
 *     channels-last; their shape is still (N,C,H,W) and their strides say so.
 *   - nc_flatten, nc_tensor_reshape-of-an-activation (through nc_flatten) and nc_gelu take part
 *     in autograd (the reference registers no node for them).
 *   - nc_tensor_zero_grad_ / nc_optimizer_zero_grad DROP a gradient that a backward pass wrote (t->grad
 *     becomes NULL until the next backward, which takes over its first contribution instead of adding it
 *     to zeros); optimizers skip a parameter without a gradient.  Gradients no backward pass ever wrote
 *     (BatchNorm running statistics) are zeroed in place and updated as in the reference.
 *   - nc_node carries extra trailing fields; code that only touches the reference's fields is
 *     unaffected because nodes are always allocated by nc_node_create.
 */
#ifndef NOCTA_B200_NOCTA_H
#define NOCTA_B200_NOCTA_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NOCTA_VERSION "0.6.0-b200"
#define NOCTA_VERSION_MAJOR 0
#define NOCTA_VERSION_MINOR 6
#define NOCTA_VERSION_PATCH 0

/* ------------------------------------------------------------------ dtypes (core/dtype.h) */
typedef enum { NC_F32, NC_F64, NC_I32, NC_I64, NC_U8, NC_BOOL, NC_DTYPE_COUNT } nc_dtype;
size_t nc_dtype_sizeof(nc_dtype dtype);
const char* nc_dtype_to_string(nc_dtype dtype);

/* ------------------------------------------------------------------ errors (core/error.h:6-55) */
typedef enum {
    NC_OK = 0,
    NC_ERR_NULL_PTR,
    NC_ERR_ALLOC,
    NC_ERR_SHAPE_MISMATCH,
    NC_ERR_DTYPE_MISMATCH,
    NC_ERR_INDEX_OUT_OF_BOUNDS,
    NC_ERR_INVALID_AXIS,
    NC_ERR_INVALID_SHAPE,
    NC_ERR_INVALID_DTYPE,
    NC_ERR_NOT_CONTIGUOUS,
    NC_ERR_NO_GRAD,
    NC_ERR_GRAPH_CYCLE,
    NC_ERR_IO,
    NC_ERR_UNKNOWN,
    NC_ERR_DEVICE /* new: tensor is not on the CUDA device, or a kernel call failed */
} nc_error;
extern nc_error nc_last_error;
extern char nc_error_context[256];
const char* nc_error_string(nc_error err);
#define NC_SET_ERROR(err, ...)                                              \
    do {                                                                    \
        nc_last_error = (err);                                              \
        snprintf(nc_error_context, sizeof(nc_error_context), __VA_ARGS__);  \
    } while (0)
static inline nc_error nc_get_error(void) { return nc_last_error; }
static inline void nc_clear_error(void) { nc_last_error = NC_OK; nc_error_context[0] = '\0'; }

/* ------------------------------------------------------------------ devices (core/device.h) */
typedef enum { NC_DEVICE_CPU = 0, NC_DEVICE_CUDA = 1 } nc_device_type;
typedef struct {
    nc_device_type type;
    int index;
    char name[256];
    size_t total_memory;
    size_t free_memory;
} nc_device_info;
void nc_set_default_device(nc_device_type type);
nc_device_type nc_get_default_device(void);
nc_device_info nc_cuda_device_info(int device_index);
/* the nc_cuda_* runtime entry points (nc_cuda_available, nc_cuda_init, ...) are declared in nocta_cuda.h */

/* ------------------------------------------------------------------ memory (core/memory.h) */
void* nc_alloc(size_t size);
void* nc_calloc(size_t count, size_t size);
void* nc_realloc(void* ptr, size_t old_size, size_t new_size);
void nc_free(void* ptr);
typedef struct {
    size_t total_allocated, total_freed, current_usage, peak_usage, allocation_count, free_count;
} nc_mem_stats;
nc_mem_stats nc_memory_stats(void);
void nc_memory_stats_reset(void);
void nc_memory_report(void);
/* new: device pool statistics (bytes held by the caching device allocator / handed out) */
typedef struct {
    size_t bytes_reserved, bytes_in_use, peak_in_use, cuda_mallocs, pool_hits;
} nc_device_pool_stats;
nc_device_pool_stats nc_device_pool_get_stats(void);
void nc_device_pool_release(void); /* return cached blocks to the driver */
/* new: cap on the bytes the pool may hold from the driver (0 = no cap, the default).  An allocation that would exceed it
 * first returns the cached blocks, then fails like a refused driver allocation: NULL + NC_ERR_ALLOC, nothing leaked. */
void nc_device_pool_set_limit(size_t bytes);
size_t nc_device_pool_get_limit(void);

typedef struct {
    void* data;      /* CPU pointer (NULL while the bytes live on the device only) */
    void* cuda_data; /* device pointer (NULL while on the CPU only) */
    size_t size;     /* bytes */
    int refcount;
    nc_device_type device;
} nc_storage;
nc_storage* nc_storage_create(size_t size);
nc_storage* nc_storage_create_on(size_t size, nc_device_type device);
nc_storage* nc_storage_retain(nc_storage* storage);
void nc_storage_release(nc_storage* storage);
int nc_storage_refcount(const nc_storage* storage);
void nc_storage_to_device(nc_storage* s, nc_device_type target);
void nc_storage_ensure_on(nc_storage* s, nc_device_type target);
void* nc_storage_data_ptr(nc_storage* s);
void nc_storage_sync_to_cpu(nc_storage* s);

/* ------------------------------------------------------------------ tensors (core/tensor.h) */
#define NC_MAX_DIMS 8
typedef struct nc_node nc_node;
typedef struct nc_tensor {
    nc_storage* storage;
    size_t offset; /* elements */
    size_t ndim;
    size_t shape[NC_MAX_DIMS];
    size_t strides[NC_MAX_DIMS]; /* elements */
    size_t numel;
    nc_dtype dtype;
    bool requires_grad;
    struct nc_tensor* grad;
    nc_node* grad_fn;
    bool is_leaf;
    bool is_contiguous;
    bool is_reachable;
} nc_tensor;

nc_tensor* nc_tensor_empty(const size_t* shape, size_t ndim, nc_dtype dtype);
nc_tensor* nc_tensor_zeros(const size_t* shape, size_t ndim, nc_dtype dtype);
nc_tensor* nc_tensor_ones(const size_t* shape, size_t ndim, nc_dtype dtype);
nc_tensor* nc_tensor_full(const size_t* shape, size_t ndim, nc_dtype dtype, double value);
nc_tensor* nc_tensor_from_data(const void* data, const size_t* shape, size_t ndim, nc_dtype dtype);
nc_tensor* nc_tensor_scalar(double value, nc_dtype dtype);
nc_tensor* nc_tensor_arange(double start, double end, double step, nc_dtype dtype);
nc_tensor* nc_tensor_rand(const size_t* shape, size_t ndim, nc_dtype dtype);
nc_tensor* nc_tensor_randn(const size_t* shape, size_t ndim, nc_dtype dtype);
nc_tensor* nc_tensor_clone(const nc_tensor* r);
void nc_tensor_free(nc_tensor* t);
/* new: seed for nc_tensor_rand/randn and the module initialisers (the reference seeds from time()) */
void nc_manual_seed(uint64_t seed);

static inline size_t nc_tensor_numel(const nc_tensor* t) { return t ? t->numel : 0; }
static inline size_t nc_tensor_ndim(const nc_tensor* t) { return t ? t->ndim : 0; }
static inline size_t nc_tensor_shape(const nc_tensor* t, size_t dim) { return (t && dim < t->ndim) ? t->shape[dim] : 0; }
static inline size_t nc_tensor_stride(const nc_tensor* t, size_t dim) { return (t && dim < t->ndim) ? t->strides[dim] : 0; }
static inline nc_dtype nc_tensor_dtype(const nc_tensor* t) { return t ? t->dtype : NC_F32; }
static inline bool nc_tensor_is_contiguous(const nc_tensor* t) { return t ? t->is_contiguous : false; }
/* CPU pointer to element 0, or NULL while the tensor lives on the device */
void* nc_tensor_data(const nc_tensor* t);
#define nc_tensor_data_f32(t) ((float*)nc_tensor_data(t))
#define nc_tensor_data_f64(t) ((double*)nc_tensor_data(t))
#define nc_tensor_data_i32(t) ((int32_t*)nc_tensor_data(t))
#define nc_tensor_data_i64(t) ((int64_t*)nc_tensor_data(t))
static inline size_t nc_tensor_nbytes(const nc_tensor* t) { return t ? t->numel * nc_dtype_sizeof(t->dtype) : 0; }

double nc_tensor_get_flat(const nc_tensor* t, size_t idx);
void nc_tensor_set_flat(nc_tensor* t, size_t idx, double value);
double nc_tensor_get(const nc_tensor* t, const size_t* indices);
void nc_tensor_set(nc_tensor* t, const size_t* indices, double value);
double nc_tensor_get1(const nc_tensor* t, size_t i);
double nc_tensor_get2(const nc_tensor* t, size_t i, size_t j);
double nc_tensor_get3(const nc_tensor* t, size_t i, size_t j, size_t k);
double nc_tensor_get4(const nc_tensor* t, size_t i, size_t j, size_t k, size_t l);
void nc_tensor_set1(nc_tensor* t, size_t i, double value);
void nc_tensor_set2(nc_tensor* t, size_t i, size_t j, double value);
void nc_tensor_set3(nc_tensor* t, size_t i, size_t j, size_t k, double value);
void nc_tensor_set4(nc_tensor* t, size_t i, size_t j, size_t k, size_t l, double value);

nc_tensor* nc_tensor_reshape(nc_tensor* t, const size_t* shape, size_t ndim);
nc_tensor* nc_tensor_flatten(nc_tensor* t);
nc_tensor* nc_tensor_transpose(nc_tensor* t, size_t dim0, size_t dim1);
nc_tensor* nc_tensor_t(nc_tensor* t);
nc_tensor* nc_tensor_contiguous(nc_tensor* t);
void nc_tensor_requires_grad_(nc_tensor* t, bool requires_grad);
nc_tensor* nc_tensor_detach(const nc_tensor* t);
void nc_tensor_zero_grad_(nc_tensor* t);
void nc_tensor_print(const nc_tensor* t);
void nc_tensor_print_shape(const nc_tensor* t);
bool nc_tensor_shape_eq(const nc_tensor* a, const nc_tensor* b);
void nc_tensor_fill_(nc_tensor* t, double value);
nc_error nc_tensor_copy_(nc_tensor* dst, const nc_tensor* src);
void nc_tensor_to_device(nc_tensor* t, nc_device_type device);

/* ------------------------------------------------------------------ autograd (autograd/node.h, backward.h) */
#define NC_MAX_INPUTS 8
/* receives the output gradient and the node's SAVED tensors; returns a nc_calloc'd array with one
 * gradient per node INPUT (entries may be NULL); the engine frees the entries and the array */
typedef nc_tensor** (*nc_backward_fn)(nc_tensor* grad_output, nc_tensor** saved, size_t n_saved);
struct nc_node {
    const char* op_name;
    nc_backward_fn backward;
    nc_tensor* inputs[NC_MAX_INPUTS];
    size_t n_inputs;
    nc_tensor* saved_tensors[NC_MAX_INPUTS];
    bool saved_tensors_owned[NC_MAX_INPUTS];
    size_t n_saved;
    nc_tensor* output;
    int visited;
    int ref_count;
    /* ---- fields beyond the reference layout ---- */
    double params[8]; /* op hyper-parameters kept on the host (stride, padding, eps, ...) */
};
nc_node* nc_node_create(const char* op_name, nc_backward_fn backward);
void nc_node_add_input(nc_node* node, nc_tensor* input);
void nc_node_save_tensor(nc_node* node, nc_tensor* t);
void nc_node_save_owned_tensor(nc_node* node, nc_tensor* t);
void nc_node_free(nc_node* node);

nc_error nc_backward(nc_tensor* t, nc_tensor* grad_output);
nc_error nc_backward_scalar(nc_tensor* loss);
nc_node** nc_build_topo(nc_tensor* t, size_t* n_nodes);
/* new: called during nc_backward each time a leaf tensor's gradient has been accumulated (its kernel is
 * queued on the stream).  Data-parallel code uses it to start the all-reduce of a gradient bucket while
 * the backward sweep continues.  Pass NULL to remove the hook. */
typedef void (*nc_grad_ready_fn)(nc_tensor* leaf, void* ctx);
void nc_set_grad_ready_hook(nc_grad_ready_fn fn, void* ctx);
typedef enum { NC_GRAD_REPLACE, NC_GRAD_ACCUMULATE } nc_grad_mode;
void nc_set_grad_mode(nc_grad_mode mode);
nc_grad_mode nc_get_grad_mode(void);
typedef struct { int prev_enabled; } nc_no_grad_guard;
nc_no_grad_guard nc_no_grad_begin(void);
void nc_no_grad_end(nc_no_grad_guard* guard);
int nc_grad_enabled(void);
void nc_set_grad_enabled(int enabled);
#define NC_NO_GRAD_BEGIN() nc_no_grad_guard _ng = nc_no_grad_begin()
#define NC_NO_GRAD_END() nc_no_grad_end(&_ng)

/* ------------------------------------------------------------------ ops (the ops headers) - the subset on the training path */
nc_tensor* nc_add(nc_tensor* a, nc_tensor* b); /* same shape, or b broadcast over the last dim */
nc_tensor* nc_sub(nc_tensor* a, nc_tensor* b);
nc_tensor* nc_mul(nc_tensor* a, nc_tensor* b); /* same shape (e.g. a supplied dropout mask) */
nc_tensor* nc_add_scalar(nc_tensor* a, double s);
nc_tensor* nc_mul_scalar(nc_tensor* a, double s);
void nc_add_(nc_tensor* a, nc_tensor* b);
void nc_mul_scalar_(nc_tensor* a, double s);
nc_tensor* nc_matmul(nc_tensor* a, nc_tensor* b); /* 2-D f32 */
nc_tensor* nc_relu(nc_tensor* x);
nc_tensor* nc_gelu(nc_tensor* x);
nc_tensor* nc_sigmoid(nc_tensor* x);
nc_tensor* nc_softmax(nc_tensor* x, int dim);
nc_tensor* nc_sum(nc_tensor* x, int axis, bool keepdim);
nc_tensor* nc_sum_all(nc_tensor* x);
nc_tensor* nc_mean_all(nc_tensor* x);
nc_tensor* nc_argmax(nc_tensor* x, int axis, bool keepdim);
nc_tensor* nc_mse_loss(nc_tensor* pred, nc_tensor* target);
nc_tensor* nc_cross_entropy_loss(nc_tensor* logits, nc_tensor* targets);
typedef enum { NC_REDUCTION_MEAN, NC_REDUCTION_SUM, NC_REDUCTION_NONE } nc_reduction;
nc_tensor* nc_cross_entropy_loss_ex(nc_tensor* logits, nc_tensor* targets, nc_reduction reduction);

/* ------------------------------------------------------------------ modules (nn/module.h) */
#define NC_MAX_PARAMS 64
#define NC_MAX_SUBMODULES 32
#define NC_MAX_NAME_LEN 64
typedef struct nc_module nc_module;
typedef nc_tensor* (*nc_forward_fn)(nc_module* self, nc_tensor* input);
struct nc_module {
    char name[NC_MAX_NAME_LEN];
    nc_tensor* params[NC_MAX_PARAMS];
    char* param_names[NC_MAX_PARAMS];
    size_t n_params;
    nc_module* submodules[NC_MAX_SUBMODULES];
    char* submodule_names[NC_MAX_SUBMODULES];
    size_t n_submodules;
    nc_forward_fn forward;
    bool training;
    void* extra;
    void (*free_extra)(void*);
};
nc_module* nc_module_create(const char* name);
void nc_module_free(nc_module* m);
nc_tensor* nc_module_forward(nc_module* m, nc_tensor* input);
void nc_module_add_param(nc_module* m, const char* name, nc_tensor* param);
void nc_module_add_submodule(nc_module* m, const char* name, nc_module* sub);
nc_tensor* nc_module_get_param(nc_module* m, const char* name);
nc_module* nc_module_get_submodule(nc_module* m, const char* name);
typedef void (*nc_param_callback)(const char* name, nc_tensor* param, void* ctx);
void nc_module_parameters(nc_module* m, nc_param_callback cb, void* ctx);
size_t nc_module_num_parameters(nc_module* m);
void nc_module_train(nc_module* m, bool mode);
static inline void nc_module_eval(nc_module* m) { nc_module_train(m, false); }
static inline bool nc_module_is_training(nc_module* m) { return m ? m->training : false; }
void nc_module_zero_grad(nc_module* m);
void nc_module_requires_grad_(nc_module* m, bool requires_grad);
void nc_module_print(nc_module* m);
/* new: move every parameter (and its gradient) of the module tree */
void nc_module_to_device(nc_module* m, nc_device_type device);

/* ------------------------------------------------------------------ layers (nn/linear.h, conv.h, batchnorm.h, dropout.h) */
nc_module* nc_linear(size_t in_features, size_t out_features, bool bias);
nc_tensor* nc_linear_weight(nc_module* linear);
nc_tensor* nc_linear_bias(nc_module* linear);
nc_tensor* nc_linear_forward(nc_tensor* input, nc_tensor* weight, nc_tensor* bias);

nc_module* nc_conv2d(size_t in_channels, size_t out_channels, size_t kernel_size, size_t stride, size_t padding, bool bias);
nc_module* nc_conv2d_simple(size_t in_channels, size_t out_channels, size_t kernel_size);
nc_tensor* nc_conv2d_weight(nc_module* conv);
nc_tensor* nc_conv2d_bias(nc_module* conv);
nc_tensor* nc_conv2d_forward(nc_tensor* input, nc_tensor* weight, nc_tensor* bias, size_t stride, size_t padding);
nc_module* nc_maxpool2d(size_t kernel_size, size_t stride);
nc_module* nc_maxpool2d_simple(size_t kernel_size);
nc_tensor* nc_maxpool2d_forward(nc_tensor* input, size_t kernel_size, size_t stride);
static inline size_t nc_conv_output_size(size_t input_size, size_t kernel_size, size_t stride, size_t padding) {
    return (input_size + 2 * padding - kernel_size) / stride + 1;
}
nc_module* nc_flatten(void);
/* new: the functional form behind nc_flatten: (N, ...) -> (N, rest), differentiable */
nc_tensor* nc_flatten_forward(nc_tensor* input);

typedef struct {
    size_t num_features;
    double eps;
    double momentum;
    bool affine;
    bool track_running_stats;
} nc_batchnorm2d_config;
static const nc_batchnorm2d_config NC_BATCHNORM2D_DEFAULT = {0, 1e-5, 0.1, true, true};
nc_module* nc_batchnorm2d(size_t num_features);
nc_module* nc_batchnorm2d_ex(nc_batchnorm2d_config config);
nc_tensor* nc_batchnorm2d_weight(nc_module* bn);
nc_tensor* nc_batchnorm2d_bias(nc_module* bn);
nc_tensor* nc_batchnorm2d_running_mean(nc_module* bn);
nc_tensor* nc_batchnorm2d_running_var(nc_module* bn);
nc_tensor* nc_batchnorm2d_forward_fn(nc_tensor* input, nc_tensor* running_mean, nc_tensor* running_var,
                                     nc_tensor* weight, nc_tensor* bias, bool training, double momentum, double eps);
/* new: BatchNorm2d followed by ReLU as ONE forward kernel pass and ONE backward pass (the output is
 * the ReLU mask); same result as nc_relu(nc_batchnorm2d_forward_fn(...)).  The module form takes a
 * module made by nc_batchnorm2d / nc_batchnorm2d_ex. */
nc_tensor* nc_batchnorm2d_relu_forward_fn(nc_tensor* input, nc_tensor* running_mean, nc_tensor* running_var,
                                          nc_tensor* weight, nc_tensor* bias, bool training, double momentum, double eps);
nc_tensor* nc_batchnorm2d_relu(nc_module* bn, nc_tensor* x);
/* new: the same followed by a 2x2 / stride-2 max-pool, as one pass each way that never stores the
 * full-resolution activation (channels-last CUDA input with C % 4 == 0 and even H, W; any other input is
 * served by the two separate ops with the same result). */
nc_tensor* nc_batchnorm2d_relu_maxpool2(nc_module* bn, nc_tensor* x);
typedef struct {
    size_t* normalized_shape;
    size_t normalized_ndim;
    double eps;
    bool elementwise_affine;
} nc_layernorm_config;
nc_module* nc_layernorm(const size_t* normalized_shape, size_t ndim);
nc_module* nc_layernorm_ex(nc_layernorm_config config);
nc_tensor* nc_layernorm_forward_fn(nc_tensor* input, const size_t* normalized_shape, size_t normalized_ndim,
                                   nc_tensor* weight, nc_tensor* bias, double eps);
/* new: dropout with a caller-supplied keep mask already scaled by 1/(1-p): y = x * mask */
nc_tensor* nc_dropout_mask_fn(nc_tensor* x, nc_tensor* mask);
/* the reference's dropout (nn/dropout.h): the keep mask is drawn with rand() on the host exactly as the reference draws it */
nc_tensor* nc_dropout_fn(nc_tensor* x, double p, bool training);
nc_module* nc_dropout(double p);
/* nn/batchnorm.h: BatchNorm1d over (N, C) or (N, C, L) */
nc_module* nc_batchnorm1d(size_t num_features);
nc_module* nc_batchnorm1d_ex(nc_batchnorm2d_config config);
nc_tensor* nc_batchnorm1d_forward_fn(nc_tensor* input, nc_tensor* running_mean, nc_tensor* running_var, nc_tensor* weight,
                                     nc_tensor* bias, bool training, double momentum, double eps);

/* ------------------------------------------------------------------ optimizers (the optim headers) */
#define NC_MAX_OPTIM_PARAMS 256
typedef struct nc_optimizer nc_optimizer;
typedef void (*nc_optim_step_fn)(nc_optimizer* self);
struct nc_optimizer {
    nc_tensor* params[NC_MAX_OPTIM_PARAMS];
    size_t n_params;
    double lr;
    nc_optim_step_fn step;
    void* state;
    void (*free_state)(void*);
    size_t t;
};
void nc_optimizer_free(nc_optimizer* opt);
void nc_optimizer_step(nc_optimizer* opt);
void nc_optimizer_zero_grad(nc_optimizer* opt);
void nc_optimizer_set_lr(nc_optimizer* opt, double lr);
double nc_optimizer_get_lr(nc_optimizer* opt);
void nc_optimizer_add_module(nc_optimizer* opt, nc_module* m);
void nc_optimizer_add_param(nc_optimizer* opt, nc_tensor* param);
/* new: gradients are multiplied by this before the update (1/world_size under data parallel) */
void nc_optimizer_set_grad_scale(nc_optimizer* opt, double scale);
/* new: move all parameter gradients into one device allocation (views at 256-byte aligned offsets);
 * returns its device address and length in floats, so data-parallel code can all-reduce one range */
void* nc_optimizer_flatten_grads(nc_optimizer* opt, size_t* n_floats);

/* ------------------------------------------------------------------ data parallel (new; the reference has no distributed layer)
 * One process per GPU, every rank a full replica on its own shard of the batch.  The step of examples/mnist.c:471-508
 * becomes: nc_optimizer_zero_grad, forward, loss, nc_backward_scalar, nc_dist_allreduce_grads, nc_optimizer_step.
 *
 * nc_bucket_plan is the host-only scheduling logic (usable without a GPU): the flat gradient arena is cut into
 * contiguous buckets of about bucket_floats elements, built from the end of the arena because the backward sweep
 * produces the last layer's gradients first.  on_ready(i) reports that entry i's gradient is final for this step and
 * returns the index of a bucket that has just become complete (or -1); next_unfired() hands out, after the sweep, the
 * buckets that did not complete by themselves; end_step() closes the step and returns how many notifications arrived
 * after their bucket had already been handed out (0 in a static graph).  Which entries report, and how often (a shared
 * weight reports once per use), is learned from the first step: that step sends nothing early. */
typedef struct nc_bucket_plan nc_bucket_plan;
nc_bucket_plan* nc_bucket_plan_create(size_t n_entries, const size_t* offsets, const size_t* numels, size_t arena_floats,
                                      size_t bucket_floats);
void nc_bucket_plan_free(nc_bucket_plan* p);
size_t nc_bucket_plan_count(const nc_bucket_plan* p);
void nc_bucket_plan_range(const nc_bucket_plan* p, size_t b, size_t* start, size_t* stop);
void nc_bucket_plan_begin_step(nc_bucket_plan* p);
int nc_bucket_plan_on_ready(nc_bucket_plan* p, size_t entry);
int nc_bucket_plan_next_unfired(nc_bucket_plan* p);
int nc_bucket_plan_end_step(nc_bucket_plan* p);

/* nc_dist: the plan driven by the backward sweep (through nc_set_grad_ready_hook, which it takes over) over one NCCL
 * communicator.  Rank 0 obtains 128 bytes from nc_dist_unique_id and hands them to every rank by any means; each rank,
 * with its device current, calls nc_dist_init, which also moves the optimizer's gradients into one arena
 * (nc_optimizer_flatten_grads) and sets the gradient scale to 1/world.  nc_dist_allreduce_grads queues whatever has
 * not been sent, makes the compute stream wait for every bucket and returns without blocking the host; it returns an
 * error (and relearns) if a gradient became final after its bucket had been sent.  NCCL is loaded at run time. */
typedef struct nc_dist nc_dist;
int nc_dist_unique_id(void* id128);
nc_dist* nc_dist_init(int rank, int world, const void* id128, nc_optimizer* opt, size_t bucket_floats);
int nc_dist_allreduce_grads(nc_dist* d);
size_t nc_dist_num_buckets(const nc_dist* d);
float* nc_dist_arena(const nc_dist* d, size_t* n_floats);
/* device time between the end of the last backward sweep and the end of its last all-reduce; blocks the host */
double nc_dist_exposed_ms(nc_dist* d);
void nc_dist_free(nc_dist* d);

/* ------------------------------------------------------------------ .ncta files (core/serialize.h)
 * Same byte layout as the reference (see nocta_b200/host/serialize.c); tensors may live on the CUDA device. */
#define NC_FILE_MAGIC 0x4154434E /* "NCTA" */
#define NC_FILE_VERSION 1
nc_error nc_tensor_save(const nc_tensor* t, const char* path);
nc_tensor* nc_tensor_load(const char* path);
nc_error nc_tensor_save_fp(const nc_tensor* t, FILE* fp, const char* name);
nc_tensor* nc_tensor_load_fp(FILE* fp, char* name_out);
typedef struct {
    char** names;
    nc_tensor** tensors;
    size_t n_tensors;
    size_t capacity;
} nc_state_dict;
nc_state_dict* nc_state_dict_create(void);
void nc_state_dict_free(nc_state_dict* sd);
void nc_state_dict_add(nc_state_dict* sd, const char* name, nc_tensor* t); /* takes ownership of t */
nc_tensor* nc_state_dict_get(nc_state_dict* sd, const char* name);
nc_error nc_state_dict_save(nc_state_dict* sd, const char* path);
nc_state_dict* nc_state_dict_load(const char* path);
nc_state_dict* nc_module_state_dict(nc_module* m);
nc_error nc_module_load_state_dict(nc_module* m, nc_state_dict* sd);
nc_error nc_module_save(nc_module* m, const char* path);
nc_error nc_module_load(nc_module* m, const char* path);
nc_error nc_module_save_desc(nc_module* m, const char* path, const char* description);
typedef struct {
    nc_state_dict* model_state;
    nc_state_dict* optimizer_state;
    size_t epoch;
    double loss;
} nc_checkpoint;
nc_error nc_checkpoint_save(nc_checkpoint* ckpt, const char* path);
nc_checkpoint* nc_checkpoint_load(const char* path);
void nc_checkpoint_free(nc_checkpoint* ckpt);
void nc_file_info(const char* path);
bool nc_file_verify(const char* path);
/* new: the optimizer's own state as named tensors ("step" = the step counter as one i64; per parameter
 * index i "velocity.i" for SGD with momentum, "m.i" / "v.i" / "vmax.i" for Adam), for the optimizer_state
 * slot of a checkpoint, and the inverse.  The reference leaves building that dict to the caller. */
nc_state_dict* nc_optimizer_state_dict(nc_optimizer* opt);
nc_error nc_optimizer_load_state_dict(nc_optimizer* opt, nc_state_dict* sd);

/* ---------------- input feeder (new; the reference assembles a batch element by element and copies it
 * synchronously, examples/mnist.c:93-111) ----------------
 * Double-buffered upload of (input, target) batches from pinned host memory on a copy stream, so the
 * copy of batch i+1 overlaps the training step on batch i.  Per slot: submit() starts the asynchronous
 * copy (after the work that last used the slot has finished), acquire() makes the compute stream wait
 * for it and hands out the slot's device tensors (owned by the feeder: do not free them), release()
 * marks the point in the compute stream after which the slot may be overwritten.  The host buffers
 * given to submit() must be pinned (nc_cuda_host_alloc) and stay unchanged until acquire() of that
 * slot has been followed by nc_feeder_wait() or by any synchronisation of the compute stream. */
typedef struct nc_feeder nc_feeder;
nc_feeder* nc_feeder_create(int slots, const size_t* x_shape, size_t x_ndim, nc_dtype x_dtype,
                            const size_t* y_shape, size_t y_ndim, nc_dtype y_dtype);
int nc_feeder_submit(nc_feeder* f, int slot, const void* x_host, const void* y_host);
int nc_feeder_acquire(nc_feeder* f, int slot, nc_tensor** x, nc_tensor** y);
int nc_feeder_release(nc_feeder* f, int slot);
int nc_feeder_wait(nc_feeder* f, int slot);  /* blocks the host until the slot's copy has finished */
void nc_feeder_free(nc_feeder* f);

typedef struct {
    double momentum;
    double dampening;
    double weight_decay;
    bool nesterov;
} nc_sgd_config;
static const nc_sgd_config NC_SGD_DEFAULT = {0.0, 0.0, 0.0, false};
nc_optimizer* nc_sgd(double lr, nc_sgd_config config);
nc_optimizer* nc_sgd_from_module(nc_module* m, double lr, nc_sgd_config config);
nc_optimizer* nc_sgd_simple(nc_module* m, double lr);
nc_optimizer* nc_sgd_momentum(nc_module* m, double lr, double momentum);

typedef struct {
    double beta1;
    double beta2;
    double eps;
    double weight_decay;
    bool amsgrad;
} nc_adam_config;
static const nc_adam_config NC_ADAM_DEFAULT = {0.9, 0.999, 1e-8, 0.0, false};
nc_optimizer* nc_adam(double lr, nc_adam_config config);
nc_optimizer* nc_adam_from_module(nc_module* m, double lr, nc_adam_config config);
nc_optimizer* nc_adam_default(nc_module* m, double lr);
nc_optimizer* nc_adamw(nc_module* m, double lr, double weight_decay);

/* ------------------------------------------------------------------ library init (nocta.h:60-74) */
void nc_init(void);    /* brings up the CUDA backend and makes it the default device */
void nc_cleanup(void); /* frees pools and library scratch */

#ifdef __cplusplus
}
#endif
#endif /* NOCTA_B200_NOCTA_H */
