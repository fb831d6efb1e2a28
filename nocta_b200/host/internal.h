/* Internal helpers shared by the host library sources (not installed). */
#ifndef NOCTA_HOST_INTERNAL_H
#define NOCTA_HOST_INTERNAL_H

#include "nocta/nocta.h"
#include "nocta_cuda.h"

/* The one stream every kernel of this process is launched on (NULL = legacy default stream). */
void* nci_stream(void);
void nci_set_stream(void* s);

/* device pool (core.c) */
void* nci_dev_alloc(size_t bytes);
void nci_dev_free(void* p, size_t bytes);

/* tensor construction without initialisation, on an explicit device */
nc_tensor* nci_empty_on(const size_t* shape, size_t ndim, nc_dtype dtype, nc_device_type dev);
/* (N,C,H,W) tensor stored channels-last on the CUDA device */
nc_tensor* nci_empty_cl(size_t N, size_t C, size_t H, size_t W);
/* same shape, strides and device as `like` (which must be dense) */
nc_tensor* nci_empty_like(const nc_tensor* like);
/* new header sharing the storage of t (no autograd state) */
nc_tensor* nci_alias(const nc_tensor* t);

bool nci_on_cuda(const nc_tensor* t);
/* Where a backward function should put the gradient of its node's input `input_index` when that input is a
 * parameter: a view of the parameter's slot in the flattened-gradient arena if that slot is still zero since it
 * was cleared (so the kernel's result lands where the all-reduce reads it, with no accumulate launch), else a new
 * tensor shaped like `like`.  Only valid inside a backward callback (autograd.c). */
nc_tensor* nci_param_grad_out(size_t input_index, const nc_tensor* like);
/* the storage is a flattened-gradient arena of some optimizer (optim.c) */
bool nci_is_grad_arena(const nc_storage* st);
void nci_forget_grad_arena(const nc_storage* st);
/* device pointer to element 0 (honours offset) */
void* nci_dptr(const nc_tensor* t);
#define nci_fptr(t) ((float*)nci_dptr(t))
/* every element of the storage range [offset, offset+numel) is used exactly once */
bool nci_is_dense(const nc_tensor* t);
bool nci_is_channels_last(const nc_tensor* t);
bool nci_same_layout(const nc_tensor* a, const nc_tensor* b);
/* returns t itself when it is already channels-last, else a new channels-last copy */
nc_tensor* nci_to_channels_last(nc_tensor* t);
/* returns g itself when its strides equal like's, else a new tensor with like's layout */
nc_tensor* nci_match_layout(nc_tensor* g, const nc_tensor* like);
/* require a CUDA-resident f32 tensor; sets the error and returns false otherwise */
bool nci_need_cuda_f32(const nc_tensor* t, const char* op);
/* In plain TF32 math mode activation / gradient kernels round their outputs to TF32 (see
 * nc_cuda_set_round_outputs); accumulations and reductions never do.  Call at the start of a wrapper. */
void nci_round_outputs(bool activation_op);
bool nci_tf32_mode(void);
/* record a failed kernel call */
bool nci_ok(int status, const char* op);
/* g is the all-ones seed nc_backward created itself for a scalar loss (its value is known without a device read) */
bool nci_is_unit_seed(const nc_tensor* g);
/* autograd wiring for an op output */
nc_node* nci_attach(nc_tensor* out, const char* name, nc_backward_fn fn);
void nci_strides4(const nc_tensor* t, size_t s[4]);

#endif
