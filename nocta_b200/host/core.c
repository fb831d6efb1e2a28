/*
 * Core of the host library: error state, tracked host allocation, device storage with a caching
 * device pool, and the nc_tensor type (creation, views, element access, device transfer).
 *
 * Public behaviour follows the reference (include/nocta/core/tensor.h, memory.h, device.h;
 * src/core/tensor.c, memory.c, device.c), with device-first storage: a tensor created while the
 * default device is CUDA owns device memory only, zero-fill is a device memset, and the pool keeps
 * freed blocks by size so a steady-state training step performs no cudaMalloc at all.
 */
#include "internal.h"
#include <math.h>
#include <stdarg.h>

/* ------------------------------------------------------------------ errors / dtypes */
nc_error nc_last_error = NC_OK;
char nc_error_context[256] = {0};

static const char* const k_err[] = {"Success", "Null pointer", "Memory allocation failed", "Shape mismatch",
                                    "Data type mismatch", "Index out of bounds", "Invalid axis", "Invalid shape",
                                    "Invalid data type", "Tensor not contiguous", "Gradient not enabled",
                                    "Cycle detected in computation graph", "I/O error", "Unknown error",
                                    "Tensor not on the CUDA device or kernel failure"};
const char* nc_error_string(nc_error err) { return ((unsigned)err <= NC_ERR_DEVICE) ? k_err[err] : "Unknown error"; }

static const size_t k_dsize[] = {4, 8, 4, 8, 1, 1};
static const char* const k_dname[] = {"float32", "float64", "int32", "int64", "uint8", "bool"};
size_t nc_dtype_sizeof(nc_dtype d) { return (unsigned)d < NC_DTYPE_COUNT ? k_dsize[d] : 0; }
const char* nc_dtype_to_string(nc_dtype d) { return (unsigned)d < NC_DTYPE_COUNT ? k_dname[d] : "unknown"; }

/* ------------------------------------------------------------------ device selection / stream */
static nc_device_type g_default_device = NC_DEVICE_CPU;
static void* g_stream = NULL;
void* nci_stream(void) { return g_stream; }
void nci_set_stream(void* s) { g_stream = s; nc_cuda_set_stream(s); }

void nc_set_default_device(nc_device_type type) {
    if (type == NC_DEVICE_CUDA && !nc_cuda_available()) {
        NC_SET_ERROR(NC_ERR_DEVICE, "CUDA requested as default device but no device is available");
        return;
    }
    g_default_device = type;
}
nc_device_type nc_get_default_device(void) { return g_default_device; }

nc_device_info nc_cuda_device_info(int index) {
    nc_device_info info;
    memset(&info, 0, sizeof(info));
    info.type = NC_DEVICE_CUDA;
    info.index = index;
    int sms = 0;
    nc_cuda_device_props(index, info.name, &info.total_memory, &info.free_memory, &sms);
    return info;
}

void nc_init(void) {
    if (!nc_cuda_available()) {
        NC_SET_ERROR(NC_ERR_DEVICE, "nc_init: no CUDA device; this library computes on the GPU only");
        return;
    }
    nc_cuda_init();
    g_default_device = NC_DEVICE_CUDA;
}
void nc_cleanup(void) {
    nc_device_pool_release();
    nc_cuda_cleanup();
}

/* ------------------------------------------------------------------ tracked host memory */
static nc_mem_stats g_mem;
#define NC_HDR 32 /* keeps 32-byte alignment and stores the block size */

void* nc_alloc(size_t size) {
    if (size == 0) size = 1;
    void* raw = NULL;
    if (posix_memalign(&raw, 32, size + NC_HDR) != 0 || !raw) {
        NC_SET_ERROR(NC_ERR_ALLOC, "host allocation of %zu bytes failed", size);
        return NULL;
    }
    *(size_t*)raw = size;
    g_mem.total_allocated += size;
    g_mem.current_usage += size;
    g_mem.allocation_count++;
    if (g_mem.current_usage > g_mem.peak_usage) g_mem.peak_usage = g_mem.current_usage;
    return (char*)raw + NC_HDR;
}
void* nc_calloc(size_t count, size_t size) {
    size_t total = count * size;
    void* p = nc_alloc(total);
    if (p) memset(p, 0, total ? total : 1);
    return p;
}
void nc_free(void* ptr) {
    if (!ptr) return;
    char* raw = (char*)ptr - NC_HDR;
    size_t size = *(size_t*)raw;
    g_mem.total_freed += size;
    g_mem.current_usage -= size;
    g_mem.free_count++;
    free(raw);
}
void* nc_realloc(void* ptr, size_t old_size, size_t new_size) {
    void* p = nc_alloc(new_size);
    if (p && ptr) memcpy(p, ptr, old_size < new_size ? old_size : new_size);
    nc_free(ptr);
    return p;
}
nc_mem_stats nc_memory_stats(void) { return g_mem; }
void nc_memory_stats_reset(void) { memset(&g_mem, 0, sizeof(g_mem)); }
void nc_memory_report(void) {
    fprintf(stderr, "[nocta] host memory: %zu allocations, %zu frees, %zu bytes live, peak %zu\n", g_mem.allocation_count,
            g_mem.free_count, g_mem.current_usage, g_mem.peak_usage);
}

/* ------------------------------------------------------------------ device pool
 * Freed device blocks are kept in per-size lists (sizes rounded to 512 B).  A training step asks
 * for the same sizes every iteration, so after the first step every request is a list pop.
 * One stream drives the device, so a block can be reused as soon as the host has released it:
 * the kernel that will write it is ordered after the kernels that read it.                      */
typedef struct pool_block { void* ptr; struct pool_block* next; } pool_block;
typedef struct pool_bucket { size_t size; pool_block* free_list; struct pool_bucket* next; } pool_bucket;
#define POOL_HASH 1024
static pool_bucket* g_buckets[POOL_HASH];
static nc_device_pool_stats g_pool;

static size_t g_pool_limit = 0; /* 0: none */
void nc_device_pool_set_limit(size_t bytes) { g_pool_limit = bytes; }
size_t nc_device_pool_get_limit(void) { return g_pool_limit; }
static size_t pool_round(size_t bytes) { return bytes == 0 ? 512 : (bytes + 511) & ~(size_t)511; }
static pool_bucket* pool_find(size_t size, bool create) {
    size_t h = (size >> 9) % POOL_HASH;
    for (pool_bucket* b = g_buckets[h]; b; b = b->next)
        if (b->size == size) return b;
    if (!create) return NULL;
    pool_bucket* b = calloc(1, sizeof(*b));
    if (!b) return NULL;
    b->size = size;
    b->next = g_buckets[h];
    g_buckets[h] = b;
    return b;
}
void* nci_dev_alloc(size_t bytes) {
    size_t size = pool_round(bytes);
    pool_bucket* b = pool_find(size, true);
    if (b && b->free_list) {
        pool_block* blk = b->free_list;
        b->free_list = blk->next;
        void* p = blk->ptr;
        free(blk);
        g_pool.pool_hits++;
        g_pool.bytes_in_use += size;
        if (g_pool.bytes_in_use > g_pool.peak_in_use) g_pool.peak_in_use = g_pool.bytes_in_use;
        return p;
    }
    if (g_pool_limit && g_pool.bytes_reserved + size > g_pool_limit) {
        nc_device_pool_release(); /* cached blocks of other sizes count against the limit: hand them back first */
        if (g_pool.bytes_reserved + size > g_pool_limit) {
            NC_SET_ERROR(NC_ERR_ALLOC, "device allocation of %zu bytes refused: %zu reserved, limit %zu", size, g_pool.bytes_reserved, g_pool_limit);
            return NULL;
        }
    }
    void* p = nc_cuda_malloc(size);
    if (!p) { /* give cached blocks back and retry once */
        nc_device_pool_release();
        nc_cuda_clear_status();
        p = nc_cuda_malloc(size);
    }
    if (!p) {
        NC_SET_ERROR(NC_ERR_ALLOC, "device allocation of %zu bytes failed", size);
        return NULL;
    }
    g_pool.cuda_mallocs++;
    g_pool.bytes_reserved += size;
    g_pool.bytes_in_use += size;
    if (g_pool.bytes_in_use > g_pool.peak_in_use) g_pool.peak_in_use = g_pool.bytes_in_use;
    return p;
}
void nci_dev_free(void* p, size_t bytes) {
    if (!p) return;
    size_t size = pool_round(bytes);
    pool_bucket* b = pool_find(size, true);
    pool_block* blk = b ? malloc(sizeof(*blk)) : NULL;
    g_pool.bytes_in_use -= size;
    if (!blk) { /* cannot cache: hand it back */
        nc_cuda_synchronize();
        nc_cuda_free(p);
        g_pool.bytes_reserved -= size;
        return;
    }
    blk->ptr = p;
    blk->next = b->free_list;
    b->free_list = blk;
}
nc_device_pool_stats nc_device_pool_get_stats(void) { return g_pool; }
void nc_device_pool_release(void) {
    bool synced = false;
    for (size_t h = 0; h < POOL_HASH; h++)
        for (pool_bucket* b = g_buckets[h]; b; b = b->next)
            while (b->free_list) {
                pool_block* blk = b->free_list;
                b->free_list = blk->next;
                if (!synced) { nc_cuda_synchronize(); synced = true; }
                nc_cuda_free(blk->ptr);
                g_pool.bytes_reserved -= b->size;
                free(blk);
            }
}

/* ------------------------------------------------------------------ storage */
nc_storage* nc_storage_create_on(size_t size, nc_device_type device) {
    nc_storage* s = nc_calloc(1, sizeof(nc_storage));
    if (!s) return NULL;
    s->size = size;
    s->refcount = 1;
    s->device = device;
    if (device == NC_DEVICE_CUDA) {
        s->cuda_data = nci_dev_alloc(size);
        if (!s->cuda_data) { nc_free(s); return NULL; }
    } else {
        s->data = nc_alloc(size);
        if (!s->data) { nc_free(s); return NULL; }
    }
    return s;
}
nc_storage* nc_storage_create(size_t size) { return nc_storage_create_on(size, g_default_device); }
nc_storage* nc_storage_retain(nc_storage* s) { if (s) s->refcount++; return s; }
void nc_storage_release(nc_storage* s) {
    if (!s) return;
    if (--s->refcount > 0) return;
    nci_forget_grad_arena(s);
    if (s->data) nc_free(s->data);
    if (s->cuda_data) nci_dev_free(s->cuda_data, s->size);
    nc_free(s);
}
int nc_storage_refcount(const nc_storage* s) { return s ? s->refcount : 0; }

void nc_storage_to_device(nc_storage* s, nc_device_type target) {
    if (!s || s->device == target) return;
    if (target == NC_DEVICE_CUDA) {
        void* d = nci_dev_alloc(s->size);
        if (!d) return;
        if (s->data && s->size) nc_cuda_memcpy_h2d(d, s->data, s->size);
        if (s->data) nc_free(s->data);
        s->data = NULL;
        s->cuda_data = d;
    } else {
        void* h = nc_alloc(s->size);
        if (!h) return;
        if (s->cuda_data && s->size) nc_cuda_memcpy_d2h(h, s->cuda_data, s->size);
        if (s->cuda_data) nci_dev_free(s->cuda_data, s->size);
        s->cuda_data = NULL;
        s->data = h;
    }
    s->device = target;
}
void nc_storage_ensure_on(nc_storage* s, nc_device_type target) { nc_storage_to_device(s, target); }
void* nc_storage_data_ptr(nc_storage* s) { return !s ? NULL : (s->device == NC_DEVICE_CUDA ? s->cuda_data : s->data); }
void nc_storage_sync_to_cpu(nc_storage* s) {
    if (!s || s->device != NC_DEVICE_CUDA) return;
    if (!s->data) s->data = nc_alloc(s->size);
    if (s->data) nc_cuda_memcpy_d2h(s->data, s->cuda_data, s->size);
}

/* ------------------------------------------------------------------ tensor helpers */
bool nci_on_cuda(const nc_tensor* t) { return t && t->storage && t->storage->device == NC_DEVICE_CUDA && t->storage->cuda_data; }
void* nci_dptr(const nc_tensor* t) {
    return (char*)t->storage->cuda_data + t->offset * nc_dtype_sizeof(t->dtype);
}
bool nci_tf32_mode(void) { return nc_cuda_get_math_mode() == NC_CUDA_MATH_TF32; }
void nci_round_outputs(bool activation_op) { nc_cuda_set_round_outputs(activation_op && nci_tf32_mode() ? 1 : 0); }
bool nci_ok(int status, const char* op) {
    if (status == 0) return true;
    NC_SET_ERROR(NC_ERR_DEVICE, "%s: kernel library status %d (%s)", op, status, nc_cuda_last_message());
    return false;
}
bool nci_need_cuda_f32(const nc_tensor* t, const char* op) {
    if (!t) { NC_SET_ERROR(NC_ERR_NULL_PTR, "%s: null tensor", op); return false; }
    if (t->dtype != NC_F32) { NC_SET_ERROR(NC_ERR_INVALID_DTYPE, "%s: float32 tensor required", op); return false; }
    if (!nci_on_cuda(t)) {
        /* a host-resident operand (created before nc_init, or by a program that never calls it) is moved to the
         * device, storage and all its views with it; there is no host compute path to fall back to */
        static int have_gpu = -1;
        if (have_gpu < 0) have_gpu = nc_cuda_available() ? 1 : 0;
        if (have_gpu && t->storage) nc_tensor_to_device((nc_tensor*)t, NC_DEVICE_CUDA);
        if (!nci_on_cuda(t)) {
            NC_SET_ERROR(NC_ERR_DEVICE, "%s: tensor is not on the CUDA device (this library has no CPU compute path)", op);
            return false;
        }
    }
    return true;
}

static void set_contiguous_strides(nc_tensor* t) {
    size_t s = 1;
    for (size_t i = t->ndim; i-- > 0;) { t->strides[i] = s; s *= t->shape[i]; }
}
static bool compute_contiguous(const nc_tensor* t) {
    size_t s = 1;
    for (size_t i = t->ndim; i-- > 0;) {
        if (t->shape[i] != 1 && t->strides[i] != s) return false;
        s *= t->shape[i];
    }
    return true;
}
static nc_tensor* tensor_header(const size_t* shape, size_t ndim, nc_dtype dtype) {
    if (ndim > NC_MAX_DIMS || (ndim > 0 && !shape)) { NC_SET_ERROR(NC_ERR_INVALID_SHAPE, "bad shape (ndim %zu)", ndim); return NULL; }
    if ((unsigned)dtype >= NC_DTYPE_COUNT) { NC_SET_ERROR(NC_ERR_INVALID_DTYPE, "bad dtype %d", (int)dtype); return NULL; }
    nc_tensor* t = nc_calloc(1, sizeof(nc_tensor));
    if (!t) return NULL;
    t->ndim = ndim;
    t->numel = 1;
    for (size_t i = 0; i < ndim; i++) { t->shape[i] = shape[i]; t->numel *= shape[i]; }
    set_contiguous_strides(t);
    t->dtype = dtype;
    t->is_leaf = true;
    t->is_contiguous = true;
    return t;
}
nc_tensor* nci_empty_on(const size_t* shape, size_t ndim, nc_dtype dtype, nc_device_type dev) {
    nc_tensor* t = tensor_header(shape, ndim, dtype);
    if (!t) return NULL;
    t->storage = nc_storage_create_on(t->numel * nc_dtype_sizeof(dtype), dev);
    if (!t->storage) { nc_free(t); return NULL; }
    return t;
}
nc_tensor* nci_empty_cl(size_t N, size_t C, size_t H, size_t W) {
    size_t shape[4] = {N, C, H, W};
    nc_tensor* t = nci_empty_on(shape, 4, NC_F32, NC_DEVICE_CUDA);
    if (!t) return NULL;
    t->strides[0] = H * W * C; t->strides[1] = 1; t->strides[2] = W * C; t->strides[3] = C;
    t->is_contiguous = compute_contiguous(t);
    return t;
}
nc_tensor* nci_empty_like(const nc_tensor* like) {
    nc_tensor* t = nci_empty_on(like->shape, like->ndim, like->dtype, like->storage->device);
    if (!t) return NULL;
    memcpy(t->strides, like->strides, sizeof(t->strides));
    t->is_contiguous = like->is_contiguous;
    return t;
}
nc_tensor* nci_alias(const nc_tensor* src) {
    nc_tensor* t = nc_calloc(1, sizeof(nc_tensor));
    if (!t) return NULL;
    *t = *src;
    t->storage = nc_storage_retain(src->storage);
    t->grad = NULL; t->grad_fn = NULL; t->requires_grad = false; t->is_leaf = true;
    return t;
}
bool nci_is_dense(const nc_tensor* t) {
    /* sort dims by stride; dense iff each stride equals the product of the smaller extents */
    size_t idx[NC_MAX_DIMS], n = 0;
    for (size_t i = 0; i < t->ndim; i++) if (t->shape[i] != 1) idx[n++] = i;
    for (size_t i = 1; i < n; i++)
        for (size_t j = i; j > 0 && t->strides[idx[j]] < t->strides[idx[j - 1]]; j--) { size_t k = idx[j]; idx[j] = idx[j - 1]; idx[j - 1] = k; }
    size_t expect = 1;
    for (size_t i = 0; i < n; i++) { if (t->strides[idx[i]] != expect) return false; expect *= t->shape[idx[i]]; }
    return true;
}
bool nci_is_channels_last(const nc_tensor* t) {
    if (t->ndim != 4) return false;
    size_t C = t->shape[1], H = t->shape[2], W = t->shape[3];
    return (t->shape[1] == 1 || t->strides[1] == 1) && (W == 1 || t->strides[3] == C) && (H == 1 || t->strides[2] == W * C) &&
           (t->shape[0] == 1 || t->strides[0] == H * W * C);
}
bool nci_same_layout(const nc_tensor* a, const nc_tensor* b) {
    if (a->ndim != b->ndim) return false;
    for (size_t i = 0; i < a->ndim; i++) {
        if (a->shape[i] != b->shape[i]) return false;
        if (a->shape[i] != 1 && a->strides[i] != b->strides[i]) return false;
    }
    return true;
}
void nci_strides4(const nc_tensor* t, size_t s[4]) { for (int i = 0; i < 4; i++) s[i] = t->strides[i]; }

static int g_relayout_round = 0; /* set while a conv input is being re-laid out in TF32 mode */
/* dst (dense, any layout) <- src (any strides), both on the device, f32, ndim <= 4 */
static bool device_relayout(nc_tensor* dst, const nc_tensor* src) {
    if (src->ndim > 4 || src->dtype != NC_F32) { NC_SET_ERROR(NC_ERR_INVALID_SHAPE, "device relayout supports f32 tensors of up to 4 dims"); return false; }
    size_t N = 1, C = 1, H = 1, W = 1;
    if (src->ndim == 4) { N = src->shape[0]; C = src->shape[1]; H = src->shape[2]; W = src->shape[3]; }
    bool src_cl = src->ndim == 4 && nci_is_channels_last(src), dst_cl = dst->ndim == 4 && nci_is_channels_last(dst);
    if (src->ndim == 4 && src->is_contiguous && dst_cl && !dst->is_contiguous)
        return nci_ok(nc_cuda_nchw_to_nhwc_f32_ex(nci_fptr(dst), nci_fptr(src), (int)N, (int)C, (int)(H * W), g_relayout_round, nci_stream()), "relayout");
    if (src_cl && dst->is_contiguous && !src->is_contiguous)
        return nci_ok(nc_cuda_nhwc_to_nchw_f32_ex(nci_fptr(dst), nci_fptr(src), (int)N, (int)C, (int)(H * W), nci_stream()), "relayout");
    if (!dst->is_contiguous) { NC_SET_ERROR(NC_ERR_NOT_CONTIGUOUS, "relayout: unsupported destination layout"); return false; }
    size_t shape[4] = {1, 1, 1, 1}, strides[4] = {0, 0, 0, 0};
    size_t pad = 4 - src->ndim;
    for (size_t i = 0; i < src->ndim; i++) { shape[pad + i] = src->shape[i]; strides[pad + i] = src->strides[i]; }
    return nci_ok(nc_cuda_strided_copy_f32_ex(nci_fptr(dst), nci_fptr(src), shape, strides, nci_stream()), "strided copy");
}
nc_tensor* nci_to_channels_last(nc_tensor* t) {
    if (nci_is_channels_last(t)) return t;
    nc_tensor* src = t;
    nc_tensor* tmp = NULL;
    if (!t->is_contiguous) { tmp = nc_tensor_contiguous(t); if (!tmp) return NULL; src = tmp; }
    nc_tensor* out = nci_empty_cl(t->shape[0], t->shape[1], t->shape[2], t->shape[3]);
    g_relayout_round = nci_tf32_mode() ? 1 : 0; /* a private copy read only by the contraction kernels */
    if (out && !device_relayout(out, src)) { nc_tensor_free(out); out = NULL; }
    g_relayout_round = 0;
    if (tmp && tmp != t) nc_tensor_free(tmp);
    return out;
}
nc_tensor* nci_match_layout(nc_tensor* g, const nc_tensor* like) {
    if (nci_same_layout(g, like)) return g;
    if (g->numel != like->numel) { NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "layout match: element counts differ"); return NULL; }
    nc_tensor* src = g;
    nc_tensor* view = NULL;
    if (g->ndim != like->ndim) { /* e.g. a (N, C*H*W) gradient for a (N,C,H,W) activation */
        view = nc_tensor_reshape(g, like->shape, like->ndim);
        if (!view) return NULL;
        src = view;
        if (nci_same_layout(src, like)) return src;
    }
    nc_tensor* out = nci_empty_like(like);
    if (out && !device_relayout(out, src)) { nc_tensor_free(out); out = NULL; }
    if (view) nc_tensor_free(view);
    return out;
}

/* ------------------------------------------------------------------ creation */
nc_tensor* nc_tensor_empty(const size_t* shape, size_t ndim, nc_dtype dtype) { return nci_empty_on(shape, ndim, dtype, g_default_device); }

void nc_tensor_fill_(nc_tensor* t, double value) {
    if (!t || !t->storage || t->numel == 0) return;
    size_t es = nc_dtype_sizeof(t->dtype);
    if (nci_on_cuda(t)) {
        if (value == 0.0 && nci_is_dense(t)) { nc_cuda_memset_async(nci_dptr(t), 0, t->numel * es, nci_stream()); return; }
        if (t->dtype == NC_F32 && nci_is_dense(t)) { nci_ok(nc_cuda_fill_f32_ex(nci_fptr(t), (float)value, t->numel, nci_stream()), "fill"); return; }
        /* rare: build on the host and upload */
        nc_tensor* h = nci_empty_on(t->shape, t->ndim, t->dtype, NC_DEVICE_CPU);
        if (!h) return;
        nc_tensor_fill_(h, value);
        nc_tensor_copy_(t, h);
        nc_tensor_free(h);
        return;
    }
    for (size_t i = 0; i < t->numel; i++) nc_tensor_set_flat(t, i, value);
}
nc_tensor* nc_tensor_full(const size_t* shape, size_t ndim, nc_dtype dtype, double value) {
    nc_tensor* t = nc_tensor_empty(shape, ndim, dtype);
    if (t) nc_tensor_fill_(t, value);
    return t;
}
nc_tensor* nc_tensor_zeros(const size_t* shape, size_t ndim, nc_dtype dtype) { return nc_tensor_full(shape, ndim, dtype, 0.0); }
nc_tensor* nc_tensor_ones(const size_t* shape, size_t ndim, nc_dtype dtype) { return nc_tensor_full(shape, ndim, dtype, 1.0); }
nc_tensor* nc_tensor_from_data(const void* data, const size_t* shape, size_t ndim, nc_dtype dtype) {
    if (!data) { NC_SET_ERROR(NC_ERR_NULL_PTR, "nc_tensor_from_data: null data"); return NULL; }
    nc_tensor* t = nc_tensor_empty(shape, ndim, dtype);
    if (!t) return NULL;
    size_t bytes = t->numel * nc_dtype_sizeof(dtype);
    if (bytes) {
        if (nci_on_cuda(t)) nc_cuda_memcpy_h2d(t->storage->cuda_data, data, bytes);
        else memcpy(t->storage->data, data, bytes);
    }
    return t;
}
nc_tensor* nc_tensor_scalar(double value, nc_dtype dtype) {
    /* scalars are host bookkeeping (saved hyper-parameters, step sizes): always CPU-resident */
    nc_tensor* t = nci_empty_on(NULL, 0, dtype, NC_DEVICE_CPU);
    if (t) nc_tensor_set_flat(t, 0, value);
    return t;
}
nc_tensor* nc_tensor_arange(double start, double end, double step, nc_dtype dtype) {
    if (step == 0.0) { NC_SET_ERROR(NC_ERR_INVALID_SHAPE, "arange: zero step"); return NULL; }
    double cnt = ceil((end - start) / step);
    size_t n = cnt > 0 ? (size_t)cnt : 0;
    nc_tensor* h = nci_empty_on(&n, 1, dtype, NC_DEVICE_CPU);
    if (!h) return NULL;
    for (size_t i = 0; i < n; i++) nc_tensor_set_flat(h, i, start + (double)i * step);
    if (g_default_device == NC_DEVICE_CUDA) nc_tensor_to_device(h, NC_DEVICE_CUDA);
    return h;
}

/* Random tensors follow the reference's generator (src/core/tensor.c:21-47): xorshift128+ with shifts 23 / 17 / 26,
 * uniform = top 53 bits / 2^53, normal = sqrt(-2 ln(u1 + 1e-10)) cos(2 pi u2); unseeded, the state starts from
 * time(NULL) as there, so a program run at the same second draws the same values from either library.
 * nc_manual_seed (new) fixes the state instead. */
static uint64_t g_rng[2] = {0, 0};
void nc_manual_seed(uint64_t seed) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull;
    for (int i = 0; i < 2; i++) {
        z += 0x9E3779B97F4A7C15ull;
        uint64_t x = z;
        x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
        x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
        g_rng[i] = x ^ (x >> 31);
    }
    if (!g_rng[0] && !g_rng[1]) g_rng[0] = 1;
}
static uint64_t rng_next(void) {
    if (g_rng[0] == 0) {
        g_rng[0] = (uint64_t)time(NULL);
        g_rng[1] = g_rng[0] ^ 0x5DEECE66DULL;
    }
    uint64_t x = g_rng[0];
    const uint64_t y = g_rng[1];
    g_rng[0] = y;
    x ^= x << 23;
    g_rng[1] = x ^ y ^ (x >> 17) ^ (y >> 26);
    return g_rng[1] + y;
}
static double rng_uniform(void) { return (double)(rng_next() >> 11) * (1.0 / 9007199254740992.0); }
static double rng_normal(void) {
    const double u1 = rng_uniform(), u2 = rng_uniform();
    return sqrt(-2.0 * log(u1 + 1e-10)) * cos(2.0 * 3.14159265358979323846 * u2);
}
static nc_tensor* random_tensor(const size_t* shape, size_t ndim, nc_dtype dtype, bool normal) {
    nc_tensor* h = nci_empty_on(shape, ndim, dtype, NC_DEVICE_CPU);
    if (!h) return NULL;
    for (size_t i = 0; i < h->numel; i++) nc_tensor_set_flat(h, i, normal ? rng_normal() : rng_uniform());
    if (g_default_device == NC_DEVICE_CUDA) nc_tensor_to_device(h, NC_DEVICE_CUDA);
    return h;
}
nc_tensor* nc_tensor_rand(const size_t* shape, size_t ndim, nc_dtype dtype) { return random_tensor(shape, ndim, dtype, false); }
nc_tensor* nc_tensor_randn(const size_t* shape, size_t ndim, nc_dtype dtype) { return random_tensor(shape, ndim, dtype, true); }

nc_tensor* nc_tensor_clone(const nc_tensor* r) {
    if (!r) { NC_SET_ERROR(NC_ERR_NULL_PTR, "clone: null tensor"); return NULL; }
    if (nci_is_dense(r)) { /* raw byte copy keeps the layout (e.g. channels-last) */
        nc_tensor* t = nci_empty_like(r);
        if (!t) return NULL;
        size_t bytes = r->numel * nc_dtype_sizeof(r->dtype);
        if (bytes) {
            if (nci_on_cuda(r)) nc_cuda_memcpy_d2d(t->storage->cuda_data, nci_dptr(r), bytes);
            else memcpy(t->storage->data, (char*)r->storage->data + r->offset * nc_dtype_sizeof(r->dtype), bytes);
        }
        t->requires_grad = r->requires_grad;
        return t;
    }
    nc_tensor* t = nc_tensor_contiguous((nc_tensor*)r);
    if (t == r) { NC_SET_ERROR(NC_ERR_UNKNOWN, "clone: unexpected aliasing"); return NULL; }
    return t;
}
void nc_tensor_free(nc_tensor* t) {
    if (!t) return;
    if (t->grad_fn) nc_node_free(t->grad_fn);
    if (t->grad) nc_tensor_free(t->grad);
    nc_storage_release(t->storage);
    nc_free(t);
}

/* ------------------------------------------------------------------ element access */
/* A raw host pointer to the elements, as the reference returns it (src/core/tensor.c).  A caller that asks for it means
 * to read or write the data behind the library's back (the script VM's optimizer natives do: src/lang/vm.c:1090-1112), so
 * a device-resident storage is moved to the host first, all its views with it (blocking copy); the next operator that
 * uses the tensor moves it back (nci_need_cuda_f32).  Correct, and slow by design: code on the hot path uses the
 * device-side optimizers instead. */
void* nc_tensor_data(const nc_tensor* t) {
    if (!t || !t->storage) return NULL;
    if (t->storage->device == NC_DEVICE_CUDA) nc_storage_to_device(t->storage, NC_DEVICE_CPU);
    if (!t->storage->data) return NULL;
    return (char*)t->storage->data + t->offset * nc_dtype_sizeof(t->dtype);
}

/* Mark bits for a caller's garbage collector (the script VM, src/lang/vm.c; reference: src/core/tensor.c:763-806): mark
 * walks the tensor, the inputs and saved tensors of its graph node and marks them; reset clears the same set.  The flag
 * of a GRADIENT tensor is left alone: this library uses it to remember whether a gradient still holds the zeros it was
 * cleared to (autograd.c), and gradients belong to their tensor, never to a collector. */
void nc_tensor_mark_reachable(nc_tensor* t) {
    if (!t || t->is_reachable) return;
    t->is_reachable = true;
    nc_node* nd = t->grad_fn;
    if (!nd) return;
    for (size_t i = 0; i < nd->n_inputs; i++) if (nd->inputs[i]) nc_tensor_mark_reachable(nd->inputs[i]);
    for (size_t i = 0; i < nd->n_saved; i++) if (nd->saved_tensors[i]) nc_tensor_mark_reachable(nd->saved_tensors[i]);
}
bool nc_tensor_is_reachable(const nc_tensor* t) { return t ? t->is_reachable : false; }
void nc_tensor_reset_reachable(nc_tensor* t) {
    if (!t || !t->is_reachable) return;
    t->is_reachable = false;
    nc_node* nd = t->grad_fn;
    if (!nd) return;
    for (size_t i = 0; i < nd->n_inputs; i++) if (nd->inputs[i]) nc_tensor_reset_reachable(nd->inputs[i]);
    for (size_t i = 0; i < nd->n_saved; i++) if (nd->saved_tensors[i]) nc_tensor_reset_reachable(nd->saved_tensors[i]);
}
static size_t flat_to_offset(const nc_tensor* t, size_t idx) {
    if (t->is_contiguous) return t->offset + idx;
    size_t off = t->offset;
    for (size_t i = t->ndim; i-- > 0;) { off += (idx % t->shape[i]) * t->strides[i]; idx /= t->shape[i]; }
    return off;
}
static double load_elem(const nc_tensor* t, size_t off) {
    size_t es = nc_dtype_sizeof(t->dtype);
    unsigned char buf[8];
    if (t->storage->device == NC_DEVICE_CUDA) nc_cuda_memcpy_d2h(buf, (char*)t->storage->cuda_data + off * es, es);
    else memcpy(buf, (char*)t->storage->data + off * es, es);
    switch (t->dtype) {
        case NC_F32: { float v; memcpy(&v, buf, 4); return v; }
        case NC_F64: { double v; memcpy(&v, buf, 8); return v; }
        case NC_I32: { int32_t v; memcpy(&v, buf, 4); return v; }
        case NC_I64: { int64_t v; memcpy(&v, buf, 8); return (double)v; }
        default: return buf[0];
    }
}
static void store_elem(nc_tensor* t, size_t off, double value) {
    size_t es = nc_dtype_sizeof(t->dtype);
    unsigned char buf[8];
    switch (t->dtype) {
        case NC_F32: { float v = (float)value; memcpy(buf, &v, 4); break; }
        case NC_F64: { memcpy(buf, &value, 8); break; }
        case NC_I32: { int32_t v = (int32_t)value; memcpy(buf, &v, 4); break; }
        case NC_I64: { int64_t v = (int64_t)value; memcpy(buf, &v, 8); break; }
        case NC_BOOL: buf[0] = value != 0.0; break;
        default: buf[0] = (unsigned char)value; break;
    }
    if (t->storage->device == NC_DEVICE_CUDA) nc_cuda_memcpy_h2d((char*)t->storage->cuda_data + off * es, buf, es);
    else memcpy((char*)t->storage->data + off * es, buf, es);
}
double nc_tensor_get_flat(const nc_tensor* t, size_t idx) {
    if (!t || !t->storage || idx >= t->numel) return 0.0;
    return load_elem(t, flat_to_offset(t, idx));
}
void nc_tensor_set_flat(nc_tensor* t, size_t idx, double value) {
    if (!t || !t->storage || idx >= t->numel) return;
    store_elem(t, flat_to_offset(t, idx), value);
}
double nc_tensor_get(const nc_tensor* t, const size_t* ix) {
    if (!t || !ix || !t->storage) return 0.0;
    size_t off = t->offset;
    for (size_t i = 0; i < t->ndim; i++) { if (ix[i] >= t->shape[i]) { NC_SET_ERROR(NC_ERR_INDEX_OUT_OF_BOUNDS, "index %zu out of range", ix[i]); return 0.0; } off += ix[i] * t->strides[i]; }
    return load_elem(t, off);
}
void nc_tensor_set(nc_tensor* t, const size_t* ix, double value) {
    if (!t || !ix || !t->storage) return;
    size_t off = t->offset;
    for (size_t i = 0; i < t->ndim; i++) { if (ix[i] >= t->shape[i]) { NC_SET_ERROR(NC_ERR_INDEX_OUT_OF_BOUNDS, "index %zu out of range", ix[i]); return; } off += ix[i] * t->strides[i]; }
    store_elem(t, off, value);
}
double nc_tensor_get1(const nc_tensor* t, size_t i) { size_t ix[1] = {i}; return (t && t->ndim == 1) ? nc_tensor_get(t, ix) : nc_tensor_get_flat(t, i); }
double nc_tensor_get2(const nc_tensor* t, size_t i, size_t j) { size_t ix[2] = {i, j}; return (t && t->ndim == 2) ? nc_tensor_get(t, ix) : 0.0; }
double nc_tensor_get3(const nc_tensor* t, size_t i, size_t j, size_t k) { size_t ix[3] = {i, j, k}; return (t && t->ndim == 3) ? nc_tensor_get(t, ix) : 0.0; }
double nc_tensor_get4(const nc_tensor* t, size_t i, size_t j, size_t k, size_t l) { size_t ix[4] = {i, j, k, l}; return (t && t->ndim == 4) ? nc_tensor_get(t, ix) : 0.0; }
void nc_tensor_set1(nc_tensor* t, size_t i, double v) { size_t ix[1] = {i}; if (t && t->ndim == 1) nc_tensor_set(t, ix, v); else nc_tensor_set_flat(t, i, v); }
void nc_tensor_set2(nc_tensor* t, size_t i, size_t j, double v) { size_t ix[2] = {i, j}; if (t && t->ndim == 2) nc_tensor_set(t, ix, v); }
void nc_tensor_set3(nc_tensor* t, size_t i, size_t j, size_t k, double v) { size_t ix[3] = {i, j, k}; if (t && t->ndim == 3) nc_tensor_set(t, ix, v); }
void nc_tensor_set4(nc_tensor* t, size_t i, size_t j, size_t k, size_t l, double v) { size_t ix[4] = {i, j, k, l}; if (t && t->ndim == 4) nc_tensor_set(t, ix, v); }

/* ------------------------------------------------------------------ views / copies */
nc_tensor* nc_tensor_contiguous(nc_tensor* t) {
    if (!t) return NULL;
    if (t->is_contiguous) return t;
    nc_tensor* out = nci_empty_on(t->shape, t->ndim, t->dtype, t->storage->device);
    if (!out) return NULL;
    if (nci_on_cuda(t)) {
        if (!device_relayout(out, t)) { nc_tensor_free(out); return NULL; }
    } else {
        size_t es = nc_dtype_sizeof(t->dtype);
        for (size_t i = 0; i < t->numel; i++)
            memcpy((char*)out->storage->data + i * es, (char*)t->storage->data + flat_to_offset(t, i) * es, es);
    }
    out->requires_grad = false;
    return out;
}
nc_tensor* nc_tensor_reshape(nc_tensor* t, const size_t* shape, size_t ndim) {
    if (!t || (!shape && ndim)) { NC_SET_ERROR(NC_ERR_NULL_PTR, "reshape: null argument"); return NULL; }
    size_t n = 1;
    for (size_t i = 0; i < ndim; i++) n *= shape[i];
    if (n != t->numel || ndim > NC_MAX_DIMS) { NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "reshape: %zu elements into %zu", t->numel, n); return NULL; }
    nc_tensor* src = t->is_contiguous ? t : nc_tensor_contiguous(t);
    if (!src) return NULL;
    nc_tensor* v = nc_calloc(1, sizeof(nc_tensor));
    if (!v) { if (src != t) nc_tensor_free(src); return NULL; }
    v->storage = nc_storage_retain(src->storage);
    v->offset = src->offset;
    v->ndim = ndim;
    v->numel = n;
    for (size_t i = 0; i < ndim; i++) v->shape[i] = shape[i];
    set_contiguous_strides(v);
    v->dtype = t->dtype;
    v->is_leaf = true;
    v->is_contiguous = true;
    if (src != t) nc_tensor_free(src);
    return v;
}
nc_tensor* nc_tensor_flatten(nc_tensor* t) { size_t n = t ? t->numel : 0; return nc_tensor_reshape(t, &n, 1); }
nc_tensor* nc_tensor_transpose(nc_tensor* t, size_t d0, size_t d1) {
    if (!t || d0 >= t->ndim || d1 >= t->ndim) { NC_SET_ERROR(NC_ERR_INVALID_AXIS, "transpose: bad dims"); return NULL; }
    nc_tensor* v = nci_alias(t);
    if (!v) return NULL;
    size_t s = v->shape[d0]; v->shape[d0] = v->shape[d1]; v->shape[d1] = s;
    s = v->strides[d0]; v->strides[d0] = v->strides[d1]; v->strides[d1] = s;
    v->is_contiguous = compute_contiguous(v);
    return v;
}
nc_tensor* nc_tensor_t(nc_tensor* t) { return (t && t->ndim == 2) ? nc_tensor_transpose(t, 0, 1) : NULL; }

void nc_tensor_requires_grad_(nc_tensor* t, bool rg) {
    if (!t) return;
    t->requires_grad = rg;
    if (rg && !t->grad) {
        t->grad = nci_empty_on(t->shape, t->ndim, t->dtype, t->storage->device);
        if (t->grad) nc_tensor_fill_(t->grad, 0.0);
    }
}
nc_tensor* nc_tensor_detach(const nc_tensor* t) { return t ? nci_alias(t) : NULL; }
/* A gradient that backward wrote since it was last cleared (marked in its is_reachable field, which is
 * otherwise unused on gradient tensors) is dropped instead of being zeroed: the next backward takes over its
 * first contribution instead of adding it to zeros.  Gradients backward never wrote (e.g. BatchNorm running
 * statistics, which the reference registers as parameters with a zero .grad) and views into the flattened
 * arena of nc_optimizer_flatten_grads are zeroed in place, as in the reference. */
void nc_tensor_zero_grad_(nc_tensor* t) {
    if (!t || !t->grad) return;
    nc_tensor* g = t->grad;
    if (g->is_reachable && g->storage && !nci_is_grad_arena(g->storage) && !g->grad_fn) {
        nc_tensor_free(g);
        t->grad = NULL;
        return;
    }
    nc_tensor_fill_(g, 0.0);
    g->is_reachable = false; /* zero since cleared */
}
bool nc_tensor_shape_eq(const nc_tensor* a, const nc_tensor* b) {
    if (!a || !b || a->ndim != b->ndim) return false;
    for (size_t i = 0; i < a->ndim; i++) if (a->shape[i] != b->shape[i]) return false;
    return true;
}
nc_error nc_tensor_copy_(nc_tensor* dst, const nc_tensor* src) {
    if (!dst || !src) return NC_ERR_NULL_PTR;
    if (dst->numel != src->numel) return NC_ERR_SHAPE_MISMATCH;
    if (dst->dtype != src->dtype) return NC_ERR_DTYPE_MISMATCH;
    size_t es = nc_dtype_sizeof(dst->dtype), bytes = dst->numel * es;
    if (!bytes) return NC_OK;
    bool same = nci_same_layout(dst, src) && nci_is_dense(dst);
    bool both_contig = dst->is_contiguous && src->is_contiguous;
    if (same || both_contig) {
        void* d = nci_on_cuda(dst) ? nci_dptr(dst) : (char*)dst->storage->data + dst->offset * es;
        const void* s = nci_on_cuda(src) ? nci_dptr(src) : (const char*)src->storage->data + src->offset * es;
        if (nci_on_cuda(dst) && nci_on_cuda(src)) nc_cuda_memcpy_d2d(d, s, bytes);
        else if (nci_on_cuda(dst)) nc_cuda_memcpy_h2d(d, s, bytes);
        else if (nci_on_cuda(src)) nc_cuda_memcpy_d2h(d, s, bytes);
        else memcpy(d, s, bytes);
        return NC_OK;
    }
    if (nci_on_cuda(dst) && nci_on_cuda(src) && dst->dtype == NC_F32 && nci_is_dense(dst))
        return device_relayout(dst, src) ? NC_OK : NC_ERR_DEVICE;
    for (size_t i = 0; i < dst->numel; i++) nc_tensor_set_flat(dst, i, nc_tensor_get_flat(src, i));
    return NC_OK;
}
void nc_tensor_to_device(nc_tensor* t, nc_device_type device) {
    if (!t || !t->storage) return;
    nc_storage_to_device(t->storage, device);
    if (t->grad) nc_tensor_to_device(t->grad, device);
}
void nc_tensor_print_shape(const nc_tensor* t) {
    if (!t) { printf("(null)\n"); return; }
    printf("(");
    for (size_t i = 0; i < t->ndim; i++) printf(i ? ", %zu" : "%zu", t->shape[i]);
    printf(") %s %s\n", nc_dtype_to_string(t->dtype), nci_on_cuda(t) ? "cuda" : "cpu");
}
void nc_tensor_print(const nc_tensor* t) {
    nc_tensor_print_shape(t);
    if (!t) return;
    size_t n = t->numel < 16 ? t->numel : 16;
    printf("[");
    for (size_t i = 0; i < n; i++) printf(i ? ", %g" : "%g", nc_tensor_get_flat(t, i));
    printf(t->numel > n ? ", ...]\n" : "]\n");
}
