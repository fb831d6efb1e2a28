/*
 * Tensor ops on the training path: elementwise arithmetic with the two broadcast forms the path
 * uses, 2-D matmul, ReLU, GELU, softmax, axis sum, argmax, cross-entropy and MSE — each a thin host
 * wrapper that allocates the result, calls one nc_cuda_* kernel and records an autograd node.
 * Semantics follow the reference CPU code (src/ops/arithmetic.c:317-533,795-817, matmul.c:33-62,
 * 503-546, activation.c:33-70,195-225,289-310,373-430, reduction.c:158-198,473-513,
 * loss.c:33-137,176-351).  GELU gets a backward here (the reference registers none).
 */
#include "internal.h"

static bool want_grad(const nc_tensor* a, const nc_tensor* b) {
    return nc_grad_enabled() && ((a && a->requires_grad) || (b && b->requires_grad));
}
static nc_tensor** grad_array(size_t n) { return nc_calloc(n, sizeof(nc_tensor*)); }

/* dense operand in the layout of `like` (same shape); returns t itself when it already matches */
static nc_tensor* operand_like(nc_tensor* t, const nc_tensor* like) { return nci_match_layout(t, like); }

/* ------------------------------------------------------------------ elementwise binary */
/* shapes equal -> plain; b is 1-D of length a.shape[last] -> row broadcast (bias add) */
/* b is one row of a: its last dimension equals a's and every other dimension of b is 1 ((8), (1, 8), (1, 1, 8) ...) */
static bool is_row_of(const nc_tensor* a, const nc_tensor* b) {
    if (a->ndim < 1 || b->ndim < 1 || b->ndim > a->ndim || !b->is_contiguous) return false;
    if (b->shape[b->ndim - 1] != a->shape[a->ndim - 1] || b->numel != b->shape[b->ndim - 1]) return false;
    return true;
}
static int classify(const nc_tensor* a, const nc_tensor* b) {
    if (nc_tensor_shape_eq(a, b)) return 0;
    if (is_row_of(a, b) && a->is_contiguous) return 1;
    if (b->numel == 1) return 2;
    return -1;
}

static nc_tensor** bwd_add(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(2);
    if (!out) return NULL;
    nc_tensor* a = saved[0];
    nc_tensor* b = saved[1];
    if (a->requires_grad) out[0] = nci_alias(g);
    if (b->requires_grad) {
        if (nc_tensor_shape_eq(a, b)) out[1] = nci_alias(g);
        else {
            /* the reference's reduce_grad_to_shape (src/ops/arithmetic.c:53-127): a 1-D operand (bias) gets the column
             * sums, a one-element operand the sum of everything, and any other broadcast operand (e.g. a (1, C)
             * matrix) gets the FIRST numel elements of the gradient, i.e. its first row only.  The last rule is
             * reproduced as it is so that programs written against the reference train identically. */
            nc_tensor* gc = nc_tensor_contiguous(g);
            out[1] = nci_empty_on(b->shape, b->ndim, NC_F32, NC_DEVICE_CUDA);
            if (gc && out[1]) {
                size_t cols = b->numel, rows = g->numel / (cols ? cols : 1);
                if (b->ndim == 1 || b->numel == 1)
                    nci_ok(nc_cuda_sum_axis_f32_ex(nci_fptr(out[1]), nci_fptr(gc), 1, rows, cols, nci_stream()), "add backward");
                else
                    nc_cuda_memcpy_d2d(nci_dptr(out[1]), nci_dptr(gc), b->numel * sizeof(float));
            }
            if (gc && gc != g) nc_tensor_free(gc);
        }
    }
    return out;
}
static nc_tensor** bwd_sub(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(2);
    if (!out) return NULL;
    if (saved[0]->requires_grad) out[0] = nci_alias(g);
    if (saved[1]->requires_grad) out[1] = nc_mul_scalar(g, -1.0);
    return out;
}
static nc_tensor** bwd_mul(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(2);
    if (!out) return NULL;
    if (saved[0]->requires_grad) out[0] = nc_mul(g, saved[1]);
    if (saved[1]->requires_grad) out[1] = nc_mul(g, saved[0]);
    return out;
}

static nc_tensor* binary(nc_tensor* a, nc_tensor* b, int op, const char* name, nc_backward_fn bwd) {
    if (!nci_need_cuda_f32(a, name) || !nci_need_cuda_f32(b, name)) return NULL;
    nci_round_outputs(true);
    int kind = classify(a, b);
    if (kind < 0 || (kind != 0 && op != 0)) {
        NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "%s: shapes must match (row-broadcast is supported for add only)", name);
        return NULL;
    }
    nc_tensor* out = NULL;
    if (kind == 0) {
        nc_tensor* ad = nci_is_dense(a) ? a : nc_tensor_contiguous(a);
        if (!ad) return NULL;
        nc_tensor* bd = operand_like(b, ad);
        if (!bd) { if (ad != a) nc_tensor_free(ad); return NULL; }
        out = nci_empty_like(ad);
        if (out && !nci_ok(nc_cuda_binary_f32_ex(op, nci_fptr(out), nci_fptr(ad), nci_fptr(bd), out->numel, nci_stream()), name)) {
            nc_tensor_free(out);
            out = NULL;
        }
        if (bd != b) nc_tensor_free(bd);
        if (ad != a) nc_tensor_free(ad);
    } else if (kind == 1) {
        out = nci_empty_like(a);
        if (out && !nci_ok(nc_cuda_add_broadcast_batch_f32_ex(nci_fptr(out), nci_fptr(a), nci_fptr(b), a->numel, (int)b->numel, nci_stream()), name)) {
            nc_tensor_free(out);
            out = NULL;
        }
    } else {
        double s = nc_tensor_get_flat(b, 0);
        return nc_add_scalar(a, s);
    }
    if (out && want_grad(a, b) && bwd) {
        nc_node* nd = nci_attach(out, name, bwd);
        if (nd) {
            nc_node_add_input(nd, a);
            nc_node_add_input(nd, b);
            nc_node_save_tensor(nd, a);
            nc_node_save_tensor(nd, b);
        }
    }
    return out;
}
nc_tensor* nc_add(nc_tensor* a, nc_tensor* b) { return binary(a, b, 0, "add", bwd_add); }
nc_tensor* nc_sub(nc_tensor* a, nc_tensor* b) { return binary(a, b, 1, "sub", bwd_sub); }
nc_tensor* nc_mul(nc_tensor* a, nc_tensor* b) { return binary(a, b, 2, "mul", bwd_mul); }

static nc_tensor** bwd_scale(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(1);
    if (out) out[0] = nc_mul_scalar(g, nc_tensor_get_flat(saved[0], 0));
    return out;
}
static nc_tensor** bwd_identity(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n; (void)saved;
    nc_tensor** out = grad_array(1);
    if (out) out[0] = nci_alias(g);
    return out;
}
static nc_tensor* scalar_op(nc_tensor* a, double s, int op, const char* name) {
    if (!nci_need_cuda_f32(a, name)) return NULL;
    nci_round_outputs(true);
    nc_tensor* ad = nci_is_dense(a) ? a : nc_tensor_contiguous(a);
    if (!ad) return NULL;
    nc_tensor* out = nci_empty_like(ad);
    if (out && !nci_ok(nc_cuda_scalar_f32_ex(op, nci_fptr(out), nci_fptr(ad), (float)s, out->numel, nci_stream()), name)) {
        nc_tensor_free(out);
        out = NULL;
    }
    if (ad != a) nc_tensor_free(ad);
    if (out && want_grad(a, NULL)) {
        nc_node* nd = nci_attach(out, name, op == 2 ? bwd_scale : bwd_identity);
        if (nd) {
            nc_node_add_input(nd, a);
            if (op == 2) nc_node_save_owned_tensor(nd, nc_tensor_scalar(s, NC_F64));
        }
    }
    return out;
}
nc_tensor* nc_add_scalar(nc_tensor* a, double s) { return scalar_op(a, s, 0, "add_scalar"); }
nc_tensor* nc_mul_scalar(nc_tensor* a, double s) { return scalar_op(a, s, 2, "mul_scalar"); }

void nc_add_(nc_tensor* a, nc_tensor* b) {
    if (!a || !b) return;
    if (!nci_need_cuda_f32(a, "add_") || !nci_need_cuda_f32(b, "add_")) return;
    if (a->numel != b->numel) { NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "add_: %zu vs %zu elements", a->numel, b->numel); return; }
    if (!nci_is_dense(a)) { NC_SET_ERROR(NC_ERR_NOT_CONTIGUOUS, "add_: destination must be dense"); return; }
    nc_tensor* bd = operand_like(b, a);
    if (!bd) return;
    nci_round_outputs(false); /* accumulation (e.g. into parameter gradients) keeps full f32 */
    nci_ok(nc_cuda_binary_f32_ex(0, nci_fptr(a), nci_fptr(a), nci_fptr(bd), a->numel, nci_stream()), "add_");
    if (bd != b) nc_tensor_free(bd);
}
void nc_mul_scalar_(nc_tensor* a, double s) {
    if (!nci_need_cuda_f32(a, "mul_scalar_") || !nci_is_dense(a)) return;
    nci_round_outputs(false);
    nci_ok(nc_cuda_scalar_f32_ex(2, nci_fptr(a), nci_fptr(a), (float)s, a->numel, nci_stream()), "mul_scalar_");
}

/* ------------------------------------------------------------------ matmul (2-D) */
/* describe a 2-D tensor to the GEMM entry: row-major (ld, trans=0) or its transpose (ld, trans=1) */
static bool mat_desc(const nc_tensor* t, int* ld, int* trans) {
    if (t->strides[1] == 1 || t->shape[1] == 1) { *ld = (int)(t->shape[0] == 1 ? t->shape[1] : t->strides[0]); *trans = 0; return true; }
    if (t->strides[0] == 1 || t->shape[0] == 1) { *ld = (int)(t->shape[1] == 1 ? t->shape[0] : t->strides[1]); *trans = 1; return true; }
    return false;
}
static nc_tensor* matmul_raw(nc_tensor* a, nc_tensor* b) {
    size_t M = a->shape[0], K = a->shape[1], N = b->shape[1];
    int lda, ta, ldb, tb;
    nc_tensor* ac = mat_desc(a, &lda, &ta) ? a : nc_tensor_contiguous(a);
    nc_tensor* bc = mat_desc(b, &ldb, &tb) ? b : nc_tensor_contiguous(b);
    nc_tensor* out = NULL;
    if (ac && bc) {
        mat_desc(ac, &lda, &ta);
        mat_desc(bc, &ldb, &tb);
        size_t shape[2] = {M, N};
        out = nci_empty_on(shape, 2, NC_F32, NC_DEVICE_CUDA);
        if (out && !nci_ok(nc_cuda_matmul_f32_ex(nci_fptr(out), (int)N, nci_fptr(ac), lda, nci_fptr(bc), ldb, (int)M, (int)N, (int)K,
                                                 1.f, 0.f, ta, tb, NULL, nci_stream()), "matmul")) {
            nc_tensor_free(out);
            out = NULL;
        }
    }
    if (ac && ac != a) nc_tensor_free(ac);
    if (bc && bc != b) nc_tensor_free(bc);
    return out;
}
static nc_tensor** bwd_matmul(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(2);
    if (!out) return NULL;
    nc_tensor* a = saved[0];
    nc_tensor* b = saved[1];
    if (a->requires_grad) { nc_tensor* bt = nc_tensor_t(b); if (bt) { out[0] = matmul_raw(g, bt); nc_tensor_free(bt); } }
    if (b->requires_grad) { nc_tensor* at = nc_tensor_t(a); if (at) { out[1] = matmul_raw(at, g); nc_tensor_free(at); } }
    return out;
}
nc_tensor* nc_matmul(nc_tensor* a, nc_tensor* b) {
    if (!nci_need_cuda_f32(a, "matmul") || !nci_need_cuda_f32(b, "matmul")) return NULL;
    if (a->ndim != 2 || b->ndim != 2 || a->shape[1] != b->shape[0]) {
        NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "matmul: expected (M,K) x (K,N)");
        return NULL;
    }
    nc_tensor* out = matmul_raw(a, b);
    if (out && want_grad(a, b)) {
        nc_node* nd = nci_attach(out, "matmul", bwd_matmul);
        if (nd) { nc_node_add_input(nd, a); nc_node_add_input(nd, b); nc_node_save_tensor(nd, a); nc_node_save_tensor(nd, b); }
    }
    return out;
}

/* ------------------------------------------------------------------ activations */
static nc_tensor** bwd_relu(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(1);
    if (!out) return NULL;
    nc_tensor* x = saved[0];
    nc_tensor* gd = operand_like(g, x);
    if (!gd) return out;
    out[0] = nci_empty_like(x);
    nci_round_outputs(true);
    if (out[0]) nci_ok(nc_cuda_relu_backward_f32_ex(nci_fptr(out[0]), nci_fptr(gd), nci_fptr(x), x->numel, nci_stream()), "relu backward");
    if (gd != g) nc_tensor_free(gd);
    return out;
}
static nc_tensor** bwd_gelu(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(1);
    if (!out) return NULL;
    nc_tensor* x = saved[0];
    nc_tensor* gd = operand_like(g, x);
    if (!gd) return out;
    out[0] = nci_empty_like(x);
    nci_round_outputs(true);
    if (out[0]) nci_ok(nc_cuda_gelu_backward_f32_ex(nci_fptr(out[0]), nci_fptr(gd), nci_fptr(x), x->numel, nci_stream()), "gelu backward");
    if (gd != g) nc_tensor_free(gd);
    return out;
}
static nc_tensor** bwd_sigmoid(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(1);
    if (!out) return NULL;
    nc_tensor* x = saved[0];
    nc_tensor* gd = operand_like(g, x);
    if (!gd) return out;
    out[0] = nci_empty_like(x);
    nci_round_outputs(true);
    if (out[0]) nci_ok(nc_cuda_sigmoid_backward_f32_ex(nci_fptr(out[0]), nci_fptr(gd), nci_fptr(x), x->numel, nci_stream()), "sigmoid backward");
    if (gd != g) nc_tensor_free(gd);
    return out;
}
typedef int (*unary_kernel)(float*, const float*, size_t, void*);
static nc_tensor* unary(nc_tensor* x, unary_kernel k, const char* name, nc_backward_fn bwd) {
    if (!nci_need_cuda_f32(x, name)) return NULL;
    nci_round_outputs(true);
    nc_tensor* xd = nci_is_dense(x) ? x : nc_tensor_contiguous(x);
    if (!xd) return NULL;
    nc_tensor* out = nci_empty_like(xd);
    if (out && !nci_ok(k(nci_fptr(out), nci_fptr(xd), out->numel, nci_stream()), name)) { nc_tensor_free(out); out = NULL; }
    if (out && want_grad(x, NULL)) {
        nc_node* nd = nci_attach(out, name, bwd);
        if (nd) {
            nc_node_add_input(nd, x);
            if (xd != x) { nc_node_save_owned_tensor(nd, xd); xd = x; } /* keep the dense copy for backward */
            else nc_node_save_tensor(nd, x);
        }
    }
    if (xd != x) nc_tensor_free(xd);
    return out;
}
nc_tensor* nc_relu(nc_tensor* x) { return unary(x, nc_cuda_relu_f32_ex, "relu", bwd_relu); }
nc_tensor* nc_gelu(nc_tensor* x) { return unary(x, nc_cuda_gelu_f32_ex, "gelu", bwd_gelu); }
nc_tensor* nc_sigmoid(nc_tensor* x) { return unary(x, nc_cuda_sigmoid_f32_ex, "sigmoid", bwd_sigmoid); }

nc_tensor* nc_softmax(nc_tensor* x, int dim) {
    if (!nci_need_cuda_f32(x, "softmax")) return NULL;
    if (dim < 0) dim += (int)x->ndim;
    if (dim != (int)x->ndim - 1 || x->ndim < 1) { NC_SET_ERROR(NC_ERR_INVALID_AXIS, "softmax: only the last dimension is supported on the device"); return NULL; }
    nc_tensor* xc = nc_tensor_contiguous(x);
    if (!xc) return NULL;
    nc_tensor* out = nci_empty_on(x->shape, x->ndim, NC_F32, NC_DEVICE_CUDA);
    size_t cols = x->shape[x->ndim - 1];
    if (out && !nci_ok(nc_cuda_softmax_f32_ex(nci_fptr(out), nci_fptr(xc), cols ? x->numel / cols : 0, cols, nci_stream()), "softmax")) {
        nc_tensor_free(out);
        out = NULL;
    }
    if (xc != x) nc_tensor_free(xc);
    return out; /* inference helper: the losses differentiate through their own fused kernel */
}

/* ------------------------------------------------------------------ reductions */
nc_tensor* nc_sum(nc_tensor* x, int axis, bool keepdim) {
    if (!nci_need_cuda_f32(x, "sum")) return NULL;
    if (axis < 0) axis += (int)x->ndim;
    if (axis < 0 || (size_t)axis >= x->ndim) { NC_SET_ERROR(NC_ERR_INVALID_AXIS, "sum: bad axis"); return NULL; }
    nc_tensor* xc = nc_tensor_contiguous(x);
    if (!xc) return NULL;
    size_t outer = 1, inner = 1, red = x->shape[axis];
    for (int i = 0; i < axis; i++) outer *= x->shape[i];
    for (size_t i = (size_t)axis + 1; i < x->ndim; i++) inner *= x->shape[i];
    size_t shape[NC_MAX_DIMS], nd = 0;
    for (size_t i = 0; i < x->ndim; i++) {
        if ((int)i == axis) { if (keepdim) shape[nd++] = 1; }
        else shape[nd++] = x->shape[i];
    }
    nc_tensor* out = nci_empty_on(shape, nd, NC_F32, NC_DEVICE_CUDA);
    if (out && !nci_ok(nc_cuda_sum_axis_f32_ex(nci_fptr(out), nci_fptr(xc), outer, red, inner, nci_stream()), "sum")) {
        nc_tensor_free(out);
        out = NULL;
    }
    if (xc != x) nc_tensor_free(xc);
    return out;
}
static nc_tensor** bwd_sum_all(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(1);
    if (!out) return NULL;
    nc_tensor* x = saved[0];
    double scale = nc_tensor_get_flat(saved[1], 0) * (nci_is_unit_seed(g) ? 1.0 : nc_tensor_get_flat(g, 0));
    out[0] = nci_empty_like(x);
    if (out[0]) nci_ok(nc_cuda_fill_f32_ex(nci_fptr(out[0]), (float)scale, x->numel, nci_stream()), "sum backward");
    return out;
}
static nc_tensor* reduce_all(nc_tensor* x, bool mean) {
    if (!nci_need_cuda_f32(x, "sum_all")) return NULL;
    nc_tensor* xd = nci_is_dense(x) ? x : nc_tensor_contiguous(x);
    if (!xd) return NULL;
    nc_tensor* out = nci_empty_on(NULL, 0, NC_F32, NC_DEVICE_CUDA);
    if (out && !nci_ok(nc_cuda_sum_axis_f32_ex(nci_fptr(out), nci_fptr(xd), 1, xd->numel, 1, nci_stream()), "sum_all")) {
        nc_tensor_free(out);
        out = NULL;
    }
    if (out && mean && x->numel) nc_mul_scalar_(out, 1.0 / (double)x->numel);
    if (out && want_grad(x, NULL) && nci_is_dense(x)) {
        nc_node* nd = nci_attach(out, mean ? "mean_all" : "sum_all", bwd_sum_all);
        if (nd) {
            nc_node_add_input(nd, x);
            nc_node_save_tensor(nd, x);
            nc_node_save_owned_tensor(nd, nc_tensor_scalar(mean && x->numel ? 1.0 / (double)x->numel : 1.0, NC_F64));
        }
    }
    if (xd != x) nc_tensor_free(xd);
    return out;
}
nc_tensor* nc_sum_all(nc_tensor* x) { return reduce_all(x, false); }
nc_tensor* nc_mean_all(nc_tensor* x) { return reduce_all(x, true); }

nc_tensor* nc_argmax(nc_tensor* x, int axis, bool keepdim) {
    if (!nci_need_cuda_f32(x, "argmax")) return NULL;
    if (axis < 0) axis += (int)x->ndim;
    if (x->ndim != 2 || axis != 1) { NC_SET_ERROR(NC_ERR_INVALID_AXIS, "argmax: only (rows, cols) over axis 1 is supported on the device"); return NULL; }
    nc_tensor* xc = nc_tensor_contiguous(x);
    if (!xc) return NULL;
    size_t shape[2] = {x->shape[0], 1};
    nc_tensor* out = nci_empty_on(shape, keepdim ? 2 : 1, NC_I64, NC_DEVICE_CUDA);
    if (out && !nci_ok(nc_cuda_argmax_rows_f32_ex((int64_t*)nci_dptr(out), nci_fptr(xc), x->shape[0], x->shape[1], nci_stream()), "argmax")) {
        nc_tensor_free(out);
        out = NULL;
    }
    if (xc != x) nc_tensor_free(xc);
    return out;
}

/* ------------------------------------------------------------------ losses
 * The forward kernel also produces the gradient w.r.t. its input for an upstream gradient of 1;
 * the node owns it and backward scales it only when the upstream value differs from 1.          */
static nc_tensor** bwd_saved_grad(nc_tensor* g, nc_tensor** saved, size_t n) {
    nc_tensor** out = grad_array(2);
    if (!out) return NULL;
    double up = nci_is_unit_seed(g) ? 1.0 : nc_tensor_get_flat(g, 0);
    nc_tensor* gi = saved[n - 1];
    out[0] = (up == 1.0) ? nci_alias(gi) : nc_mul_scalar(gi, up);
    return out;
}
static nc_tensor** bwd_mse(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(2);
    if (!out) return NULL;
    double up = nci_is_unit_seed(g) ? 1.0 : nc_tensor_get_flat(g, 0);
    nc_tensor* pred = saved[0];
    nc_tensor* target = saved[1];
    nc_tensor* gp = saved[2];
    if (pred->requires_grad) out[0] = (up == 1.0) ? nci_alias(gp) : nc_mul_scalar(gp, up);
    if (target->requires_grad) out[1] = nc_mul_scalar(gp, -up);
    return out;
}

nc_tensor* nc_cross_entropy_loss_ex(nc_tensor* logits, nc_tensor* targets, nc_reduction reduction) {
    if (!nci_need_cuda_f32(logits, "cross_entropy")) return NULL;
    if (!targets) { NC_SET_ERROR(NC_ERR_NULL_PTR, "cross_entropy: null targets"); return NULL; }
    if (logits->ndim != 2 || targets->numel != logits->shape[0]) { NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "cross_entropy: logits (N,C), targets (N)"); return NULL; }
    nc_tensor* converted = NULL;
    if (targets->dtype != NC_I64 || !nci_on_cuda(targets)) {
        /* The reference reads class indices from a tensor of any dtype (src/ops/loss.c:218-232); its script VM passes
         * float32.  The kernel wants int64 on the device: convert through the host (N values, off the hot path). */
        const size_t n = targets->numel;
        int64_t* idx = nc_alloc(sizeof(int64_t) * (n ? n : 1));
        if (!idx) return NULL;
        nc_tensor* th = nc_tensor_clone(targets);
        if (th && nci_on_cuda(th)) nc_tensor_to_device(th, NC_DEVICE_CPU);
        if (!th) { nc_free(idx); return NULL; }
        for (size_t i = 0; i < n; i++) idx[i] = (int64_t)nc_tensor_get_flat(th, i);
        nc_tensor_free(th);
        size_t shp = n;
        converted = nc_tensor_from_data(idx, &shp, 1, NC_I64);
        nc_free(idx);
        if (converted && !nci_on_cuda(converted)) nc_tensor_to_device(converted, NC_DEVICE_CUDA);
        if (!converted || !nci_on_cuda(converted)) { nc_tensor_free(converted); NC_SET_ERROR(NC_ERR_DEVICE, "cross_entropy: cannot stage the targets on the device"); return NULL; }
        nc_tensor* out = nc_cross_entropy_loss_ex(logits, converted, reduction);
        /* the node keeps the converted targets alive through its input list only while it owns them: it does not, so
         * detach them from the graph before they go (targets never receive a gradient) */
        if (out && out->grad_fn) for (size_t i = 0; i < out->grad_fn->n_inputs; i++) if (out->grad_fn->inputs[i] == converted) out->grad_fn->inputs[i] = NULL;
        nc_tensor_free(converted);
        return out;
    }
    if (reduction == NC_REDUCTION_NONE) { NC_SET_ERROR(NC_ERR_UNKNOWN, "cross_entropy: per-sample losses are not available on the device"); return NULL; }
    nc_tensor* lc = nc_tensor_contiguous(logits);
    nc_tensor* tc = nc_tensor_contiguous(targets);
    if (!lc || !tc) return NULL;
    const bool need = want_grad(logits, NULL);
    nc_tensor* loss = nci_empty_on(NULL, 0, NC_F32, NC_DEVICE_CUDA);
    nc_tensor* grad = need ? nci_empty_on(logits->shape, 2, NC_F32, NC_DEVICE_CUDA) : NULL;
    int N = (int)logits->shape[0], C = (int)logits->shape[1];
    nci_round_outputs(true);
    float gscale = reduction == NC_REDUCTION_SUM ? (float)N : 1.f;
    bool ok = loss && (!need || grad) &&
              nci_ok(nc_cuda_cross_entropy_fused_f32_ex(nci_fptr(loss), grad ? nci_fptr(grad) : NULL, nci_fptr(lc),
                                                        (const int64_t*)nci_dptr(tc), N, C, gscale, nci_stream()), "cross_entropy");
    if (ok && reduction == NC_REDUCTION_SUM) nc_mul_scalar_(loss, (double)N);
    if (lc != logits) nc_tensor_free(lc);
    if (tc != targets) nc_tensor_free(tc);
    if (!ok) { nc_tensor_free(loss); nc_tensor_free(grad); return NULL; }
    if (need) {
        nc_node* nd = nci_attach(loss, "cross_entropy", bwd_saved_grad);
        if (nd) {
            nc_node_add_input(nd, logits);
            nc_node_add_input(nd, targets);
            nc_node_save_tensor(nd, logits);
            nc_node_save_owned_tensor(nd, grad);
        } else nc_tensor_free(grad);
    }
    return loss;
}
nc_tensor* nc_cross_entropy_loss(nc_tensor* logits, nc_tensor* targets) { return nc_cross_entropy_loss_ex(logits, targets, NC_REDUCTION_MEAN); }

nc_tensor* nc_mse_loss(nc_tensor* pred, nc_tensor* target) {
    if (!nci_need_cuda_f32(pred, "mse_loss") || !nci_need_cuda_f32(target, "mse_loss")) return NULL;
    if (pred->numel != target->numel) { NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "mse_loss: element counts differ"); return NULL; }
    nc_tensor* pd = nci_is_dense(pred) ? pred : nc_tensor_contiguous(pred);
    if (!pd) return NULL;
    nc_tensor* td = operand_like(target, pd);
    if (!td) { if (pd != pred) nc_tensor_free(pd); return NULL; }
    const bool need = want_grad(pred, target);
    nc_tensor* loss = nci_empty_on(NULL, 0, NC_F32, NC_DEVICE_CUDA);
    nc_tensor* gp = need ? nci_empty_like(pd) : NULL;
    nci_round_outputs(true);
    bool ok = loss && (!need || gp) &&
              nci_ok(nc_cuda_mse_fused_f32_ex(nci_fptr(loss), gp ? nci_fptr(gp) : NULL, NULL, nci_fptr(pd), nci_fptr(td), pd->numel, 1.f,
                                              nci_stream()), "mse_loss");
    if (td != target) nc_tensor_free(td);
    if (pd != pred) nc_tensor_free(pd);
    if (!ok) { nc_tensor_free(loss); nc_tensor_free(gp); return NULL; }
    if (need) {
        nc_node* nd = nci_attach(loss, "mse_loss", bwd_mse);
        if (nd) {
            nc_node_add_input(nd, pred);
            nc_node_add_input(nd, target);
            nc_node_save_tensor(nd, pred);
            nc_node_save_tensor(nd, target);
            nc_node_save_owned_tensor(nd, gp);
        } else nc_tensor_free(gp);
    }
    return loss;
}
