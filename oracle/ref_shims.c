/*
 * Test infrastructure (not product code): small helpers linked into the reference CPU
 * library when it is built as the parity oracle.  They use only the reference's public
 * headers (nocta/nocta.h) and add what the reference lacks for whole-step runs:
 *
 *   - shim_flatten: (N,C,H,W) -> (N,C*H*W) view WITH an autograd node.  The reference's
 *     nc_flatten / nc_tensor_reshape return a leaf-like view without grad_fn
 *     (src/nn/conv.c:937-954, src/core/tensor.c:442-460), and its own example patches this
 *     in user code (examples/mnist.c:198-222).  Same idea, written fresh here.
 *   - shim_gelu: nc_gelu forward (src/ops/activation.c:289-310) plus an autograd node;
 *     the reference has no GELU backward.  The derivative is the analytic derivative of the
 *     tanh approximation used by the forward, evaluated in double.  PARITY UNPINNED for
 *     this op: there is no reference implementation of the backward to compare with.
 *   - shim_* accessors so the Python harness never depends on struct layout.
 */
#include "nocta/nocta.h"
#include <math.h>
#include <string.h>

static nc_tensor** shim_bwd_view(nc_tensor* grad, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = nc_calloc(1, sizeof(nc_tensor*));
    if (!out) return NULL;
    nc_tensor* src = saved[0];
    nc_tensor* g = nc_tensor_contiguous(grad);
    nc_tensor* v = nc_tensor_reshape(g, src->shape, src->ndim);
    /* hand back an independent copy so freeing the edge gradient never touches `grad` */
    out[0] = nc_tensor_clone(v);
    if (v != g) nc_tensor_free(v);
    if (g != grad) nc_tensor_free(g);
    return out;
}

static void shim_attach(nc_tensor* out, nc_tensor* in, const char* name, nc_backward_fn fn) {
    nc_node* nd = nc_node_create(name, fn);
    nc_node_add_input(nd, in);
    nc_node_save_tensor(nd, in);
    nd->output = out;
    out->grad_fn = nd;
    out->is_leaf = false;
    out->requires_grad = true;
}

nc_tensor* shim_flatten(nc_tensor* x) {
    if (!x) return NULL;
    size_t shp[2] = { x->shape[0], x->shape[0] ? x->numel / x->shape[0] : 0 };
    nc_tensor* y = nc_tensor_reshape(x, shp, 2);
    if (y && x->requires_grad) shim_attach(y, x, "shim_flatten", shim_bwd_view);
    return y;
}

static nc_tensor** shim_bwd_gelu(nc_tensor* grad, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = nc_calloc(1, sizeof(nc_tensor*));
    if (!out) return NULL;
    nc_tensor* x = saved[0];
    nc_tensor* dx = nc_tensor_empty(x->shape, x->ndim, x->dtype);
    const double c = sqrt(2.0 / 3.14159265358979323846), a = 0.044715;
    for (size_t i = 0; i < x->numel; i++) {
        double v = nc_tensor_get_flat(x, i);
        double u = c * (v + a * v * v * v);
        double th = tanh(u);
        double d = 0.5 * (1.0 + th) + 0.5 * v * (1.0 - th * th) * c * (1.0 + 3.0 * a * v * v);
        nc_tensor_set_flat(dx, i, nc_tensor_get_flat(grad, i) * d);
    }
    out[0] = dx;
    return out;
}

nc_tensor* shim_gelu(nc_tensor* x) {
    nc_tensor* y = nc_gelu(x);
    if (y && x->requires_grad) shim_attach(y, x, "shim_gelu", shim_bwd_gelu);
    return y;
}

/* ---- layout-independent accessors for the Python harness ---- */
void*      shim_data(nc_tensor* t)            { return nc_tensor_data(t); }
nc_tensor* shim_grad(nc_tensor* t)            { return t ? t->grad : NULL; }
size_t     shim_numel(nc_tensor* t)           { return t ? t->numel : 0; }
size_t     shim_ndim(nc_tensor* t)            { return t ? t->ndim : 0; }
size_t     shim_shape(nc_tensor* t, size_t i) { return (t && i < t->ndim) ? t->shape[i] : 0; }
size_t     shim_stride(nc_tensor* t, size_t i){ return (t && i < t->ndim) ? t->strides[i] : 0; }
int        shim_dtype(nc_tensor* t)           { return t ? (int)t->dtype : -1; }
int        shim_requires_grad(nc_tensor* t)   { return t ? (int)t->requires_grad : 0; }
int        shim_has_grad_fn(nc_tensor* t)     { return (t && t->grad_fn) ? 1 : 0; }
size_t     shim_module_nparams(nc_module* m)  { return m ? m->n_params : 0; }
nc_tensor* shim_module_param(nc_module* m, size_t i) { return (m && i < m->n_params) ? m->params[i] : NULL; }
const char* shim_module_param_name(nc_module* m, size_t i) { return (m && i < m->n_params) ? m->param_names[i] : NULL; }
size_t     shim_opt_t(nc_optimizer* o)        { return o ? o->t : 0; }
size_t     shim_opt_nparams(nc_optimizer* o)  { return o ? o->n_params : 0; }
int        shim_last_error(void)              { return (int)nc_last_error; }
