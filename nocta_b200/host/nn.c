/*
 * Modules and layers: the nc_module registry, Linear, Conv2d, MaxPool2d, Flatten, BatchNorm2d,
 * LayerNorm and mask-supplied dropout.  Each forward allocates its output from the device pool,
 * calls the kernel library and records one autograd node; each backward is one or two kernel calls.
 *
 * API and semantics follow the reference (src/nn/module.c:5-181, linear.c:45-228, conv.c:118-375,
 * 381-653,672-882,937-954, batchnorm.c:43-165,171-455,600-702,946-1085).  Device layout policy:
 * conv / batchnorm / relu / maxpool outputs are channels-last in memory (shape stays (N,C,H,W)),
 * which is the layout the tensor-core implicit-GEMM kernels read with TMA; nc_flatten converts back
 * to dense NCHW order so the Linear weights keep the reference's (C,H,W) column order.
 */
#include "internal.h"
#include <stdlib.h>
#include <math.h>

static nc_tensor** grad_array(size_t n) { return nc_calloc(n, sizeof(nc_tensor*)); }
static bool any_grad(nc_tensor* a, nc_tensor* b, nc_tensor* c) {
    return nc_grad_enabled() && ((a && a->requires_grad) || (b && b->requires_grad) || (c && c->requires_grad));
}

/* ------------------------------------------------------------------ module registry */
nc_module* nc_module_create(const char* name) {
    nc_module* m = nc_calloc(1, sizeof(nc_module));
    if (!m) return NULL;
    if (name) strncpy(m->name, name, NC_MAX_NAME_LEN - 1);
    m->training = true;
    return m;
}
void nc_module_free(nc_module* m) {
    if (!m) return;
    for (size_t i = 0; i < m->n_params; i++) { nc_tensor_free(m->params[i]); nc_free(m->param_names[i]); }
    for (size_t i = 0; i < m->n_submodules; i++) { nc_module_free(m->submodules[i]); nc_free(m->submodule_names[i]); }
    if (m->extra && m->free_extra) m->free_extra(m->extra);
    nc_free(m);
}
nc_tensor* nc_module_forward(nc_module* m, nc_tensor* input) { return (m && m->forward) ? m->forward(m, input) : NULL; }
static char* dup_name(const char* s) {
    char* d = nc_alloc(strlen(s) + 1);
    if (d) strcpy(d, s);
    return d;
}
void nc_module_add_param(nc_module* m, const char* name, nc_tensor* param) {
    if (!m || !param || !name || m->n_params >= NC_MAX_PARAMS) return;
    m->params[m->n_params] = param;
    m->param_names[m->n_params] = dup_name(name);
    m->n_params++;
    /* as in the reference, every registered tensor gets gradient tracking (src/nn/module.c:55-56) */
    nc_tensor_requires_grad_(param, true);
}
void nc_module_add_submodule(nc_module* m, const char* name, nc_module* sub) {
    if (!m || !sub || !name || m->n_submodules >= NC_MAX_SUBMODULES) return;
    m->submodules[m->n_submodules] = sub;
    m->submodule_names[m->n_submodules] = dup_name(name);
    m->n_submodules++;
}
nc_tensor* nc_module_get_param(nc_module* m, const char* name) {
    if (!m || !name) return NULL;
    for (size_t i = 0; i < m->n_params; i++) if (m->param_names[i] && !strcmp(m->param_names[i], name)) return m->params[i];
    return NULL;
}
nc_module* nc_module_get_submodule(nc_module* m, const char* name) {
    if (!m || !name) return NULL;
    for (size_t i = 0; i < m->n_submodules; i++) if (m->submodule_names[i] && !strcmp(m->submodule_names[i], name)) return m->submodules[i];
    return NULL;
}
static void walk_params(nc_module* m, const char* prefix, nc_param_callback cb, void* ctx) {
    char full[256];
    for (size_t i = 0; i < m->n_params; i++) {
        snprintf(full, sizeof(full), prefix[0] ? "%s.%s" : "%s%s", prefix, m->param_names[i] ? m->param_names[i] : "");
        cb(full, m->params[i], ctx);
    }
    for (size_t i = 0; i < m->n_submodules; i++) {
        snprintf(full, sizeof(full), prefix[0] ? "%s.%s" : "%s%s", prefix, m->submodule_names[i] ? m->submodule_names[i] : "");
        walk_params(m->submodules[i], full, cb, ctx);
    }
}
void nc_module_parameters(nc_module* m, nc_param_callback cb, void* ctx) { if (m && cb) walk_params(m, "", cb, ctx); }
static void cb_count(const char* n, nc_tensor* p, void* ctx) { (void)n; *(size_t*)ctx += p->numel; }
size_t nc_module_num_parameters(nc_module* m) { size_t c = 0; nc_module_parameters(m, cb_count, &c); return c; }
void nc_module_train(nc_module* m, bool mode) {
    if (!m) return;
    m->training = mode;
    for (size_t i = 0; i < m->n_submodules; i++) nc_module_train(m->submodules[i], mode);
}
static void cb_zero(const char* n, nc_tensor* p, void* ctx) { (void)n; (void)ctx; nc_tensor_zero_grad_(p); }
void nc_module_zero_grad(nc_module* m) { nc_module_parameters(m, cb_zero, NULL); }
static void cb_reqgrad(const char* n, nc_tensor* p, void* ctx) { (void)n; nc_tensor_requires_grad_(p, *(bool*)ctx); }
void nc_module_requires_grad_(nc_module* m, bool rg) { nc_module_parameters(m, cb_reqgrad, &rg); }
static void cb_todev(const char* n, nc_tensor* p, void* ctx) { (void)n; nc_tensor_to_device(p, *(nc_device_type*)ctx); }
void nc_module_to_device(nc_module* m, nc_device_type device) { nc_module_parameters(m, cb_todev, &device); }
static void cb_print(const char* n, nc_tensor* p, void* ctx) { (void)ctx; printf("  %-32s ", n); nc_tensor_print_shape(p); }
void nc_module_print(nc_module* m) {
    if (!m) return;
    printf("%s (%zu parameters)\n", m->name, nc_module_num_parameters(m));
    nc_module_parameters(m, cb_print, NULL);
}

/* host-initialised parameter, placed on the default device */
static nc_tensor* param_from_host(const float* host, const size_t* shape, size_t ndim) { return nc_tensor_from_data(host, shape, ndim, NC_F32); }
static nc_tensor* param_const(const size_t* shape, size_t ndim, float v) {
    size_t n = 1;
    for (size_t i = 0; i < ndim; i++) n *= shape[i];
    float* h = nc_alloc(sizeof(float) * (n ? n : 1));
    if (!h) return NULL;
    for (size_t i = 0; i < n; i++) h[i] = v;
    nc_tensor* t = param_from_host(h, shape, ndim);
    nc_free(h);
    return t;
}
static nc_tensor* param_random(const size_t* shape, size_t ndim, bool normal, double scale) {
    /* draw on the host through the seeded generator, then place on the default device */
    nc_device_type dev = nc_get_default_device();
    nc_set_default_device(NC_DEVICE_CPU);
    nc_tensor* r = normal ? nc_tensor_randn(shape, ndim, NC_F32) : nc_tensor_rand(shape, ndim, NC_F32);
    nc_set_default_device(dev);
    if (!r) return NULL;
    float* p = nc_tensor_data_f32(r);
    for (size_t i = 0; i < r->numel; i++) p[i] = (float)((normal ? p[i] : (2.0 * p[i] - 1.0)) * scale);
    if (dev == NC_DEVICE_CUDA) nc_tensor_to_device(r, NC_DEVICE_CUDA);
    return r;
}

/* ------------------------------------------------------------------ Linear */
typedef struct { size_t in_f, out_f; bool has_bias; } linear_cfg;

static nc_tensor** bwd_linear(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(3);
    if (!out) return NULL;
    nc_tensor* x = saved[0];   /* (B, in) dense rows */
    nc_tensor* W = saved[1];   /* (out, in) */
    nc_tensor* b = saved[2];   /* may be NULL */
    nc_tensor* xin = saved[3]; /* the op's input (for requires_grad and its shape) */
    nc_tensor* gc = nc_tensor_contiguous(g);
    if (!gc) return out;
    const int B = (int)(x->numel / W->shape[1]), in_f = (int)W->shape[1], out_f = (int)W->shape[0];
    if (xin->requires_grad) out[0] = nci_empty_on(xin->shape, xin->ndim, NC_F32, NC_DEVICE_CUDA);
    if (W->requires_grad) out[1] = nci_param_grad_out(1, W);
    if (b && b->requires_grad) out[2] = nci_param_grad_out(2, b);
    nci_ok(nc_cuda_linear_backward_f32_ex(out[0] ? nci_fptr(out[0]) : NULL, out[1] ? nci_fptr(out[1]) : NULL,
                                          out[2] ? nci_fptr(out[2]) : NULL, nci_fptr(gc), nci_fptr(x), nci_fptr(W), B, in_f, out_f,
                                          nci_stream()), "linear backward");
    if (gc != g) nc_tensor_free(gc);
    return out;
}
nc_tensor* nc_linear_forward(nc_tensor* input, nc_tensor* weight, nc_tensor* bias) {
    if (!nci_need_cuda_f32(input, "linear") || !nci_need_cuda_f32(weight, "linear")) return NULL;
    if (bias && !nci_need_cuda_f32(bias, "linear")) return NULL;
    if (weight->ndim != 2 || input->ndim < 1 || input->shape[input->ndim - 1] != weight->shape[1] || !weight->is_contiguous) {
        NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "linear: input (..., in) and weight (out, in) required");
        return NULL;
    }
    nc_tensor* xc = nc_tensor_contiguous(input);
    if (!xc) return NULL;
    if (nci_tf32_mode() && input->is_leaf && !input->grad_fn && input->numel / weight->shape[1] >= 128) {
        /* caller-supplied data was not written by one of our kernels: give the tensor-core GEMMs a
         * copy rounded to the nearest TF32 value (kept for the weight-gradient GEMM as well) */
        nc_tensor* xr = nci_empty_on(xc->shape, xc->ndim, NC_F32, NC_DEVICE_CUDA);
        bool ok = xr && nci_ok(nc_cuda_round_tf32_f32_ex(nci_fptr(xr), nci_fptr(xc), xc->numel, nci_stream()), "linear (operand rounding)");
        if (xc != input) nc_tensor_free(xc);
        if (!ok) { nc_tensor_free(xr); return NULL; }
        xc = xr;
    }
    size_t shape[NC_MAX_DIMS];
    for (size_t i = 0; i + 1 < input->ndim; i++) shape[i] = input->shape[i];
    shape[input->ndim - 1] = weight->shape[0];
    const int in_f = (int)weight->shape[1], out_f = (int)weight->shape[0], B = (int)(input->numel / weight->shape[1]);
    nc_tensor* y = nci_empty_on(shape, input->ndim, NC_F32, NC_DEVICE_CUDA);
    if (y && !nci_ok(nc_cuda_linear_forward_f32_ex(nci_fptr(y), nci_fptr(xc), nci_fptr(weight), bias ? nci_fptr(bias) : NULL, B, in_f, out_f,
                                                   nci_stream()), "linear")) {
        nc_tensor_free(y);
        y = NULL;
    }
    if (y && any_grad(input, weight, bias)) {
        nc_node* nd = nci_attach(y, "linear", bwd_linear);
        if (nd) {
            nc_node_add_input(nd, input);
            nc_node_add_input(nd, weight);
            if (bias) nc_node_add_input(nd, bias);
            if (xc != input) { nc_node_save_owned_tensor(nd, xc); xc = input; } else nc_node_save_tensor(nd, input);
            nc_node_save_tensor(nd, weight);
            nc_node_save_tensor(nd, bias);
            nc_node_save_tensor(nd, input);
        }
    }
    if (xc != input) nc_tensor_free(xc);
    return y;
}
static nc_tensor* linear_module_forward(nc_module* self, nc_tensor* x) {
    return nc_linear_forward(x, nc_module_get_param(self, "weight"), nc_module_get_param(self, "bias"));
}
nc_module* nc_linear(size_t in_features, size_t out_features, bool bias) {
    nc_module* m = nc_module_create("Linear");
    linear_cfg* cfg = m ? nc_alloc(sizeof(*cfg)) : NULL;
    if (!cfg) { nc_module_free(m); return NULL; }
    cfg->in_f = in_features; cfg->out_f = out_features; cfg->has_bias = bias;
    m->extra = cfg; m->free_extra = nc_free; m->forward = linear_module_forward;
    const double bound = 1.0 / sqrt((double)(in_features ? in_features : 1)); /* U(-1/sqrt(in), 1/sqrt(in)), src/nn/linear.c:204-224 */
    size_t ws[2] = {out_features, in_features};
    nc_tensor* W = param_random(ws, 2, false, bound);
    if (!W) { nc_module_free(m); return NULL; }
    nc_module_add_param(m, "weight", W);
    if (bias) {
        nc_tensor* b = param_random(&out_features, 1, false, bound);
        if (!b) { nc_module_free(m); return NULL; }
        nc_module_add_param(m, "bias", b);
    }
    return m;
}
nc_tensor* nc_linear_weight(nc_module* l) { return nc_module_get_param(l, "weight"); }
nc_tensor* nc_linear_bias(nc_module* l) { return nc_module_get_param(l, "bias"); }

/* ------------------------------------------------------------------ Conv2d */
typedef struct { size_t cin, cout, k, stride, pad; bool has_bias; } conv_cfg;

static nc_tensor** bwd_batchnorm2d(nc_tensor* g, nc_tensor** saved, size_t n);
/* If `xin` (the convolution's input, read by the kernels as `x`) was produced by a training-mode BatchNorm2d with fused ReLU
 * in channels-last layout, tell the kernel library so: see nc_cuda_offer_batchnorm_backward_sums_f32. */
static void announce_bn_backward(const nc_tensor* xin, const nc_tensor* x) {
    const nc_node* nd = xin->grad_fn;
    if (!nd || nd->backward != bwd_batchnorm2d || nd->n_saved <= 6 || x != xin || !nci_is_channels_last(x)) return;
    nc_tensor** sv = nd->saved_tensors;
    const nc_tensor* bx = sv[0];
    if (!bx || !sv[2] || !sv[3] || !sv[4] || (int)nc_tensor_get_flat(sv[4], 1) != 1 || bx->numel != x->numel || !nci_on_cuda(bx)) return;
    const size_t C = x->shape[1];
    nc_cuda_offer_batchnorm_backward_sums_f32(nci_fptr(bx), nci_fptr(sv[2]), nci_fptr(sv[3]), sv[1] ? nci_fptr(sv[1]) : NULL,
                                              sv[6] ? nci_fptr(sv[6]) : NULL, nc_tensor_get_flat(sv[4], 0), (int)C,
                                              (long long)(x->numel / C));
}

/* node params: [0] stride, [1] padding, [2] Ho, [3] Wo */
static nc_tensor** bwd_conv2d(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(3);
    if (!out) return NULL;
    nc_tensor* x = saved[0];    /* input as the forward kernel read it (channels-last when it was converted) */
    nc_tensor* W = saved[1];
    nc_tensor* b = saved[2];
    nc_tensor* xin = saved[3];  /* the op's input tensor */
    nc_tensor* hp = saved[4];   /* host scalars: stride, padding */
    const int stride = (int)nc_tensor_get_flat(hp, 0), pad = (int)nc_tensor_get_flat(hp, 1);
    const int N = (int)x->shape[0], Cin = (int)x->shape[1], H = (int)x->shape[2], Wd = (int)x->shape[3];
    const int Cout = (int)W->shape[0], kH = (int)W->shape[2], kW = (int)W->shape[3];
    const size_t Ho = (size_t)(H + 2 * pad - kH) / stride + 1, Wo = (size_t)(Wd + 2 * pad - kW) / stride + 1;
    /* the kernels want dy channels-last */
    nc_tensor* like = nci_empty_cl((size_t)N, (size_t)Cout, Ho, Wo);
    if (!like) return out;
    nc_tensor* gd = nci_match_layout(g, like);
    nc_tensor_free(like);
    if (!gd) return out;
    size_t xs[4], ys[4];
    nci_strides4(x, xs);
    nci_strides4(gd, ys);
    const bool need_w = W->requires_grad, need_b = b && b->requires_grad;
    if (need_w) out[1] = nci_param_grad_out(1, W);
    if (need_b) out[2] = nci_param_grad_out(2, b);
    if (need_w || need_b)
        nci_ok(nc_cuda_conv2d_backward_weight_f32_ex(out[1] ? nci_fptr(out[1]) : NULL, out[2] ? nci_fptr(out[2]) : NULL, nci_fptr(gd), ys,
                                                     nci_fptr(x), xs, N, Cin, H, Wd, Cout, kH, kW, stride, pad, nci_stream()),
               "conv2d backward (weight)");
    /* the input gradient goes last: when the input is the output of a BatchNorm with fused ReLU, the kernel that writes the
     * gradient also sums what that BatchNorm's backward needs, and the offer only holds while nothing else is launched
     * between this call and that backward (the next node of a chain) */
    if (xin->requires_grad) {
        out[0] = nci_empty_like(x);
        if (out[0]) {
            announce_bn_backward(xin, x);
            nci_ok(nc_cuda_conv2d_backward_input_f32_ex(nci_fptr(out[0]), xs, nci_fptr(gd), ys, nci_fptr(W), N, Cin, H, Wd, Cout, kH, kW,
                                                        stride, pad, nci_stream()), "conv2d backward (input)");
        }
    }
    if (gd != g) nc_tensor_free(gd);
    return out;
}
nc_tensor* nc_conv2d_forward(nc_tensor* input, nc_tensor* weight, nc_tensor* bias, size_t stride, size_t padding) {
    if (!nci_need_cuda_f32(input, "conv2d") || !nci_need_cuda_f32(weight, "conv2d")) return NULL;
    if (bias && !nci_need_cuda_f32(bias, "conv2d")) return NULL;
    if (input->ndim != 4 || weight->ndim != 4 || !weight->is_contiguous) { NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "conv2d: input (N,C,H,W), weight (Cout,Cin,kH,kW)"); return NULL; }
    const size_t N = input->shape[0], Cin = input->shape[1], H = input->shape[2], Wd = input->shape[3];
    const size_t Cout = weight->shape[0], kH = weight->shape[2], kW = weight->shape[3];
    if (weight->shape[1] != Cin || stride == 0 || H + 2 * padding < kH || Wd + 2 * padding < kW || (bias && bias->numel != Cout)) {
        NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "conv2d: channel / kernel / bias sizes do not fit the input");
        return NULL;
    }
    const size_t Ho = (H + 2 * padding - kH) / stride + 1, Wo = (Wd + 2 * padding - kW) / stride + 1;
    /* wide inputs are re-laid out channels-last once so the tensor-core kernels can read them with TMA */
    nc_tensor* x = input;
    if (Cin >= 16 && !nci_is_channels_last(input)) { x = nci_to_channels_last(input); if (!x) return NULL; }
    nc_tensor* y = nci_empty_cl(N, Cout, Ho, Wo);
    size_t xs[4], ys[4];
    if (y) { nci_strides4(x, xs); nci_strides4(y, ys); }
    /* in a training graph the kernel also leaves per-channel sums of y for a BatchNorm called right after it */
    const int prev_stats = nc_cuda_set_conv_stats(nc_grad_enabled() ? 1 : 0);
    const bool conv_ok = y && nci_ok(nc_cuda_conv2d_forward_f32_ex(nci_fptr(y), ys, nci_fptr(x), xs, nci_fptr(weight), bias ? nci_fptr(bias) : NULL, (int)N,
                                                                   (int)Cin, (int)H, (int)Wd, (int)Cout, (int)kH, (int)kW, (int)stride, (int)padding,
                                                                   nci_stream()), "conv2d");
    nc_cuda_set_conv_stats(prev_stats); /* an offer already made stays valid until the next launch */
    if (y && !conv_ok) {
        nc_tensor_free(y);
        y = NULL;
    }
    /* as in the reference, autograd is wired when the input or the weight asks for it (src/nn/conv.c:560) */
    if (y && nc_grad_enabled() && (input->requires_grad || weight->requires_grad)) {
        nc_node* nd = nci_attach(y, "conv2d", bwd_conv2d);
        if (nd) {
            nc_node_add_input(nd, input);
            nc_node_add_input(nd, weight);
            if (bias) nc_node_add_input(nd, bias);
            if (x != input) { nc_node_save_owned_tensor(nd, x); x = input; } else nc_node_save_tensor(nd, input);
            nc_node_save_tensor(nd, weight);
            nc_node_save_tensor(nd, bias);
            nc_node_save_tensor(nd, input);
            size_t two = 2;
            nc_tensor* hp = nci_empty_on(&two, 1, NC_F64, NC_DEVICE_CPU);
            if (hp) { nc_tensor_set_flat(hp, 0, (double)stride); nc_tensor_set_flat(hp, 1, (double)padding); }
            nc_node_save_owned_tensor(nd, hp);
        }
    }
    if (x != input) nc_tensor_free(x);
    return y;
}
static nc_tensor* conv_module_forward(nc_module* self, nc_tensor* x) {
    conv_cfg* c = self->extra;
    return nc_conv2d_forward(x, nc_module_get_param(self, "weight"), nc_module_get_param(self, "bias"), c->stride, c->pad);
}
nc_module* nc_conv2d(size_t cin, size_t cout, size_t k, size_t stride, size_t padding, bool bias) {
    nc_module* m = nc_module_create("Conv2D");
    conv_cfg* cfg = m ? nc_alloc(sizeof(*cfg)) : NULL;
    if (!cfg) { nc_module_free(m); return NULL; }
    cfg->cin = cin; cfg->cout = cout; cfg->k = k; cfg->stride = stride; cfg->pad = padding; cfg->has_bias = bias;
    m->extra = cfg; m->free_extra = nc_free; m->forward = conv_module_forward;
    size_t ws[4] = {cout, cin, k, k};
    double fan_in = (double)(cin * k * k);
    nc_tensor* W = param_random(ws, 4, true, sqrt(2.0 / (fan_in > 0 ? fan_in : 1.0))); /* Kaiming normal, src/nn/conv.c:633-641 */
    if (!W) { nc_module_free(m); return NULL; }
    nc_module_add_param(m, "weight", W);
    if (bias) {
        nc_tensor* b = param_const(&cout, 1, 0.f);
        if (!b) { nc_module_free(m); return NULL; }
        nc_module_add_param(m, "bias", b);
    }
    return m;
}
nc_module* nc_conv2d_simple(size_t cin, size_t cout, size_t k) { return nc_conv2d(cin, cout, k, 1, 0, true); }
nc_tensor* nc_conv2d_weight(nc_module* c) { return nc_module_get_param(c, "weight"); }
nc_tensor* nc_conv2d_bias(nc_module* c) { return nc_module_get_param(c, "bias"); }

/* ------------------------------------------------------------------ MaxPool2d */
typedef struct { size_t k, stride; } pool_cfg;
static int layout_of(const nc_tensor* t) { return (t->is_contiguous) ? 0 : 1; } /* 0 = NCHW dense, 1 = channels-last */

/* saved: [input (shape and layout), argmax, host scalars (k, stride)] */
static nc_tensor** bwd_maxpool(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(1);
    if (!out) return NULL;
    nc_tensor* x = saved[0];
    nc_tensor* idx = saved[1];
    const int k = (int)nc_tensor_get_flat(saved[2], 0), stride = (int)nc_tensor_get_flat(saved[2], 1);
    const int layout = (int)nc_tensor_get_flat(saved[2], 2);
    /* gradient in the layout of the forward output (= layout of idx) */
    nc_tensor* like = nci_alias(idx);
    if (!like) return out;
    like->dtype = NC_F32;
    nc_tensor* gd = nci_match_layout(g, like);
    nc_tensor_free(like);
    if (!gd) return out;
    size_t shape[4] = {x->shape[0], x->shape[1], x->shape[2], x->shape[3]};
    out[0] = layout ? nci_empty_cl(shape[0], shape[1], shape[2], shape[3]) : nci_empty_on(shape, 4, NC_F32, NC_DEVICE_CUDA);
    if (out[0])
        nci_ok(nc_cuda_maxpool2d_backward_idx_f32_ex(nci_fptr(out[0]), nci_fptr(gd), (const uint8_t*)nci_dptr(idx), (int)shape[0], (int)shape[1],
                                                     (int)shape[2], (int)shape[3], k, stride, layout, nci_stream()), "maxpool backward");
    if (gd != g) nc_tensor_free(gd);
    return out;
}
nc_tensor* nc_maxpool2d_forward(nc_tensor* input, size_t k, size_t stride) {
    if (!nci_need_cuda_f32(input, "maxpool2d")) return NULL;
    if (input->ndim != 4 || k == 0 || stride == 0 || input->shape[2] < k || input->shape[3] < k || k * k > 255) {
        NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "maxpool2d: 4-D input at least as large as the window required");
        return NULL;
    }
    nc_tensor* x = input;
    if (!input->is_contiguous && !nci_is_channels_last(input)) { x = nc_tensor_contiguous(input); if (!x) return NULL; }
    const int layout = layout_of(x);
    const size_t N = x->shape[0], C = x->shape[1], H = x->shape[2], W = x->shape[3];
    const size_t Ho = (H - k) / stride + 1, Wo = (W - k) / stride + 1;
    size_t oshape[4] = {N, C, Ho, Wo};
    nc_tensor* y = layout ? nci_empty_cl(N, C, Ho, Wo) : nci_empty_on(oshape, 4, NC_F32, NC_DEVICE_CUDA);
    const bool need = nc_grad_enabled() && input->requires_grad;
    nc_tensor* idx = NULL;
    if (y && need) {
        idx = nci_empty_on(oshape, 4, NC_U8, NC_DEVICE_CUDA);
        if (idx) { memcpy(idx->strides, y->strides, sizeof(idx->strides)); idx->is_contiguous = y->is_contiguous; }
    }
    if (y && !nci_ok(nc_cuda_maxpool2d_forward_idx_f32_ex(nci_fptr(y), idx ? (uint8_t*)nci_dptr(idx) : NULL, nci_fptr(x), (int)N, (int)C, (int)H,
                                                          (int)W, (int)k, (int)stride, layout, nci_stream()), "maxpool2d")) {
        nc_tensor_free(y);
        nc_tensor_free(idx);
        y = NULL;
        idx = NULL;
    }
    if (y && need && idx) {
        nc_node* nd = nci_attach(y, "maxpool2d", bwd_maxpool);
        if (nd) {
            nc_node_add_input(nd, input);
            nc_node_save_tensor(nd, input);
            nc_node_save_owned_tensor(nd, idx);
            size_t three = 3;
            nc_tensor* hp = nci_empty_on(&three, 1, NC_F64, NC_DEVICE_CPU);
            if (hp) { nc_tensor_set_flat(hp, 0, (double)k); nc_tensor_set_flat(hp, 1, (double)stride); nc_tensor_set_flat(hp, 2, (double)layout); }
            nc_node_save_owned_tensor(nd, hp);
        } else nc_tensor_free(idx);
    }
    if (x != input) nc_tensor_free(x);
    return y;
}
static nc_tensor* pool_module_forward(nc_module* self, nc_tensor* x) { pool_cfg* c = self->extra; return nc_maxpool2d_forward(x, c->k, c->stride); }
nc_module* nc_maxpool2d(size_t k, size_t stride) {
    nc_module* m = nc_module_create("MaxPool2D");
    pool_cfg* cfg = m ? nc_alloc(sizeof(*cfg)) : NULL;
    if (!cfg) { nc_module_free(m); return NULL; }
    cfg->k = k; cfg->stride = stride;
    m->extra = cfg; m->free_extra = nc_free; m->forward = pool_module_forward;
    return m;
}
nc_module* nc_maxpool2d_simple(size_t k) { return nc_maxpool2d(k, k); }

/* ------------------------------------------------------------------ Flatten */
static nc_tensor** bwd_flatten(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(1);
    if (!out) return NULL;
    nc_tensor* r = nci_match_layout(g, saved[0]);
    out[0] = (r == g) ? nci_alias(g) : r;
    return out;
}
nc_tensor* nc_flatten_forward(nc_tensor* x) {
    if (!x || x->ndim < 1) { NC_SET_ERROR(NC_ERR_NULL_PTR, "flatten: null or 0-d input"); return NULL; }
    size_t shape[2] = {x->shape[0], x->shape[0] ? x->numel / x->shape[0] : 0};
    nc_tensor* y = nc_tensor_reshape(x, shape, 2); /* copies into dense (C,H,W) order when x is channels-last */
    if (y && nc_grad_enabled() && x->requires_grad) {
        nc_node* nd = nci_attach(y, "flatten", bwd_flatten);
        if (nd) { nc_node_add_input(nd, x); nc_node_save_tensor(nd, x); }
    }
    return y;
}
static nc_tensor* flatten_module_forward(nc_module* self, nc_tensor* x) { (void)self; return nc_flatten_forward(x); }
nc_module* nc_flatten(void) {
    nc_module* m = nc_module_create("Flatten");
    if (m) m->forward = flatten_module_forward;
    return m;
}

/* ------------------------------------------------------------------ BatchNorm2d */
typedef struct { size_t num_features; double eps, momentum; bool affine, track; size_t batches; } bn_cfg;

/* saved: [x (as normalised), gamma, batch_mean, batch_var, host scalars (eps, layout), input] */
static nc_tensor** bwd_batchnorm2d(nc_tensor* g, nc_tensor** saved, size_t n) {
    nc_tensor** out = grad_array(3);
    if (!out) return NULL;
    nc_tensor* x = saved[0];
    nc_tensor* gamma = saved[1];
    nc_tensor* mean = saved[2];
    nc_tensor* var = saved[3];
    const double eps = nc_tensor_get_flat(saved[4], 0);
    const int layout = (int)nc_tensor_get_flat(saved[4], 1);
    const bool fused_relu = n > 6;                 /* fused ReLU: the mask is recomputed from x, gamma and beta */
    nc_tensor* beta = fused_relu ? saved[6] : NULL; /* may be NULL for a layer without affine parameters */
    nc_tensor* gd = nci_match_layout(g, x);
    if (!gd) return out;
    const int N = (int)x->shape[0], C = (int)x->shape[1], S = (int)(x->shape[2] * x->shape[3]);
    size_t cs = (size_t)C;
    nci_round_outputs(true);
    out[0] = nci_empty_like(x);
    /* node inputs are (input[, weight, bias]): parameter gradients exist only for an affine layer */
    if (gamma) { out[1] = nci_param_grad_out(1, gamma); out[2] = nci_param_grad_out(2, gamma); }
    if (out[0] && (!gamma || (out[1] && out[2])))
        nci_ok(nc_cuda_batchnorm_backward_f32_ex(nci_fptr(out[0]), gamma ? nci_fptr(out[1]) : NULL, gamma ? nci_fptr(out[2]) : NULL, nci_fptr(gd), nci_fptr(x),
                                                 gamma ? nci_fptr(gamma) : NULL, nci_fptr(mean), nci_fptr(var), NULL, beta ? nci_fptr(beta) : NULL,
                                                 fused_relu ? 1 : 0, N, C, S, eps, layout, nci_stream()), "batchnorm backward");
    if (gd != g) nc_tensor_free(gd);
    return out;
}
static nc_tensor* bn_forward(nc_tensor* input, nc_tensor* running_mean, nc_tensor* running_var, nc_tensor* weight,
                             nc_tensor* bias, bool training, double momentum, double eps, int relu) {
    if (!input || input->ndim != 4) { NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "BatchNorm2D requires 4D input (N,C,H,W)"); return NULL; }
    if (!nci_need_cuda_f32(input, "batchnorm2d")) return NULL;
    nc_tensor* opt[4] = {running_mean, running_var, weight, bias};
    for (int i = 0; i < 4; i++)
        if (opt[i] && (!nci_need_cuda_f32(opt[i], "batchnorm2d") || opt[i]->numel != input->shape[1])) {
            if (nc_last_error == NC_OK) NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "batchnorm2d: per-channel tensor of the wrong size");
            return NULL;
        }
    nc_tensor* x = input;
    if (!input->is_contiguous && !nci_is_channels_last(input)) { x = nc_tensor_contiguous(input); if (!x) return NULL; }
    const int layout = layout_of(x);
    const int N = (int)x->shape[0], C = (int)x->shape[1], S = (int)(x->shape[2] * x->shape[3]);
    size_t cs = (size_t)C;
    nci_round_outputs(true);
    nc_tensor* y = nci_empty_like(x);
    nc_tensor* mean = nci_empty_on(&cs, 1, NC_F32, NC_DEVICE_CUDA);
    nc_tensor* var = nci_empty_on(&cs, 1, NC_F32, NC_DEVICE_CUDA);
    bool ok = y && mean && var &&
              nci_ok(nc_cuda_batchnorm_forward_f32_ex(nci_fptr(y), nci_fptr(x), weight ? nci_fptr(weight) : NULL, bias ? nci_fptr(bias) : NULL,
                                                      running_mean ? nci_fptr(running_mean) : NULL, running_var ? nci_fptr(running_var) : NULL,
                                                      nci_fptr(mean), nci_fptr(var), N, C, S, momentum, eps, training ? 1 : 0, layout, relu,
                                                      nci_stream()), "batchnorm2d");
    bool wired = false;
    if (ok && any_grad(input, weight, bias)) {
        nc_node* nd = nci_attach(y, "batchnorm2d", bwd_batchnorm2d);
        if (nd) {
            nc_node_add_input(nd, input);
            if (weight) nc_node_add_input(nd, weight);
            if (bias) nc_node_add_input(nd, bias);
            if (x != input) { nc_node_save_owned_tensor(nd, x); x = input; } else nc_node_save_tensor(nd, input);
            nc_node_save_tensor(nd, weight);
            nc_node_save_owned_tensor(nd, mean);
            nc_node_save_owned_tensor(nd, var);
            size_t two = 2;
            nc_tensor* hp = nci_empty_on(&two, 1, NC_F64, NC_DEVICE_CPU);
            if (hp) { nc_tensor_set_flat(hp, 0, eps); nc_tensor_set_flat(hp, 1, (double)layout); }
            nc_node_save_owned_tensor(nd, hp);
            nc_node_save_tensor(nd, input);
            if (relu) nc_node_save_tensor(nd, bias); /* backward recomputes the ReLU mask from x, gamma, beta */
            wired = true;
        }
    }
    if (!wired) { nc_tensor_free(mean); nc_tensor_free(var); }
    if (x != input) nc_tensor_free(x);
    if (!ok) { nc_tensor_free(y); return NULL; }
    return y;
}
nc_tensor* nc_batchnorm2d_forward_fn(nc_tensor* input, nc_tensor* running_mean, nc_tensor* running_var, nc_tensor* weight,
                                     nc_tensor* bias, bool training, double momentum, double eps) {
    return bn_forward(input, running_mean, running_var, weight, bias, training, momentum, eps, 0);
}
nc_tensor* nc_batchnorm2d_relu_forward_fn(nc_tensor* input, nc_tensor* running_mean, nc_tensor* running_var, nc_tensor* weight,
                                          nc_tensor* bias, bool training, double momentum, double eps) {
    return bn_forward(input, running_mean, running_var, weight, bias, training, momentum, eps, 1);
}
nc_tensor* nc_batchnorm2d_relu(nc_module* bn, nc_tensor* x) {
    if (!bn || !bn->extra) { NC_SET_ERROR(NC_ERR_NULL_PTR, "batchnorm2d_relu: not a BatchNorm2D module"); return NULL; }
    bn_cfg* c = bn->extra;
    if (bn->training) c->batches++;
    return bn_forward(x, nc_module_get_param(bn, "running_mean"), nc_module_get_param(bn, "running_var"), nc_module_get_param(bn, "weight"),
                      nc_module_get_param(bn, "bias"), bn->training, c->momentum, c->eps, 1);
}
/* ---- BatchNorm2d + ReLU + MaxPool(2, 2) as one forward pass and one backward pass ----
 * saved: [x, gamma, batch_mean, batch_var, host scalar (eps), beta, window offsets] */
static nc_tensor** bwd_bn_relu_pool(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(3);
    if (!out) return NULL;
    nc_tensor* x = saved[0];
    nc_tensor* gamma = saved[1];
    nc_tensor* mean = saved[2];
    nc_tensor* var = saved[3];
    const double eps = nc_tensor_get_flat(saved[4], 0);
    nc_tensor* beta = saved[5];
    nc_tensor* idx = saved[6];
    /* gradient in the layout of the pooled output (= layout of idx) */
    nc_tensor* like = nci_alias(idx);
    if (!like) return out;
    like->dtype = NC_F32;
    nc_tensor* gd = nci_match_layout(g, like);
    nc_tensor_free(like);
    if (!gd) return out;
    const int N = (int)x->shape[0], C = (int)x->shape[1], H = (int)x->shape[2], W = (int)x->shape[3];
    size_t cs = (size_t)C;
    nci_round_outputs(true);
    out[0] = nci_empty_like(x);
    if (gamma) { out[1] = nci_param_grad_out(1, gamma); out[2] = nci_param_grad_out(2, gamma); }
    if (out[0] && (!gamma || (out[1] && out[2])))
        nci_ok(nc_cuda_batchnorm_relu_maxpool2_backward_f32_ex(nci_fptr(out[0]), gamma ? nci_fptr(out[1]) : NULL, gamma ? nci_fptr(out[2]) : NULL,
                                                               nci_fptr(gd), (const uint8_t*)nci_dptr(idx), nci_fptr(x), gamma ? nci_fptr(gamma) : NULL,
                                                               beta ? nci_fptr(beta) : NULL, nci_fptr(mean), nci_fptr(var), N, C, H, W, eps,
                                                               nci_stream()), "batchnorm+relu+maxpool backward");
    if (gd != g) nc_tensor_free(gd);
    return out;
}
nc_tensor* nc_batchnorm2d_relu_maxpool2(nc_module* bn, nc_tensor* input) {
    if (!bn || !bn->extra) { NC_SET_ERROR(NC_ERR_NULL_PTR, "batchnorm2d_relu_maxpool2: not a BatchNorm2D module"); return NULL; }
    if (!input || input->ndim != 4) { NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "BatchNorm2D requires 4D input (N,C,H,W)"); return NULL; }
    const size_t N = input->shape[0], C = input->shape[1], H = input->shape[2], W = input->shape[3];
    const bool fusable = nci_on_cuda(input) && input->dtype == NC_F32 && nci_is_channels_last(input) && nci_is_dense(input) &&
                         (C % 4 == 0) && (H % 2 == 0) && (W % 2 == 0) && H >= 2 && W >= 2;
    if (!fusable) { /* same result from the two separate ops */
        nc_tensor* y = nc_batchnorm2d_relu(bn, input);
        nc_tensor* p = y ? nc_maxpool2d_forward(y, 2, 2) : NULL;
        /* y is invisible to the caller: the pool node takes ownership when there is a graph, else it goes now */
        if (y && p && p->grad_fn) nc_node_save_owned_tensor(p->grad_fn, y);
        else if (y) nc_tensor_free(y);
        return p;
    }
    bn_cfg* c = bn->extra;
    if (bn->training) c->batches++;
    nc_tensor* weight = nc_module_get_param(bn, "weight");
    nc_tensor* bias = nc_module_get_param(bn, "bias");
    nc_tensor* rm = nc_module_get_param(bn, "running_mean");
    nc_tensor* rv = nc_module_get_param(bn, "running_var");
    size_t cs = C, oshape[4] = {N, C, H / 2, W / 2};
    nci_round_outputs(true);
    nc_tensor* y = nci_empty_cl(N, C, H / 2, W / 2);
    nc_tensor* mean = nci_empty_on(&cs, 1, NC_F32, NC_DEVICE_CUDA);
    nc_tensor* var = nci_empty_on(&cs, 1, NC_F32, NC_DEVICE_CUDA);
    const bool need = nc_grad_enabled() && any_grad(input, weight, bias);
    nc_tensor* idx = NULL;
    if (y && need) {
        idx = nci_empty_on(oshape, 4, NC_U8, NC_DEVICE_CUDA);
        if (idx) { memcpy(idx->strides, y->strides, sizeof(idx->strides)); idx->is_contiguous = y->is_contiguous; }
    }
    bool ok = y && mean && var && (!need || idx) &&
              nci_ok(nc_cuda_batchnorm_relu_maxpool2_forward_f32_ex(nci_fptr(y), idx ? (uint8_t*)nci_dptr(idx) : NULL, nci_fptr(input),
                                                                    weight ? nci_fptr(weight) : NULL, bias ? nci_fptr(bias) : NULL,
                                                                    rm ? nci_fptr(rm) : NULL, rv ? nci_fptr(rv) : NULL, nci_fptr(mean), nci_fptr(var),
                                                                    (int)N, (int)C, (int)H, (int)W, c->momentum, c->eps, bn->training ? 1 : 0,
                                                                    nci_stream()), "batchnorm+relu+maxpool");
    bool wired = false;
    if (ok && need) {
        nc_node* nd = nci_attach(y, "batchnorm2d_relu_maxpool2", bwd_bn_relu_pool);
        if (nd) {
            nc_node_add_input(nd, input);
            if (weight) nc_node_add_input(nd, weight);
            if (bias) nc_node_add_input(nd, bias);
            nc_node_save_tensor(nd, input);
            nc_node_save_tensor(nd, weight);
            nc_node_save_owned_tensor(nd, mean);
            nc_node_save_owned_tensor(nd, var);
            size_t one = 1;
            nc_tensor* hp = nci_empty_on(&one, 1, NC_F64, NC_DEVICE_CPU);
            if (hp) nc_tensor_set_flat(hp, 0, c->eps);
            nc_node_save_owned_tensor(nd, hp);
            nc_node_save_tensor(nd, bias);
            nc_node_save_owned_tensor(nd, idx);
            wired = true;
        }
    }
    if (!wired) { nc_tensor_free(mean); nc_tensor_free(var); nc_tensor_free(idx); }
    if (!ok) { nc_tensor_free(y); return NULL; }
    return y;
}
static nc_tensor* bn_module_forward(nc_module* self, nc_tensor* x) {
    bn_cfg* c = self->extra;
    if (self->training) c->batches++;
    return nc_batchnorm2d_forward_fn(x, nc_module_get_param(self, "running_mean"), nc_module_get_param(self, "running_var"),
                                     nc_module_get_param(self, "weight"), nc_module_get_param(self, "bias"), self->training, c->momentum,
                                     c->eps);
}
nc_module* nc_batchnorm2d_ex(nc_batchnorm2d_config config) {
    nc_module* m = nc_module_create("BatchNorm2D");
    bn_cfg* cfg = m ? nc_alloc(sizeof(*cfg)) : NULL;
    if (!cfg) { nc_module_free(m); return NULL; }
    cfg->num_features = config.num_features; cfg->eps = config.eps; cfg->momentum = config.momentum;
    cfg->affine = config.affine; cfg->track = config.track_running_stats; cfg->batches = 0;
    m->extra = cfg; m->free_extra = nc_free; m->forward = bn_module_forward;
    size_t cs = config.num_features;
    if (config.affine) {
        nc_module_add_param(m, "weight", param_const(&cs, 1, 1.f));
        nc_module_add_param(m, "bias", param_const(&cs, 1, 0.f));
    }
    if (config.track_running_stats) {
        /* registered like parameters, as in the reference (src/nn/batchnorm.c:447-451): they end up with
         * requires_grad = true and a zero gradient, so e.g. AdamW decays them */
        nc_module_add_param(m, "running_mean", param_const(&cs, 1, 0.f));
        nc_module_add_param(m, "running_var", param_const(&cs, 1, 1.f));
    }
    return m;
}
nc_module* nc_batchnorm2d(size_t num_features) {
    nc_batchnorm2d_config c = NC_BATCHNORM2D_DEFAULT;
    c.num_features = num_features;
    return nc_batchnorm2d_ex(c);
}
/* ------------------------------------------------------------------ BatchNorm1d (src/nn/batchnorm.c:705-860)
 * input (N, C) or (N, C, L): statistics per channel over N (and L).  (N, C) row-major is the channels-last case of the
 * 2-D kernels with one pixel per row; (N, C, L) is their channel-major case.
 * saved: [x (dense), gamma, batch_mean, batch_var, host scalars (eps, layout, N, C, L)] */
static nc_tensor** bwd_batchnorm1d(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(3);
    if (!out) return NULL;
    nc_tensor* x = saved[0];
    nc_tensor* gamma = saved[1];
    const double eps = nc_tensor_get_flat(saved[4], 0);
    const int layout = (int)nc_tensor_get_flat(saved[4], 1);
    const int N = (int)nc_tensor_get_flat(saved[4], 2), C = (int)nc_tensor_get_flat(saved[4], 3), L = (int)nc_tensor_get_flat(saved[4], 4);
    nc_tensor* gd = g->is_contiguous ? g : nc_tensor_contiguous(g);
    if (!gd) return out;
    nci_round_outputs(true);
    out[0] = nci_empty_on(x->shape, x->ndim, NC_F32, NC_DEVICE_CUDA);
    if (gamma) { out[1] = nci_param_grad_out(1, gamma); out[2] = nci_param_grad_out(2, gamma); }
    if (out[0] && (!gamma || (out[1] && out[2])))
        nci_ok(nc_cuda_batchnorm_backward_f32_ex(nci_fptr(out[0]), gamma ? nci_fptr(out[1]) : NULL, gamma ? nci_fptr(out[2]) : NULL, nci_fptr(gd),
                                                 nci_fptr(x), gamma ? nci_fptr(gamma) : NULL, nci_fptr(saved[2]), nci_fptr(saved[3]), NULL, NULL, 0,
                                                 N, C, L, eps, layout, nci_stream()), "batchnorm1d backward");
    if (gd != g) nc_tensor_free(gd);
    return out;
}
nc_tensor* nc_batchnorm1d_forward_fn(nc_tensor* input, nc_tensor* running_mean, nc_tensor* running_var, nc_tensor* weight,
                                     nc_tensor* bias, bool training, double momentum, double eps) {
    if (!input || (input->ndim != 2 && input->ndim != 3)) { NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "BatchNorm1D requires (N,C) or (N,C,L) input"); return NULL; }
    if (!nci_need_cuda_f32(input, "batchnorm1d")) return NULL;
    nc_tensor* opt[4] = {running_mean, running_var, weight, bias};
    for (int i = 0; i < 4; i++)
        if (opt[i] && (!nci_need_cuda_f32(opt[i], "batchnorm1d") || opt[i]->numel != input->shape[1])) {
            if (nc_last_error == NC_OK) NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "batchnorm1d: per-channel tensor of the wrong size");
            return NULL;
        }
    nc_tensor* x = input->is_contiguous ? input : nc_tensor_contiguous(input);
    if (!x) return NULL;
    const int N = (int)x->shape[0], C = (int)x->shape[1], L = x->ndim == 3 ? (int)x->shape[2] : 1;
    const int layout = x->ndim == 2 ? 1 : 0;
    size_t cs = (size_t)C;
    nci_round_outputs(true);
    nc_tensor* y = nci_empty_on(x->shape, x->ndim, NC_F32, NC_DEVICE_CUDA);
    nc_tensor* mean = nci_empty_on(&cs, 1, NC_F32, NC_DEVICE_CUDA);
    nc_tensor* var = nci_empty_on(&cs, 1, NC_F32, NC_DEVICE_CUDA);
    bool ok = y && mean && var &&
              nci_ok(nc_cuda_batchnorm_forward_f32_ex(nci_fptr(y), nci_fptr(x), weight ? nci_fptr(weight) : NULL, bias ? nci_fptr(bias) : NULL,
                                                      running_mean ? nci_fptr(running_mean) : NULL, running_var ? nci_fptr(running_var) : NULL,
                                                      nci_fptr(mean), nci_fptr(var), N, C, L, momentum, eps, training ? 1 : 0, layout, 0,
                                                      nci_stream()), "batchnorm1d");
    bool wired = false;
    if (ok && any_grad(input, weight, bias)) {
        nc_node* nd = nci_attach(y, "batchnorm1d", bwd_batchnorm1d);
        if (nd) {
            nc_node_add_input(nd, input);
            if (weight) nc_node_add_input(nd, weight);
            if (bias) nc_node_add_input(nd, bias);
            if (x != input) { nc_node_save_owned_tensor(nd, x); x = input; } else nc_node_save_tensor(nd, input);
            nc_node_save_tensor(nd, weight);
            nc_node_save_owned_tensor(nd, mean);
            nc_node_save_owned_tensor(nd, var);
            size_t five = 5;
            nc_tensor* hp = nci_empty_on(&five, 1, NC_F64, NC_DEVICE_CPU);
            if (hp) {
                nc_tensor_set_flat(hp, 0, eps); nc_tensor_set_flat(hp, 1, (double)layout); nc_tensor_set_flat(hp, 2, (double)N);
                nc_tensor_set_flat(hp, 3, (double)C); nc_tensor_set_flat(hp, 4, (double)L);
            }
            nc_node_save_owned_tensor(nd, hp);
            wired = true;
        }
    }
    if (!wired) { nc_tensor_free(mean); nc_tensor_free(var); }
    if (x != input) nc_tensor_free(x);
    if (!ok) { nc_tensor_free(y); return NULL; }
    return y;
}
static nc_tensor* bn1d_module_forward(nc_module* self, nc_tensor* x) {
    bn_cfg* c = self->extra;
    if (self->training) c->batches++;
    return nc_batchnorm1d_forward_fn(x, nc_module_get_param(self, "running_mean"), nc_module_get_param(self, "running_var"),
                                     nc_module_get_param(self, "weight"), nc_module_get_param(self, "bias"), self->training, c->momentum,
                                     c->eps);
}
nc_module* nc_batchnorm1d_ex(nc_batchnorm2d_config config) {
    nc_module* m = nc_batchnorm2d_ex(config); /* same parameters and buffers */
    if (m) { snprintf(m->name, sizeof(m->name), "BatchNorm1D"); m->forward = bn1d_module_forward; }
    return m;
}
nc_module* nc_batchnorm1d(size_t num_features) {
    nc_batchnorm2d_config c = NC_BATCHNORM2D_DEFAULT;
    c.num_features = num_features;
    return nc_batchnorm1d_ex(c);
}

nc_tensor* nc_batchnorm2d_weight(nc_module* bn) { return nc_module_get_param(bn, "weight"); }
nc_tensor* nc_batchnorm2d_bias(nc_module* bn) { return nc_module_get_param(bn, "bias"); }
nc_tensor* nc_batchnorm2d_running_mean(nc_module* bn) { return nc_module_get_param(bn, "running_mean"); }
nc_tensor* nc_batchnorm2d_running_var(nc_module* bn) { return nc_module_get_param(bn, "running_var"); }

/* ------------------------------------------------------------------ LayerNorm */
typedef struct { size_t shape[NC_MAX_DIMS]; size_t ndim; double eps; bool affine; } ln_cfg;

/* saved: [x (contiguous), gamma, host scalars (norm_size, eps), input] */
static nc_tensor** bwd_layernorm(nc_tensor* g, nc_tensor** saved, size_t n) {
    (void)n;
    nc_tensor** out = grad_array(3);
    if (!out) return NULL;
    nc_tensor* x = saved[0];
    nc_tensor* gamma = saved[1];
    const size_t cols = (size_t)nc_tensor_get_flat(saved[2], 0);
    const double eps = nc_tensor_get_flat(saved[2], 1);
    nc_tensor* gc = nc_tensor_contiguous(g);
    if (!gc) return out;
    const size_t rows = cols ? x->numel / cols : 0;
    nci_round_outputs(true);
    out[0] = nci_empty_on(x->shape, x->ndim, NC_F32, NC_DEVICE_CUDA);
    if (gamma) { out[1] = nci_empty_on(&cols, 1, NC_F32, NC_DEVICE_CUDA); out[2] = nci_empty_on(&cols, 1, NC_F32, NC_DEVICE_CUDA); }
    if (out[0] && (!gamma || (out[1] && out[2])))
        nci_ok(nc_cuda_layernorm_backward_f32_ex(nci_fptr(out[0]), gamma ? nci_fptr(out[1]) : NULL, gamma ? nci_fptr(out[2]) : NULL, nci_fptr(gc),
                                                 nci_fptr(x), gamma ? nci_fptr(gamma) : NULL, rows, cols, eps, nci_stream()), "layernorm backward");
    if (gc != g) nc_tensor_free(gc);
    return out;
}
nc_tensor* nc_layernorm_forward_fn(nc_tensor* input, const size_t* normalized_shape, size_t normalized_ndim, nc_tensor* weight,
                                   nc_tensor* bias, double eps) {
    if (!nci_need_cuda_f32(input, "layernorm")) return NULL;
    size_t cols = 1;
    for (size_t i = 0; i < normalized_ndim; i++) cols *= normalized_shape[i];
    if (cols == 0 || input->numel % cols || (weight && weight->numel != cols) || (bias && bias->numel != cols)) {
        NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "layernorm: normalized shape does not divide the input");
        return NULL;
    }
    if ((weight && !nci_need_cuda_f32(weight, "layernorm")) || (bias && !nci_need_cuda_f32(bias, "layernorm"))) return NULL;
    nc_tensor* x = nc_tensor_contiguous(input);
    if (!x) return NULL;
    nci_round_outputs(true);
    nc_tensor* y = nci_empty_on(input->shape, input->ndim, NC_F32, NC_DEVICE_CUDA);
    if (y && !nci_ok(nc_cuda_layernorm_forward_f32_ex(nci_fptr(y), nci_fptr(x), weight ? nci_fptr(weight) : NULL, bias ? nci_fptr(bias) : NULL,
                                                      input->numel / cols, cols, eps, nci_stream()), "layernorm")) {
        nc_tensor_free(y);
        y = NULL;
    }
    if (y && any_grad(input, weight, bias)) {
        nc_node* nd = nci_attach(y, "layernorm", bwd_layernorm);
        if (nd) {
            nc_node_add_input(nd, input);
            if (weight) nc_node_add_input(nd, weight);
            if (bias) nc_node_add_input(nd, bias);
            if (x != input) { nc_node_save_owned_tensor(nd, x); x = input; } else nc_node_save_tensor(nd, input);
            nc_node_save_tensor(nd, weight);
            size_t two = 2;
            nc_tensor* hp = nci_empty_on(&two, 1, NC_F64, NC_DEVICE_CPU);
            if (hp) { nc_tensor_set_flat(hp, 0, (double)cols); nc_tensor_set_flat(hp, 1, eps); }
            nc_node_save_owned_tensor(nd, hp);
            nc_node_save_tensor(nd, input);
        }
    }
    if (x != input) nc_tensor_free(x);
    return y;
}
static nc_tensor* ln_module_forward(nc_module* self, nc_tensor* x) {
    ln_cfg* c = self->extra;
    return nc_layernorm_forward_fn(x, c->shape, c->ndim, nc_module_get_param(self, "weight"), nc_module_get_param(self, "bias"), c->eps);
}
nc_module* nc_layernorm_ex(nc_layernorm_config config) {
    if (config.normalized_ndim > NC_MAX_DIMS || (config.normalized_ndim && !config.normalized_shape)) {
        NC_SET_ERROR(NC_ERR_INVALID_SHAPE, "layernorm: bad normalized shape");
        return NULL;
    }
    nc_module* m = nc_module_create("LayerNorm");
    ln_cfg* cfg = m ? nc_calloc(1, sizeof(*cfg)) : NULL;
    if (!cfg) { nc_module_free(m); return NULL; }
    size_t cols = 1;
    for (size_t i = 0; i < config.normalized_ndim; i++) { cfg->shape[i] = config.normalized_shape[i]; cols *= cfg->shape[i]; }
    cfg->ndim = config.normalized_ndim; cfg->eps = config.eps; cfg->affine = config.elementwise_affine;
    m->extra = cfg; m->free_extra = nc_free; m->forward = ln_module_forward;
    if (config.elementwise_affine) {
        nc_module_add_param(m, "weight", param_const(&cols, 1, 1.f));
        nc_module_add_param(m, "bias", param_const(&cols, 1, 0.f));
    }
    return m;
}
nc_module* nc_layernorm(const size_t* normalized_shape, size_t ndim) {
    nc_layernorm_config c = {(size_t*)normalized_shape, ndim, 1e-5, true}; /* eps fixed at 1e-5 (src/nn/batchnorm.c:1056) */
    return nc_layernorm_ex(c);
}

/* ------------------------------------------------------------------ dropout with a supplied mask */
nc_tensor* nc_dropout_mask_fn(nc_tensor* x, nc_tensor* mask) { return nc_mul(x, mask); }
/* Dropout with the reference's mask rule (src/nn/dropout.c:52-97): element i (logical order) is kept when
 * rand() / RAND_MAX > p and scaled by 1 / (1 - p).  The mask is drawn on the host from the C library generator,
 * exactly as the reference draws it, so the same srand() seed gives the same mask; it is uploaded already scaled and
 * the device does y = x * mask (the gradient is g * mask).  Evaluation mode, p == 0 and an invalid p return a copy. */
nc_tensor* nc_dropout_fn(nc_tensor* x, double p, bool training) {
    if (!x) { NC_SET_ERROR(NC_ERR_NULL_PTR, "dropout: null input"); return NULL; }
    if (!training || p == 0.0 || p < 0.0 || p >= 1.0) return nc_tensor_clone(x);
    if (!nci_need_cuda_f32(x, "dropout")) return NULL;
    const float scale = (float)(1.0 / (1.0 - p));
    float* h = nc_alloc(sizeof(float) * (x->numel ? x->numel : 1));
    if (!h) return NULL;
    for (size_t i = 0; i < x->numel; i++) h[i] = ((double)rand() / RAND_MAX > p) ? scale : 0.f;
    nc_device_type dev = nc_get_default_device();
    nc_set_default_device(NC_DEVICE_CUDA);
    nc_tensor* mask = nc_tensor_from_data(h, x->shape, x->ndim, NC_F32);
    nc_set_default_device(dev);
    nc_free(h);
    if (!mask) return NULL;
    nc_tensor* y = nc_mul(x, mask);
    /* with a graph the multiply node needs the mask in backward: hand it over; else it is done */
    if (y && y->grad_fn) nc_node_save_owned_tensor(y->grad_fn, mask);
    else nc_tensor_free(mask);
    return y;
}
typedef struct { double p; } dropout_cfg;
static nc_tensor* dropout_module_forward(nc_module* self, nc_tensor* x) { return nc_dropout_fn(x, ((dropout_cfg*)self->extra)->p, self->training); }
nc_module* nc_dropout(double p) {
    nc_module* m = nc_module_create("Dropout");
    dropout_cfg* cfg = m ? nc_alloc(sizeof(*cfg)) : NULL;
    if (!cfg) { nc_module_free(m); return NULL; }
    cfg->p = p;
    m->extra = cfg; m->free_extra = nc_free; m->forward = dropout_module_forward;
    return m;
}
