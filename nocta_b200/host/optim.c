/*
 * Optimizers: SGD (momentum, dampening, Nesterov, L2) and Adam / AdamW / AMSGrad.  The update of
 * one parameter tensor is one fused kernel that also applies the gradient scale (1/world under
 * data parallel).  Rules follow the reference CPU path (src/optim/optimizer.c:3-51,
 * src/optim/sgd.c:13-171, src/optim/adam.c:11-131): the step counter t is per optimizer; SGD uses
 * v = g on the very first step (t == 0) and increments t after the sweep; Adam increments t first
 * and derives the bias corrections from it in double on the host.
 */
#include "internal.h"
#include <math.h>

typedef struct { double grad_scale; const nc_storage* arena; size_t arena_bytes; } opt_common;
typedef struct { opt_common c; nc_sgd_config cfg; nc_tensor* velocity[NC_MAX_OPTIM_PARAMS]; } sgd_state;
typedef struct { opt_common c; nc_adam_config cfg; nc_tensor* m[NC_MAX_OPTIM_PARAMS]; nc_tensor* v[NC_MAX_OPTIM_PARAMS]; nc_tensor* vmax[NC_MAX_OPTIM_PARAMS]; } adam_state;

void nc_optimizer_free(nc_optimizer* opt) {
    if (!opt) return;
    if (opt->state && opt->free_state) opt->free_state(opt->state);
    nc_free(opt);
}
void nc_optimizer_step(nc_optimizer* opt) { if (opt && opt->step) opt->step(opt); }
void nc_optimizer_zero_grad(nc_optimizer* opt) {
    if (!opt) return;
    opt_common* c = opt->state;
    if (c && c->arena) {
        /* flattened gradients: one memset for the whole range when every gradient still lives there */
        bool all = true;
        for (size_t i = 0; i < opt->n_params && all; i++) all = opt->params[i]->grad && opt->params[i]->grad->storage == c->arena;
        if (all) {
            nc_cuda_memset_async(c->arena->cuda_data, 0, c->arena_bytes, nci_stream());
            for (size_t i = 0; i < opt->n_params; i++) opt->params[i]->grad->is_reachable = false; /* zero since cleared */
            return;
        }
    }
    for (size_t i = 0; i < opt->n_params; i++) nc_tensor_zero_grad_(opt->params[i]);
}
void nc_optimizer_set_lr(nc_optimizer* opt, double lr) { if (opt) opt->lr = lr; }
double nc_optimizer_get_lr(nc_optimizer* opt) { return opt ? opt->lr : 0.0; }
void nc_optimizer_add_param(nc_optimizer* opt, nc_tensor* param) {
    if (!opt || !param || opt->n_params >= NC_MAX_OPTIM_PARAMS) return;
    opt->params[opt->n_params++] = param;
}
static void cb_add(const char* name, nc_tensor* p, void* ctx) { (void)name; nc_optimizer_add_param(ctx, p); }
void nc_optimizer_add_module(nc_optimizer* opt, nc_module* m) { if (opt && m) nc_module_parameters(m, cb_add, opt); }
void nc_optimizer_set_grad_scale(nc_optimizer* opt, double scale) { if (opt && opt->state) ((opt_common*)opt->state)->grad_scale = scale; }

/* Re-homes every parameter gradient of the optimizer into ONE device allocation (each gradient becomes a
 * view at a 256-byte aligned offset) and returns its device address and length in floats.  A data-parallel
 * caller sums that single range across ranks instead of one small buffer per parameter; padding between
 * views is zero and stays zero.  Gradients keep their values. */
/* storages that hold flattened gradients: views into them are written in place although they share storage */
#define NCI_MAX_ARENAS 16
static const nc_storage* g_arenas[NCI_MAX_ARENAS];
bool nci_is_grad_arena(const nc_storage* st) {
    if (!st) return false;
    for (int i = 0; i < NCI_MAX_ARENAS; i++) if (g_arenas[i] == st) return true;
    return false;
}
/* called by nc_storage_release when a storage dies: a later storage at the same address must not pass for an arena */
void nci_forget_grad_arena(const nc_storage* st) {
    for (int i = 0; i < NCI_MAX_ARENAS; i++) if (g_arenas[i] == st) g_arenas[i] = NULL;
}
void* nc_optimizer_flatten_grads(nc_optimizer* opt, size_t* n_floats) {
    if (!opt || !n_floats) return NULL;
    size_t total = 0;
    for (size_t i = 0; i < opt->n_params; i++) {
        nc_tensor* p = opt->params[i];
        if (!p || p->dtype != NC_F32 || !nci_on_cuda(p)) { NC_SET_ERROR(NC_ERR_DEVICE, "flatten_grads: f32 CUDA parameters required"); return NULL; }
        total += (p->numel + 63) & ~(size_t)63;
    }
    if (!total) return NULL;
    int slot = -1;
    for (int i = 0; i < NCI_MAX_ARENAS && slot < 0; i++) if (!g_arenas[i]) slot = i;
    if (slot < 0) { NC_SET_ERROR(NC_ERR_ALLOC, "flatten_grads: %d gradient arenas are alive already", NCI_MAX_ARENAS); return NULL; }
    nc_storage* arena = nc_storage_create_on(total * sizeof(float), NC_DEVICE_CUDA);
    if (!arena) return NULL;
    nc_cuda_memset_async(arena->cuda_data, 0, total * sizeof(float), nci_stream());
    g_arenas[slot] = arena;
    size_t off = 0;
    for (size_t i = 0; i < opt->n_params; i++) {
        nc_tensor* p = opt->params[i];
        nc_tensor* g = nc_calloc(1, sizeof(nc_tensor));
        if (!g) { nc_storage_release(arena); return NULL; }
        g->storage = nc_storage_retain(arena);
        g->offset = off;
        g->ndim = p->ndim;
        g->numel = p->numel;
        memcpy(g->shape, p->shape, sizeof(g->shape));
        memcpy(g->strides, p->strides, sizeof(g->strides));
        g->dtype = NC_F32;
        g->is_leaf = true;
        g->is_contiguous = true;
        if (p->grad) { nc_tensor_copy_(g, p->grad); g->is_reachable = true; /* holds values: accumulate, do not take over */ nc_tensor_free(p->grad); }
        p->grad = g;
        p->requires_grad = true;
        off += (p->numel + 63) & ~(size_t)63;
    }
    void* base = arena->cuda_data;
    if (opt->state) { ((opt_common*)opt->state)->arena = arena; ((opt_common*)opt->state)->arena_bytes = total * sizeof(float); }
    nc_storage_release(arena); /* the views keep it alive */
    *n_floats = total;
    return base;
}

static nc_tensor* state_like(const nc_tensor* p) {
    nc_tensor* s = nci_empty_on(p->shape, p->ndim, p->dtype, p->storage->device);
    if (s) nc_tensor_fill_(s, 0.0);
    return s;
}
static bool param_ready(const nc_tensor* p, const char* who) {
    if (!p->grad) return false;
    if (!nci_need_cuda_f32(p, who) || !nci_need_cuda_f32(p->grad, who)) return false;
    if (!p->is_contiguous || !p->grad->is_contiguous) { NC_SET_ERROR(NC_ERR_NOT_CONTIGUOUS, "%s: parameters must be contiguous", who); return false; }
    return true;
}

/* ------------------------------------------------------------------ SGD */
static void sgd_step(nc_optimizer* self) {
    /* one launch for all parameters that have a gradient (tables of device pointers gathered here) */
    sgd_state* st = self->state;
    static float* P[NC_MAX_OPTIM_PARAMS]; static float* V[NC_MAX_OPTIM_PARAMS]; static float* G[NC_MAX_OPTIM_PARAMS];
    static size_t Nn[NC_MAX_OPTIM_PARAMS];
    int count = 0;
    for (size_t i = 0; i < self->n_params; i++) {
        nc_tensor* p = self->params[i];
        if (!param_ready(p, "sgd")) continue;
        float* vel = NULL;
        if (st->cfg.momentum != 0.0) {
            if (!st->velocity[i]) st->velocity[i] = state_like(p);
            if (!st->velocity[i]) continue;
            vel = nci_fptr(st->velocity[i]);
        }
        P[count] = nci_fptr(p); V[count] = vel; G[count] = nci_fptr(p->grad); Nn[count] = p->numel;
        count++;
    }
    if (count)
        nci_ok(nc_cuda_sgd_update_multi_f32_ex(count, P, V, G, Nn, self->lr, st->cfg.momentum, st->cfg.dampening, st->cfg.weight_decay,
                                               st->cfg.nesterov ? 1 : 0, self->t == 0 ? 1 : 0, st->c.grad_scale, nci_stream()), "sgd step");
    self->t++;
}
static void sgd_free(void* state) {
    sgd_state* st = state;
    for (size_t i = 0; i < NC_MAX_OPTIM_PARAMS; i++) if (st->velocity[i]) nc_tensor_free(st->velocity[i]);
    nc_free(st);
}
nc_optimizer* nc_sgd(double lr, nc_sgd_config config) {
    nc_optimizer* o = nc_calloc(1, sizeof(nc_optimizer));
    sgd_state* st = o ? nc_calloc(1, sizeof(sgd_state)) : NULL;
    if (!st) { nc_free(o); return NULL; }
    st->c.grad_scale = 1.0;
    st->cfg = config;
    o->lr = lr; o->step = sgd_step; o->state = st; o->free_state = sgd_free;
    return o;
}
nc_optimizer* nc_sgd_from_module(nc_module* m, double lr, nc_sgd_config config) {
    nc_optimizer* o = nc_sgd(lr, config);
    if (o) nc_optimizer_add_module(o, m);
    return o;
}
nc_optimizer* nc_sgd_simple(nc_module* m, double lr) { return nc_sgd_from_module(m, lr, NC_SGD_DEFAULT); }
nc_optimizer* nc_sgd_momentum(nc_module* m, double lr, double momentum) {
    nc_sgd_config c = NC_SGD_DEFAULT;
    c.momentum = momentum;
    return nc_sgd_from_module(m, lr, c);
}

/* ------------------------------------------------------------------ Adam / AdamW */
static void adam_step(nc_optimizer* self) {
    adam_state* st = self->state;
    self->t++;
    const double bc1 = 1.0 - pow(st->cfg.beta1, (double)self->t), bc2 = 1.0 - pow(st->cfg.beta2, (double)self->t);
    static float* P[NC_MAX_OPTIM_PARAMS]; static float* M[NC_MAX_OPTIM_PARAMS]; static float* V[NC_MAX_OPTIM_PARAMS];
    static float* X[NC_MAX_OPTIM_PARAMS]; static float* G[NC_MAX_OPTIM_PARAMS];
    static size_t Nn[NC_MAX_OPTIM_PARAMS];
    int count = 0;
    for (size_t i = 0; i < self->n_params; i++) {
        nc_tensor* p = self->params[i];
        if (!param_ready(p, "adam")) continue;
        if (!st->m[i]) {
            st->m[i] = state_like(p);
            st->v[i] = state_like(p);
            if (st->cfg.amsgrad) st->vmax[i] = state_like(p);
        }
        if (!st->m[i] || !st->v[i]) continue;
        P[count] = nci_fptr(p); M[count] = nci_fptr(st->m[i]); V[count] = nci_fptr(st->v[i]);
        X[count] = st->vmax[i] ? nci_fptr(st->vmax[i]) : NULL; G[count] = nci_fptr(p->grad); Nn[count] = p->numel;
        count++;
    }
    if (count)
        nci_ok(nc_cuda_adam_update_multi_f32_ex(count, P, M, V, X, G, Nn, self->lr, st->cfg.beta1, st->cfg.beta2, st->cfg.eps,
                                                st->cfg.weight_decay, bc1, bc2, st->c.grad_scale, nci_stream()), "adam step");
}
static void adam_free(void* state) {
    adam_state* st = state;
    for (size_t i = 0; i < NC_MAX_OPTIM_PARAMS; i++) {
        if (st->m[i]) nc_tensor_free(st->m[i]);
        if (st->v[i]) nc_tensor_free(st->v[i]);
        if (st->vmax[i]) nc_tensor_free(st->vmax[i]);
    }
    nc_free(st);
}
nc_optimizer* nc_adam(double lr, nc_adam_config config) {
    nc_optimizer* o = nc_calloc(1, sizeof(nc_optimizer));
    adam_state* st = o ? nc_calloc(1, sizeof(adam_state)) : NULL;
    if (!st) { nc_free(o); return NULL; }
    st->c.grad_scale = 1.0;
    st->cfg = config;
    o->lr = lr; o->step = adam_step; o->state = st; o->free_state = adam_free;
    return o;
}
nc_optimizer* nc_adam_from_module(nc_module* m, double lr, nc_adam_config config) {
    nc_optimizer* o = nc_adam(lr, config);
    if (o) nc_optimizer_add_module(o, m);
    return o;
}
nc_optimizer* nc_adam_default(nc_module* m, double lr) { return nc_adam_from_module(m, lr, NC_ADAM_DEFAULT); }
nc_optimizer* nc_adamw(nc_module* m, double lr, double weight_decay) {
    nc_adam_config c = NC_ADAM_DEFAULT;
    c.weight_decay = weight_decay;
    return nc_adam_from_module(m, lr, c);
}

/* ------------------------------------------------------------------ optimizer state <-> named tensors */
static void sd_add_clone(nc_state_dict* sd, const char* prefix, size_t i, const nc_tensor* t) {
    if (!t) return;
    char name[NC_MAX_NAME_LEN];
    snprintf(name, sizeof(name), "%s.%zu", prefix, i);
    nc_tensor* c = nc_tensor_clone(t);
    if (c) nc_state_dict_add(sd, name, c);
}
nc_state_dict* nc_optimizer_state_dict(nc_optimizer* opt) {
    if (!opt) return NULL;
    nc_state_dict* sd = nc_state_dict_create();
    if (!sd) return NULL;
    const int64_t t = (int64_t)opt->t;
    const size_t one = 1;
    nc_device_type dev = nc_get_default_device();
    nc_set_default_device(NC_DEVICE_CPU);  /* the counter is host bookkeeping */
    nc_tensor* step = nc_tensor_from_data(&t, &one, 1, NC_I64);
    nc_set_default_device(dev);
    if (step) nc_state_dict_add(sd, "step", step);
    if (opt->step == sgd_step) {
        sgd_state* st = opt->state;
        for (size_t i = 0; i < opt->n_params; i++) sd_add_clone(sd, "velocity", i, st->velocity[i]);
    } else if (opt->step == adam_step) {
        adam_state* st = opt->state;
        for (size_t i = 0; i < opt->n_params; i++) {
            sd_add_clone(sd, "m", i, st->m[i]);
            sd_add_clone(sd, "v", i, st->v[i]);
            sd_add_clone(sd, "vmax", i, st->vmax[i]);
        }
    }
    return sd;
}
static nc_error restore_slot(nc_state_dict* sd, const char* prefix, size_t i, const nc_tensor* param, nc_tensor** slot) {
    char name[NC_MAX_NAME_LEN];
    snprintf(name, sizeof(name), "%s.%zu", prefix, i);
    nc_tensor* src = nc_state_dict_get(sd, name);
    if (!src) return NC_OK;
    if (!nc_tensor_shape_eq(param, src)) { NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "optimizer state %s does not fit parameter %zu", name, i); return NC_ERR_SHAPE_MISMATCH; }
    if (!*slot) *slot = state_like(param);
    if (!*slot) return NC_ERR_ALLOC;
    return nc_tensor_copy_(*slot, src);
}
nc_error nc_optimizer_load_state_dict(nc_optimizer* opt, nc_state_dict* sd) {
    if (!opt || !sd) return NC_ERR_NULL_PTR;
    nc_tensor* step = nc_state_dict_get(sd, "step");
    if (step && step->numel == 1) opt->t = (size_t)nc_tensor_get_flat(step, 0);
    nc_error err = NC_OK;
    for (size_t i = 0; i < opt->n_params && err == NC_OK; i++) {
        if (opt->step == sgd_step) {
            err = restore_slot(sd, "velocity", i, opt->params[i], &((sgd_state*)opt->state)->velocity[i]);
        } else if (opt->step == adam_step) {
            adam_state* st = opt->state;
            err = restore_slot(sd, "m", i, opt->params[i], &st->m[i]);
            if (err == NC_OK) err = restore_slot(sd, "v", i, opt->params[i], &st->v[i]);
            if (err == NC_OK) err = restore_slot(sd, "vmax", i, opt->params[i], &st->vmax[i]);
        }
    }
    return err;
}
