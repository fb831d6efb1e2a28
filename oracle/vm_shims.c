/* TEST INFRASTRUCTURE ONLY (linked into oracle/_ref/apps/noc_vm, never into the product libraries).
 *
 * The reference's script interpreter (src/lang/vm.c:1173-1264) registers natives for every operator of the reference,
 * including the ones outside the training hot path that this repository does not build (tanh, SiLU, average pooling,
 * BCE, ...).  To link the UNMODIFIED interpreter against libnocta.so, those entry points are defined here as stubs that
 * record an error and return NULL, which the interpreter turns into nil: a script that stays on the training path
 * (convolution, BatchNorm, ReLU, max-pool, matmul, cross-entropy, backward, SGD) never reaches them. */
#include "nocta/nocta.h"
#include <stdio.h>

static nc_tensor* off_path(const char* name) {
    fprintf(stderr, "[vm_shims] %s is not on the training path this library implements\n", name);
    return NULL;
}
#define UNARY(fn) nc_tensor* fn(nc_tensor* x) { (void)x; return off_path(#fn); }
UNARY(nc_tanh_act) UNARY(nc_silu) UNARY(nc_sqrt) UNARY(nc_exp) UNARY(nc_log) UNARY(nc_abs)
UNARY(nc_min_all) UNARY(nc_max_all)
nc_tensor* nc_mean(nc_tensor* x, int axis, bool keep) { (void)x; (void)axis; (void)keep; return off_path("nc_mean"); }
nc_tensor* nc_leaky_relu(nc_tensor* x, double a) { (void)x; (void)a; return off_path("nc_leaky_relu"); }
nc_tensor* nc_clamp(nc_tensor* x, double lo, double hi) { (void)x; (void)lo; (void)hi; return off_path("nc_clamp"); }
nc_tensor* nc_pow_scalar(nc_tensor* x, double e) { (void)x; (void)e; return off_path("nc_pow_scalar"); }
nc_tensor* nc_sub_scalar(nc_tensor* x, double s) { (void)x; (void)s; return off_path("nc_sub_scalar"); }
nc_tensor* nc_div_scalar(nc_tensor* x, double s) { (void)x; (void)s; return off_path("nc_div_scalar"); }
nc_tensor* nc_div(nc_tensor* a, nc_tensor* b) { (void)a; (void)b; return off_path("nc_div"); }
nc_tensor* nc_var(nc_tensor* x, int axis, bool keep, bool unbiased) { (void)x; (void)axis; (void)keep; (void)unbiased; return off_path("nc_var"); }
nc_tensor* nc_std(nc_tensor* x, int axis, bool keep, bool unbiased) { (void)x; (void)axis; (void)keep; (void)unbiased; return off_path("nc_std"); }
nc_tensor* nc_norm(nc_tensor* x, double p) { (void)x; (void)p; return off_path("nc_norm"); }
nc_tensor* nc_bce_loss(nc_tensor* p, nc_tensor* t) { (void)p; (void)t; return off_path("nc_bce_loss"); }
nc_tensor* nc_avgpool2d_forward(nc_tensor* x, size_t k, size_t s) { (void)x; (void)k; (void)s; return off_path("nc_avgpool2d_forward"); }
void nc_adam_step_single(nc_tensor* param, nc_tensor* grad, nc_tensor* m, nc_tensor* v, nc_tensor* v_max, nc_adam_config* config,
                         double lr, int t) {
    (void)param; (void)grad; (void)m; (void)v; (void)v_max; (void)config; (void)lr; (void)t;
    off_path("nc_adam_step_single");
}
