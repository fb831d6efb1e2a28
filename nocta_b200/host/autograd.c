/*
 * Autograd tape: nodes and the reverse sweep.
 *
 * Contract kept from the reference (include/nocta/autograd/node.h:15-53, src/autograd/backward.c:
 * 127-252): a node's backward callback gets (grad_output, saved tensors, n_saved) and returns a
 * nc_calloc'd array with one gradient per node input; inputs and saved tensors are borrowed unless
 * saved with nc_node_save_owned_tensor; user code may register its own nodes.
 *
 * What differs is cost, not meaning: an edge gradient that arrives first is adopted (no clone),
 * later arrivals are added in place, and a gradient whose storage is shared is copied before it is
 * written (copy-on-write), so every activation gradient is touched once instead of twice.
 */
#include "internal.h"
#include <string.h>

static int g_grad_enabled = 1;
static nc_grad_mode g_grad_mode = NC_GRAD_ACCUMULATE;

void nc_set_grad_mode(nc_grad_mode mode) { g_grad_mode = mode; }
nc_grad_mode nc_get_grad_mode(void) { return g_grad_mode; }
int nc_grad_enabled(void) { return g_grad_enabled; }
void nc_set_grad_enabled(int enabled) { g_grad_enabled = enabled ? 1 : 0; }
nc_no_grad_guard nc_no_grad_begin(void) {
    nc_no_grad_guard g = {g_grad_enabled};
    g_grad_enabled = 0;
    return g;
}
void nc_no_grad_end(nc_no_grad_guard* guard) { if (guard) g_grad_enabled = guard->prev_enabled; }

nc_node* nc_node_create(const char* op_name, nc_backward_fn backward) {
    nc_node* n = nc_calloc(1, sizeof(nc_node));
    if (!n) return NULL;
    n->op_name = op_name;
    n->backward = backward;
    return n;
}
void nc_node_add_input(nc_node* node, nc_tensor* input) {
    if (node && node->n_inputs < NC_MAX_INPUTS) node->inputs[node->n_inputs++] = input;
}
void nc_node_save_tensor(nc_node* node, nc_tensor* t) {
    if (!node || node->n_saved >= NC_MAX_INPUTS) return;
    node->saved_tensors[node->n_saved] = t;
    node->saved_tensors_owned[node->n_saved++] = false;
}
void nc_node_save_owned_tensor(nc_node* node, nc_tensor* t) {
    if (!node || node->n_saved >= NC_MAX_INPUTS) return;
    node->saved_tensors[node->n_saved] = t;
    node->saved_tensors_owned[node->n_saved++] = true;
}
void nc_node_free(nc_node* node) {
    if (!node) return;
    for (size_t i = 0; i < node->n_saved; i++)
        if (node->saved_tensors_owned[i] && node->saved_tensors[i]) nc_tensor_free(node->saved_tensors[i]);
    nc_free(node);
}
nc_node* nci_attach(nc_tensor* out, const char* name, nc_backward_fn fn) {
    nc_node* n = nc_node_create(name, fn);
    if (!n) return NULL;
    n->output = out;
    out->grad_fn = n;
    out->is_leaf = false;
    out->requires_grad = true;
    return n;
}

/* iterative post-order DFS over grad_fn edges; returns nodes with producers before consumers */
typedef struct { nc_node* node; size_t next; } dfs_frame;
nc_node** nc_build_topo(nc_tensor* t, size_t* n_nodes) {
    *n_nodes = 0;
    if (!t || !t->grad_fn) return NULL;
    size_t cap = 64, n = 0, scap = 64, sp = 0;
    nc_node** order = nc_alloc(cap * sizeof(*order));
    dfs_frame* stack = nc_alloc(scap * sizeof(*stack));
    if (!order || !stack) { nc_free(order); nc_free(stack); return NULL; }
    stack[sp++] = (dfs_frame){t->grad_fn, 0};
    t->grad_fn->visited = 1;
    while (sp) {
        dfs_frame* f = &stack[sp - 1];
        if (f->next < f->node->n_inputs) {
            nc_tensor* in = f->node->inputs[f->next++];
            if (in && in->grad_fn && !in->grad_fn->visited) {
                in->grad_fn->visited = 1;
                if (sp == scap) {
                    dfs_frame* ns = nc_realloc(stack, scap * sizeof(*stack), 2 * scap * sizeof(*stack));
                    if (!ns) { nc_free(order); return NULL; }
                    stack = ns; scap *= 2;
                }
                stack[sp++] = (dfs_frame){in->grad_fn, 0};
            }
        } else {
            if (n == cap) {
                nc_node** no = nc_realloc(order, cap * sizeof(*order), 2 * cap * sizeof(*order));
                if (!no) { nc_free(stack); return NULL; }
                order = no; cap *= 2;
            }
            order[n++] = f->node;
            sp--;
        }
    }
    nc_free(stack);
    for (size_t i = 0; i < n; i++) { order[i]->visited = 0; order[i]->ref_count = (int)i; /* index for O(1) lookup */ }
    *n_nodes = n;
    return order;
}

/* a += b where a may share storage with another header: copy first */
static nc_tensor* add_into(nc_tensor* a, nc_tensor* b) {
    if (a->storage->refcount > 1) {
        nc_tensor* c = nc_tensor_clone(a);
        nc_tensor_free(a);
        a = c;
        if (!a) return NULL;
    }
    nc_add_(a, b);
    return a;
}

static nc_grad_ready_fn g_ready_fn = NULL;
static void* g_ready_ctx = NULL;
void nc_set_grad_ready_hook(nc_grad_ready_fn fn, void* ctx) { g_ready_fn = fn; g_ready_ctx = ctx; }

/* destinations offered to the backward callback that is running (see nci_param_grad_out) */
static nc_tensor* g_dest[NC_MAX_INPUTS];
nc_tensor* nci_param_grad_out(size_t input_index, const nc_tensor* like) {
    nc_tensor* d = input_index < NC_MAX_INPUTS ? g_dest[input_index] : NULL;
    if (d && d->dtype == like->dtype && d->is_contiguous && nc_tensor_shape_eq(d, like)) {
        nc_tensor* a = nci_alias(d);
        if (a) return a;
    }
    return nci_empty_on(like->shape, like->ndim, like->dtype, NC_DEVICE_CUDA);
}
static void offer_destinations(const nc_node* node) {
    for (size_t j = 0; j < NC_MAX_INPUTS; j++) {
        const nc_tensor* in = j < node->n_inputs ? node->inputs[j] : NULL;
        g_dest[j] = (in && in->is_leaf && in->requires_grad && in->grad && !in->grad->is_reachable && in->grad->storage &&
                     nci_is_grad_arena(in->grad->storage)) ? in->grad : NULL;
    }
}

static void accumulate_leaf(nc_tensor* leaf, nc_tensor* g) {
    if (!leaf->requires_grad || leaf->numel != g->numel) return;
    if (leaf->grad && g->storage == leaf->grad->storage && g->offset == leaf->grad->offset) {
        /* the backward kernel wrote straight into the parameter's (cleared) arena slot */
        leaf->grad->is_reachable = true;
        if (g_ready_fn) g_ready_fn(leaf, g_ready_ctx);
        return;
    }
    if (!leaf->grad) {
        /* first contribution since the gradient was cleared: take it over instead of adding it to zeros.  The
         * new header shares g's storage; a later in-place add goes through add_into, which copies first while
         * the storage is still shared. */
        if (g->dtype == leaf->dtype && g->storage->device == leaf->storage->device && g->is_contiguous && nci_is_dense(g) &&
            nc_tensor_shape_eq(g, leaf)) {
            leaf->grad = nci_alias(g);
            if (leaf->grad) {
                leaf->grad->is_leaf = true;
                leaf->grad->is_reachable = true; /* written by backward: see nc_tensor_zero_grad_ */
                if (g_ready_fn) g_ready_fn(leaf, g_ready_ctx);
                return;
            }
        }
        leaf->grad = nci_empty_on(leaf->shape, leaf->ndim, leaf->dtype, leaf->storage->device);
        if (!leaf->grad) return;
        nc_tensor_fill_(leaf->grad, 0.0);
    }
    if (leaf->grad->storage->refcount > 1 && !nci_is_grad_arena(leaf->grad->storage)) {
        /* taken over earlier in this sweep and still shared with the tensor it came from */
        nc_tensor* own = add_into(leaf->grad, g);
        if (own) { leaf->grad = own; own->is_leaf = true; own->is_reachable = true; }
        if (g_ready_fn) g_ready_fn(leaf, g_ready_ctx);
        return;
    }
    nc_add_(leaf->grad, g);
    leaf->grad->is_reachable = true;
    /* the accumulate kernel is queued: a data-parallel caller may now queue this gradient's all-reduce
     * behind it while the rest of the backward sweep keeps the device busy */
    if (g_ready_fn) g_ready_fn(leaf, g_ready_ctx);
}

/* The seed nc_backward itself filled with ones: a loss node that receives it knows the upstream value on the host
 * and does not have to read a device scalar back (which would drain the whole forward pass before backward starts). */
static const nc_tensor* g_unit_seed = NULL;
bool nci_is_unit_seed(const nc_tensor* g) { return g && g == g_unit_seed; }

nc_error nc_backward(nc_tensor* t, nc_tensor* grad_output) {
    if (!t) return NC_ERR_NULL_PTR;
    nc_tensor* seed = NULL;
    g_unit_seed = NULL;
    if (grad_output) {
        if (grad_output->numel != t->numel) { NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "backward: gradient has %zu elements, output %zu", grad_output->numel, t->numel); return NC_ERR_SHAPE_MISMATCH; }
        seed = nci_alias(grad_output);
    } else {
        if (t->numel != 1) { NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "backward: output must be scalar, got %zu elements", t->numel); return NC_ERR_SHAPE_MISMATCH; }
        seed = nci_empty_on(t->shape, t->ndim, t->dtype, t->storage->device);
        if (seed) nc_tensor_fill_(seed, 1.0);
        g_unit_seed = seed;
    }
    if (!seed) return NC_ERR_ALLOC;
    if (!t->grad_fn) {
        if (t->requires_grad) accumulate_leaf(t, seed);
        g_unit_seed = NULL;
        nc_tensor_free(seed);
        return NC_OK;
    }
    size_t n = 0;
    nc_node** topo = nc_build_topo(t, &n);
    if (!topo || !n) { g_unit_seed = NULL; nc_tensor_free(seed); nc_free(topo); return NC_OK; }
    nc_tensor** pending = nc_calloc(n, sizeof(*pending));
    if (!pending) { g_unit_seed = NULL; nc_tensor_free(seed); nc_free(topo); return NC_ERR_ALLOC; }
    pending[n - 1] = seed;
    const int prev = g_grad_enabled;
    g_grad_enabled = 0;
    nc_error rc = NC_OK;
    for (size_t i = n; i-- > 0;) {
        nc_node* node = topo[i];
        nc_tensor* g = pending[i];
        if (!node || !g || !node->backward) continue;
        offer_destinations(node);
        nc_tensor** in_grads = node->backward(g, node->saved_tensors, node->n_saved);
        memset(g_dest, 0, sizeof(g_dest));
        if (!in_grads) { if (nc_last_error != NC_OK) rc = nc_last_error; continue; }
        /* callbacks return one distinct tensor object per input (views may share storage) */
        for (size_t j = 0; j < node->n_inputs; j++) {
            nc_tensor* in = node->inputs[j];
            nc_tensor* ig = in_grads[j];
            if (!ig) continue;
            bool adopted = false;
            if (in) {
                if (in->requires_grad && in->is_leaf) accumulate_leaf(in, ig);
                if (in->grad_fn) {
                    size_t k = (size_t)in->grad_fn->ref_count;
                    if (k < n && topo[k] == in->grad_fn) {
                        if (!pending[k]) {
                            if (ig != g) { pending[k] = ig; adopted = true; }
                            else pending[k] = nc_tensor_clone(ig);
                        } else {
                            pending[k] = add_into(pending[k], ig);
                        }
                    }
                }
            }
            if (!adopted && ig != g) nc_tensor_free(ig);
        }
        nc_free(in_grads);
        if (g == g_unit_seed) g_unit_seed = NULL;   /* only the root node ever sees it */
        nc_tensor_free(g);
        pending[i] = NULL;
    }
    g_unit_seed = NULL;
    g_grad_enabled = prev;
    for (size_t i = 0; i < n; i++) if (pending[i]) nc_tensor_free(pending[i]);
    for (size_t i = 0; i < n; i++) topo[i]->ref_count = 0;
    nc_free(pending);
    nc_free(topo);
    return rc;
}
nc_error nc_backward_scalar(nc_tensor* loss) { return nc_backward(loss, NULL); }
