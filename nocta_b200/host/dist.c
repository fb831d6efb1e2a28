/*
 * Data-parallel gradient exchange for a C caller: one process per GPU, every rank a full replica, the parameter
 * gradients of one optimizer summed across ranks once per step (the 1/world factor is folded into the optimizer kernel).
 * The reference has no distributed layer; the training step it would wrap is examples/mnist.c:471-508
 * (zero_grad, forward, loss, nc_backward, optimizer step) with nc_dist_allreduce_grads between backward and step.
 *
 *   nc_bucket_plan   pure host logic: cuts the flat gradient arena into contiguous buckets and decides, from the
 *                    "gradient of leaf i is final" notifications of the backward sweep, when a bucket may be sent.
 *                    No device or NCCL call: the CPU tests drive it over gloo.
 *   nc_dist          the plan + one NCCL communicator + a communication stream ordered against the compute stream by
 *                    events.  A bucket's all-reduce is queued as soon as the kernel that wrote its last gradient has been
 *                    queued, so the exchange of late layers overlaps the backward of early ones; the host never waits.
 *
 * NCCL is bound at run time (dlopen "libnccl.so.2"): a process that never calls nc_dist_init needs no NCCL, and a host
 * program that already loaded one (a Python process that imported torch) shares that copy.
 */
#include "internal.h"
#include <dlfcn.h>
#include <stdio.h>

/* ------------------------------------------------------------------ bucket plan */
struct nc_bucket_plan {
    size_t n_entries;
    size_t* offset;      /* arena offset of entry i (ascending) */
    int* bucket_of;
    int* expected;       /* ready notifications entry i produced in the step the plan learned from */
    int* seen;           /* ... in the current step */
    size_t n_buckets;
    size_t* start;       /* bucket b covers arena floats [start[b], stop[b]); bucket 0 is the END of the arena */
    size_t* stop;
    int* pending;        /* expected notifications not yet seen; < 0: never fire early */
    bool* fired;
    bool learned, relearn;
    int late;            /* notifications that arrived after their bucket had been sent (this step) */
};

nc_bucket_plan* nc_bucket_plan_create(size_t n_entries, const size_t* offsets, const size_t* numels, size_t arena_floats,
                                      size_t bucket_floats) {
    if (!n_entries || !offsets || !numels || !arena_floats) return NULL;
    for (size_t i = 0; i < n_entries; i++)
        if (offsets[i] + numels[i] > arena_floats || (i && offsets[i] < offsets[i - 1] + numels[i - 1])) {
            NC_SET_ERROR(NC_ERR_INVALID_SHAPE, "bucket plan: entries must lie inside the arena in ascending order");
            return NULL;
        }
    nc_bucket_plan* p = nc_calloc(1, sizeof(*p));
    if (!p) return NULL;
    p->n_entries = n_entries;
    p->offset = nc_calloc(n_entries, sizeof(size_t));
    p->bucket_of = nc_calloc(n_entries, sizeof(int));
    p->expected = nc_calloc(n_entries, sizeof(int));
    p->seen = nc_calloc(n_entries, sizeof(int));
    p->start = nc_calloc(n_entries, sizeof(size_t));
    p->stop = nc_calloc(n_entries, sizeof(size_t));
    p->pending = nc_calloc(n_entries, sizeof(int));
    p->fired = nc_calloc(n_entries, sizeof(bool));
    if (!p->offset || !p->bucket_of || !p->expected || !p->seen || !p->start || !p->stop || !p->pending || !p->fired) {
        nc_bucket_plan_free(p);
        return NULL;
    }
    /* The backward sweep produces gradients from the end of the arena (last layer) towards its start: buckets are built
     * from the end so that the first one to complete is tight.  A bucket closes once it holds bucket_floats or more. */
    size_t b = 0, hi = arena_floats;
    for (size_t k = n_entries; k-- > 0;) {
        p->offset[k] = offsets[k];
        p->bucket_of[k] = (int)b;
        const bool close = (hi - offsets[k] >= bucket_floats) || k == 0;
        if (close) {
            p->start[b] = k == 0 ? 0 : offsets[k];
            p->stop[b] = hi;
            hi = p->start[b];
            b++;
        }
    }
    p->n_buckets = b;
    nc_bucket_plan_begin_step(p);
    return p;
}
void nc_bucket_plan_free(nc_bucket_plan* p) {
    if (!p) return;
    nc_free(p->offset); nc_free(p->bucket_of); nc_free(p->expected); nc_free(p->seen);
    nc_free(p->start); nc_free(p->stop); nc_free(p->pending); nc_free(p->fired);
    nc_free(p);
}
size_t nc_bucket_plan_count(const nc_bucket_plan* p) { return p ? p->n_buckets : 0; }
void nc_bucket_plan_range(const nc_bucket_plan* p, size_t b, size_t* start, size_t* stop) {
    if (!p || b >= p->n_buckets) return;
    if (start) *start = p->start[b];
    if (stop) *stop = p->stop[b];
}
void nc_bucket_plan_begin_step(nc_bucket_plan* p) {
    if (!p) return;
    for (size_t b = 0; b < p->n_buckets; b++) { p->fired[b] = false; p->pending[b] = p->learned ? 0 : -1; }
    for (size_t i = 0; i < p->n_entries; i++) {
        p->seen[i] = 0;
        /* Entries that never report (parameters no backward reaches, e.g. BatchNorm running statistics registered as
         * parameters) do not hold their bucket back; an entry that reports twice (a shared weight) is waited for twice. */
        if (p->learned) p->pending[p->bucket_of[i]] += p->expected[i];
    }
    if (p->learned)
        for (size_t b = 0; b < p->n_buckets; b++) if (p->pending[b] == 0) p->pending[b] = -1;  /* nothing ever reports: leave it to finish */
    p->late = 0;
}
int nc_bucket_plan_on_ready(nc_bucket_plan* p, size_t entry) {
    if (!p || entry >= p->n_entries) return -1;
    const int b = p->bucket_of[entry];
    p->seen[entry]++;
    if (p->fired[b]) { p->late++; p->relearn = true; return -1; }   /* the graph changed since the plan learned it */
    if (!p->learned || p->pending[b] < 0) return -1;
    if (p->seen[entry] > p->expected[entry]) { p->relearn = true; return -1; }
    if (--p->pending[b] == 0) { p->fired[b] = true; return b; }
    return -1;
}
int nc_bucket_plan_next_unfired(nc_bucket_plan* p) {
    if (!p) return -1;
    for (size_t b = 0; b < p->n_buckets; b++)
        if (!p->fired[b]) { p->fired[b] = true; return (int)b; }
    return -1;
}
int nc_bucket_plan_end_step(nc_bucket_plan* p) {
    if (!p) return 0;
    const int late = p->late;
    if (!p->learned || p->relearn) {
        for (size_t i = 0; i < p->n_entries; i++) p->expected[i] = p->seen[i];
        p->learned = true;
        p->relearn = false;
    } else {
        for (size_t i = 0; i < p->n_entries; i++) if (p->seen[i] != p->expected[i]) p->relearn = true;  /* applies from the step after next */
    }
    nc_bucket_plan_begin_step(p);
    return late;
}

/* ------------------------------------------------------------------ NCCL, bound at run time */
typedef struct { char internal[128]; } nccl_unique_id;   /* ncclUniqueId: 128 opaque bytes (nccl.h) */
typedef void* nccl_comm;
enum { NCCL_FLOAT32 = 7, NCCL_SUM = 0 };                 /* ncclFloat32 / ncclSum (nccl.h) */
static struct {
    void* handle;
    int (*get_unique_id)(nccl_unique_id*);
    int (*comm_init_rank)(nccl_comm*, int, nccl_unique_id, int);
    int (*all_reduce)(const void*, void*, size_t, int, int, nccl_comm, void*);
    int (*comm_destroy)(nccl_comm);
    const char* (*error_string)(int);
} g_nccl;

static bool nccl_bind(void) {
    if (g_nccl.handle) return true;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) { NC_SET_ERROR(NC_ERR_DEVICE, "nc_dist: cannot load libnccl.so.2 (%s)", dlerror()); return false; }
    *(void**)&g_nccl.get_unique_id = dlsym(h, "ncclGetUniqueId");
    *(void**)&g_nccl.comm_init_rank = dlsym(h, "ncclCommInitRank");
    *(void**)&g_nccl.all_reduce = dlsym(h, "ncclAllReduce");
    *(void**)&g_nccl.comm_destroy = dlsym(h, "ncclCommDestroy");
    *(void**)&g_nccl.error_string = dlsym(h, "ncclGetErrorString");
    if (!g_nccl.get_unique_id || !g_nccl.comm_init_rank || !g_nccl.all_reduce || !g_nccl.comm_destroy) {
        NC_SET_ERROR(NC_ERR_DEVICE, "nc_dist: libnccl lacks a required symbol");
        dlclose(h);
        return false;
    }
    g_nccl.handle = h;
    return true;
}
static bool nccl_ok(int rc, const char* what) {
    if (rc == 0) return true;
    NC_SET_ERROR(NC_ERR_DEVICE, "nc_dist: %s failed: %s", what, g_nccl.error_string ? g_nccl.error_string(rc) : "NCCL error");
    return false;
}

/* ------------------------------------------------------------------ nc_dist */
struct nc_dist {
    int rank, world;
    nc_optimizer* opt;
    nc_bucket_plan* plan;
    nccl_comm comm;
    float* arena;
    size_t arena_floats;
    void* comm_stream;
    void** ready_ev;    /* compute stream: the bucket's last gradient kernel has been queued */
    void** done_ev;     /* communication stream: the bucket's all-reduce has finished */
    void* bwd_end_ev;
    int status;         /* first failure of the current step */
    int late_total;
};

int nc_dist_unique_id(void* id128) {
    if (!id128) return NC_ERR_NULL_PTR;
    if (!nccl_bind()) return NC_ERR_DEVICE;
    nccl_unique_id id;
    if (!nccl_ok(g_nccl.get_unique_id(&id), "ncclGetUniqueId")) return NC_ERR_DEVICE;
    memcpy(id128, &id, sizeof(id));
    return NC_OK;
}

static void dist_fire(nc_dist* d, int b) {
    size_t s = 0, e = 0;
    nc_bucket_plan_range(d->plan, (size_t)b, &s, &e);
    if (e <= s) return;
    if (nc_cuda_event_record(d->ready_ev[b], nci_stream()) || nc_cuda_stream_wait_event(d->comm_stream, d->ready_ev[b])) { d->status = NC_ERR_DEVICE; return; }
    if (!nccl_ok(g_nccl.all_reduce(d->arena + s, d->arena + s, e - s, NCCL_FLOAT32, NCCL_SUM, d->comm, d->comm_stream), "ncclAllReduce")) { d->status = NC_ERR_DEVICE; return; }
    if (nc_cuda_event_record(d->done_ev[b], d->comm_stream)) d->status = NC_ERR_DEVICE;
}
static void dist_on_ready(nc_tensor* leaf, void* ctx) {
    nc_dist* d = ctx;
    for (size_t i = 0; i < d->opt->n_params; i++)
        if (d->opt->params[i] == leaf) {
            const int b = nc_bucket_plan_on_ready(d->plan, i);
            if (b >= 0) dist_fire(d, b);
            return;
        }
}

nc_dist* nc_dist_init(int rank, int world, const void* id128, nc_optimizer* opt, size_t bucket_floats) {
    if (!id128 || !opt || world < 1 || rank < 0 || rank >= world) { NC_SET_ERROR(NC_ERR_INVALID_SHAPE, "nc_dist_init: bad argument"); return NULL; }
    if (!nccl_bind()) return NULL;
    nc_dist* d = nc_calloc(1, sizeof(*d));
    if (!d) return NULL;
    d->rank = rank; d->world = world; d->opt = opt;
    size_t n = 0;
    d->arena = nc_optimizer_flatten_grads(opt, &n);
    d->arena_floats = n;
    if (!d->arena) { nc_free(d); return NULL; }
    size_t offs[NC_MAX_OPTIM_PARAMS], nums[NC_MAX_OPTIM_PARAMS], off = 0;
    for (size_t i = 0; i < opt->n_params; i++) {   /* the layout nc_optimizer_flatten_grads produced */
        offs[i] = off; nums[i] = opt->params[i]->numel;
        off += (opt->params[i]->numel + 63) & ~(size_t)63;
    }
    d->plan = nc_bucket_plan_create(opt->n_params, offs, nums, n, bucket_floats ? bucket_floats : ((size_t)1 << 21));
    if (!d->plan) { nc_free(d); return NULL; }
    nccl_unique_id id;
    memcpy(&id, id128, sizeof(id));
    if (!nccl_ok(g_nccl.comm_init_rank(&d->comm, world, id, rank), "ncclCommInitRank")) { nc_bucket_plan_free(d->plan); nc_free(d); return NULL; }
    const size_t nb = nc_bucket_plan_count(d->plan);
    d->comm_stream = nc_cuda_stream_create();
    d->ready_ev = nc_calloc(nb, sizeof(void*));
    d->done_ev = nc_calloc(nb, sizeof(void*));
    d->bwd_end_ev = nc_cuda_event_create_timed();
    bool ok = d->comm_stream && d->ready_ev && d->done_ev && d->bwd_end_ev;
    for (size_t b = 0; ok && b < nb; b++) {
        d->ready_ev[b] = nc_cuda_event_create();
        d->done_ev[b] = nc_cuda_event_create_timed();
        ok = d->ready_ev[b] && d->done_ev[b];
    }
    if (!ok) { NC_SET_ERROR(NC_ERR_DEVICE, "nc_dist_init: stream / event creation failed"); nc_dist_free(d); return NULL; }
    nc_set_grad_ready_hook(dist_on_ready, d);
    nc_optimizer_set_grad_scale(opt, 1.0 / (double)world);
    return d;
}

int nc_dist_allreduce_grads(nc_dist* d) {
    if (!d) return NC_ERR_NULL_PTR;
    nc_cuda_event_record(d->bwd_end_ev, nci_stream());
    int b;
    while ((b = nc_bucket_plan_next_unfired(d->plan)) >= 0) dist_fire(d, b);
    const size_t nb = nc_bucket_plan_count(d->plan);
    for (size_t k = 0; k < nb; k++)   /* the optimizer kernel, queued next on the compute stream, waits for every bucket */
        if (nc_cuda_stream_wait_event(nci_stream(), d->done_ev[k])) d->status = NC_ERR_DEVICE;
    const int late = nc_bucket_plan_end_step(d->plan);
    d->late_total += late;
    int rc = d->status;
    d->status = NC_OK;
    if (late > 0 && rc == NC_OK) {
        /* a gradient was still being accumulated after its bucket had been sent: this step's sum is incomplete */
        NC_SET_ERROR(NC_ERR_INVALID_SHAPE, "nc_dist: %d gradient(s) became final after their bucket was sent (the graph changed); "
                     "the plan has been relearned, repeat the step", late);
        rc = NC_ERR_INVALID_SHAPE;
    }
    return rc;
}

size_t nc_dist_num_buckets(const nc_dist* d) { return d ? nc_bucket_plan_count(d->plan) : 0; }
float* nc_dist_arena(const nc_dist* d, size_t* n_floats) {
    if (!d) return NULL;
    if (n_floats) *n_floats = d->arena_floats;
    return d->arena;
}
/* Device time from the end of the backward sweep to the end of the last bucket's all-reduce in the step just queued
 * (the communication the backward did not hide).  Blocks the host until that step's exchange has finished. */
double nc_dist_exposed_ms(nc_dist* d) {
    if (!d) return -1.0;
    double worst = 0.0;
    const size_t nb = nc_bucket_plan_count(d->plan);
    if (nc_cuda_event_synchronize(d->bwd_end_ev)) return -1.0;
    for (size_t b = 0; b < nb; b++) {
        float ms = 0.f;
        if (nc_cuda_event_synchronize(d->done_ev[b])) return -1.0;
        if (nc_cuda_event_elapsed_ms(d->bwd_end_ev, d->done_ev[b], &ms)) return -1.0;
        if ((double)ms > worst) worst = (double)ms;
    }
    return worst;
}
void nc_dist_free(nc_dist* d) {
    if (!d) return;
    nc_set_grad_ready_hook(NULL, NULL);
    nc_cuda_synchronize();
    const size_t nb = d->plan ? nc_bucket_plan_count(d->plan) : 0;
    for (size_t b = 0; b < nb; b++) {
        if (d->ready_ev && d->ready_ev[b]) nc_cuda_event_destroy(d->ready_ev[b]);
        if (d->done_ev && d->done_ev[b]) nc_cuda_event_destroy(d->done_ev[b]);
    }
    if (d->bwd_end_ev) nc_cuda_event_destroy(d->bwd_end_ev);
    if (d->comm_stream) nc_cuda_stream_destroy(d->comm_stream);
    if (d->comm) g_nccl.comm_destroy(d->comm);
    nc_free(d->ready_ev);
    nc_free(d->done_ev);
    nc_bucket_plan_free(d->plan);
    nc_free(d);
}
