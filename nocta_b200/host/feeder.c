/* Double-buffered input upload: pinned host batches -> device tensors on a copy stream that overlaps
 * the compute stream.  No counterpart in the reference, whose example copies each batch synchronously
 * (examples/mnist.c:93-111); the tensors it hands out are ordinary nc_tensor inputs of the path. */
#include "internal.h"

#include <stdlib.h>
#include <string.h>

#define NC_FEEDER_MAX_SLOTS 8

struct nc_feeder {
    int slots;
    void* copy_stream;
    nc_tensor* x[NC_FEEDER_MAX_SLOTS];
    nc_tensor* y[NC_FEEDER_MAX_SLOTS];
    void* copied[NC_FEEDER_MAX_SLOTS];    /* recorded on the copy stream after a slot's upload */
    void* released[NC_FEEDER_MAX_SLOTS];  /* recorded on the compute stream when the user is done with a slot */
    bool in_flight[NC_FEEDER_MAX_SLOTS];
    bool ever_released[NC_FEEDER_MAX_SLOTS];
    size_t x_bytes, y_bytes;
};

void nc_feeder_free(nc_feeder* f) {
    if (!f) return;
    if (f->copy_stream) nc_cuda_stream_synchronize(f->copy_stream);
    nc_cuda_stream_synchronize(nci_stream());
    for (int i = 0; i < f->slots; i++) {
        if (f->x[i]) nc_tensor_free(f->x[i]);
        if (f->y[i]) nc_tensor_free(f->y[i]);
        nc_cuda_event_destroy(f->copied[i]);
        nc_cuda_event_destroy(f->released[i]);
    }
    nc_cuda_stream_destroy(f->copy_stream);
    free(f);
}

nc_feeder* nc_feeder_create(int slots, const size_t* x_shape, size_t x_ndim, nc_dtype x_dtype,
                            const size_t* y_shape, size_t y_ndim, nc_dtype y_dtype) {
    if (slots < 1 || slots > NC_FEEDER_MAX_SLOTS || !x_shape) {
        NC_SET_ERROR(NC_ERR_INVALID_SHAPE, "nc_feeder_create: 1..%d slots and an input shape are required", NC_FEEDER_MAX_SLOTS);
        return NULL;
    }
    nc_feeder* f = (nc_feeder*)calloc(1, sizeof(nc_feeder));
    if (!f) { NC_SET_ERROR(NC_ERR_ALLOC, "nc_feeder_create: out of memory"); return NULL; }
    f->slots = slots;
    f->copy_stream = nc_cuda_stream_create();
    if (!f->copy_stream) { NC_SET_ERROR(NC_ERR_DEVICE, "nc_feeder_create: no copy stream"); nc_feeder_free(f); return NULL; }
    for (int i = 0; i < slots; i++) {
        f->x[i] = nci_empty_on(x_shape, x_ndim, x_dtype, NC_DEVICE_CUDA);
        f->y[i] = y_shape ? nci_empty_on(y_shape, y_ndim, y_dtype, NC_DEVICE_CUDA) : NULL;
        f->copied[i] = nc_cuda_event_create();
        f->released[i] = nc_cuda_event_create();
        if (!f->x[i] || (y_shape && !f->y[i]) || !f->copied[i] || !f->released[i]) {
            NC_SET_ERROR(NC_ERR_ALLOC, "nc_feeder_create: slot %d could not be set up", i);
            nc_feeder_free(f);
            return NULL;
        }
    }
    f->x_bytes = f->x[0]->numel * nc_dtype_sizeof(x_dtype);
    f->y_bytes = f->y[0] ? f->y[0]->numel * nc_dtype_sizeof(y_dtype) : 0;
    return f;
}

static bool slot_ok(nc_feeder* f, int slot, const char* what) {
    if (!f || slot < 0 || slot >= f->slots) {
        NC_SET_ERROR(NC_ERR_INDEX_OUT_OF_BOUNDS, "%s: bad feeder or slot %d", what, slot);
        return false;
    }
    return true;
}

int nc_feeder_submit(nc_feeder* f, int slot, const void* x_host, const void* y_host) {
    if (!slot_ok(f, slot, "nc_feeder_submit")) return -1;
    if (!x_host || (f->y[slot] && !y_host)) { NC_SET_ERROR(NC_ERR_NULL_PTR, "nc_feeder_submit: null host buffer"); return -1; }
    if (f->in_flight[slot]) { NC_SET_ERROR(NC_ERR_INVALID_SHAPE, "nc_feeder_submit: slot %d was submitted and not yet acquired", slot); return -1; }
    /* the previous user of this slot's device buffers must have finished before they are overwritten */
    if (f->ever_released[slot] && nc_cuda_stream_wait_event(f->copy_stream, f->released[slot]) != 0) return -1;
    if (nc_cuda_memcpy_h2d_async(nci_dptr(f->x[slot]), x_host, f->x_bytes, f->copy_stream) != 0) return -1;
    if (f->y[slot] && nc_cuda_memcpy_h2d_async(nci_dptr(f->y[slot]), y_host, f->y_bytes, f->copy_stream) != 0) return -1;
    if (nc_cuda_event_record(f->copied[slot], f->copy_stream) != 0) return -1;
    f->in_flight[slot] = true;
    return 0;
}

int nc_feeder_acquire(nc_feeder* f, int slot, nc_tensor** x, nc_tensor** y) {
    if (!slot_ok(f, slot, "nc_feeder_acquire")) return -1;
    if (!f->in_flight[slot]) { NC_SET_ERROR(NC_ERR_INVALID_SHAPE, "nc_feeder_acquire: slot %d has no submitted batch", slot); return -1; }
    if (nc_cuda_stream_wait_event(nci_stream(), f->copied[slot]) != 0) return -1;
    f->in_flight[slot] = false;
    if (x) *x = f->x[slot];
    if (y) *y = f->y[slot];
    return 0;
}

int nc_feeder_release(nc_feeder* f, int slot) {
    if (!slot_ok(f, slot, "nc_feeder_release")) return -1;
    if (nc_cuda_event_record(f->released[slot], nci_stream()) != 0) return -1;
    f->ever_released[slot] = true;
    return 0;
}

int nc_feeder_wait(nc_feeder* f, int slot) {
    if (!slot_ok(f, slot, "nc_feeder_wait")) return -1;
    return nc_cuda_event_synchronize(f->copied[slot]) == 0 ? 0 : -1;
}
