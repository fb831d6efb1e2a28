/*
 * .ncta files: tensors, state dicts, module parameters and training checkpoints, for tensors that live
 * on the CUDA device as well as on the host.  The byte layout is the reference's
 * (include/nocta/core/serialize.h:9-37, src/core/serialize.c:32-101, 223-306, 431-546):
 *
 *   file header    u32 magic "NCTA" | u32 version 1 | u32 n_tensors | u32 flags | char description[64]
 *   checkpoint     (flags == 1) u64 epoch | f64 loss | u32 n_model | u32 n_optimizer, then the tensors
 *   tensor record  char name[64] | u32 dtype | u32 ndim | u64 shape[8] | u64 data_size | data bytes
 *
 * all little-endian, data in logical (row-major) order whatever the tensor's strides are.  A file written
 * here from device tensors is byte-identical to the one the reference writes from the same values on
 * the host.  Differences: the reference reads the CPU pointer only (serialize.c:52-56) and does not
 * validate record headers; here device data is staged through the host, loaded tensors are placed on the
 * default device, and malformed records are rejected (NC_ERR_IO) instead of being trusted.
 */
#include "internal.h"

#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    uint32_t magic, version, n_tensors, flags;
    char description[64];
} file_header;

typedef struct {
    char name[NC_MAX_NAME_LEN];
    uint32_t dtype, ndim;
    uint64_t shape[NC_MAX_DIMS];
    uint64_t data_size;
} tensor_header;

_Static_assert(sizeof(file_header) == 80, "file header is 80 bytes on disk");
_Static_assert(sizeof(tensor_header) == 144, "tensor record header is 144 bytes on disk");

static void header_init(file_header* h, uint32_t n, uint32_t flags, const char* description) {
    memset(h, 0, sizeof(*h));
    h->magic = NC_FILE_MAGIC;
    h->version = NC_FILE_VERSION;
    h->n_tensors = n;
    h->flags = flags;
    if (description) strncpy(h->description, description, sizeof(h->description) - 1);
}
static bool header_read(FILE* fp, file_header* h) {
    return fread(h, sizeof(*h), 1, fp) == 1 && h->magic == NC_FILE_MAGIC;
}

/* dense row-major bytes of t in a malloc'ed host buffer */
static void* host_bytes(const nc_tensor* t, size_t bytes) {
    void* buf = malloc(bytes ? bytes : 1);
    if (!buf) return NULL;
    const nc_tensor* src = t;
    nc_tensor* tmp = NULL;
    if (!t->is_contiguous) {
        tmp = nc_tensor_contiguous((nc_tensor*)t);
        if (!tmp) { free(buf); return NULL; }
        src = tmp;
    }
    if (bytes) {
        if (nci_on_cuda(src)) nc_cuda_memcpy_d2h(buf, nci_dptr(src), bytes);
        else memcpy(buf, (const char*)src->storage->data + src->offset * nc_dtype_sizeof(src->dtype), bytes);
    }
    if (tmp) nc_tensor_free(tmp);
    return buf;
}

nc_error nc_tensor_save_fp(const nc_tensor* t, FILE* fp, const char* name) {
    if (!t || !fp) return NC_ERR_NULL_PTR;
    tensor_header th;
    memset(&th, 0, sizeof(th));
    if (name) strncpy(th.name, name, NC_MAX_NAME_LEN - 1);
    th.dtype = (uint32_t)t->dtype;
    th.ndim = (uint32_t)t->ndim;
    for (size_t i = 0; i < t->ndim; i++) th.shape[i] = t->shape[i];
    th.data_size = (uint64_t)t->numel * nc_dtype_sizeof(t->dtype);
    if (fwrite(&th, sizeof(th), 1, fp) != 1) return NC_ERR_IO;
    void* buf = host_bytes(t, (size_t)th.data_size);
    if (!buf) return NC_ERR_ALLOC;
    const bool ok = fwrite(buf, 1, (size_t)th.data_size, fp) == (size_t)th.data_size;
    free(buf);
    return ok ? NC_OK : NC_ERR_IO;
}

nc_tensor* nc_tensor_load_fp(FILE* fp, char* name_out) {
    if (!fp) return NULL;
    tensor_header th;
    if (fread(&th, sizeof(th), 1, fp) != 1) { NC_SET_ERROR(NC_ERR_IO, "tensor record: header is truncated"); return NULL; }
    if (th.ndim > NC_MAX_DIMS || th.dtype >= (uint32_t)NC_DTYPE_COUNT) {
        NC_SET_ERROR(NC_ERR_IO, "tensor record: ndim %u / dtype %u out of range", th.ndim, th.dtype);
        return NULL;
    }
    size_t shape[NC_MAX_DIMS], numel = 1;
    for (uint32_t i = 0; i < th.ndim; i++) {
        shape[i] = (size_t)th.shape[i];
        if (th.shape[i] && numel > SIZE_MAX / 16 / th.shape[i]) { NC_SET_ERROR(NC_ERR_IO, "tensor record: shape overflows"); return NULL; }
        numel *= shape[i];
    }
    const size_t bytes = numel * nc_dtype_sizeof((nc_dtype)th.dtype);
    if (th.data_size != (uint64_t)bytes) {
        NC_SET_ERROR(NC_ERR_IO, "tensor record: data_size %llu does not match the shape (%zu bytes)", (unsigned long long)th.data_size, bytes);
        return NULL;
    }
    void* buf = malloc(bytes ? bytes : 1);
    if (!buf) { NC_SET_ERROR(NC_ERR_ALLOC, "tensor record: %zu bytes", bytes); return NULL; }
    if (fread(buf, 1, bytes, fp) != bytes) {
        free(buf);
        NC_SET_ERROR(NC_ERR_IO, "tensor record: data is truncated");
        return NULL;
    }
    nc_tensor* t = bytes ? nc_tensor_from_data(buf, shape, th.ndim, (nc_dtype)th.dtype) : nc_tensor_empty(shape, th.ndim, (nc_dtype)th.dtype);
    free(buf);
    if (t && name_out) {
        memcpy(name_out, th.name, NC_MAX_NAME_LEN - 1);
        name_out[NC_MAX_NAME_LEN - 1] = 0;
    }
    return t;
}

nc_error nc_tensor_save(const nc_tensor* t, const char* path) {
    if (!t || !path) return NC_ERR_NULL_PTR;
    FILE* fp = fopen(path, "wb");
    if (!fp) { NC_SET_ERROR(NC_ERR_IO, "cannot open %s", path); return NC_ERR_IO; }
    file_header h;
    header_init(&h, 1, 0, "Single tensor");
    nc_error err = fwrite(&h, sizeof(h), 1, fp) == 1 ? nc_tensor_save_fp(t, fp, "tensor") : NC_ERR_IO;
    if (fclose(fp) != 0 && err == NC_OK) err = NC_ERR_IO;
    return err;
}

nc_tensor* nc_tensor_load(const char* path) {
    if (!path) return NULL;
    FILE* fp = fopen(path, "rb");
    if (!fp) { NC_SET_ERROR(NC_ERR_IO, "cannot open %s", path); return NULL; }
    file_header h;
    nc_tensor* t = NULL;
    if (header_read(fp, &h)) t = nc_tensor_load_fp(fp, NULL);
    else NC_SET_ERROR(NC_ERR_IO, "%s is not an .ncta file", path);
    fclose(fp);
    return t;
}

/* ------------------------------------------------------------------ state dict */
nc_state_dict* nc_state_dict_create(void) {
    nc_state_dict* sd = nc_calloc(1, sizeof(nc_state_dict));
    if (!sd) return NULL;
    sd->capacity = 16;
    sd->names = nc_calloc(sd->capacity, sizeof(char*));
    sd->tensors = nc_calloc(sd->capacity, sizeof(nc_tensor*));
    if (!sd->names || !sd->tensors) { nc_state_dict_free(sd); return NULL; }
    return sd;
}
void nc_state_dict_free(nc_state_dict* sd) {
    if (!sd) return;
    for (size_t i = 0; i < sd->n_tensors; i++) {
        nc_free(sd->names[i]);
        nc_tensor_free(sd->tensors[i]);
    }
    nc_free(sd->names);
    nc_free(sd->tensors);
    nc_free(sd);
}
void nc_state_dict_add(nc_state_dict* sd, const char* name, nc_tensor* t) {
    if (!sd || !name || !t) return;
    if (sd->n_tensors == sd->capacity) {
        const size_t cap = sd->capacity * 2;
        char** names = nc_realloc(sd->names, sd->capacity * sizeof(char*), cap * sizeof(char*));
        if (!names) return;
        sd->names = names;
        nc_tensor** tensors = nc_realloc(sd->tensors, sd->capacity * sizeof(nc_tensor*), cap * sizeof(nc_tensor*));
        if (!tensors) return;
        sd->tensors = tensors;
        sd->capacity = cap;
    }
    const size_t len = strlen(name);
    char* copy = nc_alloc(len + 1);
    if (!copy) return;
    memcpy(copy, name, len + 1);
    sd->names[sd->n_tensors] = copy;
    sd->tensors[sd->n_tensors] = t;
    sd->n_tensors++;
}
nc_tensor* nc_state_dict_get(nc_state_dict* sd, const char* name) {
    if (!sd || !name) return NULL;
    for (size_t i = 0; i < sd->n_tensors; i++)
        if (!strcmp(sd->names[i], name)) return sd->tensors[i];
    return NULL;
}

static nc_error write_tensors(FILE* fp, nc_state_dict* sd) {
    for (size_t i = 0; sd && i < sd->n_tensors; i++) {
        nc_error err = nc_tensor_save_fp(sd->tensors[i], fp, sd->names[i]);
        if (err != NC_OK) return err;
    }
    return NC_OK;
}
static nc_error save_dict(nc_state_dict* sd, const char* path, const char* description) {
    if (!sd || !path) return NC_ERR_NULL_PTR;
    FILE* fp = fopen(path, "wb");
    if (!fp) { NC_SET_ERROR(NC_ERR_IO, "cannot open %s", path); return NC_ERR_IO; }
    file_header h;
    header_init(&h, (uint32_t)sd->n_tensors, 0, description);
    nc_error err = fwrite(&h, sizeof(h), 1, fp) == 1 ? write_tensors(fp, sd) : NC_ERR_IO;
    if (fclose(fp) != 0 && err == NC_OK) err = NC_ERR_IO;
    return err;
}
nc_error nc_state_dict_save(nc_state_dict* sd, const char* path) { return save_dict(sd, path, "State dict"); }

static nc_state_dict* read_tensors(FILE* fp, uint32_t n) {
    nc_state_dict* sd = nc_state_dict_create();
    for (uint32_t i = 0; sd && i < n; i++) {
        char name[NC_MAX_NAME_LEN] = {0};
        nc_tensor* t = nc_tensor_load_fp(fp, name);
        if (!t) { nc_state_dict_free(sd); return NULL; }
        nc_state_dict_add(sd, name, t);
    }
    return sd;
}
nc_state_dict* nc_state_dict_load(const char* path) {
    if (!path) return NULL;
    FILE* fp = fopen(path, "rb");
    if (!fp) { NC_SET_ERROR(NC_ERR_IO, "cannot open %s", path); return NULL; }
    file_header h;
    nc_state_dict* sd = NULL;
    if (header_read(fp, &h)) sd = read_tensors(fp, h.n_tensors);
    else NC_SET_ERROR(NC_ERR_IO, "%s is not an .ncta file", path);
    fclose(fp);
    return sd;
}

/* ------------------------------------------------------------------ modules */
static void cb_collect(const char* name, nc_tensor* p, void* ctx) {
    nc_tensor* c = nc_tensor_clone(p);
    if (c) nc_state_dict_add(ctx, name, c);
}
nc_state_dict* nc_module_state_dict(nc_module* m) {
    if (!m) return NULL;
    nc_state_dict* sd = nc_state_dict_create();
    if (sd) nc_module_parameters(m, cb_collect, sd);
    return sd;
}
typedef struct { nc_state_dict* sd; nc_error err; size_t matched; } load_ctx;
static void cb_assign(const char* name, nc_tensor* p, void* ctx) {
    load_ctx* lc = ctx;
    nc_tensor* src = nc_state_dict_get(lc->sd, name);
    if (!src || lc->err != NC_OK) return;
    if (!nc_tensor_shape_eq(p, src)) {
        NC_SET_ERROR(NC_ERR_SHAPE_MISMATCH, "shape mismatch for %s", name);
        lc->err = NC_ERR_SHAPE_MISMATCH;
        return;
    }
    nc_error e = nc_tensor_copy_(p, src);
    if (e != NC_OK) lc->err = e;
    else lc->matched++;
}
/* Every parameter of the module tree whose dotted name is in the dict is overwritten (the reference
 * matches top-level names only and skips nested ones, src/core/serialize.c:333-341). */
nc_error nc_module_load_state_dict(nc_module* m, nc_state_dict* sd) {
    if (!m || !sd) return NC_ERR_NULL_PTR;
    load_ctx lc = {sd, NC_OK, 0};
    nc_module_parameters(m, cb_assign, &lc);
    return lc.err;
}
nc_error nc_module_save_desc(nc_module* m, const char* path, const char* description) {
    if (!m || !path) return NC_ERR_NULL_PTR;
    nc_state_dict* sd = nc_module_state_dict(m);
    if (!sd) return NC_ERR_ALLOC;
    nc_error err = save_dict(sd, path, description);
    nc_state_dict_free(sd);
    return err;
}
nc_error nc_module_save(nc_module* m, const char* path) { return nc_module_save_desc(m, path, "State dict"); }
nc_error nc_module_load(nc_module* m, const char* path) {
    if (!m || !path) return NC_ERR_NULL_PTR;
    nc_state_dict* sd = nc_state_dict_load(path);
    if (!sd) return NC_ERR_IO;
    nc_error err = nc_module_load_state_dict(m, sd);
    nc_state_dict_free(sd);
    return err;
}

/* ------------------------------------------------------------------ checkpoints */
nc_error nc_checkpoint_save(nc_checkpoint* ckpt, const char* path) {
    if (!ckpt || !path) return NC_ERR_NULL_PTR;
    FILE* fp = fopen(path, "wb");
    if (!fp) { NC_SET_ERROR(NC_ERR_IO, "cannot open %s", path); return NC_ERR_IO; }
    const uint32_t n_model = ckpt->model_state ? (uint32_t)ckpt->model_state->n_tensors : 0;
    const uint32_t n_optim = ckpt->optimizer_state ? (uint32_t)ckpt->optimizer_state->n_tensors : 0;
    char desc[64];
    snprintf(desc, sizeof(desc), "Checkpoint epoch=%zu loss=%.6f", ckpt->epoch, ckpt->loss);
    file_header h;
    header_init(&h, n_model + n_optim, 1, desc);
    const uint64_t epoch = (uint64_t)ckpt->epoch;
    nc_error err = NC_OK;
    if (fwrite(&h, sizeof(h), 1, fp) != 1 || fwrite(&epoch, sizeof(epoch), 1, fp) != 1 || fwrite(&ckpt->loss, sizeof(double), 1, fp) != 1 ||
        fwrite(&n_model, sizeof(n_model), 1, fp) != 1 || fwrite(&n_optim, sizeof(n_optim), 1, fp) != 1)
        err = NC_ERR_IO;
    if (err == NC_OK) err = write_tensors(fp, ckpt->model_state);
    if (err == NC_OK) err = write_tensors(fp, ckpt->optimizer_state);
    if (fclose(fp) != 0 && err == NC_OK) err = NC_ERR_IO;
    return err;
}
nc_checkpoint* nc_checkpoint_load(const char* path) {
    if (!path) return NULL;
    FILE* fp = fopen(path, "rb");
    if (!fp) { NC_SET_ERROR(NC_ERR_IO, "cannot open %s", path); return NULL; }
    file_header h;
    uint64_t epoch = 0;
    double loss = 0.0;
    uint32_t n_model = 0, n_optim = 0;
    nc_checkpoint* ck = NULL;
    if (header_read(fp, &h) && h.flags == 1 && fread(&epoch, sizeof(epoch), 1, fp) == 1 && fread(&loss, sizeof(loss), 1, fp) == 1 &&
        fread(&n_model, sizeof(n_model), 1, fp) == 1 && fread(&n_optim, sizeof(n_optim), 1, fp) == 1 &&
        (uint64_t)n_model + n_optim == h.n_tensors)
        ck = nc_calloc(1, sizeof(nc_checkpoint));
    else
        NC_SET_ERROR(NC_ERR_IO, "%s is not a checkpoint file", path);
    if (ck) {
        ck->epoch = (size_t)epoch;
        ck->loss = loss;
        if (n_model) ck->model_state = read_tensors(fp, n_model);
        if (n_optim && (!n_model || ck->model_state)) ck->optimizer_state = read_tensors(fp, n_optim);
        if ((n_model && !ck->model_state) || (n_optim && !ck->optimizer_state)) {
            nc_checkpoint_free(ck);
            ck = NULL;
        }
    }
    fclose(fp);
    return ck;
}
void nc_checkpoint_free(nc_checkpoint* ckpt) {
    if (!ckpt) return;
    nc_state_dict_free(ckpt->model_state);
    nc_state_dict_free(ckpt->optimizer_state);
    nc_free(ckpt);
}

/* ------------------------------------------------------------------ inspection */
/* Walks the records without loading the data; returns false on any inconsistency. */
static bool walk_file(const char* path, bool print) {
    FILE* fp = path ? fopen(path, "rb") : NULL;
    if (!fp) return false;
    file_header h;
    bool ok = header_read(fp, &h) && h.version == NC_FILE_VERSION;
    if (ok && print) printf("%s: version %u, %u tensors, flags %u, \"%.63s\"\n", path, h.version, h.n_tensors, h.flags, h.description);
    if (ok && h.flags == 1) ok = fseek(fp, 8 + 8 + 4 + 4, SEEK_CUR) == 0;
    for (uint32_t i = 0; ok && i < h.n_tensors; i++) {
        tensor_header th;
        ok = fread(&th, sizeof(th), 1, fp) == 1 && th.ndim <= NC_MAX_DIMS && th.dtype < (uint32_t)NC_DTYPE_COUNT;
        if (!ok) break;
        uint64_t numel = 1;
        for (uint32_t d = 0; d < th.ndim; d++) numel *= th.shape[d];
        ok = th.data_size == numel * nc_dtype_sizeof((nc_dtype)th.dtype);
        if (ok && print) {
            printf("  %-40.63s %s (", th.name, nc_dtype_to_string((nc_dtype)th.dtype));
            for (uint32_t d = 0; d < th.ndim; d++) printf(d ? ", %llu" : "%llu", (unsigned long long)th.shape[d]);
            printf(") %llu bytes\n", (unsigned long long)th.data_size);
        }
        if (ok) {
            /* the data must really be there */
            const long here = ftell(fp);
            ok = here >= 0 && fseek(fp, 0, SEEK_END) == 0 && (uint64_t)(ftell(fp) - here) >= th.data_size &&
                 fseek(fp, here + (long)th.data_size, SEEK_SET) == 0;
        }
    }
    fclose(fp);
    return ok;
}
void nc_file_info(const char* path) {
    if (!walk_file(path, true)) printf("%s: not a readable .ncta file\n", path ? path : "(null)");
}
bool nc_file_verify(const char* path) { return walk_file(path, false); }
