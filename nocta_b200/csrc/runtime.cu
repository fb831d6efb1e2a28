// Device/runtime part of the nc_cuda_* ABI: memory, streams, status, library scratch.
// Replaces the reference's src/cuda/cuda_device.cu:22-136 (which prints and drops CUDA errors).
#include "nc_common.cuh"
#include "../../include/nocta_cuda.h"
#include <stdarg.h>
#include <string.h>
#include <stdlib.h>

namespace ncc {

static int g_status = NC_CUDA_OK;
static char g_message[512] = {0};
static cudaStream_t g_stream = nullptr;
static int g_sm_count = 0;
// Default TF32; a program that cannot call nc_cuda_set_math_mode (one built against the reference's API only) can
// choose through the environment: NOCTA_CUDA_MATH_MODE = 0 (TF32), 1 (TF32 rounded in the kernel), 2 (3xTF32), 3 (FP32).
static int initial_math_mode() {
    const char* e = getenv("NOCTA_CUDA_MATH_MODE");
    if (e && e[0] >= '0' && e[0] <= '3' && e[1] == 0) return e[0] - '0';
    return NC_CUDA_MATH_TF32;
}
static int g_math_mode = initial_math_mode();
unsigned long long g_launches = 0;
unsigned long long g_epoch = 0;

static const int kScratchSlots = 10;
static void* g_scratch[kScratchSlots] = {nullptr};
static size_t g_scratch_bytes[kScratchSlots] = {0};
static unsigned int* g_err_word = nullptr;

int set_status(int code, const char* fmt, ...) {
    g_status = code;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_message, sizeof(g_message), fmt, ap);
    va_end(ap);
    if (code != NC_CUDA_OK) fprintf(stderr, "[nocta-cuda] error %d: %s\n", code, g_message);
    return code;
}
int last_status() { return g_status; }
const char* last_message() { return g_message; }
cudaStream_t current_stream() { return g_stream; }
int math_mode() { return g_math_mode; }
static int g_round_outputs = 0;
bool round_outputs() { return g_round_outputs != 0; }
int set_round_outputs(int on) { int p = g_round_outputs; g_round_outputs = on ? 1 : 0; return p; }

int sm_count() {
    if (g_sm_count == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            g_sm_count <= 0)
            g_sm_count = 148;
    }
    return g_sm_count;
}

void* scratch(int slot, size_t bytes, cudaStream_t st) {
    if (slot < 0 || slot >= kScratchSlots) return nullptr;
    if (bytes <= g_scratch_bytes[slot] && g_scratch[slot]) return g_scratch[slot];
    // Growing: earlier work on any stream may still read the old block, so drain first.
    (void)st;
    cudaDeviceSynchronize();
    if (g_scratch[slot]) cudaFree(g_scratch[slot]);
    size_t want = bytes + (bytes >> 2) + 4096;
    void* p = nullptr;
    if (cudaMalloc(&p, want) != cudaSuccess) {
        g_scratch[slot] = nullptr;
        g_scratch_bytes[slot] = 0;
        set_status(NC_CUDA_ERR_RUNTIME, "scratch slot %d: cudaMalloc(%zu) failed", slot, want);
        return nullptr;
    }
    g_scratch[slot] = p;
    g_scratch_bytes[slot] = want;
    return p;
}

// ---- per-channel statistics captured by a forward convolution for the BatchNorm that follows ----
// A convolution kernel whose epilogue threads own whole output channels can sum its output (and its
// square) per channel on the way out.  While the switch is on, the forward convolution entry point
// publishes such partial sums together with the output pointer; a training-mode BatchNorm forward that
// is the very next kernel-launching call of the library, on exactly that tensor, takes them instead of
// reading the tensor again.  Any other library launch in between (which could have changed the tensor)
// invalidates the offer.
static int g_conv_stats_on = 0;
static struct { const float* y; int C; long long rows; int slabs; double* partial; unsigned long long stamp; bool valid; } g_offer = {};
int set_conv_stats(int on) { int p = g_conv_stats_on; g_conv_stats_on = on ? 1 : 0; return p; }  // an offer already made stays
bool conv_stats_wanted() { return g_conv_stats_on != 0; }
double* conv_stats_buffer(size_t slabs, int C, cudaStream_t st) { return (double*)scratch(8, sizeof(double) * 2 * slabs * (size_t)C, st); }
void conv_stats_publish(const float* y, int C, long long rows, int slabs, double* partial) {
    g_offer.y = y; g_offer.C = C; g_offer.rows = rows; g_offer.slabs = slabs; g_offer.partial = partial;
    g_offer.stamp = g_epoch;
    g_offer.valid = true;
}
bool conv_stats_take(const float* x, int C, long long rows, double** partial, int* slabs) {
    const bool hit = g_offer.valid && g_offer.y == x && g_offer.C == C && g_offer.rows == rows && g_offer.stamp == g_epoch;
    g_offer.valid = false;
    if (hit) { *partial = g_offer.partial; *slabs = g_offer.slabs; }
    return hit;
}

// BatchNorm-backward sums folded into the input-gradient convolution that produces the upstream gradient.
static BnFold g_fold_pending = {}, g_fold_now = {};
static bool g_fold_pending_valid = false, g_fold_now_valid = false;
static struct { const float* dy; BnFold f; int slabs; double* partial; unsigned long long stamp; bool valid; } g_fold_offer = {};
unsigned long long g_bn_fold_hits = 0;
static int initial_bn_fold() { const char* e = getenv("NOCTA_BN_FOLD"); return (e && e[0] == '0') ? 0 : 1; }   // NOCTA_BN_FOLD=0: off at start
static int g_bn_fold_on = initial_bn_fold();
void bn_fold_announce(const BnFold& f) { g_fold_pending = f; g_fold_pending_valid = true; }
void bn_fold_enter() { g_fold_now = g_fold_pending; g_fold_now_valid = g_fold_pending_valid; g_fold_pending_valid = false; g_fold_offer.valid = false; }
void bn_fold_leave() { g_fold_now_valid = false; }
const BnFold* bn_fold_active() { return g_fold_now_valid ? &g_fold_now : nullptr; }
double* bn_fold_buffer(size_t slabs, int C, cudaStream_t st) { return (double*)scratch(9, sizeof(double) * 2 * slabs * (size_t)C, st); }
void bn_fold_publish(const float* dy, int slabs, double* partial) {
    g_fold_offer.dy = dy; g_fold_offer.f = g_fold_now; g_fold_offer.slabs = slabs;
    g_fold_offer.partial = partial; g_fold_offer.stamp = g_epoch; g_fold_offer.valid = true;
}
bool bn_fold_take(const float* dy, const BnFold& want, double** partial, int* slabs) {
    const BnFold& f = g_fold_offer.f;
    const bool hit = g_fold_offer.valid && g_fold_offer.dy == dy && g_fold_offer.stamp == g_epoch && f.x == want.x && f.mean == want.mean &&
                     f.var == want.var && f.gamma == want.gamma && f.beta == want.beta && f.eps == want.eps && f.C == want.C &&
                     f.rows == want.rows;
    g_fold_offer.valid = false;
    if (hit) { *partial = g_fold_offer.partial; *slabs = g_fold_offer.slabs; ++g_bn_fold_hits; }
    return hit;
}

unsigned int* device_error_word() {
    if (!g_err_word) {
        if (cudaMalloc((void**)&g_err_word, 64) != cudaSuccess) return nullptr;
        cudaMemset(g_err_word, 0, 64);
    }
    return g_err_word;
}

// ---- per-category device timing ----
static const char* const kProfNames[PROF_CATEGORIES] = {
    "conv_fwd", "conv_dx", "conv_dw", "gemm_nt", "gemm_nn", "gemm_tn", "gemm_tt", "conv_first", "batchnorm", "layernorm",
    "activation", "elementwise", "maxpool", "loss", "sgd", "adam", "reduce", "relayout"};
static const int kProfCap = 32768;
static struct {
    bool on = false;
    int n = 0, depth = 0, role = PROF_GEMM_NT;
    cudaEvent_t* start = nullptr;
    cudaEvent_t* stop = nullptr;
    unsigned char* cat = nullptr;
    double* work = nullptr;
} g_prof;
bool prof_armed() { return g_prof.on; }
void prof_set_role(int cat) { g_prof.role = cat; }
int prof_role() { return g_prof.role; }
ProfScope::ProfScope(int cat, double work, cudaStream_t stream, bool kernel_level) : slot(-1), st(stream), outer(false) {
    if (!g_prof.on) return;
    if (!kernel_level) {
        outer = true;
        if (g_prof.depth++ > 0) return;
    }
    if (g_prof.n >= kProfCap || cat < 0 || cat >= PROF_CATEGORIES) return;
    slot = g_prof.n++;
    g_prof.cat[slot] = (unsigned char)cat;
    g_prof.work[slot] = work;
    cudaEventRecord(g_prof.start[slot], st);
}
void ProfScope::add_work(double more) { if (slot >= 0) g_prof.work[slot] += more; }
ProfScope::~ProfScope() {
    if (outer) g_prof.depth--;
    if (slot >= 0) cudaEventRecord(g_prof.stop[slot], st);
}

static void release_all() {
    for (int i = 0; i < kScratchSlots; i++) {
        if (g_scratch[i]) cudaFree(g_scratch[i]);
        g_scratch[i] = nullptr;
        g_scratch_bytes[i] = 0;
    }
    if (g_err_word) cudaFree(g_err_word);
    g_err_word = nullptr;
}

}  // namespace ncc

using namespace ncc;

extern "C" {

bool nc_cuda_available(void) {
    int n = 0;
    return cudaGetDeviceCount(&n) == cudaSuccess && n > 0;
}
int nc_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
    return n;
}
void nc_cuda_set_device(int index) {
    if (cudaSetDevice(index) != cudaSuccess) set_status(NC_CUDA_ERR_RUNTIME, "cudaSetDevice(%d) failed", index);
    g_sm_count = 0;
}
void nc_cuda_synchronize(void) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) set_status(NC_CUDA_ERR_RUNTIME, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
}
void nc_cuda_init(void) {
    if (!nc_cuda_available()) {
        set_status(NC_CUDA_ERR_RUNTIME, "no CUDA device");
        return;
    }
    cudaFree(0);
    (void)sm_count();
    (void)device_error_word();
}
void nc_cuda_cleanup(void) {
    cudaDeviceSynchronize();
    release_all();
}
void* nc_cuda_malloc(size_t size) {
    void* p = nullptr;
    if (size == 0) size = 16;
    cudaError_t e = cudaMalloc(&p, size);
    if (e != cudaSuccess) {
        set_status(NC_CUDA_ERR_RUNTIME, "cudaMalloc(%zu): %s", size, cudaGetErrorString(e));
        return nullptr;
    }
    return p;
}
void nc_cuda_free(void* ptr) {
    if (ptr) cudaFree(ptr);
}
void nc_cuda_memcpy_h2d(void* dst, const void* src, size_t size) {
    ++g_epoch;
    cudaError_t e = cudaMemcpyAsync(dst, src, size, cudaMemcpyHostToDevice, g_stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g_stream);
    if (e != cudaSuccess) set_status(NC_CUDA_ERR_RUNTIME, "memcpy_h2d: %s", cudaGetErrorString(e));
}
void nc_cuda_memcpy_d2h(void* dst, const void* src, size_t size) {
    cudaError_t e = cudaMemcpyAsync(dst, src, size, cudaMemcpyDeviceToHost, g_stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g_stream);
    if (e != cudaSuccess) set_status(NC_CUDA_ERR_RUNTIME, "memcpy_d2h: %s", cudaGetErrorString(e));
}
void nc_cuda_memcpy_d2d(void* dst, const void* src, size_t size) {
    ++g_epoch;
    cudaError_t e = cudaMemcpyAsync(dst, src, size, cudaMemcpyDeviceToDevice, g_stream);
    if (e != cudaSuccess) set_status(NC_CUDA_ERR_RUNTIME, "memcpy_d2d: %s", cudaGetErrorString(e));
}
void nc_cuda_memset(void* ptr, int value, size_t size) {
    ++g_epoch;
    cudaError_t e = cudaMemsetAsync(ptr, value, size, g_stream);
    if (e != cudaSuccess) set_status(NC_CUDA_ERR_RUNTIME, "memset: %s", cudaGetErrorString(e));
}
int nc_cuda_device_props(int index, char* name256, size_t* total_bytes, size_t* free_bytes, int* sms) {
    cudaDeviceProp p;
    NCC_TRY(cudaGetDeviceProperties(&p, index));
    if (name256) {
        strncpy(name256, p.name, 255);
        name256[255] = 0;
    }
    if (sms) *sms = p.multiProcessorCount;
    if (total_bytes) *total_bytes = p.totalGlobalMem;
    if (free_bytes) {
        size_t f = 0, t = 0;
        int cur = 0;
        cudaGetDevice(&cur);
        if (cur == index && cudaMemGetInfo(&f, &t) == cudaSuccess) *free_bytes = f;
        else *free_bytes = 0;
    }
    return NC_CUDA_OK;
}
void nc_cuda_set_stream(void* stream) { g_stream = (cudaStream_t)stream; }
void* nc_cuda_get_stream(void) { return (void*)g_stream; }
int nc_cuda_memcpy_h2d_async(void* dst, const void* src, size_t size, void* stream) {
    ++g_epoch;
    NCC_TRY(cudaMemcpyAsync(dst, src, size, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return NC_CUDA_OK;
}
int nc_cuda_memcpy_d2h_async(void* dst, const void* src, size_t size, void* stream) {
    NCC_TRY(cudaMemcpyAsync(dst, src, size, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return NC_CUDA_OK;
}
int nc_cuda_memset_async(void* ptr, int value, size_t size, void* stream) {
    ++g_epoch;
    NCC_TRY(cudaMemsetAsync(ptr, value, size, (cudaStream_t)stream));
    return NC_CUDA_OK;
}
void* nc_cuda_host_alloc(size_t size) {
    void* p = nullptr;
    if (cudaHostAlloc(&p, size ? size : 16, cudaHostAllocDefault) != cudaSuccess) {
        set_status(NC_CUDA_ERR_RUNTIME, "cudaHostAlloc(%zu) failed", size);
        return nullptr;
    }
    return p;
}
void nc_cuda_host_free(void* ptr) {
    if (ptr) cudaFreeHost(ptr);
}
int nc_cuda_stream_synchronize(void* stream) {
    NCC_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    return NC_CUDA_OK;
}
void* nc_cuda_stream_create(void) {
    cudaStream_t st = nullptr;
    if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) {
        set_status(NC_CUDA_ERR_RUNTIME, "cudaStreamCreate failed");
        return nullptr;
    }
    return st;
}
void nc_cuda_stream_destroy(void* stream) {
    if (stream) cudaStreamDestroy((cudaStream_t)stream);
}
void* nc_cuda_event_create(void) {
    cudaEvent_t ev = nullptr;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) {
        set_status(NC_CUDA_ERR_RUNTIME, "cudaEventCreate failed");
        return nullptr;
    }
    return ev;
}
void* nc_cuda_event_create_timed(void) {
    cudaEvent_t ev = nullptr;
    if (cudaEventCreate(&ev) != cudaSuccess) {
        set_status(NC_CUDA_ERR_RUNTIME, "cudaEventCreate failed");
        return nullptr;
    }
    return ev;
}
int nc_cuda_event_elapsed_ms(void* start, void* stop, float* ms) {
    NCC_REQUIRE(start && stop && ms, "event_elapsed: null argument");
    NCC_TRY(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return NC_CUDA_OK;
}
void nc_cuda_event_destroy(void* event) {
    if (event) cudaEventDestroy((cudaEvent_t)event);
}
int nc_cuda_event_record(void* event, void* stream) {
    NCC_REQUIRE(event, "event_record: null event");
    NCC_TRY(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream));
    return NC_CUDA_OK;
}
int nc_cuda_stream_wait_event(void* stream, void* event) {
    NCC_REQUIRE(event, "stream_wait_event: null event");
    NCC_TRY(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0));
    return NC_CUDA_OK;
}
int nc_cuda_event_synchronize(void* event) {
    NCC_REQUIRE(event, "event_synchronize: null event");
    NCC_TRY(cudaEventSynchronize((cudaEvent_t)event));
    return NC_CUDA_OK;
}
int nc_cuda_last_status(void) { return g_status; }
const char* nc_cuda_last_message(void) { return g_message; }
void nc_cuda_clear_status(void) {
    g_status = NC_CUDA_OK;
    g_message[0] = 0;
}
int nc_cuda_set_math_mode(int mode) {
    int prev = g_math_mode;
    if (mode >= NC_CUDA_MATH_TF32 && mode <= NC_CUDA_MATH_FP32_SIMT) g_math_mode = mode;
    else set_status(NC_CUDA_ERR_ARG, "unknown math mode %d", mode);
    return prev;
}
int nc_cuda_get_math_mode(void) { return g_math_mode; }
int nc_cuda_set_round_outputs(int on) { return ncc::set_round_outputs(on); }
int nc_cuda_set_conv_stats(int on) { return set_conv_stats(on); }
int nc_cuda_offer_batchnorm_backward_sums_f32(const float* x, const float* mean, const float* var, const float* gamma, const float* beta,
                                              double eps, int C, long long rows) {
    NCC_REQUIRE(x && mean && var && C > 0 && rows > 0, "offer_batchnorm_backward_sums: null pointer or empty shape");
    BnFold f = {x, mean, var, gamma, beta, (float)eps, C, rows};
    if (g_bn_fold_on) bn_fold_announce(f);
    return NC_CUDA_OK;
}
int nc_cuda_set_batchnorm_backward_fold(int on) { int p = g_bn_fold_on; g_bn_fold_on = on ? 1 : 0; return p; }
unsigned long long nc_cuda_batchnorm_backward_fold_count(void) { return g_bn_fold_hits; }
unsigned int nc_cuda_device_error_word(void) {
    unsigned int* w = device_error_word();
    unsigned int h = 0;
    if (!w) return 0;
    if (cudaMemcpy(&h, w, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return 0xffffffffu;
    if (h) cudaMemset(w, 0, sizeof(h));
    return h;
}
int nc_cuda_profile_begin(void) {
    if (!g_prof.start) {
        g_prof.start = new cudaEvent_t[kProfCap];
        g_prof.stop = new cudaEvent_t[kProfCap];
        g_prof.cat = new unsigned char[kProfCap];
        g_prof.work = new double[kProfCap];
        for (int i = 0; i < kProfCap; i++)
            if (cudaEventCreate(&g_prof.start[i]) != cudaSuccess || cudaEventCreate(&g_prof.stop[i]) != cudaSuccess)
                return set_status(NC_CUDA_ERR_RUNTIME, "profile: cudaEventCreate failed");
    }
    g_prof.n = 0;
    g_prof.depth = 0;
    g_prof.on = true;
    return NC_CUDA_OK;
}
int nc_cuda_profile_end(void) {
    g_prof.on = false;
    if (g_prof.n > 0 && cudaEventSynchronize(g_prof.stop[g_prof.n - 1]) != cudaSuccess)
        return set_status(NC_CUDA_ERR_RUNTIME, "profile: cudaEventSynchronize failed");
    return NC_CUDA_OK;
}
int nc_cuda_profile_categories(void) { return PROF_CATEGORIES; }
const char* nc_cuda_profile_category_name(int category) {
    return (category >= 0 && category < PROF_CATEGORIES) ? kProfNames[category] : "";
}
int nc_cuda_profile_read(int category, double* total_ms, unsigned long long* calls, double* work) {
    if (g_prof.on) return set_status(NC_CUDA_ERR_ARG, "profile_read: call nc_cuda_profile_end first");
    double ms = 0.0, w = 0.0;
    unsigned long long n = 0;
    for (int i = 0; i < g_prof.n; i++) {
        if (g_prof.cat[i] != category) continue;
        float t = 0.f;
        if (cudaEventElapsedTime(&t, g_prof.start[i], g_prof.stop[i]) != cudaSuccess) continue;
        ms += t; w += g_prof.work[i]; n++;
    }
    if (total_ms) *total_ms = ms;
    if (calls) *calls = n;
    if (work) *work = w;
    return NC_CUDA_OK;
}
unsigned long long nc_cuda_launch_count(void) { return g_launches; }
void nc_cuda_reset_launch_count(void) { g_launches = 0; }  // the epoch keeps counting

}  // extern "C"
