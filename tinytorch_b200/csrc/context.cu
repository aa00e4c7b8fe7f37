/* Process-wide device context: one GPU, one compute stream, a stream-ordered
 * memory pool, the last-error text and per-kernel-class event timing.
 *
 * The reference keeps no such state (it is host code over malloc); this file
 * is what "L0 hardware" becomes once storage moves into HBM. */
#include "tt_internal.h"

#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <unordered_map>
#include <vector>

TTContext g_tt = {0, 0, 0, 0, nullptr, nullptr, nullptr, -1, -1, -1, -1, 1, 0, 0, 0};    /* -1: take the setting from the environment */

static char g_err[512] = "";

void tt_set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    if (getenv("TT_VERBOSE")) fprintf(stderr, "tinytorch-b200: %s\n", g_err);
}

int tt_cuda_ok(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return 1;
    tt_set_error("%s: %s", what, cudaGetErrorString(e));
    return 0;
}

static int env_int(const char *name, int dflt) {
    const char *s = getenv(name);
    if (!s || !*s) return dflt;
    return atoi(s);
}

static int ctx_open(int device) {
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count <= 0) {
        tt_set_error("no CUDA device available (%s): this library has no CPU path",
                     e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
        g_tt.ready = -1;
        return -1;
    }
    if (device < 0 || device >= count) {
        tt_set_error("device %d out of range (%d visible)", device, count);
        g_tt.ready = -1;
        return -1;
    }
    if (!tt_cuda_ok(cudaSetDevice(device), "cudaSetDevice")) { g_tt.ready = -1; return -1; }
    cudaDeviceProp prop;
    if (!tt_cuda_ok(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties")) { g_tt.ready = -1; return -1; }
    if (prop.major != 10) {
        tt_set_error("device %d is sm_%d%d; this library carries sm_100a code only",
                     device, prop.major, prop.minor);
        g_tt.ready = -1;
        return -1;
    }
    g_tt.device = device;
    g_tt.sm_count = prop.multiProcessorCount;
    g_tt.gemm_sms = env_int("TT_GEMM_SMS", g_tt.sm_count);
    if (g_tt.gemm_sms < 1 || g_tt.gemm_sms > g_tt.sm_count) g_tt.gemm_sms = g_tt.sm_count;
    if (!tt_cuda_ok(cudaStreamCreateWithFlags(&g_tt.stream, cudaStreamNonBlocking), "cudaStreamCreate") ||
        !tt_cuda_ok(cudaStreamCreateWithFlags(&g_tt.comm_stream, cudaStreamNonBlocking), "cudaStreamCreate") ||
        !tt_cuda_ok(cudaStreamCreateWithFlags(&g_tt.copy_stream, cudaStreamNonBlocking), "cudaStreamCreate")) {
        g_tt.ready = -1;
        return -1;
    }
    /* Keep freed blocks in the pool: the training loop allocates the same
     * sizes every step and must not go back to the driver for them. */
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
        unsigned long long keep = ~0ull;
        cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    if (g_tt.gemm_path < 0) g_tt.gemm_path = env_int("TT_GEMM_PATH", 0);
    if (g_tt.fuse_padones < 0) g_tt.fuse_padones = env_int("TT_FUSE_PADONES", 1);
    if (g_tt.fuse_relu < 0) g_tt.fuse_relu = env_int("TT_FUSE_RELU", 1);
    if (g_tt.conv_implicit < 0) g_tt.conv_implicit = env_int("TT_CONV_IMPLICIT", 1);
    g_tt.ready = 1;
    return 0;
}

int tt_ctx_init(void) {
    if (g_tt.ready == 1) return 0;
    if (g_tt.ready == -1) return -1;
    int dev = env_int("TT_DEVICE", env_int("LOCAL_RANK", 0));
    return ctx_open(dev);
}

extern "C" int ttb_device_count(void) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) { cudaGetLastError(); return 0; }
    return count;
}

extern "C" int ttb_init(int device) {
    if (g_tt.ready == 1) {
        if (device == g_tt.device) return 0;
        tt_set_error("ttb_init(%d): the library already runs on device %d", device, g_tt.device);
        return -1;
    }
    g_tt.ready = 0;
    return ctx_open(device);
}

extern "C" const char *ttb_last_error(void) { return g_err; }

extern "C" int ttb_sync(void) {
    if (tt_ctx_init() != 0) return -1;
    if (!tt_cuda_ok(cudaStreamSynchronize(g_tt.stream), "cudaStreamSynchronize")) return -1;
    if (!tt_cuda_ok(cudaStreamSynchronize(g_tt.comm_stream), "cudaStreamSynchronize(comm)")) return -1;
    if (!tt_cuda_ok(cudaStreamSynchronize(g_tt.copy_stream), "cudaStreamSynchronize(copy)")) return -1;
    if (gemm_tc_poll_status()) return -1;
    return 0;
}

extern "C" long ttb_launch_count(void) { return g_tt.launches; }

/* Device memory for tensors and scratch.  Underneath is the stream-ordered pool (cudaMallocAsync on
 * the compute stream); in front of it sit free lists by exact size for blocks of up to 64 MB, because
 * a training loop asks for the same few sizes thousands of times per second and the two driver
 * calls per tensor were a third of the host's time per launch.  A block goes back on its list at
 * release and is handed out again to the next request of that size: every use is ordered on the
 * compute stream, so reuse needs no further synchronisation -- the same guarantee cudaFreeAsync on
 * that stream gives.  The lists hold at most TT_CACHE_MB (default 4096) megabytes; beyond that, and
 * for larger blocks, release goes to the pool.  TT_CACHE_MB=0 switches the lists off. */
struct DevBlockCache {
    std::unordered_map<size_t, std::vector<void *>> free_by_size;
    std::unordered_map<void *, size_t> size_of;          /* blocks handed out that may come back to a list */
    size_t cached_bytes = 0;
    size_t limit_bytes = 0;
    bool configured = false;
};
static DevBlockCache g_cache;
static const size_t CACHE_MAX_BLOCK = (size_t)64 << 20;

void *tt_dev_alloc(size_t bytes) {
    if (tt_ctx_init() != 0) return nullptr;
    if (!g_cache.configured) {
        g_cache.limit_bytes = (size_t)env_int("TT_CACHE_MB", 4096) << 20;
        g_cache.configured = true;
    }
    if (bytes == 0) bytes = 4;
    bytes = (bytes + 255) & ~(size_t)255;
    const bool cacheable = g_cache.limit_bytes > 0 && bytes <= CACHE_MAX_BLOCK;
    if (cacheable) {
        auto it = g_cache.free_by_size.find(bytes);
        if (it != g_cache.free_by_size.end() && !it->second.empty()) {
            void *p = it->second.back();
            it->second.pop_back();
            g_cache.cached_bytes -= bytes;
            g_cache.size_of[p] = bytes;
            return p;
        }
    }
    void *p = nullptr;
    if (!tt_cuda_ok(cudaMallocAsync(&p, bytes, g_tt.stream), "cudaMallocAsync")) return nullptr;
    if (cacheable) g_cache.size_of[p] = bytes;
    return p;
}

void tt_dev_free(void *p) {
    if (!p || g_tt.ready != 1) return;
    auto it = g_cache.size_of.find(p);
    if (it != g_cache.size_of.end()) {
        const size_t bytes = it->second;
        g_cache.size_of.erase(it);
        if (g_cache.cached_bytes + bytes <= g_cache.limit_bytes) {
            g_cache.free_by_size[bytes].push_back(p);
            g_cache.cached_bytes += bytes;
            return;
        }
    }
    cudaFreeAsync(p, g_tt.stream);
}

/* Device memory as the driver and the stream-ordered pool see it: {free bytes on the GPU, bytes the
 * pool has reserved from the driver, bytes of the pool handed out}.  Equal before and after a call
 * means the call neither went to the driver nor took a block from the pool. */
extern "C" int ttb_mem_info(unsigned long long out[3]) {
    if (!out || tt_ctx_init() != 0) return -1;
    size_t free_b = 0, total_b = 0;
    if (!tt_cuda_ok(cudaMemGetInfo(&free_b, &total_b), "cudaMemGetInfo")) return -1;
    cudaMemPool_t pool;
    unsigned long long reserved = 0, used = 0;
    if (!tt_cuda_ok(cudaDeviceGetDefaultMemPool(&pool, g_tt.device), "cudaDeviceGetDefaultMemPool") ||
        !tt_cuda_ok(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemCurrent, &reserved), "cudaMemPoolGetAttribute") ||
        !tt_cuda_ok(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemCurrent, &used), "cudaMemPoolGetAttribute")) return -1;
    out[0] = (unsigned long long)free_b; out[1] = reserved; out[2] = used;
    return 0;
}

extern "C" void *ttb_pinned_alloc(size_t bytes) {
    if (tt_ctx_init() != 0) return nullptr;
    void *p = nullptr;
    if (!tt_cuda_ok(cudaHostAlloc(&p, bytes ? bytes : 4, cudaHostAllocDefault), "cudaHostAlloc")) return nullptr;
    return p;
}
extern "C" void ttb_pinned_free(void *p) { if (p) cudaFreeHost(p); }

/* ---- events ---------------------------------------------------------------*/
extern "C" void *ttb_event_create(void) {
    if (tt_ctx_init() != 0) return nullptr;
    cudaEvent_t ev;
    if (!tt_cuda_ok(cudaEventCreate(&ev), "cudaEventCreate")) return nullptr;
    return (void *)ev;
}
extern "C" void ttb_event_record(void *ev) {
    if (ev && g_tt.ready == 1) cudaEventRecord((cudaEvent_t)ev, g_tt.stream);
}
extern "C" float ttb_event_elapsed_ms(void *a, void *b) {
    float ms = -1.0f;
    if (!a || !b) return ms;
    if (!tt_cuda_ok(cudaEventSynchronize((cudaEvent_t)b), "cudaEventSynchronize")) return -1.0f;
    if (!tt_cuda_ok(cudaEventElapsedTime(&ms, (cudaEvent_t)a, (cudaEvent_t)b), "cudaEventElapsedTime")) return -1.0f;
    return ms;
}
extern "C" void ttb_event_destroy(void *ev) { if (ev) cudaEventDestroy((cudaEvent_t)ev); }

/* ---- per-class tracing ----------------------------------------------------
 * Event pairs come from a growing pool and are resolved when read. */
typedef struct TracePair { cudaEvent_t a, b; int kind; double work; } TracePair;
static TracePair *g_pairs = nullptr;
static long g_npairs = 0, g_cap_pairs = 0, g_made_pairs = 0;

extern "C" void ttb_trace_enable(int on) { g_tt.trace = on ? 1 : 0; }
extern "C" void ttb_trace_reset(void) { g_npairs = 0; tt_dist_trace_reset(); }

void tt_trace_begin(int kind) {
    if (!g_tt.trace) return;
    if (g_npairs == g_cap_pairs) {
        long nc = g_cap_pairs ? g_cap_pairs * 2 : 1024;
        TracePair *np = (TracePair *)realloc(g_pairs, sizeof(TracePair) * (size_t)nc);
        if (!np) { g_tt.trace = 0; return; }
        g_pairs = np; g_cap_pairs = nc;
    }
    TracePair *p = &g_pairs[g_npairs];
    if (g_npairs >= g_made_pairs) {
        if (cudaEventCreate(&p->a) != cudaSuccess || cudaEventCreate(&p->b) != cudaSuccess) { g_tt.trace = 0; return; }
        g_made_pairs = g_npairs + 1;
    }
    p->kind = kind;
    cudaEventRecord(p->a, g_tt.stream);
}

void tt_trace_end(int kind, double work) {
    if (!g_tt.trace) return;
    TracePair *p = &g_pairs[g_npairs];
    (void)kind;
    p->work = work;
    cudaEventRecord(p->b, g_tt.stream);
    g_npairs++;
}

extern "C" int ttb_trace_read(int kind, double *total_ms, long *launches, double *work) {
    if (g_tt.ready != 1) return -1;
    if (!tt_cuda_ok(cudaStreamSynchronize(g_tt.stream), "cudaStreamSynchronize")) return -1;
    double t = 0.0, w = 0.0; long n = 0;
    for (long i = 0; i < g_npairs; i++) {
        if (g_pairs[i].kind != kind) continue;
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, g_pairs[i].a, g_pairs[i].b) != cudaSuccess) continue;
        t += ms; w += g_pairs[i].work; n++;
    }
    if (total_ms) *total_ms = t;
    if (launches) *launches = n;
    if (work) *work = w;
    return 0;
}
