/* Data-parallel gradient reduction over NCCL (NVLink 5 / NVSwitch).
 *
 * The reference is a single-process library with no communication layer;
 * this file is new.  One process drives one GPU and holds a full replica of
 * the parameters; the batch is split by rows and every rank's loss seed is
 * scaled by 1/global_batch, so a SUM all-reduce of each parameter gradient
 * reproduces the full-batch gradient.  The reduction of a gradient is
 * enqueued on a second stream the moment the backward pass has finished
 * accumulating into it (see run_backward in autograd.cu), ordered after the
 * producing kernels by an event, and overlaps the remaining backward GEMMs.
 *
 * NCCL is bound at run time with dlopen, so the library loads and the
 * single-GPU path works on a machine without NCCL, and a process that has
 * already loaded an NCCL (for instance through PyTorch) shares that copy
 * instead of pulling in a second one.  Gradients that fit the peer-memory
 * block of peer_reduce.cu (when the ranks have exchanged its handles) are
 * reduced by that kernel instead of ncclAllReduce.  Failures are reported, never waited
 * on: the communicator is created in blocking mode, every call's result is
 * checked, and ttb_dist_join polls ncclCommGetAsyncError. */
#include "tt_internal.h"

#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

/* The handful of NCCL declarations this file needs (public API, nccl.h). */
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;          /* 0 = ncclSuccess, 7 = ncclInProgress */
enum { NCCL_FLOAT32 = 7, NCCL_SUM = 0 };

/* ncclConfig_t as of NCCL 2.18 (the first fields of every later version, which accept it by its size and
 * version fields): what ncclCommInitRankConfig / ncclCommSplit need to cap a communicator's CTAs. */
typedef struct {
    size_t size; unsigned int magic; unsigned int version;
    int blocking; int cgaClusterSize; int minCTAs; int maxCTAs; const char *netName; int splitShare;
} TtNcclConfig;
#define TT_NCCL_UNDEF_INT ((int)0x80000000)
static TtNcclConfig nccl_config(int max_ctas) {
    TtNcclConfig c = {sizeof(TtNcclConfig), 0xcafebeefu, 21803u, TT_NCCL_UNDEF_INT, TT_NCCL_UNDEF_INT, TT_NCCL_UNDEF_INT,
                      max_ctas, nullptr, TT_NCCL_UNDEF_INT};
    return c;
}

typedef ncclResult_t (*fn_GetUniqueId)(ncclUniqueId *);
typedef ncclResult_t (*fn_CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, TtNcclConfig *);
typedef ncclResult_t (*fn_CommSplit)(ncclComm_t, int, int, ncclComm_t *, TtNcclConfig *);
typedef ncclResult_t (*fn_CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
typedef ncclResult_t (*fn_AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t);
typedef ncclResult_t (*fn_CommDestroy)(ncclComm_t);
typedef ncclResult_t (*fn_CommAbort)(ncclComm_t);
typedef ncclResult_t (*fn_CommGetAsyncError)(ncclComm_t, ncclResult_t *);
typedef const char *(*fn_GetErrorString)(ncclResult_t);

static struct {
    void *handle;
    fn_GetUniqueId GetUniqueId;
    fn_CommInitRank CommInitRank;
    fn_AllReduce AllReduce;
    fn_CommDestroy CommDestroy;
    fn_CommAbort CommAbort;
    fn_CommGetAsyncError CommGetAsyncError;
    fn_GetErrorString GetErrorString;
    fn_CommInitRankConfig CommInitRankConfig;      /* optional (NCCL >= 2.14) */
    fn_CommSplit CommSplit;                        /* optional (NCCL >= 2.18) */
} nccl;

static ncclComm_t g_comm = nullptr;
/* Optional (TT_DP_TAIL_COMM=1): a second communicator over the same ranks for the reductions nothing is left
 * to hide behind (the last row block of the last weight gradient of a pass).  The first one is held to the
 * CTAs that fit beside the GEMMs, this one may take the SMs the finished backward pass has left idle.  Without
 * it those reductions run on the first communicator. */
static ncclComm_t g_comm_tail = nullptr;
static int g_world = 1, g_rank = 0;
static cudaEvent_t g_ev_ready = nullptr, g_ev_done = nullptr;
static int g_inflight = 0;

static int nccl_bind(void) {
    if (nccl.handle) return 0;
    const char *names[] = {getenv("TT_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (int i = 0; i < 3 && !nccl.handle; i++)
        if (names[i] && *names[i]) nccl.handle = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    if (!nccl.handle) { tt_set_error("NCCL not found (dlopen libnccl.so.2): %s", dlerror()); return -1; }
    nccl.GetUniqueId = (fn_GetUniqueId)dlsym(nccl.handle, "ncclGetUniqueId");
    nccl.CommInitRank = (fn_CommInitRank)dlsym(nccl.handle, "ncclCommInitRank");
    nccl.AllReduce = (fn_AllReduce)dlsym(nccl.handle, "ncclAllReduce");
    nccl.CommDestroy = (fn_CommDestroy)dlsym(nccl.handle, "ncclCommDestroy");
    nccl.CommAbort = (fn_CommAbort)dlsym(nccl.handle, "ncclCommAbort");
    nccl.CommGetAsyncError = (fn_CommGetAsyncError)dlsym(nccl.handle, "ncclCommGetAsyncError");
    nccl.GetErrorString = (fn_GetErrorString)dlsym(nccl.handle, "ncclGetErrorString");
    nccl.CommInitRankConfig = (fn_CommInitRankConfig)dlsym(nccl.handle, "ncclCommInitRankConfig");
    nccl.CommSplit = (fn_CommSplit)dlsym(nccl.handle, "ncclCommSplit");
    if (!nccl.GetUniqueId || !nccl.CommInitRank || !nccl.AllReduce || !nccl.CommDestroy ||
        !nccl.CommAbort || !nccl.CommGetAsyncError || !nccl.GetErrorString) {
        tt_set_error("NCCL library lacks a required symbol");
        dlclose(nccl.handle);
        memset(&nccl, 0, sizeof nccl);
        return -1;
    }
    return 0;
}

static int nccl_ok(ncclResult_t r, const char *what) {
    if (r == 0) return 1;
    tt_set_error("%s: %s", what, nccl.GetErrorString ? nccl.GetErrorString(r) : "NCCL error");
    return 0;
}

extern "C" int ttb_dist_unique_id(char id_out[128]) {
    if (!id_out) return -1;
    if (nccl_bind() != 0) return -1;
    ncclUniqueId id;
    if (!nccl_ok(nccl.GetUniqueId(&id), "ncclGetUniqueId")) return -1;
    memcpy(id_out, id.internal, 128);
    return 0;
}

extern "C" int ttb_dist_init(int rank, int world, const char id_in[128]) {
    if (g_comm) { tt_set_error("ttb_dist_init: already initialised"); return -1; }
    if (world < 1 || rank < 0 || rank >= world || !id_in) { tt_set_error("ttb_dist_init: bad rank/world"); return -1; }
    if (tt_ctx_init() != 0) return -1;
    if (world == 1) { g_world = 1; g_rank = 0; return 0; }
    if (nccl_bind() != 0) return -1;
    /* From four ranks on the GEMMs leave the SMs their wave count does not need to the collective
     * (gemm_tc.cu, TT_TC_FIT); NCCL is then held to the CTAs that fit there, unless the caller has
     * set NCCL_MAX_CTAS.  Measured together on an earlier build: 8 GPUs 2.65 -> 2.53 ms per step; either one
     * alone loses. */
    int fit = 1, from = 4;
#ifdef TT_TUNING
    {
        const char *f = getenv("TT_TC_FIT"), *fw = getenv("TT_TC_FIT_WORLD");
        if (f && *f) fit = atoi(f);
        if (fw && *fw) from = atoi(fw);
    }
#endif
    const bool cap = fit && world >= from && !getenv("NCCL_MAX_CTAS");
    ncclUniqueId id;
    memcpy(id.internal, id_in, 128);
    /* How many CTAs NCCL gets was measured on the benchmark MLP with 4 and 8 GPUs: ONE communicator with 24 CTAs.
     * Eight GPUs: 2.49-2.50 ms per step (16 CTAs plus a second communicator for the last reduction of a step:
     * 2.65; 32 CTAs: 2.50); four GPUs: 3.59 (16 + second communicator 3.65).  What is exposed at the end of the
     * backward pass shrinks by more (8 GPUs 0.65 -> 0.39 ms) than the GEMMs lose to the eight extra CTAs (1.82
     * -> 1.96 ms).  The second communicator remains available: TT_DP_TAIL_COMM=1. */
    const int main_ctas = 24;
    const bool want_tail = nccl.CommSplit && getenv("TT_DP_TAIL_COMM") && atoi(getenv("TT_DP_TAIL_COMM")) == 1;
    if (cap && nccl.CommInitRankConfig) {
        /* main communicator capped by its configuration (not by the environment, which would cap the
         * second one too); tail communicator split off it with NCCL's own default */
        TtNcclConfig main_cfg = nccl_config(main_ctas);
        if (!nccl_ok(nccl.CommInitRankConfig(&g_comm, world, id, rank, &main_cfg), "ncclCommInitRankConfig")) { g_comm = nullptr; return -1; }
        if (want_tail) {
            TtNcclConfig tail_cfg = nccl_config(TT_NCCL_UNDEF_INT);
            if (nccl.CommSplit(g_comm, 0, rank, &g_comm_tail, &tail_cfg) != 0) g_comm_tail = nullptr;     /* optional: the main one serves */
        }
    } else {
        if (cap) setenv("NCCL_MAX_CTAS", "24", 0);
        if (!nccl_ok(nccl.CommInitRank(&g_comm, world, id, rank), "ncclCommInitRank")) { g_comm = nullptr; return -1; }
    }
    if (!tt_cuda_ok(cudaEventCreateWithFlags(&g_ev_ready, cudaEventDisableTiming), "cudaEventCreate") ||
        !tt_cuda_ok(cudaEventCreateWithFlags(&g_ev_done, cudaEventDisableTiming), "cudaEventCreate")) return -1;
    g_world = world; g_rank = rank;
    /* TT_GEMM_SMS can keep SMs free for NCCL's kernels while a persistent GEMM runs.  Measured
     * on the benchmark MLP, reserving 20 SMs cost more GEMM time than the reductions gained
     * (2 GPUs: 2.45 -> 2.49 ms per step on the 8-GPU job's per-GPU shapes), so the default is
     * to reserve none. */
    return 0;
}

extern "C" int ttb_dist_world(void) { return g_world; }
int tt_dist_active(void) { return g_comm != nullptr && g_world > 1; }
/* Work was put on the communication stream outside an all-reduce (a fused optimiser step):
 * ttb_dist_join must order the compute stream after it. */
void tt_dist_note_comm_work(void) { g_inflight++; }

/* ---- per-collective timing (while ttb_trace_enable is on) ---------------------------------
 * Every reduction is bracketed by an event pair on the communication stream, and every
 * ttb_dist_join by one event at the compute stream's tail (before it is made to wait) and
 * one at the communication stream's tail: the second minus the first is the time the
 * collectives and the updates behind them were NOT hidden by compute in that step. */
struct CommPair { cudaEvent_t a, b; double bytes; };
static std::vector<CommPair> g_cpairs, g_jpairs;      /* event pools, reused across resets */
static size_t g_ncpairs = 0, g_njpairs = 0;

void tt_dist_trace_reset(void) { g_ncpairs = 0; g_njpairs = 0; }

static CommPair *pair_from(std::vector<CommPair> &pool, size_t &used) {
    if (used == pool.size()) {
        CommPair c = {nullptr, nullptr, 0.0};
        if (cudaEventCreate(&c.a) != cudaSuccess || cudaEventCreate(&c.b) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        pool.push_back(c);
    }
    return &pool[used++];
}

/* Sum count floats at p over all ranks in place: ordered after everything already on the
 * compute stream, runs on the communication stream. */
static int reduce_on_comm_stream(float *p, size_t count, int tail = 0) {
    if (!tt_cuda_ok(cudaEventRecord(g_ev_ready, g_tt.stream), "cudaEventRecord") ||
        !tt_cuda_ok(cudaStreamWaitEvent(g_tt.comm_stream, g_ev_ready, 0), "cudaStreamWaitEvent")) return -1;
    CommPair *tp = g_tt.trace ? pair_from(g_cpairs, g_ncpairs) : nullptr;
    if (tp) { tp->bytes = 4.0 * (double)count; cudaEventRecord(tp->a, g_tt.comm_stream); }
    int rc = 0;
    if (tt_peer_usable(p, count)) {
        if (tt_peer_allreduce(p, count, g_tt.comm_stream) != 0) rc = -1;
    } else if (!nccl_ok(nccl.AllReduce(p, p, count, NCCL_FLOAT32, NCCL_SUM, (tail && g_comm_tail) ? g_comm_tail : g_comm, g_tt.comm_stream), "ncclAllReduce")) rc = -1;
    if (tp) cudaEventRecord(tp->b, g_tt.comm_stream);
    if (rc == 0) g_inflight++;
    return rc;
}

/* Order the communication stream after everything enqueued on the compute stream so far. */
int tt_dist_comm_after_compute(void) {
    if (!tt_dist_active()) return 0;
    if (!tt_cuda_ok(cudaEventRecord(g_ev_ready, g_tt.stream), "cudaEventRecord") ||
        !tt_cuda_ok(cudaStreamWaitEvent(g_tt.comm_stream, g_ev_ready, 0), "cudaStreamWaitEvent")) return -1;
    return 0;
}

/* The reduction of a gradient whose producing GEMM already pushed its first pushed_floats values to
 * their owners (fused reduce-scatter): peer-memory kernel only. */
int tt_dist_allreduce_pushed(float *p, size_t count, size_t pushed_floats) {
    if (!tt_dist_active() || !count) return 0;
    if (!tt_cuda_ok(cudaEventRecord(g_ev_ready, g_tt.stream), "cudaEventRecord") ||
        !tt_cuda_ok(cudaStreamWaitEvent(g_tt.comm_stream, g_ev_ready, 0), "cudaStreamWaitEvent")) return -1;
    CommPair *tp = g_tt.trace ? pair_from(g_cpairs, g_ncpairs) : nullptr;
    if (tp) { tp->bytes = 4.0 * (double)count; cudaEventRecord(tp->a, g_tt.comm_stream); }
    const int rc = tt_peer_allreduce_pushed(p, count, pushed_floats, g_tt.comm_stream);
    if (tp) cudaEventRecord(tp->b, g_tt.comm_stream);
    if (rc == 0) g_inflight++;
    return rc;
}

int tt_dist_allreduce_async(Tensor *t) {
    if (!tt_dist_active()) return 0;
    float *p = tt_dev_rw(t);
    if (!p) return -1;
    if (reduce_on_comm_stream(p, (size_t)t->numel) != 0) return -1;
    tt_mark_busy(t, g_tt.comm_stream);
    return 0;
}

int tt_dist_allreduce_range(float *p, size_t count) {
    if (!tt_dist_active() || !count) return 0;
    return reduce_on_comm_stream(p, count);
}
/* The same for a reduction that no compute is left to overlap with: it may use the tail communicator. */
int tt_dist_allreduce_tail(float *p, size_t count) {
    if (!tt_dist_active() || !count) return 0;
    return reduce_on_comm_stream(p, count, 1);
}

extern "C" int ttb_dist_allreduce(Tensor *t) {
    if (!t) return -1;
    return tt_dist_allreduce_async(t);
}

/* Sums since the last ttb_trace_reset: {collectives, bytes reduced, ms inside collectives (event
 * pairs on the communication stream, waiting for the slowest rank included), joins, exposed ms
 * (communication stream's tail minus compute stream's tail at each join, when positive), longest
 * collective in ms}.  Waits for both streams. */
extern "C" int ttb_dist_comm_read(double out[6]) {
    if (!out || g_tt.ready != 1) return -1;
    if (!tt_cuda_ok(cudaStreamSynchronize(g_tt.stream), "cudaStreamSynchronize") ||
        !tt_cuda_ok(cudaStreamSynchronize(g_tt.comm_stream), "cudaStreamSynchronize(comm)")) return -1;
    for (int i = 0; i < 6; i++) out[i] = 0.0;
    for (size_t i = 0; i < g_ncpairs; i++) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, g_cpairs[i].a, g_cpairs[i].b) != cudaSuccess) { cudaGetLastError(); continue; }
        out[0] += 1.0; out[1] += g_cpairs[i].bytes; out[2] += ms;
        if (ms > out[5]) out[5] = ms;
    }
    for (size_t i = 0; i < g_njpairs; i++) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, g_jpairs[i].a, g_jpairs[i].b) != cudaSuccess) { cudaGetLastError(); continue; }
        out[3] += 1.0;
        if (ms > 0.0f) out[4] += ms;
    }
    return 0;
}

/* Make the compute stream wait for every reduction enqueued so far. */
extern "C" int ttb_dist_join(void) {
    if (g_comm == nullptr && !g_inflight) return 0;
    if (g_inflight) {
        if (g_tt.trace) {
            CommPair *jp = pair_from(g_jpairs, g_njpairs);
            if (jp) { cudaEventRecord(jp->a, g_tt.stream); cudaEventRecord(jp->b, g_tt.comm_stream); }
        }
        if (!tt_cuda_ok(cudaEventRecord(g_ev_done, g_tt.comm_stream), "cudaEventRecord") ||
            !tt_cuda_ok(cudaStreamWaitEvent(g_tt.stream, g_ev_done, 0), "cudaStreamWaitEvent")) return -1;
        g_inflight = 0;
    }
    if (!tt_dist_active()) return 0;
    if (tt_peer_poll_status()) return -1;
    ncclResult_t async = 0;
    if (!nccl_ok(nccl.CommGetAsyncError(g_comm, &async), "ncclCommGetAsyncError")) return -1;
    if (async != 0 && async != 7) {
        nccl_ok(async, "NCCL asynchronous error");
        if (g_comm_tail) { nccl.CommAbort(g_comm_tail); g_comm_tail = nullptr; }
        nccl.CommAbort(g_comm);
        g_comm = nullptr; g_world = 1;
        return -1;
    }
    return 0;
}

extern "C" void ttb_dist_finalize(void) {
    tt_peer_finalize();
    if (g_comm) {
        cudaStreamSynchronize(g_tt.comm_stream);
        if (g_comm_tail) { nccl.CommDestroy(g_comm_tail); g_comm_tail = nullptr; }
        nccl.CommDestroy(g_comm);
        g_comm = nullptr;
    }
    if (g_ev_ready) { cudaEventDestroy(g_ev_ready); g_ev_ready = nullptr; }
    if (g_ev_done) { cudaEventDestroy(g_ev_done); g_ev_done = nullptr; }
    g_world = 1; g_rank = 0; g_inflight = 0;
    g_tt.gemm_sms = g_tt.sm_count;
}
