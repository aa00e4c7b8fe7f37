/* Gradient all-reduce over peer memory (NVLink 5 / NVSwitch), without NCCL's kernels.
 *
 * The reference is a single-process library; this file is new.  Why it exists: the GEMM of
 * this library is a persistent kernel whose CTAs fill an SM's shared memory, so a library
 * collective that brings its own large CTAs cannot share an SM with it -- the two take SMs
 * from each other and both slow down.  The kernel below needs four bytes of shared memory and few
 * registers per thread, so its CTAs sit beside the GEMM's on the same SMs, and it moves the
 * bytes with plain peer loads and stores.
 *
 * Every rank owns one device allocation (cudaMalloc, exported with cudaIpcGetMemHandle and
 * opened by the other ranks): a block of flags, a staging area of `world` slots, and a
 * result area.  One launch per gradient, the same on every rank; CTA b of every rank works
 * on slice b of every chunk, so the CTAs with the same index form an independent group and
 * no grid-wide barrier is needed:
 *   1. push    rank r stores slice b of chunk c of its gradient into slot r of rank c's
 *              staging area, for every c != r;
 *      flags   r writes the launch number into flag[0][r][b] of every peer and waits until
 *              its own flag[0][p][b] carries it for every p;
 *   2. reduce  r adds slice b of chunk r over all ranks IN RANK ORDER (its own part from the
 *              gradient, the others from its staging slots), writes the sums into its own
 *              gradient and into the result area of every peer;
 *      flags   as before, on flag[1];
 *   3. copy    r copies the chunks c != r from its result area into its gradient.
 * Every rank ends with bit-identical sums (each chunk is added once, by one rank).
 *
 * Every wait is bounded: when the limit passes (about two seconds; ttb_dist_set_wait_limit_ms
 * changes it), the kernel writes a code into a host-mapped status word and stops waiting (its
 * output is then wrong and ttb_dist_join reports the failure); it never spins forever.  A
 * failure is sticky and spreads: the rank that gave up sets a poison word in its own flag
 * block and in every peer's, every wait polls the waiter's poison words and every launch
 * looks at them first, so a peer whose launches have fallen out of step with the rank that
 * gave up reports the failure instead of passing its waits on stale flags and summing
 * left-over staging data.  After a failure this process launches no further peer
 * reductions (they return -1); the job has to tear the peer path down.  A launch may reuse the staging and result areas of the
 * previous one because a rank leaves a launch only after every peer has signalled the end
 * of its phase 2, and enters phase 2 only after every peer has entered the launch. */
#include "tt_internal.h"

#include <stdlib.h>
#include <string.h>

#define PR_MAX_WORLD 8
#define PR_MAX_CTAS 64
#define PR_THREADS 256
#define PR_FLAG_WORDS (2 * PR_MAX_WORLD * PR_MAX_CTAS)
#define PR_POISON_WORD PR_FLAG_WORDS             /* + rank: set by `rank` when one of its waits ran out */
#define PR_FLAG_BYTES 16384                      /* flags block, padded */
#define PR_WAIT_LIMIT (1u << 24)                 /* polls of ~128 ns: about two seconds */
#define PR_POLLS_PER_MS 8192u

struct PeerParams {
    float *g;                       /* this rank's gradient (or a contiguous part of it) */
    long count4;                    /* its length in 128-bit words */
    long chunk4;                    /* words per chunk */
    long slot4;                     /* words between staging slots */
    int rank, world;
    unsigned epoch;                 /* launch number, the value the flags take */
    long push_from4;                /* words below this index were pushed to their owners by the producing GEMM's epilogue */
    float *stage[PR_MAX_WORLD];     /* staging area (the one of this launch) of rank p as mapped in this process */
    float *result[PR_MAX_WORLD];    /* result area of rank p */
    unsigned *flags[PR_MAX_WORLD];  /* flag block of rank p */
    unsigned *status;               /* host-mapped: 0 = fine */
    unsigned wait_limit;            /* polls before a wait gives up */
};

/* Has any rank (this one included) given up on a wait of this job? */
__device__ __forceinline__ int pr_poisoned(const PeerParams &p) {
    const volatile unsigned *mine = p.flags[p.rank] + PR_POISON_WORD;
    int bad = 0;
    for (int q = 0; q < p.world; q++) bad |= mine[q] != 0u;
    return bad;
}
/* Tell everybody, this rank's later launches included, that this rank stopped waiting. */
__device__ __forceinline__ void pr_poison_all(const PeerParams &p) {
    for (int q = 0; q < p.world; q++) *(volatile unsigned *)(p.flags[q] + PR_POISON_WORD + p.rank) = 1u;
    __threadfence_system();
}

__device__ __forceinline__ void pr_signal_and_wait(const PeerParams &p, int phase, int b, bool &ok, int *gave_up) {
    /* each thread orders its own peer stores before the flag that announces them */
    __threadfence_system();
    __syncthreads();
    const int t = threadIdx.x;
    if (t < p.world && t != p.rank) {
        volatile unsigned *theirs = p.flags[t] + (phase * PR_MAX_WORLD + p.rank) * PR_MAX_CTAS + b;
        *theirs = p.epoch;
        if (ok) {
            volatile unsigned *mine = p.flags[p.rank] + (phase * PR_MAX_WORLD + t) * PR_MAX_CTAS + b;
            unsigned n = 0;
            while ((int)(*mine - p.epoch) < 0) {
                if (++n > p.wait_limit) {
                    *(volatile unsigned *)p.status = 0x100u | ((unsigned)phase << 4) | (unsigned)t;
                    *(volatile int *)gave_up = 1;
                    pr_poison_all(p);
                    break;
                }
                if ((n & 63u) == 0u && pr_poisoned(p)) {          /* somebody else gave up (another rank, or another CTA of this one): so do we */
                    if (*(volatile unsigned *)p.status == 0u)      /* the first report stands: it names the wait that ran out */
                        *(volatile unsigned *)p.status = 0x200u | ((unsigned)phase << 4) | (unsigned)t;
                    *(volatile int *)gave_up = 1;
                    break;
                }
                __nanosleep(128);
            }
        }
    }
    __syncthreads();
    if (*(volatile int *)gave_up) ok = false;            /* a wait of this CTA ran out: signal on, but wait no more */
    __threadfence_system();
}

/* At most 80 registers x 256 threads: a CTA of this kernel fits into the registers a GEMM CTA
 * (448 threads x 96) leaves free on its SM. */
__global__ void __launch_bounds__(PR_THREADS, 3) peer_allreduce_kernel(PeerParams p) {
    const int b = blockIdx.x, nb = gridDim.x, t = threadIdx.x;
    const long per = (p.chunk4 + nb - 1) / nb;
    const long s0 = (long)b * per < p.chunk4 ? (long)b * per : p.chunk4;
    const long s1 = s0 + per < p.chunk4 ? s0 + per : p.chunk4;
    float4 *g4 = (float4 *)p.g;
    bool ok = true;
    __shared__ int gave_up;
    if (t == 0) {
        gave_up = 0;
        if (pr_poisoned(p)) {            /* a wait ran out earlier, here or on a peer: flags and staging are not to be trusted */
            gave_up = 1;
            if (*(volatile unsigned *)p.status == 0u) *(volatile unsigned *)p.status = 0x300u | (unsigned)p.rank;
        }
    }
    __syncthreads();
    if (gave_up) return;

    /* 1. push my part of every foreign chunk to its owner (four independent 128-bit loads per
     * thread and peer in flight: the stores are posted, the loads set the pace) */
    for (int i = 1; i < p.world; i++) {
        const int c = (p.rank + i) % p.world;
        const long base = (long)c * p.chunk4;
        float4 *dst = (float4 *)p.stage[c] + (long)p.rank * p.slot4;
        long hi = p.count4 - base < s1 ? p.count4 - base : s1;          /* the last chunk may be short */
        long lo = p.push_from4 - base > s0 ? p.push_from4 - base : s0;  /* the GEMM's epilogue delivered what lies below push_from4 */
        long k = lo + t;
        for (; k + 3 * PR_THREADS < hi; k += 4 * PR_THREADS) {
            const float4 v0 = g4[base + k], v1 = g4[base + k + PR_THREADS];
            const float4 v2 = g4[base + k + 2 * PR_THREADS], v3 = g4[base + k + 3 * PR_THREADS];
            dst[k] = v0; dst[k + PR_THREADS] = v1; dst[k + 2 * PR_THREADS] = v2; dst[k + 3 * PR_THREADS] = v3;
        }
        for (; k < hi; k += PR_THREADS) dst[k] = g4[base + k];
    }
    pr_signal_and_wait(p, 0, b, ok, &gave_up);

    /* 2. add my chunk over the ranks, in rank order; hand the sums to everybody */
    {
        const long base = (long)p.rank * p.chunk4;
        const float4 *slots = (const float4 *)p.stage[p.rank];
        const long hi = p.count4 - base < s1 ? p.count4 - base : s1;
        for (long k = s0 + t; k < hi; k += PR_THREADS) {
            /* the loads of all ranks' parts are issued before the first add */
            float4 a[PR_MAX_WORLD];
            #pragma unroll
            for (int q = 0; q < PR_MAX_WORLD; q++)
                if (q < p.world) a[q] = q == p.rank ? g4[base + k] : __ldcg(slots + (long)q * p.slot4 + k);
            float4 acc = a[0];
            #pragma unroll
            for (int q = 1; q < PR_MAX_WORLD; q++)
                if (q < p.world) { acc.x += a[q].x; acc.y += a[q].y; acc.z += a[q].z; acc.w += a[q].w; }
            g4[base + k] = acc;
            for (int i = 1; i < p.world; i++) {
                const int c = (p.rank + i) % p.world;
                ((float4 *)p.result[c])[base + k] = acc;
            }
        }
    }
    pr_signal_and_wait(p, 1, b, ok, &gave_up);

    /* 3. take the other chunks' sums */
    {
        const float4 *res = (const float4 *)p.result[p.rank];
        for (int i = 1; i < p.world; i++) {
            const int c = (p.rank + i) % p.world;
            const long base = (long)c * p.chunk4;
            long hi = p.count4 - base < s1 ? p.count4 - base : s1;
            long k = s0 + t;
            for (; k + 3 * PR_THREADS < hi; k += 4 * PR_THREADS) {
                const float4 v0 = __ldcg(res + base + k), v1 = __ldcg(res + base + k + PR_THREADS);
                const float4 v2 = __ldcg(res + base + k + 2 * PR_THREADS), v3 = __ldcg(res + base + k + 3 * PR_THREADS);
                g4[base + k] = v0; g4[base + k + PR_THREADS] = v1;
                g4[base + k + 2 * PR_THREADS] = v2; g4[base + k + 3 * PR_THREADS] = v3;
            }
            for (; k < hi; k += PR_THREADS) g4[base + k] = __ldcg(res + base + k);
        }
    }
}

/* ---- host side -----------------------------------------------------------------------*/
static struct {
    int active, rank, world, ctas;
    size_t max_floats;
    long slot4;
    char *base[PR_MAX_WORLD];        /* allocation of rank p as mapped here; [rank] is our own */
    unsigned epoch;
    unsigned *status_host, *status_dev;
    unsigned wait_limit;             /* 0 = the default */
    int failed;                      /* sticky: a bounded wait ran out in this job */
    cudaEvent_t done[2];             /* end of the last launch that used staging area 0 / 1 */
    int done_valid[2];
} g_peer;

/* How long a device-side wait on another rank may last before the kernel gives up and the
 * failure is reported (default about two seconds).  For tests of the failure path and for
 * jobs that want to learn of a dead peer sooner. */
extern "C" int ttb_dist_set_wait_limit_ms(int ms) {
    if (ms < 1 || ms > 60000) { tt_set_error("ttb_dist_set_wait_limit_ms: 1..60000"); return -1; }
    g_peer.wait_limit = (unsigned)ms * PR_POLLS_PER_MS;
    return 0;
}

static size_t pr_slot_floats(size_t max_floats, int world) {
    size_t c = (max_floats + world - 1) / world;
    return (c + 31) & ~(size_t)31;                  /* chunks are whole 32-float blocks: a GEMM epilogue stores such blocks */
}
static long pr_chunk4(size_t count, int world) {
    const long count4 = (long)(count / 4);
    const long c = (count4 + world - 1) / world;
    return (c + 7) & ~7l;
}
static size_t pr_total_bytes(size_t max_floats, int world) {
    /* two staging areas of world slots, used by alternate launches (the epilogue of a weight-gradient GEMM
     * may be filling one while the previous reduction still reads the other), and a result area */
    size_t padded = pr_slot_floats(max_floats, world) * world;
    return PR_FLAG_BYTES + 3 * padded * sizeof(float);
}

/* Allocate this rank's block for gradients of up to max_floats values in a job of `world`
 * ranks and return the 64-byte handle the other ranks open it with. */
extern "C" int ttb_dist_peer_export(size_t max_floats, int world, char handle_out[64]) {
    if (!handle_out || max_floats == 0 || world < 2 || world > PR_MAX_WORLD) {
        tt_set_error("ttb_dist_peer_export: bad arguments (2..%d ranks)", PR_MAX_WORLD);
        return -1;
    }
    if (g_peer.base[0] || g_peer.active) { tt_set_error("ttb_dist_peer_export: already set up"); return -1; }
    if (tt_ctx_init() != 0) return -1;
    void *p = nullptr;
    const size_t bytes = pr_total_bytes(max_floats, world);
    if (!tt_cuda_ok(cudaMalloc(&p, bytes), "cudaMalloc(peer block)")) return -1;
    if (!tt_cuda_ok(cudaMemset(p, 0, PR_FLAG_BYTES), "cudaMemset(peer flags)")) { cudaFree(p); return -1; }
    static_assert((PR_POISON_WORD + PR_MAX_WORLD) * sizeof(unsigned) <= PR_FLAG_BYTES, "flag block too small");
    cudaIpcMemHandle_t h;
    if (!tt_cuda_ok(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle")) { cudaFree(p); return -1; }
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle_out, &h, 64);
    g_peer.base[0] = (char *)p;              /* parked here until the import knows our rank */
    g_peer.max_floats = max_floats;
    g_peer.world = world;
    return 0;
}

/* Open the blocks of the other ranks (handles: world x 64 bytes, in rank order) and switch
 * the gradient reductions of this process to the peer kernel. */
extern "C" int ttb_dist_peer_import(int rank, int world, const char *handles) {
    if (!handles || !g_peer.base[0] || g_peer.active || world != g_peer.world || rank < 0 || rank >= world) {
        tt_set_error("ttb_dist_peer_import: call ttb_dist_peer_export first, with the same number of ranks");
        return -1;
    }
    char *own = g_peer.base[0];
    g_peer.base[0] = nullptr;
    for (int p = 0; p < world; p++) {
        if (p == rank) { g_peer.base[p] = own; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + 64 * (size_t)p, 64);
        void *m = nullptr;
        if (!tt_cuda_ok(cudaIpcOpenMemHandle(&m, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")) {
            for (int q = 0; q < p; q++) if (q != rank && g_peer.base[q]) { cudaIpcCloseMemHandle(g_peer.base[q]); g_peer.base[q] = nullptr; }
            g_peer.base[0] = own;
            return -1;
        }
        g_peer.base[p] = (char *)m;
    }
    if (!g_peer.status_host) {
        if (!tt_cuda_ok(cudaHostAlloc((void **)&g_peer.status_host, sizeof(unsigned), cudaHostAllocMapped), "cudaHostAlloc")) return -1;
        *g_peer.status_host = 0;
        if (!tt_cuda_ok(cudaHostGetDevicePointer((void **)&g_peer.status_dev, g_peer.status_host, 0), "cudaHostGetDevicePointer")) return -1;
    }
    g_peer.rank = rank;
    g_peer.slot4 = (long)(pr_slot_floats(g_peer.max_floats, world) / 4);
    g_peer.epoch = 0;
    g_peer.failed = 0;
    const char *e = getenv("TT_PEER_CTAS");
    g_peer.ctas = (e && *e) ? atoi(e) : 64;
    if (g_peer.ctas < 1) g_peer.ctas = 1;
    if (g_peer.ctas > PR_MAX_CTAS) g_peer.ctas = PR_MAX_CTAS;
    g_peer.active = 1;
    return 0;
}

/* Can the peer kernel take this reduction?  (Otherwise the caller uses NCCL.) */
int tt_peer_usable(const float *p, size_t count) {
    return g_peer.active && count > 0 && count <= g_peer.max_floats && (count & 3) == 0 && (((uintptr_t)p) & 15u) == 0;
}

static float *pr_stage_of(int q, unsigned epoch) {
    const size_t padded_floats = (size_t)g_peer.slot4 * 4 * g_peer.world;
    return (float *)(g_peer.base[q] + PR_FLAG_BYTES) + (size_t)(epoch & 1u) * padded_floats;
}

/* The reduction that follows will be launch number epoch + 1 and use staging area (epoch + 1) & 1.
 * Tell a GEMM where to push; the compute stream first waits for the launch that used that area
 * last (two launches ago), so nothing it still reads is overwritten. */
int tt_peer_push_plan(const float *grad, size_t count, PeerPush *out) {
    if (!tt_peer_usable(grad, count) || g_peer.failed) return 0;
    const unsigned next = g_peer.epoch + 1;
    const int buf = (int)(next & 1u);
    if (g_peer.done_valid[buf] && cudaStreamWaitEvent(g_tt.stream, g_peer.done[buf], 0) != cudaSuccess) { cudaGetLastError(); return 0; }
    memset(out, 0, sizeof *out);
    out->world = g_peer.world; out->rank = g_peer.rank;
    out->chunk_floats = pr_chunk4(count, g_peer.world) * 4;
    out->slot_floats = g_peer.slot4 * 4;
    for (int q = 0; q < g_peer.world; q++) out->stage[q] = pr_stage_of(q, next);
    return 1;
}

int tt_peer_allreduce_pushed(float *p, size_t count, size_t pushed_floats, cudaStream_t stream) {
    if (g_peer.failed || tt_peer_poll_status()) {
        tt_set_error("peer all-reduce: a bounded wait ran out earlier in this job; the peer path is shut");
        return -1;
    }
    PeerParams k;
    memset(&k, 0, sizeof k);
    const size_t padded_floats = (size_t)g_peer.slot4 * 4 * g_peer.world;
    k.g = p;
    k.count4 = (long)(count / 4);
    k.chunk4 = pr_chunk4(count, g_peer.world);
    k.slot4 = g_peer.slot4;
    k.rank = g_peer.rank; k.world = g_peer.world;
    k.epoch = ++g_peer.epoch;
    k.push_from4 = (long)(pushed_floats / 4);
    k.status = g_peer.status_dev;
    k.wait_limit = g_peer.wait_limit ? g_peer.wait_limit : PR_WAIT_LIMIT;
    for (int q = 0; q < g_peer.world; q++) {
        k.flags[q] = (unsigned *)g_peer.base[q];
        k.stage[q] = pr_stage_of(q, k.epoch);
        k.result[q] = (float *)(g_peer.base[q] + PR_FLAG_BYTES) + 2 * padded_floats;
    }
    peer_allreduce_kernel<<<g_peer.ctas, PR_THREADS, 0, stream>>>(k);
    g_tt.launches++;
    const int buf = (int)(k.epoch & 1u);
    if (!g_peer.done[buf] && cudaEventCreateWithFlags(&g_peer.done[buf], cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); g_peer.done[buf] = nullptr; }
    if (g_peer.done[buf]) { cudaEventRecord(g_peer.done[buf], stream); g_peer.done_valid[buf] = 1; }
    return tt_cuda_ok(cudaGetLastError(), "peer all-reduce launch") ? 0 : -1;
}

int tt_peer_allreduce(float *p, size_t count, cudaStream_t stream) { return tt_peer_allreduce_pushed(p, count, 0, stream); }

/* Non-zero when a peer kernel gave up on a wait since the last call. */
int tt_peer_poll_status(void) {
    if (!g_peer.status_host) return 0;
    unsigned v = *(volatile unsigned *)g_peer.status_host;
    if (v) {
        g_peer.failed = 1;
        if ((v & 0xf00u) == 0x100u)
            tt_set_error("peer all-reduce: bounded wait expired (phase %u, waiting for rank %u)", (v >> 4) & 0xfu, v & 0xfu);
        else if ((v & 0xf00u) == 0x200u)
            tt_set_error("peer all-reduce: another rank gave up on a wait (seen in phase %u while waiting for rank %u)", (v >> 4) & 0xfu, v & 0xfu);
        else
            tt_set_error("peer all-reduce: launched after a rank of the job had given up on a wait");
        return (int)v;
    }
    return 0;
}

extern "C" int ttb_dist_peer_active(void) { return g_peer.active; }

/* Tear-down is in two halves because CUDA leaves it undefined to free an exported block while
 * another process still has it open: first EVERY rank closes what it imported
 * (ttb_dist_peer_close), then, after a rendezvous of all ranks, each rank frees its own block
 * (ttb_dist_finalize).  tinytorch_b200.dist.finalize() does barrier / close / barrier / finalize. */
extern "C" void ttb_dist_peer_close(void) {
    if (!g_peer.active) return;
    cudaDeviceSynchronize();
    for (int p = 0; p < PR_MAX_WORLD; p++) {
        if (!g_peer.base[p] || p == g_peer.rank) continue;
        cudaIpcCloseMemHandle(g_peer.base[p]);
        g_peer.base[p] = nullptr;
    }
    /* our own block moves to the parking slot the export used; the peer kernel is off from here on */
    char *own = g_peer.base[g_peer.rank];
    g_peer.base[g_peer.rank] = nullptr;
    g_peer.base[0] = own;
    g_peer.active = 0;
}

void tt_peer_finalize(void) {
    if (g_peer.active) ttb_dist_peer_close();
    if (g_peer.base[0]) { cudaDeviceSynchronize(); cudaFree(g_peer.base[0]); g_peer.base[0] = nullptr; }
    g_peer.epoch = 0;
    g_peer.failed = 0;
    for (int b = 0; b < 2; b++) { if (g_peer.done[b]) cudaEventDestroy(g_peer.done[b]); g_peer.done[b] = nullptr; g_peer.done_valid[b] = 0; }
    if (g_peer.status_host) *g_peer.status_host = 0;
}
