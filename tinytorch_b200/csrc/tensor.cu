/* Tensor storage: the payload lives in HBM, the public record's `data` is a
 * lazily synchronised host mirror.
 *
 * Mirrors the contract of the reference's src/tensor.c (shape validation and
 * overflow guard :10-18, zero fill :21, contiguous strides :29-32, refcount
 * :48-61, accessors :63-75) with device memory in place of calloc. */
#include "tt_internal.h"

#include <limits.h>
#include <stdlib.h>
#include <string.h>

#define TT_MAX_NUMEL (1L << 40)    /* same cap as the reference (src/tensor.c:8) */

/* Shape check shared by every constructor.  Returns numel, or -1. */
static long checked_numel(const long *shape, int ndim) {
    if (!shape || ndim <= 0 || ndim > 8) return -1;
    long n = 1;
    for (int i = 0; i < ndim; i++) {
        if (shape[i] <= 0) return -1;
        if (n > LONG_MAX / shape[i]) return -1;
        n *= shape[i];
    }
    if (n > TT_MAX_NUMEL) return -1;
    return n;
}

static TTensor *record_new(const long *shape, int ndim, long numel) {
    TTensor *t = (TTensor *)calloc(1, sizeof(TTensor));
    if (!t) return nullptr;
    t->pub.shape = (long *)malloc(sizeof(long) * (size_t)ndim);
    t->pub.strides = (long *)malloc(sizeof(long) * (size_t)ndim);
    if (!t->pub.shape || !t->pub.strides) {
        free(t->pub.shape); free(t->pub.strides); free(t);
        return nullptr;
    }
    for (int i = 0; i < ndim; i++) t->pub.shape[i] = shape[i];
    t->pub.strides[ndim - 1] = 1;
    for (int i = ndim - 2; i >= 0; i--)
        t->pub.strides[i] = t->pub.strides[i + 1] * shape[i + 1];
    t->pub.ndim = ndim;
    t->pub.numel = numel;
    t->pub.refcount = 1;
    return t;
}

static void record_free(TTensor *t) {
    free(t->pub.data);
    free(t->pub.shape);
    free(t->pub.strides);
    free(t);
}

Tensor *tt_new_uninit(const long *shape, int ndim) {
    long numel = checked_numel(shape, ndim);
    if (numel < 0) return nullptr;
    TTensor *t = record_new(shape, ndim, numel);
    if (!t) return nullptr;
    t->dev = (float *)tt_dev_alloc(sizeof(float) * (size_t)numel);
    if (!t->dev) { record_free(t); return nullptr; }
    t->dev_valid = 1;
    return &t->pub;
}

extern "C" Tensor *tt_new(const long *shape, int ndim) {
    Tensor *t = tt_new_uninit(shape, ndim);
    if (!t) return nullptr;
    if (!tt_cuda_ok(cudaMemsetAsync(TT(t)->dev, 0, sizeof(float) * (size_t)t->numel, g_tt.stream),
                    "cudaMemsetAsync")) {
        tt_release(t);
        return nullptr;
    }
    return t;
}

Tensor *tt_new_like(const Tensor *a, int zero) {
    return zero ? tt_new(a->shape, a->ndim) : tt_new_uninit(a->shape, a->ndim);
}

extern "C" Tensor *tt_fromdata(const float *data, const long *shape, int ndim) {
    /* The shape is judged before `data` is looked at: a hostile shape with a
     * NULL pointer must fail here (reference: tests/test_ops.py:330-332). */
    long numel = checked_numel(shape, ndim);
    if (numel < 0 || !data) return nullptr;
    Tensor *t = tt_new_uninit(shape, ndim);
    if (!t) return nullptr;
    /* From pageable memory this returns once the source has been staged, so
     * the caller may reuse `data` at once; from pinned memory it is a true
     * asynchronous copy and the caller keeps the buffer alive until the next
     * synchronising call, as with any CUDA stream. */
    if (!tt_cuda_ok(cudaMemcpyAsync(TT(t)->dev, data, sizeof(float) * (size_t)numel,
                                    cudaMemcpyHostToDevice, g_tt.stream), "cudaMemcpyAsync(H2D)")) {
        tt_release(t);
        return nullptr;
    }
    return t;
}

Tensor *tt_new_lazy_padones(Tensor *src) {
    if (!src || src->ndim != 2) return nullptr;
    long shp[2] = {src->shape[0], src->shape[1] + 1};
    long numel = checked_numel(shp, 2);
    if (numel < 0) return nullptr;
    TTensor *t = record_new(shp, 2, numel);
    if (!t) return nullptr;
    t->lazy_kind = TT_LAZY_PADONES;
    t->lazy_src = TT(tt_retain(src));
    return &t->pub;
}

/* A product that is not launched yet (see TT_LAZY_MATMUL).  Shapes are the caller's business. */
Tensor *tt_new_lazy_matmul(Tensor *x, Tensor *w, int pad) {
    if (!x || !w || x->ndim != 2 || w->ndim != 2) return nullptr;
    long shp[2] = {x->shape[0], w->shape[1]};
    long numel = checked_numel(shp, 2);
    if (numel < 0) return nullptr;
    TTensor *t = record_new(shp, 2, numel);
    if (!t) return nullptr;
    t->lazy_kind = TT_LAZY_MATMUL;
    t->lazy_pad = pad ? 1 : 0;
    t->lazy_src = TT(tt_retain(x));
    t->lazy_src2 = TT(tt_retain(w));
    return &t->pub;
}

int tt_is_deferred_matmul(const Tensor *t) { return t && TT(t)->lazy_kind == TT_LAZY_MATMUL; }

/* Launch the product of a TT_LAZY_MATMUL tensor into dst[M,N]. */
static int run_deferred_matmul(const TTensor *t, float *dst, int relu) {
    const Tensor *x = &t->lazy_src->pub, *w = &t->lazy_src2->pub;
    const float *px = tt_dev_ro(x), *pw = tt_dev_ro(w);
    if (!px || !pw) return -1;
    GemmArgs g;
    memset(&g, 0, sizeof g);
    g.M = (int)t->pub.shape[0]; g.N = (int)t->pub.shape[1]; g.K = (int)w->shape[0];
    g.A = px; g.lda = x->shape[1]; g.a_pad_ones = t->lazy_pad;
    g.B = pw; g.ldb = g.N; g.C = dst; g.ldc = g.N;
    g.relu = relu;
    return tt_gemm(&g);
}

Tensor *tt_deferred_matmul_relu(const Tensor *ct) {
    const TTensor *t = TT(ct);
    if (!t || t->lazy_kind != TT_LAZY_MATMUL) return nullptr;
    Tensor *out = tt_new_uninit(t->pub.shape, 2);
    if (!out) return nullptr;
    if (run_deferred_matmul(t, TT(out)->dev, 1) != 0) { tt_release(out); return nullptr; }
    return out;
}

extern "C" Tensor *tt_retain(Tensor *t) {
    if (!t) return nullptr;
    t->refcount++;
    return t;
}

extern "C" void tt_release(Tensor *t) {
    if (!t) return;
    if (--t->refcount > 0) return;
    TTensor *x = TT(t);
    if (x->ready) {
        if (x->ready_pending && g_tt.ready == 1) cudaStreamWaitEvent(g_tt.stream, x->ready, 0);   /* the free is stream-ordered */
        cudaEventDestroy(x->ready);
    }
    if (x->busy) {
        /* a download, reduction or fused update on another stream may still be using the block:
         * whoever gets it next (the free is ordered on the compute stream) comes after that work */
        if (x->busy_pending && g_tt.ready == 1) cudaStreamWaitEvent(g_tt.stream, x->busy, 0);
        cudaEventDestroy(x->busy);
    }
    if (x->dev) tt_dev_free(x->dev);
    if (x->lazy_src) tt_release(&x->lazy_src->pub);
    if (x->lazy_src2) tt_release(&x->lazy_src2->pub);
    record_free(x);
}

void tt_mark_busy(Tensor *ct, cudaStream_t s) {
    TTensor *t = TT(ct);
    if (!t || g_tt.ready != 1) return;
    if (!t->busy && cudaEventCreateWithFlags(&t->busy, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        t->busy = nullptr;
        cudaStreamSynchronize(s);            /* no event to be had: fall back to waiting here */
        return;
    }
    if (cudaEventRecord(t->busy, s) == cudaSuccess) t->busy_pending = 1;
}

/* Produce a deferred payload. */
static int materialise(TTensor *t) {
    if (t->lazy_kind == TT_LAZY_NONE) return 1;
    float *dev = (float *)tt_dev_alloc(sizeof(float) * (size_t)t->pub.numel);
    if (!dev) return 0;
    if (t->lazy_kind == TT_LAZY_PADONES) {
        const float *src = tt_dev_ro(&t->lazy_src->pub);
        if (!src) { tt_dev_free(dev); return 0; }     /* stays deferred; nothing is kept */
        k_padones(dev, src, (int)t->lazy_src->pub.shape[0], (int)t->lazy_src->pub.shape[1]);
    } else if (t->lazy_kind == TT_LAZY_MATMUL) {
        if (run_deferred_matmul(t, dev, 0) != 0) { tt_dev_free(dev); return 0; }
        tt_release(&t->lazy_src2->pub);
        t->lazy_src2 = nullptr;
    }
    t->dev = dev;
    tt_release(&t->lazy_src->pub);
    t->lazy_src = nullptr;
    t->lazy_kind = TT_LAZY_NONE;
    t->dev_valid = 1;
    return 1;
}

/* An upload queued by ttb_upload_async must land before anything else touches the payload. */
static int await_upload(TTensor *t) {
    if (!t->ready_pending) return 1;
    if (!tt_cuda_ok(cudaStreamWaitEvent(g_tt.stream, t->ready, 0), "cudaStreamWaitEvent(upload)")) return 0;
    t->ready_pending = 0;
    return 1;
}

float *tt_dev_ro(const Tensor *ct) {
    TTensor *t = TT(ct);
    if (!t) return nullptr;
    if (!materialise(t)) return nullptr;
    if (!await_upload(t)) return nullptr;
    if (t->host_exposed) {
        /* The caller holds the mirror and may have written to it. */
        if (!tt_cuda_ok(cudaMemcpyAsync(t->dev, t->pub.data, sizeof(float) * (size_t)t->pub.numel,
                                        cudaMemcpyHostToDevice, g_tt.stream), "cudaMemcpyAsync(H2D)"))
            return nullptr;
        t->host_exposed = 0;
        t->dev_valid = 1;
    }
    return t->dev;
}

float *tt_dev_rw(Tensor *ct) {
    float *p = tt_dev_ro(ct);
    if (p) TT(ct)->host_valid = 0;
    return p;
}

extern "C" float *ttb_device_ptr(Tensor *t) { return t ? tt_dev_ro(t) : nullptr; }

/* Input pipeline: copy host data into an EXISTING tensor on the copy stream, so that the
 * transfer of the next batch runs under the kernels of the current one.  The copy is ordered
 * after all compute work enqueued so far (which may still read the old contents); the
 * tensor's next use on the compute stream waits for it. */
extern "C" int ttb_upload_async(Tensor *dst, const float *src) {
    TTensor *t = TT(dst);
    if (!t || !src) { tt_set_error("ttb_upload_async: NULL argument"); return -1; }
    if (!materialise(t) || !await_upload(t)) return -1;
    static cudaEvent_t fence = nullptr;
    if (!fence && !tt_cuda_ok(cudaEventCreateWithFlags(&fence, cudaEventDisableTiming), "cudaEventCreate")) return -1;
    if (!t->ready && !tt_cuda_ok(cudaEventCreateWithFlags(&t->ready, cudaEventDisableTiming), "cudaEventCreate")) return -1;
    if (!tt_cuda_ok(cudaEventRecord(fence, g_tt.stream), "cudaEventRecord") ||
        !tt_cuda_ok(cudaStreamWaitEvent(g_tt.copy_stream, fence, 0), "cudaStreamWaitEvent") ||
        !tt_cuda_ok(cudaMemcpyAsync(t->dev, src, sizeof(float) * (size_t)t->pub.numel, cudaMemcpyHostToDevice,
                                    g_tt.copy_stream), "cudaMemcpyAsync(H2D)") ||
        !tt_cuda_ok(cudaEventRecord(t->ready, g_tt.copy_stream), "cudaEventRecord"))
        return -1;
    t->ready_pending = 1;
    t->dev_valid = 1; t->host_valid = 0; t->host_exposed = 0;
    return 0;
}

/* Output side of the pipeline: copy a tensor's payload into caller memory (pinned, for a copy that is
 * really asynchronous) on the copy stream, ordered after the compute work enqueued so far -- so the host
 * can enqueue the next step before it looks at this one's result.  ttb_download_wait blocks until every
 * such copy has landed (and reports a tensor-core kernel that gave up meanwhile). */
extern "C" int ttb_download_async(const Tensor *src, float *dst) {
    TTensor *t = TT(src);
    if (!t || !dst) { tt_set_error("ttb_download_async: NULL argument"); return -1; }
    const float *p = tt_dev_ro(src);
    if (!p) return -1;
    static cudaEvent_t fence = nullptr;
    if (!fence && !tt_cuda_ok(cudaEventCreateWithFlags(&fence, cudaEventDisableTiming), "cudaEventCreate")) return -1;
    if (!tt_cuda_ok(cudaEventRecord(fence, g_tt.stream), "cudaEventRecord") ||
        !tt_cuda_ok(cudaStreamWaitEvent(g_tt.copy_stream, fence, 0), "cudaStreamWaitEvent") ||
        !tt_cuda_ok(cudaMemcpyAsync(dst, p, sizeof(float) * (size_t)t->pub.numel, cudaMemcpyDeviceToHost,
                                    g_tt.copy_stream), "cudaMemcpyAsync(D2H)"))
        return -1;
    tt_mark_busy(&t->pub, g_tt.copy_stream);      /* src may be released before ttb_download_wait */
    return 0;
}
extern "C" int ttb_download_wait(void) {
    if (tt_ctx_init() != 0) return -1;
    if (!tt_cuda_ok(cudaStreamSynchronize(g_tt.copy_stream), "cudaStreamSynchronize(copy)")) return -1;
    return gemm_tc_poll_status() ? -1 : 0;
}

extern "C" float *tt_data(const Tensor *ct) {
    TTensor *t = TT(ct);
    if (!t) return nullptr;
    if (!materialise(t)) return nullptr;
    if (!await_upload(t)) return nullptr;
    size_t bytes = sizeof(float) * (size_t)t->pub.numel;
    if (!t->pub.data) {
        t->pub.data = (float *)malloc(bytes);
        if (!t->pub.data) return nullptr;
        t->host_valid = 0;
    }
    if (!t->host_valid && !t->host_exposed) {
        if (!tt_cuda_ok(cudaMemcpyAsync(t->pub.data, t->dev, bytes, cudaMemcpyDeviceToHost, g_tt.stream),
                        "cudaMemcpyAsync(D2H)"))
            return nullptr;
        if (!tt_cuda_ok(cudaStreamSynchronize(g_tt.stream), "cudaStreamSynchronize"))
            return nullptr;
        if (gemm_tc_poll_status()) return nullptr;     /* a kernel upstream gave up: the numbers are not to be trusted */
        t->host_valid = 1;
    }
    t->host_exposed = 1;
    return t->pub.data;
}

extern "C" long tt_numel(const Tensor *t) { return t ? t->numel : 0; }
extern "C" int  tt_ndim(const Tensor *t) { return t ? t->ndim : 0; }

extern "C" void tt_shape(const Tensor *t, long *out) {
    if (!t || !out) return;
    for (int i = 0; i < t->ndim; i++) out[i] = t->shape[i];
}

extern "C" void tt_strides(const Tensor *t, long *out) {
    if (!t || !out) return;
    for (int i = 0; i < t->ndim; i++) out[i] = t->strides[i];
}
