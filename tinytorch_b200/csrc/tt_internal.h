/* Private declarations shared by the translation units of libtinytorch.so. */
#ifndef TT_INTERNAL_H
#define TT_INTERNAL_H

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "tensor.h"
#include "autograd.h"
#include "tt_b200.h"

/* ---- tensor record --------------------------------------------------------
 * The public struct comes first, so a Tensor* is also a TTensor*. */
/* TT_LAZY_PADONES: [M,K] -> [M,K+1] with a ones column, from lazy_src.
 * TT_LAZY_MATMUL:  lazy_src * lazy_src2 (lazy_pad: lazy_src carries a virtual ones column, so the
 *                  last row of lazy_src2 is added to every row), not launched yet: the builder that
 *                  consumes it may fuse its own step into the product's epilogue instead. */
enum { TT_LAZY_NONE = 0, TT_LAZY_PADONES = 1, TT_LAZY_MATMUL = 2 };

typedef struct TTensor {
    Tensor  pub;
    float  *dev;           /* device payload, numel floats */
    uint8_t dev_valid;     /* device payload is current */
    uint8_t host_valid;    /* host mirror (pub.data) is current */
    uint8_t host_exposed;  /* tt_data() handed the mirror out since the last upload */
    uint8_t lazy_kind;     /* payload not produced yet: TT_LAZY_* */
    struct TTensor *lazy_src;   /* retained source of a deferred payload */
    struct TTensor *lazy_src2;  /* second retained source (TT_LAZY_MATMUL: the right-hand operand) */
    uint8_t lazy_pad;           /* TT_LAZY_MATMUL: lazy_src has a virtual ones column */
    cudaEvent_t ready;     /* upload on the copy stream that the next device use must wait for */
    uint8_t ready_pending;
    cudaEvent_t busy;      /* last use on another stream (download, all-reduce, fused update): release waits for it */
    uint8_t busy_pending;
} TTensor;

static inline TTensor *TT(const Tensor *t) { return (TTensor *)t; }

/* ---- context --------------------------------------------------------------*/
typedef struct TTContext {
    int          ready;        /* 1 after a successful init, -1 after a failed one */
    int          device;
    int          sm_count;
    int          gemm_sms;     /* CTAs a persistent GEMM may occupy: all SMs, fewer while NCCL kernels share the GPU */
    cudaStream_t stream;       /* all compute */
    cudaStream_t comm_stream;  /* NCCL all-reduce */
    cudaStream_t copy_stream;  /* asynchronous input uploads */
    int          gemm_path;    /* 0 auto, 1 tensor core, 2 exact fp32 */
    int          fuse_padones; /* fold padones into the adjoining GEMM */
    int          fuse_relu;    /* fold relu and its gradient mask into the adjoining GEMMs' epilogues */
    int          conv_implicit; /* convolutions as implicit GEMMs (no im2col matrix) where the shape allows */
    int          grad_enabled; /* 0: builders record no graph (forward-only / evaluation batches) */
    int          trace;
    long         launches;
    long         gemm_pushed_floats;  /* set by tt_gemm: leading floats of C whose foreign chunks went to their owners */
} TTContext;

extern TTContext g_tt;

int   tt_ctx_init(void);                       /* 0 ok, -1 failed (message stored) */
void  tt_set_error(const char *fmt, ...);
int   tt_cuda_ok(cudaError_t e, const char *what);   /* 1 ok, 0 failed (message stored) */
void *tt_dev_alloc(size_t bytes);              /* stream-ordered, NULL on failure */
void  tt_dev_free(void *p);

/* Tensor helpers (tensor.cu). */
Tensor *tt_new_uninit(const long *shape, int ndim);    /* device payload left unwritten */
Tensor *tt_new_like(const Tensor *a, int zero);
float  *tt_dev_ro(const Tensor *t);            /* device pointer for reading (uploads / materialises) */
float  *tt_dev_rw(Tensor *t);                  /* device pointer for writing; mirror becomes stale */
Tensor *tt_new_lazy_padones(Tensor *src);      /* [M,K] -> [M,K+1], produced on first use */
Tensor *tt_new_lazy_matmul(Tensor *x, Tensor *w, int pad);   /* x[M,K] (pad: virtual ones column) times w, produced on first use */
int     tt_is_deferred_matmul(const Tensor *t);   /* a TT_LAZY_MATMUL tensor whose product has not been launched */
/* The deferred product of `t` with a relu fused into its epilogue, as a new tensor; t stays deferred. */
Tensor *tt_deferred_matmul_relu(const Tensor *t);
/* The payload is being read or written on `s` (not the compute stream): its block must not be
 * handed to another allocation before that work has finished.  tt_release orders the free after it. */
void    tt_mark_busy(Tensor *t, cudaStream_t s);

/* Tracing (context.cu): bracket a launch of class `kind`. */
void tt_trace_begin(int kind);
void tt_trace_end(int kind, double work);

/* ---- kernel launchers (all on g_tt.stream) -------------------------------- */
/* kernels_elementwise.cu */
void k_fill(float *p, long n, float v);
void k_copy(float *dst, const float *src, long n);
void k_add(float *o, const float *a, const float *b, long n);
void k_mul(float *o, const float *a, const float *b, long n);
void k_addscalar(float *o, const float *a, float s, long n);
void k_mulscalar(float *o, const float *a, float s, long n);
void k_accum(float *dst, const float *src, long n);            /* dst += src */
void k_relu(float *o, const float *x, long n);
void k_relu_bwd(float *dx, const float *x, const float *g, long n, int accumulate);
void k_padones(float *o, const float *x, int M, int K);
void k_slice_cols(float *o, const float *g, int M, int K, int ldg, int accumulate);
void k_softmax(float *o, const float *x, long rows, int N);
void k_softmax_bwd(float *dx, const float *s, const float *g, long rows, int N);
void k_softmax_xent(const float *logits, const float *labels, long rows, int N,
                    float scale, float *dlogits, float *row_loss);
void k_mean(const float *x, long n, float *out);               /* out[0] = sum(x)/n */
int  k_colsum(const float *g, int M, int N, int ldg, float *out, int accumulate);   /* 0, or -1 when its scratch cannot be had */
void k_sgd(float *w, const float *g, float lr, long n);
void k_sgd_momentum(float *w, float *v, const float *g, float lr, float mu, long n);
void k_adam(float *w, float *m, float *v, const float *g, float lr_t, float b1,
            float b2, float omb1, float omb2, float eps, long n);
void k_transpose(float *o, const float *x, int R, int C);      /* o[C,R] = x[R,C]^T */

/* kernels_spatial.cu */
void k_im2col(const float *x, int N, int C, int H, int W, int HH, int WW,
              int ph, int pw, int sh, int sw, int Ho, int Wo, float *col);
void k_col2im(const float *col, int N, int C, int H, int W, int HH, int WW,
              int ph, int pw, int sh, int sw, int Ho, int Wo, float *x);
void k_conv_unpermute_bias(const float *om, const float *bias, int N, int F, long sp, float *out);
void k_conv_permute(const float *g, int N, int F, long sp, float *gp);
void k_conv_bias_grad(const float *g, int N, int F, long sp, float *db);
void k_maxpool(const float *x, long NC, int H, int W, int ph, int pw, int sh, int sw,
               int Ho, int Wo, float *out);
void k_maxpool_bwd(const float *x, const float *g, long NC, int H, int W, int ph, int pw,
                   int sh, int sw, int Ho, int Wo, float *dx);
void k_maxpool_argmax(const float *x, long NC, int H, int W, int ph, int pw, int sh, int sw,
                      int Ho, int Wo, long long *idx);
void k_avgpool(const float *x, long NC, int H, int W, int ph, int pw, int sh, int sw,
               int Ho, int Wo, float *out);
void k_avgpool_bwd(const float *g, long NC, int H, int W, int ph, int pw, int sh, int sw,
                   int Ho, int Wo, float *dx);

/* ---- GEMM -----------------------------------------------------------------
 * C[M,N] (+)= op(A) * op(B) (+ bias[n]) with row-major storage everywhere:
 *   ta == 0: A is [M,K] with row pitch lda;  ta == 1: A is stored [K,M]
 *   tb == 0: B is [K,N] with row pitch ldb;  tb == 1: B is stored [N,K]
 * accumulate != 0 adds into C.  bias (may be NULL) is one value per column.
 * Returns 0, or -1 with the reason stored. */
/* Where the epilogue of a weight-gradient product sends what other ranks own (peer_reduce.cu): the
 * gradient, seen as one flat array, is cut into `world` chunks of chunk_floats; the part of chunk c
 * computed here goes straight into slot `rank` of rank c's staging area (plain peer stores) instead
 * of local memory, so the reduce-scatter's transfer happens inside the GEMM. */
typedef struct PeerPush {
    float *stage[8];         /* staging area of every rank as mapped in this process */
    int world, rank;
    long chunk_floats, slot_floats;
} PeerPush;

typedef struct GemmArgs {
    int ta, tb;
    int M, N, K;
    const float *A; long lda;
    const float *B; long ldb;
    float *C; long ldc;
    const float *bias;
    int accumulate;
    /* A carries a virtual last column of ones (ta == 0: logical K = stored
     * columns + 1) or a virtual last row (ta == 1: logical M = stored rows of
     * A^T + 1): a padones node consumed without materialising it. */
    int a_pad_ones;
    /* Which reference loop the exact-fp32 path reproduces bit for bit:
     * 0 forward sgemm, 1 backward dot/axpy products, 2 naive tt_matmul. */
    int rule;
    /* Fused elementwise steps of the epilogue, applied to the finished product (bias included)
     * BEFORE it is stored or added into C:
     *   relu  v = v > 0 ? v : 0                      (tt_relu, src/ops.c:104-106)
     *   mask  v = mask[m * ldmask + n] > 0 ? v : 0   (backward_relu, src/autograd.c:318-327, with
     *         the relu's OUTPUT as the mask: y > 0 exactly when x > 0, NaN included) */
    int relu;
    const float *mask; long ldmask;
    /* Optional: push the parts of C that other ranks own to them (see PeerPush).  Honoured by the
     * tensor-core kernel for a plain product into a contiguous C (ldc == N, N a multiple of 32);
     * g_tt.gemm_pushed_floats tells the caller how many leading floats of C were handled that way. */
    const PeerPush *push;
} GemmArgs;

int tt_gemm(const GemmArgs *g);                 /* dispatch by g_tt.gemm_path */
int gemm_simt(const GemmArgs *g);               /* gemm_simt.cu: exact fp32, k ascending */
int gemm_tc(const GemmArgs *g);                 /* gemm_tc.cu: tcgen05 3xTF32 */
int gemm_tc_usable(const GemmArgs *g);          /* alignment rules of the TMA path */
int gemm_tc_poll_status(void);                  /* non-zero (reason stored) when a kernel gave up on a bounded wait */

/* ---- implicit-GEMM convolution (conv_tc.cu) -----------------------------------
 * x [N,C,H,W], filters [F,C,HH,WW], strides (sh,sw), zero padding (ph,pw), output [N,F,Ho,Wo]. */
typedef struct ConvGeom { int N, C, H, W, F, HH, WW, sh, sw, ph, pw, Ho, Wo; } ConvGeom;
int conv_tc_usable(const ConvGeom *g, int need_dgrad);      /* 1 when the gathered tensor-core kernel takes this shape */
int conv_tc_fprop(const ConvGeom *g, const float *x, const float *w, const float *bias, float *out);
int conv_tc_dgrad(const ConvGeom *g, const float *grad_out, const float *w, float *dx, int accumulate);
int conv_tc_wgrad(const ConvGeom *g, const float *x, const float *grad_out, float *dw, int accumulate);
int conv_tc_poll_status(void);

/* dist.cu: called by the backward pass when a marked leaf's gradient is final. */
int tt_dist_active(void);
int tt_dist_allreduce_async(Tensor *t);
int tt_dist_allreduce_range(float *p, size_t count);     /* same, for a contiguous part of a gradient */
int tt_dist_allreduce_tail(float *p, size_t count);      /* same, when nothing is left to overlap it with */
/* peer-memory all-reduce (peer_reduce.cu) */
int tt_peer_usable(const float *p, size_t count);
int tt_peer_allreduce(float *p, size_t count, cudaStream_t stream);
int tt_peer_poll_status(void);
void tt_peer_finalize(void);
/* Fused reduce-scatter: plan the push of the next reduction (1 when the gradient qualifies), and run
 * that reduction for a gradient whose first pushed_floats values were pushed by the GEMM. */
int tt_peer_push_plan(const float *grad, size_t count, PeerPush *out);
int tt_peer_allreduce_pushed(float *p, size_t count, size_t pushed_floats, cudaStream_t stream);
int tt_dist_allreduce_pushed(float *p, size_t count, size_t pushed_floats);
/* dist.cu: per-collective timing while tracing is on */
void tt_dist_trace_reset(void);

#endif
