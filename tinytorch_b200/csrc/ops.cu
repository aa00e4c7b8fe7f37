/* Tensor operators of the C ABI: validation and shape logic on the host,
 * arithmetic in the CUDA kernels.  Every entry point keeps the reference's
 * contract (fresh output, NULL on any invalid argument); the reference
 * function each one stands in for is named at its definition. */
#include "tt_internal.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

static int same_shape(const Tensor *a, const Tensor *b) {
    if (a->ndim != b->ndim) return 0;
    for (int i = 0; i < a->ndim; i++)
        if (a->shape[i] != b->shape[i]) return 0;
    return 1;
}

/* ---- GEMM dispatch ---------------------------------------------------------
 * Tensor-core kernel for shapes large enough to fill a 128-row tile and whose
 * operands TMA can address; exact-fp32 kernel otherwise.  A virtual ones
 * column on A is native to the exact kernel; for the tensor-core kernel it is
 * peeled off: as a bias row in the epilogue (forward), or as a column sum
 * written to the last row of C (weight gradient). */
static int tc_wanted(const GemmArgs *g) {
    if (g_tt.gemm_path == 2) return 0;
    if (g_tt.gemm_path == 1) return 1;
    return g->M >= 16 && g->N >= 8 && g->K >= 8 && (long)g->M * g->N * g->K >= (1l << 21);
}

/* TMA needs 16-byte aligned rows.  A small operand whose pitch is not a multiple of four
 * floats (a [32,27] convolution filter bank, a [K,10] classifier weight) is copied into
 * pool scratch with a padded pitch; large ones are left to the exact kernel. */
static const float *repitched(const float *src, long rows, long cols, long *pitch, float **scratch) {
    *scratch = nullptr;
    if ((*pitch & 3) == 0 && ((((uintptr_t)src) & 15u) == 0)) return src;
    if (rows * cols > (4l << 20)) return nullptr;
    long np = (cols + 3) & ~3l;
    float *buf = (float *)tt_dev_alloc(sizeof(float) * (size_t)rows * np);
    if (!buf) return nullptr;
    if (cudaMemcpy2DAsync(buf, np * sizeof(float), src, *pitch * sizeof(float), cols * sizeof(float), rows,
                          cudaMemcpyDeviceToDevice, g_tt.stream) != cudaSuccess) {
        cudaGetLastError();
        tt_dev_free(buf);
        return nullptr;
    }
    *scratch = buf; *pitch = np;
    return buf;
}

int tt_gemm(const GemmArgs *g) {
    g_tt.gemm_pushed_floats = 0;
    if (g->M <= 0 || g->N <= 0 || g->K <= 0) { tt_set_error("gemm: empty shape"); return -1; }
    GemmArgs core = *g;
    if (g->a_pad_ones) {
        if (!g->ta) core.K = g->K - 1; else core.M = g->M - 1;
        core.a_pad_ones = 0;
    }
    float *sa = nullptr, *sb = nullptr;
    int use_tc = core.M > 0 && core.K > 0 && tc_wanted(&core);
    if (use_tc && !gemm_tc_usable(&core) && g_tt.gemm_path != 1) {
        const float *a = repitched(core.A, core.ta ? core.K : core.M, core.ta ? core.M : core.K, &core.lda, &sa);
        const float *b = a ? repitched(core.B, core.tb ? core.N : core.K, core.tb ? core.K : core.N, &core.ldb, &sb) : nullptr;
        if (a && b) { core.A = a; core.B = b; }
    }
    use_tc = use_tc && gemm_tc_usable(&core);
    struct Cleanup { float *a, *b; ~Cleanup() { if (a) tt_dev_free(a); if (b) tt_dev_free(b); } } cleanup = {sa, sb};
    if (g_tt.gemm_path == 1 && !use_tc) {
        tt_set_error("gemm: tensor-core path forced but the shape cannot be fed by TMA");
        return -1;
    }
    if (!use_tc) return gemm_simt(g);
    if (g->a_pad_ones && !g->ta) {
        if (g->tb) return gemm_simt(g);                 /* bias row must be a row of B */
        core.bias = g->B + (long)core.K * g->ldb;        /* the ones column times the last row of B (always the caller's B) */
        return gemm_tc(&core);
    }
    if (g->a_pad_ones && g->ta) {
        if (g->tb) return gemm_simt(g);
        if (gemm_tc(&core) != 0) return -1;
        /* last row of A^T is all ones: that row of C is the column sum of B */
        return k_colsum(g->B, g->K, g->N, (int)g->ldb, g->C + (long)core.M * g->ldc, g->accumulate);
    }
    return gemm_tc(&core);
}

extern "C" void ttb_set_gemm_path(int path) {
    if (path >= 0 && path <= 2) g_tt.gemm_path = path;
}

/* ---- elementwise (src/ops.c:26-82,104-106) ---------------------------------*/
typedef void (*BinK)(float *, const float *, const float *, long);

static Tensor *binary_op(const Tensor *a, const Tensor *b, BinK k) {
    if (!a || !b || !same_shape(a, b)) return nullptr;
    const float *pa = tt_dev_ro(a), *pb = tt_dev_ro(b);
    if (!pa || !pb) return nullptr;
    Tensor *out = tt_new_like(a, 0);
    if (!out) return nullptr;
    k(TT(out)->dev, pa, pb, a->numel);
    return out;
}
extern "C" Tensor *tt_add(const Tensor *a, const Tensor *b) { return binary_op(a, b, k_add); }
extern "C" Tensor *tt_mul(const Tensor *a, const Tensor *b) { return binary_op(a, b, k_mul); }

extern "C" Tensor *tt_addscalar(const Tensor *a, float s) {
    if (!a) return nullptr;
    const float *pa = tt_dev_ro(a);
    if (!pa) return nullptr;
    Tensor *out = tt_new_like(a, 0);
    if (!out) return nullptr;
    k_addscalar(TT(out)->dev, pa, s, a->numel);
    return out;
}
extern "C" Tensor *tt_mulscalar(const Tensor *a, float s) {
    if (!a) return nullptr;
    const float *pa = tt_dev_ro(a);
    if (!pa) return nullptr;
    Tensor *out = tt_new_like(a, 0);
    if (!out) return nullptr;
    k_mulscalar(TT(out)->dev, pa, s, a->numel);
    return out;
}
extern "C" Tensor *tt_relu(const Tensor *a) {
    if (!a) return nullptr;
    const float *pa = tt_dev_ro(a);
    if (!pa) return nullptr;
    Tensor *out = tt_new_like(a, 0);
    if (!out) return nullptr;
    k_relu(TT(out)->dev, pa, a->numel);
    return out;
}
extern "C" Tensor *ttb_relu_bwd(const Tensor *x, const Tensor *g) {
    if (!x || !g || x->numel != g->numel) return nullptr;
    const float *px = tt_dev_ro(x), *pg = tt_dev_ro(g);
    if (!px || !pg) return nullptr;
    Tensor *out = tt_new_like(x, 0);
    if (!out) return nullptr;
    k_relu_bwd(TT(out)->dev, px, pg, x->numel, 0);
    return out;
}

extern "C" Tensor *ttb_colsum(const Tensor *g) {
    if (!g || g->ndim != 2 || g->shape[0] > 0x7fffffffL || g->shape[1] > 0x7fffffffL) return nullptr;
    const float *pg = tt_dev_ro(g);
    if (!pg) return nullptr;
    long shp[1] = {g->shape[1]};
    Tensor *out = tt_new_uninit(shp, 1);
    if (!out) return nullptr;
    if (k_colsum(pg, (int)g->shape[0], (int)g->shape[1], (int)g->shape[1], TT(out)->dev, 0) != 0) {
        tt_release(out);
        return nullptr;
    }
    return out;
}

/* ---- softmax (src/ops.c:108-145, src/autograd.c:329-346) -------------------*/
extern "C" Tensor *tt_softmax(const Tensor *a) {
    if (!a || a->ndim < 1) return nullptr;
    const float *pa = tt_dev_ro(a);
    if (!pa) return nullptr;
    Tensor *out = tt_new_like(a, 0);
    if (!out) return nullptr;
    int N = (int)a->shape[a->ndim - 1];
    k_softmax(TT(out)->dev, pa, a->numel / N, N);
    return out;
}
extern "C" Tensor *ttb_softmax_bwd(const Tensor *s, const Tensor *g) {
    if (!s || !g || s->ndim < 1 || !same_shape(s, g)) return nullptr;
    const float *ps = tt_dev_ro(s), *pg = tt_dev_ro(g);
    if (!ps || !pg) return nullptr;
    Tensor *out = tt_new_like(s, 0);
    if (!out) return nullptr;
    int N = (int)s->shape[s->ndim - 1];
    k_softmax_bwd(TT(out)->dev, ps, pg, s->numel / N, N);
    return out;
}
extern "C" Tensor *ttb_softmax_xent(const Tensor *logits, const Tensor *labels, float scale, Tensor **dlogits) {
    if (!logits || !labels || !dlogits || logits->ndim != 2) return nullptr;
    long rows = logits->shape[0];
    int N = (int)logits->shape[1];
    if (labels->numel != rows) return nullptr;
    const float *pz = tt_dev_ro(logits), *py = tt_dev_ro(labels);
    if (!pz || !py) return nullptr;
    Tensor *dz = tt_new_like(logits, 0);
    long one = 1;
    Tensor *loss = tt_new_uninit(&one, 1);
    float *row_loss = (float *)tt_dev_alloc(sizeof(float) * (size_t)rows);
    if (!dz || !loss || !row_loss) {
        tt_release(dz); tt_release(loss); tt_dev_free(row_loss);
        return nullptr;
    }
    k_softmax_xent(pz, py, rows, N, scale, TT(dz)->dev, row_loss);
    k_mean(row_loss, rows, TT(loss)->dev);
    tt_dev_free(row_loss);
    *dlogits = dz;
    return loss;
}

/* ---- matmul (src/ops.c:84-102, src/gemm.c:644-671) -------------------------*/
static Tensor *matmul_rule(const Tensor *a, const Tensor *b, int rule) {
    if (!a || !b || a->ndim != 2 || b->ndim != 2) return nullptr;
    if (a->shape[1] != b->shape[0]) return nullptr;
    if (a->shape[0] > 0x7fffffffL || a->shape[1] > 0x7fffffffL || b->shape[1] > 0x7fffffffL) return nullptr;
    const float *pa = tt_dev_ro(a), *pb = tt_dev_ro(b);
    if (!pa || !pb) return nullptr;
    long shp[2] = {a->shape[0], b->shape[1]};
    Tensor *out = tt_new_uninit(shp, 2);
    if (!out) return nullptr;
    GemmArgs g;
    memset(&g, 0, sizeof g);
    g.M = (int)shp[0]; g.N = (int)shp[1]; g.K = (int)a->shape[1];
    g.A = pa; g.lda = g.K; g.B = pb; g.ldb = g.N; g.C = TT(out)->dev; g.ldc = g.N;
    g.rule = rule;
    if (tt_gemm(&g) != 0) { tt_release(out); return nullptr; }
    return out;
}
extern "C" Tensor *tt_matmul(const Tensor *a, const Tensor *b) { return matmul_rule(a, b, 2); }
extern "C" Tensor *tt_matmul_fast(const Tensor *a, const Tensor *b) { return matmul_rule(a, b, 0); }
extern "C" Tensor *tt_matmul_omp(const Tensor *a, const Tensor *b, int nthreads) {
    (void)nthreads;
    return matmul_rule(a, b, 0);
}

/* R[M,N] = X[M,K] * Y[N,K]^T   (src/autograd.c:66-84) */
extern "C" Tensor *ttb_matmul_nt(const Tensor *x, const Tensor *y) {
    if (!x || !y || x->ndim != 2 || y->ndim != 2 || x->shape[1] != y->shape[1]) return nullptr;
    const float *px = tt_dev_ro(x), *py = tt_dev_ro(y);
    if (!px || !py) return nullptr;
    long shp[2] = {x->shape[0], y->shape[0]};
    Tensor *out = tt_new_uninit(shp, 2);
    if (!out) return nullptr;
    GemmArgs g;
    memset(&g, 0, sizeof g);
    g.tb = 1; g.M = (int)shp[0]; g.N = (int)shp[1]; g.K = (int)x->shape[1];
    g.A = px; g.lda = g.K; g.B = py; g.ldb = g.K; g.C = TT(out)->dev; g.ldc = g.N;
    g.rule = 1;
    if (tt_gemm(&g) != 0) { tt_release(out); return nullptr; }
    return out;
}
/* R[M,N] = X[K,M]^T * Y[K,N]   (src/autograd.c:87-103) */
extern "C" Tensor *ttb_matmul_tn(const Tensor *x, const Tensor *y) {
    if (!x || !y || x->ndim != 2 || y->ndim != 2 || x->shape[0] != y->shape[0]) return nullptr;
    const float *px = tt_dev_ro(x), *py = tt_dev_ro(y);
    if (!px || !py) return nullptr;
    long shp[2] = {x->shape[1], y->shape[1]};
    Tensor *out = tt_new_uninit(shp, 2);
    if (!out) return nullptr;
    GemmArgs g;
    memset(&g, 0, sizeof g);
    g.ta = 1; g.M = (int)shp[0]; g.N = (int)shp[1]; g.K = (int)x->shape[0];
    g.A = px; g.lda = g.M; g.B = py; g.ldb = g.N; g.C = TT(out)->dev; g.ldc = g.N;
    g.rule = 1;
    if (tt_gemm(&g) != 0) { tt_release(out); return nullptr; }
    return out;
}

/* Host-pointer sgemm (src/gemm.c:569).  Stages through device memory. */
extern "C" int tt_sgemm_rowmajor(int M, int N, int K, const float *A, const float *B, float *C, int nthreads) {
    (void)nthreads;
    if (M <= 0 || N <= 0 || K <= 0 || !A || !B || !C) return -1;
    long sa[2] = {M, K}, sb[2] = {K, N};
    Tensor *ta = tt_fromdata(A, sa, 2), *tb = tt_fromdata(B, sb, 2);
    Tensor *tc = (ta && tb) ? tt_matmul_fast(ta, tb) : nullptr;
    int rc = -1;
    if (tc) {
        const float *h = tt_data(tc);
        if (h) { memcpy(C, h, sizeof(float) * (size_t)M * N); rc = 0; }
    }
    tt_release(ta); tt_release(tb); tt_release(tc);
    return rc;
}

/* ---- reshape (src/ops_spatial.c:22-34): a copy, never a view ---------------*/
extern "C" Tensor *tt_reshape(const Tensor *a, const long *new_shape, int new_ndim) {
    if (!a || !new_shape || new_ndim <= 0 || new_ndim > 8) return nullptr;
    long numel = 1;
    for (int i = 0; i < new_ndim; i++) {
        if (new_shape[i] <= 0) return nullptr;
        if (numel > a->numel / new_shape[i] + 1) return nullptr;   /* cannot match, and must not overflow */
        numel *= new_shape[i];
    }
    if (numel != a->numel) return nullptr;
    const float *pa = tt_dev_ro(a);
    if (!pa) return nullptr;
    Tensor *out = tt_new_uninit(new_shape, new_ndim);
    if (!out) return nullptr;
    k_copy(TT(out)->dev, pa, numel);
    return out;
}

/* ---- convolution (src/ops_spatial.c:71-127) ---------------------------------
 * im2col, one GEMM W[F, C*kh*kw] x col, then the permute to NCHW with the
 * bias added.  Same validation order as the reference. */
static int conv_geometry(const Tensor *a, const Tensor *w, const Tensor *b, int sh, int sw, int ph, int pw,
                         int *Ho, int *Wo) {
    if (!a || !w || a->ndim != 4 || w->ndim != 4) return 0;
    long C = a->shape[1], H = a->shape[2], W = a->shape[3];
    long F = w->shape[0], Cw = w->shape[1], HH = w->shape[2], WW = w->shape[3];
    if (C != Cw) return 0;
    if (b && (b->ndim != 1 || b->shape[0] != F)) return 0;
    if (!(HH > 0 && WW > 0 && sh > 0 && sw > 0 && ph >= 0 && pw >= 0)) return 0;
    long ho = (H + 2l * ph - HH) / sh + 1, wo = (W + 2l * pw - WW) / sw + 1;
    if (H + 2l * ph - HH < 0 || W + 2l * pw - WW < 0) return 0;
    if (ho <= 0 || wo <= 0) return 0;
    if (ho > 0x7fffffffL || wo > 0x7fffffffL) return 0;
    *Ho = (int)ho; *Wo = (int)wo;
    return 1;
}

extern "C" Tensor *tt_conv2d(const Tensor *a, const Tensor *w, const Tensor *b,
                             int stride_h, int stride_w, int pad_h, int pad_w) {
    int Ho, Wo;
    if (!conv_geometry(a, w, b, stride_h, stride_w, pad_h, pad_w, &Ho, &Wo)) return nullptr;
    int N = (int)a->shape[0], C = (int)a->shape[1], H = (int)a->shape[2], W = (int)a->shape[3];
    int F = (int)w->shape[0], HH = (int)w->shape[2], WW = (int)w->shape[3];
    long sp = (long)Ho * Wo, ncol = (long)N * sp;
    int kc = C * HH * WW;
    if (ncol > 0x7fffffffL) return nullptr;
    const float *px = tt_dev_ro(a), *pw_ = tt_dev_ro(w), *pb = b ? tt_dev_ro(b) : nullptr;
    if (!px || !pw_ || (b && !pb)) return nullptr;
    long shp[4] = {N, F, Ho, Wo};
    Tensor *out = tt_new_uninit(shp, 4);
    /* implicit GEMM: the image is read through the index map, no col matrix, no permute pass.  Small
     * problems and the exact-fp32 setting keep the literal im2col + sgemm route below (bit-identical
     * to the reference). */
    const ConvGeom cg = {N, C, H, W, F, HH, WW, stride_h, stride_w, pad_h, pad_w, Ho, Wo};
    if (out && g_tt.conv_implicit && g_tt.gemm_path != 2 && (double)ncol * F * kc >= (double)(1l << 21) &&
        conv_tc_usable(&cg, 0)) {
        if (conv_tc_fprop(&cg, px, pw_, pb, TT(out)->dev) != 0) { tt_release(out); return nullptr; }
        return out;
    }
    float *col = (float *)tt_dev_alloc(sizeof(float) * (size_t)kc * ncol);
    float *om = (float *)tt_dev_alloc(sizeof(float) * (size_t)F * ncol);
    if (!out || !col || !om) { tt_release(out); tt_dev_free(col); tt_dev_free(om); return nullptr; }
    k_im2col(px, N, C, H, W, HH, WW, pad_h, pad_w, stride_h, stride_w, Ho, Wo, col);
    GemmArgs g;
    memset(&g, 0, sizeof g);
    g.M = F; g.N = (int)ncol; g.K = kc;
    g.A = pw_; g.lda = kc; g.B = col; g.ldb = ncol; g.C = om; g.ldc = ncol;
    int rc = tt_gemm(&g);
    if (rc == 0) k_conv_unpermute_bias(om, pb, N, F, sp, TT(out)->dev);
    tt_dev_free(col); tt_dev_free(om);
    if (rc != 0) { tt_release(out); return nullptr; }
    return out;
}

extern "C" Tensor *ttb_im2col(const Tensor *x, int kh, int kw, int stride_h, int stride_w, int pad_h, int pad_w) {
    if (!x || x->ndim != 4) return nullptr;
    if (!(kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 && pad_h >= 0 && pad_w >= 0)) return nullptr;
    long N = x->shape[0], C = x->shape[1], H = x->shape[2], W = x->shape[3];
    if (H + 2l * pad_h - kh < 0 || W + 2l * pad_w - kw < 0) return nullptr;
    long Ho = (H + 2l * pad_h - kh) / stride_h + 1, Wo = (W + 2l * pad_w - kw) / stride_w + 1;
    const float *px = tt_dev_ro(x);
    if (!px) return nullptr;
    long shp[2] = {C * kh * kw, N * Ho * Wo};
    Tensor *col = tt_new_uninit(shp, 2);
    if (!col) return nullptr;
    k_im2col(px, (int)N, (int)C, (int)H, (int)W, kh, kw, pad_h, pad_w, stride_h, stride_w, (int)Ho, (int)Wo, TT(col)->dev);
    return col;
}
extern "C" Tensor *ttb_col2im(const Tensor *col, int N, int C, int H, int W, int kh, int kw,
                              int stride_h, int stride_w, int pad_h, int pad_w) {
    if (!col || col->ndim != 2 || N <= 0 || C <= 0 || H <= 0 || W <= 0) return nullptr;
    if (!(kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 && pad_h >= 0 && pad_w >= 0)) return nullptr;
    if (H + 2l * pad_h - kh < 0 || W + 2l * pad_w - kw < 0) return nullptr;
    long Ho = (H + 2l * pad_h - kh) / stride_h + 1, Wo = (W + 2l * pad_w - kw) / stride_w + 1;
    if (col->shape[0] != (long)C * kh * kw || col->shape[1] != (long)N * Ho * Wo) return nullptr;
    const float *pc = tt_dev_ro(col);
    if (!pc) return nullptr;
    long shp[4] = {N, C, H, W};
    Tensor *x = tt_new_uninit(shp, 4);
    if (!x) return nullptr;
    k_col2im(pc, N, C, H, W, kh, kw, pad_h, pad_w, stride_h, stride_w, (int)Ho, (int)Wo, TT(x)->dev);
    return x;
}

/* ---- pooling (src/ops_spatial.c:129-201, src/autograd.c:555-628) -----------*/
static int pool_geometry(const Tensor *a, int ph, int pw, int sh, int sw, int *Ho, int *Wo) {
    if (!a || a->ndim != 4) return 0;
    if (!(ph > 0 && pw > 0 && sh > 0 && sw > 0)) return 0;
    long H = a->shape[2], W = a->shape[3];
    if (H - ph < 0 || W - pw < 0) return 0;
    long ho = (H - ph) / sh + 1, wo = (W - pw) / sw + 1;
    if (ho <= 0 || wo <= 0) return 0;
    *Ho = (int)ho; *Wo = (int)wo;
    return 1;
}
extern "C" Tensor *tt_maxpool2d(const Tensor *a, int pool_h, int pool_w, int stride_h, int stride_w) {
    int Ho, Wo;
    if (!pool_geometry(a, pool_h, pool_w, stride_h, stride_w, &Ho, &Wo)) return nullptr;
    const float *pa = tt_dev_ro(a);
    if (!pa) return nullptr;
    long shp[4] = {a->shape[0], a->shape[1], Ho, Wo};
    Tensor *out = tt_new_uninit(shp, 4);
    if (!out) return nullptr;
    k_maxpool(pa, a->shape[0] * a->shape[1], (int)a->shape[2], (int)a->shape[3], pool_h, pool_w,
              stride_h, stride_w, Ho, Wo, TT(out)->dev);
    return out;
}
extern "C" Tensor *tt_avgpool2d(const Tensor *a, int pool_h, int pool_w, int stride_h, int stride_w) {
    int Ho, Wo;
    if (!pool_geometry(a, pool_h, pool_w, stride_h, stride_w, &Ho, &Wo)) return nullptr;
    const float *pa = tt_dev_ro(a);
    if (!pa) return nullptr;
    long shp[4] = {a->shape[0], a->shape[1], Ho, Wo};
    Tensor *out = tt_new_uninit(shp, 4);
    if (!out) return nullptr;
    k_avgpool(pa, a->shape[0] * a->shape[1], (int)a->shape[2], (int)a->shape[3], pool_h, pool_w,
              stride_h, stride_w, Ho, Wo, TT(out)->dev);
    return out;
}
extern "C" Tensor *ttb_maxpool_bwd(const Tensor *x, const Tensor *g, int pool_h, int pool_w, int stride_h, int stride_w) {
    int Ho, Wo;
    if (!pool_geometry(x, pool_h, pool_w, stride_h, stride_w, &Ho, &Wo)) return nullptr;
    if (!g || g->ndim != 4 || g->shape[0] != x->shape[0] || g->shape[1] != x->shape[1] ||
        g->shape[2] != Ho || g->shape[3] != Wo) return nullptr;
    const float *px = tt_dev_ro(x), *pg = tt_dev_ro(g);
    if (!px || !pg) return nullptr;
    Tensor *dx = tt_new_like(x, 0);
    if (!dx) return nullptr;
    k_maxpool_bwd(px, pg, x->shape[0] * x->shape[1], (int)x->shape[2], (int)x->shape[3], pool_h, pool_w,
                  stride_h, stride_w, Ho, Wo, TT(dx)->dev);
    return dx;
}
extern "C" int ttb_maxpool_argmax(const Tensor *x, int pool_h, int pool_w, int stride_h, int stride_w, long *idx_out) {
    int Ho, Wo;
    if (!idx_out || !pool_geometry(x, pool_h, pool_w, stride_h, stride_w, &Ho, &Wo)) return -1;
    const float *px = tt_dev_ro(x);
    if (!px) return -1;
    long total = x->shape[0] * x->shape[1] * Ho * Wo;
    long long *d = (long long *)tt_dev_alloc(sizeof(long long) * (size_t)total);
    if (!d) return -1;
    k_maxpool_argmax(px, x->shape[0] * x->shape[1], (int)x->shape[2], (int)x->shape[3], pool_h, pool_w,
                     stride_h, stride_w, Ho, Wo, d);
    int ok = tt_cuda_ok(cudaMemcpyAsync(idx_out, d, sizeof(long long) * (size_t)total, cudaMemcpyDeviceToHost, g_tt.stream),
                        "cudaMemcpyAsync(D2H)") &&
             tt_cuda_ok(cudaStreamSynchronize(g_tt.stream), "cudaStreamSynchronize");
    tt_dev_free(d);
    return ok ? 0 : -1;
}
extern "C" Tensor *ttb_avgpool_bwd(const Tensor *g, int N, int C, int H, int W, int pool_h, int pool_w,
                                   int stride_h, int stride_w) {
    if (!g || g->ndim != 4 || N <= 0 || C <= 0 || H <= 0 || W <= 0) return nullptr;
    if (!(pool_h > 0 && pool_w > 0 && stride_h > 0 && stride_w > 0) || H < pool_h || W < pool_w) return nullptr;
    int Ho = (H - pool_h) / stride_h + 1, Wo = (W - pool_w) / stride_w + 1;
    if (g->shape[0] != N || g->shape[1] != C || g->shape[2] != Ho || g->shape[3] != Wo) return nullptr;
    const float *pg = tt_dev_ro(g);
    if (!pg) return nullptr;
    long shp[4] = {N, C, H, W};
    Tensor *dx = tt_new_uninit(shp, 4);
    if (!dx) return nullptr;
    k_avgpool_bwd(pg, (long)N * C, H, W, pool_h, pool_w, stride_h, stride_w, Ho, Wo, TT(dx)->dev);
    return dx;
}

/* ---- optimiser steps ---------------------------------------------------------*/
extern "C" int ttb_sgd_step(Tensor *w, const Tensor *g, float lr) {
    if (!w || !g || w->numel != g->numel) { tt_set_error("ttb_sgd_step: shape mismatch"); return -1; }
    const float *pg = tt_dev_ro(g);
    float *pw_ = tt_dev_rw(w);
    if (!pg || !pw_) return -1;
    k_sgd(pw_, pg, lr, w->numel);
    return 0;
}
extern "C" int ttb_sgd_momentum_step(Tensor *w, Tensor *v, const Tensor *g, float lr, float mu) {
    if (!w || !v || !g || w->numel != g->numel || v->numel != w->numel) { tt_set_error("ttb_sgd_momentum_step: shape mismatch"); return -1; }
    const float *pg = tt_dev_ro(g);
    float *pw_ = tt_dev_rw(w), *pv = tt_dev_rw(v);
    if (!pg || !pw_ || !pv) return -1;
    k_sgd_momentum(pw_, pv, pg, lr, mu, w->numel);
    return 0;
}
extern "C" int ttb_adam_step(Tensor *w, Tensor *m, Tensor *v, const Tensor *g, double lr,
                             double beta1, double beta2, double eps, int t) {
    if (!w || !m || !v || !g || t < 1 || w->numel != g->numel || m->numel != w->numel || v->numel != w->numel) {
        tt_set_error("ttb_adam_step: bad arguments");
        return -1;
    }
    const float *pg = tt_dev_ro(g);
    float *pw_ = tt_dev_rw(w), *pm = tt_dev_rw(m), *pv = tt_dev_rw(v);
    if (!pg || !pw_ || !pm || !pv) return -1;
    /* scalars formed in double and rounded once, as NumPy does with Python floats */
    double lr_t = lr * (sqrt(1.0 - pow(beta2, (double)t)) / (1.0 - pow(beta1, (double)t)));
    k_adam(pw_, pm, pv, pg, (float)lr_t, (float)beta1, (float)beta2, (float)(1.0 - beta1), (float)(1.0 - beta2),
           (float)eps, w->numel);
    return 0;
}
