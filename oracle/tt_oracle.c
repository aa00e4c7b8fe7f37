/* CPU oracle for the tinytorch training hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain scalar C, the
 * arithmetic of the reference CPU implementation (kanqzkokelo/tinytorch) for
 * the operators on the training hot path.  It is the checker that the CUDA
 * kernels are compared against; nothing in the product library links, loads
 * or calls it.  Only the test-suite, the smoke check and the CPU-baseline leg
 * of the benchmark may use it.
 *
 * Parity of this restatement is PINNED: tests/test_oracle.py compares every
 * function below with the reference library compiled from its own sources
 * (oracle/Makefile -> oracle/_ref/libtinytorch_ref.so) when that build is
 * present, and with fixtures generated from that library
 * (tests/golden/, made by tests/golden/make_golden.py) everywhere else.
 *
 * Summation orders follow the reference exactly (citations are
 * file:line inside the reference project), so on the same host the results
 * are bit-identical to the reference library built from C:
 *   - forward sgemm: per output one accumulator, fused multiply-add, k
 *     ascending (the K blocks of the kernel reload the accumulator from C, so
 *     they do not change the chain); the rows beyond the last multiple of 6
 *     and the columns beyond the last multiple of 16 use separately rounded
 *     multiply and add and skip exact zeros of A (src/gemm.c:52-62,569-641).
 *   - backward GEMMs: one accumulator, separately rounded multiply and add,
 *     k ascending (src/autograd.c:66-103,439-454).
 * Build with -ffp-contract=off so that only the explicit fmaf() fuses.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#define ORC_MR 6      /* src/gemm.c:22-24 */
#define ORC_NR 16     /* src/gemm.c:25-27 */

/* Scalar edge path of the forward sgemm: C[i, n0:n1] += A[i,k] * B[k, n0:n1],
 * zero entries of A skipped (src/gemm.c:52-62). */
static void orc_edge(int M, int N, int K, const float *A, const float *B,
                     float *C, int n0, int n1) {
    for (int i = 0; i < M; i++) {
        for (int k = 0; k < K; k++) {
            float a = A[(long)i * K + k];
            if (a == 0.0f) continue;
            for (int j = n0; j < n1; j++) {
                float p = a * B[(long)k * N + j];
                C[(long)i * N + j] = C[(long)i * N + j] + p;
            }
        }
    }
}

/* Forward sgemm, row-major, C must be zero on entry (src/gemm.c:569-641).
 * The 6x16 register tile of src/gemm.c:70-567 is one k-ascending FMA chain
 * per output: the first 384-wide K block starts the accumulators at zero
 * (:83-95), every later block reloads them from C (:264-280) and carries on,
 * so the K blocking leaves no trace in the arithmetic. */
int orc_sgemm(int M, int N, int K, const float *A, const float *B, float *C) {
    int nfull = (N / ORC_NR) * ORC_NR;
    int mfull = (M / ORC_MR) * ORC_MR;
    if (nfull <= 0 || K <= 0) {
        if (nfull < N) orc_edge(M, N, K, A, B, C, nfull, N);
        return 0;
    }
    if (mfull == 0) {
        orc_edge(M, N, K, A, B, C, 0, N);
        return 0;
    }
    #pragma omp parallel for schedule(static)
    for (int i = 0; i < mfull; i++) {
        for (int j = 0; j < nfull; j++) {
            float acc = 0.0f;
            for (int k = 0; k < K; k++)
                acc = fmaf(A[(long)i * K + k], B[(long)k * N + j], acc);
            C[(long)i * N + j] = acc;
        }
    }
    if (mfull < M)
        orc_edge(M - mfull, N, K, A + (long)mfull * K, B, C + (long)mfull * N, 0, nfull);
    if (nfull < N)
        orc_edge(M, N, K, A, B, C, nfull, N);
    return 0;
}

/* Naive matmul of the tensor API (src/ops.c:84-102): row-by-row axpy with
 * zero entries of A skipped. */
void orc_matmul_naive(int M, int N, int K, const float *A, const float *B, float *C) {
    memset(C, 0, sizeof(float) * (size_t)M * N);
    orc_edge(M, N, K, A, B, C, 0, N);
}

/* R[M,N] = X[M,K] * Y[N,K]^T, dot products, k ascending
 * (src/autograd.c:66-84; the same loop is sgemm_A_Bt_local, :439-454). */
void orc_matmul_nt(int M, int N, long K, const float *X, const float *Y, float *R) {
    #pragma omp parallel for collapse(2) schedule(static)
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            float s = 0.0f;
            for (long k = 0; k < K; k++) {
                float p = X[(long)m * K + k] * Y[(long)n * K + k];
                s = s + p;
            }
            R[(long)m * N + n] = s;
        }
}

/* R[M,N] = X[K,M]^T * Y[K,N], axpy over k ascending into a zeroed R
 * (src/autograd.c:87-103). */
void orc_matmul_tn(int M, int N, int K, const float *X, const float *Y, float *R) {
    #pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        for (int n = 0; n < N; n++) R[(long)m * N + n] = 0.0f;
        for (int k = 0; k < K; k++) {
            float x = X[(long)k * M + m];
            for (int n = 0; n < N; n++) {
                float p = x * Y[(long)k * N + n];
                R[(long)m * N + n] = R[(long)m * N + n] + p;
            }
        }
    }
}

/* Elementwise operators (src/ops.c:44-82, 104-106). */
void orc_add(long n, const float *a, const float *b, float *o) { for (long i = 0; i < n; i++) o[i] = a[i] + b[i]; }
void orc_mul(long n, const float *a, const float *b, float *o) { for (long i = 0; i < n; i++) o[i] = a[i] * b[i]; }
void orc_addscalar(long n, const float *a, float s, float *o) { for (long i = 0; i < n; i++) o[i] = a[i] + s; }
void orc_mulscalar(long n, const float *a, float s, float *o) { for (long i = 0; i < n; i++) o[i] = a[i] * s; }
void orc_relu(long n, const float *a, float *o) { for (long i = 0; i < n; i++) o[i] = a[i] > 0.0f ? a[i] : 0.0f; }

/* dx = x > 0 ? g : 0, mask taken from the forward INPUT (src/autograd.c:318-327). */
void orc_relu_bwd(long n, const float *x, const float *g, float *dx) {
    for (long i = 0; i < n; i++) dx[i] = x[i] > 0.0f ? g[i] : 0.0f;
}

/* Softmax over the last axis: max, exp(x-max), sequential sum, divide; a row
 * whose maximum is -Inf becomes uniform (src/ops.c:108-145). */
void orc_softmax(long rows, int N, const float *x, float *o) {
    for (long r = 0; r < rows; r++) {
        const float *xr = x + r * N;
        float *orow = o + r * N;
        float mx = -INFINITY;
        for (int j = 0; j < N; j++) if (xr[j] > mx) mx = xr[j];
        if (mx == -INFINITY) {
            for (int j = 0; j < N; j++) orow[j] = 1.0f / (float)N;
        } else {
            float sum = 0.0f;
            for (int j = 0; j < N; j++) { float e = expf(xr[j] - mx); orow[j] = e; sum = sum + e; }
            for (int j = 0; j < N; j++) orow[j] = orow[j] / sum;
        }
    }
}

/* dx = s * (g - sum_j g_j s_j) per row (src/autograd.c:329-346). */
void orc_softmax_bwd(long rows, int N, const float *s, const float *g, float *dx) {
    for (long r = 0; r < rows; r++) {
        const float *sr = s + r * N, *gr = g + r * N;
        float dot = 0.0f;
        for (int j = 0; j < N; j++) { float p = gr[j] * sr[j]; dot = dot + p; }
        for (int j = 0; j < N; j++) dx[r * N + j] = sr[j] * (gr[j] - dot);
    }
}

/* Append a column of ones / drop the last gradient column
 * (src/autograd.c:195-212, 348-359). */
void orc_padones(int M, int K, const float *x, float *o) {
    for (int m = 0; m < M; m++) {
        memcpy(o + (long)m * (K + 1), x + (long)m * K, sizeof(float) * (size_t)K);
        o[(long)m * (K + 1) + K] = 1.0f;
    }
}
void orc_padones_bwd(int M, int K, const float *g, float *dx) {
    for (int m = 0; m < M; m++)
        memcpy(dx + (long)m * K, g + (long)m * (K + 1), sizeof(float) * (size_t)K);
}

/* col[(c,kh,kw), (n,ho,wo)] = x[n, c, ho*sh-ph+kh, wo*sw-pw+kw] or 0
 * (src/ops_spatial.c:37-69; identical copy at src/autograd.c:371-404). */
void orc_im2col(const float *x, int N, int C, int H, int W, int HH, int WW,
                int ph, int pw, int sh, int sw, float *col) {
    int Ho = (H + 2 * ph - HH) / sh + 1, Wo = (W + 2 * pw - WW) / sw + 1;
    long sp = (long)Ho * Wo, ncol = (long)N * sp;
    int kc = C * HH * WW;
    #pragma omp parallel for schedule(static)
    for (int c = 0; c < kc; c++) {
        int kw = c % WW, kh = (c / WW) % HH, ci = c / (HH * WW);
        for (int n = 0; n < N; n++)
            for (int ho = 0; ho < Ho; ho++)
                for (int wo = 0; wo < Wo; wo++) {
                    int r = ho * sh - ph + kh, q = wo * sw - pw + kw;
                    float v = 0.0f;
                    if (r >= 0 && r < H && q >= 0 && q < W)
                        v = x[(((long)n * C + ci) * H + r) * W + q];
                    col[(long)c * ncol + (long)n * sp + (long)ho * Wo + wo] = v;
                }
    }
}

/* Scatter-add of col back to the image, (c,kh,kw) outermost then n, ho, wo
 * (src/autograd.c:406-434). */
void orc_col2im(const float *col, int N, int C, int H, int W, int HH, int WW,
                int ph, int pw, int sh, int sw, float *x) {
    int Ho = (H + 2 * ph - HH) / sh + 1, Wo = (W + 2 * pw - WW) / sw + 1;
    long sp = (long)Ho * Wo, ncol = (long)N * sp;
    int kc = C * HH * WW;
    memset(x, 0, sizeof(float) * (size_t)N * C * H * W);
    for (int c = 0; c < kc; c++) {
        int kw = c % WW, kh = (c / WW) % HH, ci = c / (HH * WW);
        for (int n = 0; n < N; n++)
            for (int ho = 0; ho < Ho; ho++)
                for (int wo = 0; wo < Wo; wo++) {
                    int r = ho * sh - ph + kh, q = wo * sw - pw + kw;
                    if (r >= 0 && r < H && q >= 0 && q < W) {
                        long o = (((long)n * C + ci) * H + r) * W + q;
                        x[o] = x[o] + col[(long)c * ncol + (long)n * sp + (long)ho * Wo + wo];
                    }
                }
    }
}

/* conv2d forward = im2col, one sgemm W[F,C*HH*WW] x col, then the permute
 * [F, N*sp] -> [N,F,sp] with the bias added (src/ops_spatial.c:71-127).
 * bias may be NULL.  Returns 0, or -1 when memory runs out. */
int orc_conv2d(const float *x, const float *w, const float *bias,
               int N, int C, int H, int W, int F, int HH, int WW,
               int sh, int sw, int ph, int pw, float *out) {
    int Ho = (H + 2 * ph - HH) / sh + 1, Wo = (W + 2 * pw - WW) / sw + 1;
    long sp = (long)Ho * Wo, ncol = (long)N * sp;
    int kc = C * HH * WW;
    float *col = (float *)malloc(sizeof(float) * (size_t)kc * ncol);
    float *om = (float *)calloc((size_t)F * ncol, sizeof(float));
    if (!col || !om) { free(col); free(om); return -1; }
    orc_im2col(x, N, C, H, W, HH, WW, ph, pw, sh, sw, col);
    orc_sgemm(F, (int)ncol, kc, w, col, om);
    for (int n = 0; n < N; n++)
        for (int f = 0; f < F; f++) {
            float b = bias ? bias[f] : 0.0f;
            for (long i = 0; i < sp; i++)
                out[((long)n * F + f) * sp + i] = om[(long)f * ncol + (long)n * sp + i] + b;
        }
    free(col); free(om);
    return 0;
}

/* conv2d backward (src/autograd.c:456-553).  Any of db, dw, dx may be NULL
 * (the reference skips the parts whose parent needs no gradient).
 *   db[f]   = sum over n, ho, wo of g                        (:467-482)
 *   dw      = g_perm[F, N*sp] x col^T  via dot products      (:487-513)
 *   dx      = col2im( W^T[kc,F] x g_perm )  forward sgemm    (:515-552) */
int orc_conv2d_bwd(const float *x, const float *w, const float *g,
                   int N, int C, int H, int W, int F, int HH, int WW,
                   int sh, int sw, int ph, int pw,
                   float *dx, float *dw, float *db) {
    int Ho = (H + 2 * ph - HH) / sh + 1, Wo = (W + 2 * pw - WW) / sw + 1;
    long sp = (long)Ho * Wo, ncol = (long)N * sp;
    int kc = C * HH * WW;
    if (db) {
        for (int f = 0; f < F; f++) {
            float s = 0.0f;
            for (int n = 0; n < N; n++)
                for (long i = 0; i < sp; i++) s = s + g[((long)n * F + f) * sp + i];
            db[f] = s;
        }
    }
    float *gp = (float *)malloc(sizeof(float) * (size_t)F * ncol);
    if (!gp) return -1;
    for (int f = 0; f < F; f++)
        for (int n = 0; n < N; n++)
            memcpy(gp + (long)f * ncol + (long)n * sp, g + ((long)n * F + f) * sp, sizeof(float) * (size_t)sp);
    if (dw) {
        float *col = (float *)malloc(sizeof(float) * (size_t)kc * ncol);
        if (!col) { free(gp); return -1; }
        orc_im2col(x, N, C, H, W, HH, WW, ph, pw, sh, sw, col);
        orc_matmul_nt(F, kc, ncol, gp, col, dw);
        free(col);
    }
    if (dx) {
        float *wt = (float *)malloc(sizeof(float) * (size_t)F * kc);
        float *dcol = (float *)calloc((size_t)kc * ncol, sizeof(float));
        if (!wt || !dcol) { free(wt); free(dcol); free(gp); return -1; }
        for (int f = 0; f < F; f++)
            for (int k = 0; k < kc; k++) wt[(long)k * F + f] = w[(long)f * kc + k];
        orc_sgemm(kc, (int)ncol, F, wt, gp, dcol);
        orc_col2im(dcol, N, C, H, W, HH, WW, ph, pw, sh, sw, dx);
        free(wt); free(dcol);
    }
    free(gp);
    return 0;
}

/* Max pooling without padding; start at -Inf, strict '>' so a NaN never
 * wins (src/ops_spatial.c:129-164). */
void orc_maxpool(const float *x, int N, int C, int H, int W, int ph, int pw,
                 int sh, int sw, float *out) {
    int Ho = (H - ph) / sh + 1, Wo = (W - pw) / sw + 1;
    for (long nc = 0; nc < (long)N * C; nc++)
        for (int ho = 0; ho < Ho; ho++)
            for (int wo = 0; wo < Wo; wo++) {
                float m = -INFINITY;
                for (int kh = 0; kh < ph; kh++)
                    for (int kw = 0; kw < pw; kw++) {
                        float v = x[(nc * H + ho * sh + kh) * W + wo * sw + kw];
                        if (v > m) m = v;
                    }
                out[(nc * Ho + ho) * Wo + wo] = m;
            }
}

/* Argmax routing (src/autograd.c:555-594): per window the first strict
 * maximum in (kh, kw) scan order, the window origin when nothing beats
 * -Inf; the window's gradient is added there.  idx (may be NULL) receives
 * the flat input offset chosen for every output element. */
void orc_maxpool_bwd(const float *x, const float *g, int N, int C, int H, int W,
                     int ph, int pw, int sh, int sw, float *dx, long *idx) {
    int Ho = (H - ph) / sh + 1, Wo = (W - pw) / sw + 1;
    memset(dx, 0, sizeof(float) * (size_t)N * C * H * W);
    for (long nc = 0; nc < (long)N * C; nc++)
        for (int ho = 0; ho < Ho; ho++)
            for (int wo = 0; wo < Wo; wo++) {
                float m = -INFINITY;
                int bh = ho * sh, bw = wo * sw;
                for (int kh = 0; kh < ph; kh++)
                    for (int kw = 0; kw < pw; kw++) {
                        float v = x[(nc * H + ho * sh + kh) * W + wo * sw + kw];
                        if (v > m) { m = v; bh = ho * sh + kh; bw = wo * sw + kw; }
                    }
                long o = (nc * H + bh) * W + bw;
                dx[o] = dx[o] + g[(nc * Ho + ho) * Wo + wo];
                if (idx) idx[(nc * Ho + ho) * Wo + wo] = o;
            }
}

/* Mean pooling and its backward (src/ops_spatial.c:166-201,
 * src/autograd.c:596-628). */
void orc_avgpool(const float *x, int N, int C, int H, int W, int ph, int pw,
                 int sh, int sw, float *out) {
    int Ho = (H - ph) / sh + 1, Wo = (W - pw) / sw + 1;
    float norm = 1.0f / (float)(ph * pw);
    for (long nc = 0; nc < (long)N * C; nc++)
        for (int ho = 0; ho < Ho; ho++)
            for (int wo = 0; wo < Wo; wo++) {
                float s = 0.0f;
                for (int kh = 0; kh < ph; kh++)
                    for (int kw = 0; kw < pw; kw++)
                        s = s + x[(nc * H + ho * sh + kh) * W + wo * sw + kw];
                out[(nc * Ho + ho) * Wo + wo] = s * norm;
            }
}
void orc_avgpool_bwd(const float *g, int N, int C, int H, int W, int ph, int pw,
                     int sh, int sw, float *dx) {
    int Ho = (H - ph) / sh + 1, Wo = (W - pw) / sw + 1;
    float norm = 1.0f / (float)(ph * pw);
    memset(dx, 0, sizeof(float) * (size_t)N * C * H * W);
    for (long nc = 0; nc < (long)N * C; nc++)
        for (int ho = 0; ho < Ho; ho++)
            for (int wo = 0; wo < Wo; wo++) {
                float gv = g[(nc * Ho + ho) * Wo + wo] * norm;
                for (int kh = 0; kh < ph; kh++)
                    for (int kw = 0; kw < pw; kw++) {
                        long o = (nc * H + ho * sh + kh) * W + wo * sw + kw;
                        dx[o] = dx[o] + gv;
                    }
            }
}

/* Gradient accumulation: dst += src (src/autograd.c:52-54). */
void orc_accum(long n, float *dst, const float *src) {
    for (long i = 0; i < n; i++) dst[i] = dst[i] + src[i];
}
