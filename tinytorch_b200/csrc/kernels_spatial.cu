/* Spatial kernels of the hot path: batched im2col and its adjoint, the
 * permutes around the convolution GEMMs, the bias gradient, max/avg pooling
 * forward and backward.
 *
 * Index arithmetic is integer-exact and follows the reference's maps, so
 * im2col, pooling and arg-max routing are bit-exact.  The two adjoints that
 * the reference writes as serial scatter-adds (col2im, pooling backward) are
 * written as GATHERS: one thread owns one image element and adds its
 * contributions in the order the reference's loops produce them, which needs
 * no atomics and reproduces the reference sums bit for bit.  All kernels are
 * HBM-bound: consecutive threads touch consecutive addresses on both sides. */
#include "tt_internal.h"

#include <math.h>

#define TPB 256

static inline int grid_for(long items) {
    long want = (items + TPB - 1) / TPB;
    long cap = (long)g_tt.sm_count * 8;
    if (want < 1) want = 1;
    return (int)(want < cap ? want : cap);
}

#define LAUNCH(kern, grid, block, smem, ...)                         \
    do {                                                             \
        kern<<<(grid), (block), (smem), g_tt.stream>>>(__VA_ARGS__); \
        g_tt.launches++;                                             \
    } while (0)

/* col[(c,kh,kw), (n,ho,wo)] = x[n, c, ho*sh-ph+kh, wo*sw-pw+kw] or 0
 * (src/ops_spatial.c:37-69; same map at src/autograd.c:371-404).
 * One thread per col element, wo fastest: reads and writes are both runs of
 * consecutive addresses for stride 1. */
__global__ void __launch_bounds__(TPB) im2col_kernel(const float *__restrict__ x, int N, int C, int H, int W,
                                                      int HH, int WW, int ph, int pw, int sh, int sw,
                                                      int Ho, int Wo, float *__restrict__ col) {
    long sp = (long)Ho * Wo, ncol = (long)N * sp;
    long total = (long)C * HH * WW * ncol;
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        long c = i / ncol, r = i - c * ncol;
        int n = (int)(r / sp);
        int s = (int)(r - (long)n * sp);
        int ho = s / Wo, wo = s - ho * Wo;
        int kw = (int)(c % WW), kh = (int)((c / WW) % HH), ci = (int)(c / ((long)HH * WW));
        int row = ho * sh - ph + kh, q = wo * sw - pw + kw;
        float v = 0.0f;
        if (row >= 0 && row < H && q >= 0 && q < W)
            v = x[(((long)n * C + ci) * H + row) * W + q];
        col[i] = v;
    }
}
void k_im2col(const float *x, int N, int C, int H, int W, int HH, int WW,
              int ph, int pw, int sh, int sw, int Ho, int Wo, float *col) {
    long total = (long)C * HH * WW * N * Ho * Wo;
    tt_trace_begin(TTB_K_SPATIAL);
    LAUNCH(im2col_kernel, grid_for(total), TPB, 0, x, N, C, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo, col);
    tt_trace_end(TTB_K_SPATIAL, 4.0 * ((double)total + (double)N * C * H * W));
}

/* Adjoint of im2col (src/autograd.c:406-434), as a gather: the element
 * x[n,ci,h,w] receives col[(ci,kh,kw),(n,ho,wo)] for every (kh,kw) with
 * ho*sh-ph+kh == h and wo*sw-pw+kw == w.  The reference adds them with
 * (kh,kw) ascending (its outer loop is c = (ci,kh,kw)); so does this. */
__global__ void __launch_bounds__(TPB) col2im_kernel(const float *__restrict__ col, int N, int C, int H, int W,
                                                      int HH, int WW, int ph, int pw, int sh, int sw,
                                                      int Ho, int Wo, float *__restrict__ x) {
    long sp = (long)Ho * Wo, ncol = (long)N * sp;
    long total = (long)N * C * H * W;
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int w = (int)(i % W);
        long t = i / W;
        int h = (int)(t % H); t /= H;
        int ci = (int)(t % C);
        int n = (int)(t / C);
        float acc = 0.0f;
        for (int kh = 0; kh < HH; kh++) {
            int hn = h + ph - kh;
            if (hn < 0 || hn % sh) continue;
            int ho = hn / sh;
            if (ho >= Ho) continue;
            for (int kw = 0; kw < WW; kw++) {
                int wn = w + pw - kw;
                if (wn < 0 || wn % sw) continue;
                int wo = wn / sw;
                if (wo >= Wo) continue;
                long c = ((long)ci * HH + kh) * WW + kw;
                acc = acc + col[c * ncol + (long)n * sp + (long)ho * Wo + wo];
            }
        }
        x[i] = acc;
    }
}
void k_col2im(const float *col, int N, int C, int H, int W, int HH, int WW,
              int ph, int pw, int sh, int sw, int Ho, int Wo, float *x) {
    long total = (long)N * C * H * W;
    tt_trace_begin(TTB_K_SPATIAL);
    LAUNCH(col2im_kernel, grid_for(total), TPB, 0, col, N, C, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo, x);
    tt_trace_end(TTB_K_SPATIAL, 4.0 * ((double)total + (double)C * HH * WW * N * Ho * Wo));
}

/* out[n,f,i] = om[f, n*sp+i] + bias[f]   (src/ops_spatial.c:105-119) */
__global__ void __launch_bounds__(TPB) conv_unpermute_bias_kernel(const float *__restrict__ om, const float *__restrict__ bias,
                                                                   int N, int F, long sp, float *__restrict__ out) {
    long total = (long)N * F * sp;
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        long s = i % sp;
        long t = i / sp;
        int f = (int)(t % F);
        long n = t / F;
        float b = bias ? bias[f] : 0.0f;
        out[i] = om[(long)f * N * sp + n * sp + s] + b;
    }
}
void k_conv_unpermute_bias(const float *om, const float *bias, int N, int F, long sp, float *out) {
    long total = (long)N * F * sp;
    tt_trace_begin(TTB_K_SPATIAL);
    LAUNCH(conv_unpermute_bias_kernel, grid_for(total), TPB, 0, om, bias, N, F, sp, out);
    tt_trace_end(TTB_K_SPATIAL, 8.0 * (double)total);
}

/* gp[f, n*sp+i] = g[n,f,i]   (src/autograd.c:494-501) */
__global__ void __launch_bounds__(TPB) conv_permute_kernel(const float *__restrict__ g, int N, int F, long sp,
                                                            float *__restrict__ gp) {
    long total = (long)N * F * sp;
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        long s = i % sp;
        long t = i / sp;
        long n = t % N;
        long f = t / N;
        gp[i] = g[(n * F + f) * sp + s];
    }
}
void k_conv_permute(const float *g, int N, int F, long sp, float *gp) {
    long total = (long)N * F * sp;
    tt_trace_begin(TTB_K_SPATIAL);
    LAUNCH(conv_permute_kernel, grid_for(total), TPB, 0, g, N, F, sp, gp);
    tt_trace_end(TTB_K_SPATIAL, 8.0 * (double)total);
}

/* db[f] = sum over n, ho, wo of g[n,f,ho,wo]   (src/autograd.c:467-482).
 * Two deterministic phases: blocks (f, slab of n) reduce with a fixed tree,
 * then the slab sums are added in order. */
__global__ void __launch_bounds__(TPB) bias_grad_partial_kernel(const float *__restrict__ g, int N, int F, long sp,
                                                                 int n_per_slab, float *__restrict__ part) {
    __shared__ float sh[TPB / 32];
    int f = blockIdx.x, slab = blockIdx.y;
    int n0 = slab * n_per_slab;
    int n1 = n0 + n_per_slab < N ? n0 + n_per_slab : N;
    float acc = 0.0f;
    for (int n = n0; n < n1; n++) {
        const float *p = g + ((long)n * F + f) * sp;
        for (long i = threadIdx.x; i < sp; i += TPB) acc += p[i];
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int k = 0; k < TPB / 32; k++) s += sh[k];
        part[(long)f * gridDim.y + slab] = s;
    }
}
__global__ void bias_grad_final_kernel(const float *__restrict__ part, int F, int slabs, float *__restrict__ db) {
    int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= F) return;
    float s = 0.0f;
    for (int k = 0; k < slabs; k++) s += part[(long)f * slabs + k];
    db[f] = s;
}
void k_conv_bias_grad(const float *g, int N, int F, long sp, float *db) {
    int slabs = (g_tt.sm_count * 8 + F - 1) / F;
    if (slabs > N) slabs = N;
    if (slabs < 1) slabs = 1;
    int n_per_slab = (N + slabs - 1) / slabs;
    slabs = (N + n_per_slab - 1) / n_per_slab;
    float *part = (float *)tt_dev_alloc(sizeof(float) * (size_t)F * slabs);
    if (!part) return;
    tt_trace_begin(TTB_K_REDUCE);
    LAUNCH(bias_grad_partial_kernel, dim3(F, slabs), TPB, 0, g, N, F, sp, n_per_slab, part);
    LAUNCH(bias_grad_final_kernel, (F + 127) / 128, 128, 0, part, F, slabs, db);
    tt_trace_end(TTB_K_REDUCE, 4.0 * (double)N * F * sp);
    tt_dev_free(part);
}

/* ---- pooling ---------------------------------------------------------------
 * Window scan shared by forward, backward and the arg-max probe: start at
 * -Inf with the index at the window origin, strict '>' in (kh,kw) order, so a
 * NaN never wins and ties keep the first maximum
 * (src/ops_spatial.c:151-157, src/autograd.c:575-586). */
__device__ __forceinline__ void window_argmax(const float *__restrict__ plane, int W, int h0, int w0,
                                              int ph, int pw, float &best, int &bh, int &bw) {
    best = -INFINITY; bh = h0; bw = w0;
    for (int kh = 0; kh < ph; kh++)
        for (int kw = 0; kw < pw; kw++) {
            float v = plane[(long)(h0 + kh) * W + (w0 + kw)];
            if (v > best) { best = v; bh = h0 + kh; bw = w0 + kw; }
        }
}

__global__ void __launch_bounds__(TPB) maxpool_kernel(const float *__restrict__ x, long NC, int H, int W, int ph, int pw,
                                                       int sh, int sw, int Ho, int Wo, float *__restrict__ out) {
    long total = NC * Ho * Wo;
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int wo = (int)(i % Wo);
        long t = i / Wo;
        int ho = (int)(t % Ho);
        long nc = t / Ho;
        float best; int bh, bw;
        window_argmax(x + nc * H * W, W, ho * sh, wo * sw, ph, pw, best, bh, bw);
        out[i] = best;
    }
}
void k_maxpool(const float *x, long NC, int H, int W, int ph, int pw, int sh, int sw,
               int Ho, int Wo, float *out) {
    long total = NC * Ho * Wo;
    tt_trace_begin(TTB_K_SPATIAL);
    LAUNCH(maxpool_kernel, grid_for(total), TPB, 0, x, NC, H, W, ph, pw, sh, sw, Ho, Wo, out);
    tt_trace_end(TTB_K_SPATIAL, 4.0 * ((double)NC * H * W + (double)total));
}

__global__ void __launch_bounds__(TPB) maxpool_argmax_kernel(const float *__restrict__ x, long NC, int H, int W, int ph, int pw,
                                                              int sh, int sw, int Ho, int Wo, long long *__restrict__ idx) {
    long total = NC * Ho * Wo;
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int wo = (int)(i % Wo);
        long t = i / Wo;
        int ho = (int)(t % Ho);
        long nc = t / Ho;
        float best; int bh, bw;
        window_argmax(x + nc * H * W, W, ho * sh, wo * sw, ph, pw, best, bh, bw);
        idx[i] = (long long)((nc * H + bh) * W + bw);
    }
}
void k_maxpool_argmax(const float *x, long NC, int H, int W, int ph, int pw, int sh, int sw,
                      int Ho, int Wo, long long *idx) {
    long total = NC * Ho * Wo;
    LAUNCH(maxpool_argmax_kernel, grid_for(total), TPB, 0, x, NC, H, W, ph, pw, sh, sw, Ho, Wo, idx);
}

/* Gradient routing (src/autograd.c:555-594) as a gather over the input:
 * element (h,w) looks at every window that contains it, in (ho,wo) ascending
 * order -- the order in which the reference's loops reach it -- re-derives
 * that window's arg-max and adds the window's gradient when it is the
 * winner.  For the non-overlapping 2x2/2 case that is one window per
 * element; elements outside every window get 0. */
__global__ void __launch_bounds__(TPB) maxpool_bwd_kernel(const float *__restrict__ x, const float *__restrict__ g, long NC,
                                                           int H, int W, int ph, int pw, int sh, int sw,
                                                           int Ho, int Wo, float *__restrict__ dx) {
    long total = NC * H * W;
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int w = (int)(i % W);
        long t = i / W;
        int h = (int)(t % H);
        long nc = t / H;
        const float *plane = x + nc * H * W;
        int ho_lo = h - ph + 1 <= 0 ? 0 : (h - ph + 1 + sh - 1) / sh;
        int ho_hi = h / sh < Ho - 1 ? h / sh : Ho - 1;
        int wo_lo = w - pw + 1 <= 0 ? 0 : (w - pw + 1 + sw - 1) / sw;
        int wo_hi = w / sw < Wo - 1 ? w / sw : Wo - 1;
        float acc = 0.0f;
        for (int ho = ho_lo; ho <= ho_hi; ho++)
            for (int wo = wo_lo; wo <= wo_hi; wo++) {
                float best; int bh, bw;
                window_argmax(plane, W, ho * sh, wo * sw, ph, pw, best, bh, bw);
                if (bh == h && bw == w) acc = acc + g[(nc * Ho + ho) * Wo + wo];
            }
        dx[i] = acc;
    }
}
void k_maxpool_bwd(const float *x, const float *g, long NC, int H, int W, int ph, int pw,
                   int sh, int sw, int Ho, int Wo, float *dx) {
    long total = NC * H * W;
    tt_trace_begin(TTB_K_SPATIAL);
    LAUNCH(maxpool_bwd_kernel, grid_for(total), TPB, 0, x, g, NC, H, W, ph, pw, sh, sw, Ho, Wo, dx);
    tt_trace_end(TTB_K_SPATIAL, 4.0 * (2.0 * (double)total + (double)NC * Ho * Wo));
}

/* Mean pooling (src/ops_spatial.c:166-201) and its adjoint
 * (src/autograd.c:596-628), the latter again as a gather in (ho,wo) order. */
__global__ void __launch_bounds__(TPB) avgpool_kernel(const float *__restrict__ x, long NC, int H, int W, int ph, int pw,
                                                       int sh, int sw, int Ho, int Wo, float *__restrict__ out) {
    long total = NC * Ho * Wo;
    float norm = 1.0f / (float)(ph * pw);
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int wo = (int)(i % Wo);
        long t = i / Wo;
        int ho = (int)(t % Ho);
        long nc = t / Ho;
        const float *plane = x + nc * H * W;
        float s = 0.0f;
        for (int kh = 0; kh < ph; kh++)
            for (int kw = 0; kw < pw; kw++)
                s = s + plane[(long)(ho * sh + kh) * W + (wo * sw + kw)];
        out[i] = s * norm;
    }
}
void k_avgpool(const float *x, long NC, int H, int W, int ph, int pw, int sh, int sw,
               int Ho, int Wo, float *out) {
    long total = NC * Ho * Wo;
    tt_trace_begin(TTB_K_SPATIAL);
    LAUNCH(avgpool_kernel, grid_for(total), TPB, 0, x, NC, H, W, ph, pw, sh, sw, Ho, Wo, out);
    tt_trace_end(TTB_K_SPATIAL, 4.0 * ((double)NC * H * W + (double)total));
}

__global__ void __launch_bounds__(TPB) avgpool_bwd_kernel(const float *__restrict__ g, long NC, int H, int W, int ph, int pw,
                                                           int sh, int sw, int Ho, int Wo, float *__restrict__ dx) {
    long total = NC * H * W;
    float norm = 1.0f / (float)(ph * pw);
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int w = (int)(i % W);
        long t = i / W;
        int h = (int)(t % H);
        long nc = t / H;
        int ho_lo = h - ph + 1 <= 0 ? 0 : (h - ph + 1 + sh - 1) / sh;
        int ho_hi = h / sh < Ho - 1 ? h / sh : Ho - 1;
        int wo_lo = w - pw + 1 <= 0 ? 0 : (w - pw + 1 + sw - 1) / sw;
        int wo_hi = w / sw < Wo - 1 ? w / sw : Wo - 1;
        float acc = 0.0f;
        for (int ho = ho_lo; ho <= ho_hi; ho++)
            for (int wo = wo_lo; wo <= wo_hi; wo++)
                acc = acc + g[(nc * Ho + ho) * Wo + wo] * norm;
        dx[i] = acc;
    }
}
void k_avgpool_bwd(const float *g, long NC, int H, int W, int ph, int pw, int sh, int sw,
                   int Ho, int Wo, float *dx) {
    long total = NC * H * W;
    tt_trace_begin(TTB_K_SPATIAL);
    LAUNCH(avgpool_bwd_kernel, grid_for(total), TPB, 0, g, NC, H, W, ph, pw, sh, sw, Ho, Wo, dx);
    tt_trace_end(TTB_K_SPATIAL, 4.0 * ((double)total + (double)NC * Ho * Wo));
}
