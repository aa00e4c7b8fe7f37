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
 * One block row per row of col, four consecutive columns per thread (one
 * 128-bit store), wo fastest: reads and writes are both runs of consecutive
 * addresses for stride 1, and the index decode is 32-bit. */
__global__ void __launch_bounds__(TPB) im2col_kernel(const float *__restrict__ x, int N, int C, int H, int W,
                                                      int HH, int WW, int ph, int pw, int sh, int sw,
                                                      int Ho, int Wo, float *__restrict__ col) {
    /* blockIdx.y = row of col (c_im, kh, kw); each thread produces four consecutive columns */
    const int c = blockIdx.y;
    const int kw = c % WW, kh = (c / WW) % HH, ci = c / (HH * WW);
    const int sp = Ho * Wo;
    const long ncol = (long)N * sp;
    const long r0 = ((long)blockIdx.x * TPB + threadIdx.x) * 4;
    if (r0 >= ncol) return;
    float *dst = col + (long)c * ncol + r0;
    int n = (int)(r0 / sp);
    int s = (int)(r0 - (long)n * sp);
    int ho = s / Wo, wo = s - ho * Wo;
    float v[4];
    #pragma unroll
    for (int j = 0; j < 4; j++) {
        v[j] = 0.0f;
        if (r0 + j < ncol) {
            const int row = ho * sh - ph + kh, q = wo * sw - pw + kw;
            if (row >= 0 && row < H && q >= 0 && q < W)
                v[j] = x[(((long)n * C + ci) * H + row) * W + q];
        }
        if (++wo == Wo) { wo = 0; if (++ho == Ho) { ho = 0; n++; } }
    }
    if (r0 + 3 < ncol && ((ncol & 3) == 0) && ((((uintptr_t)col) & 15u) == 0)) {
        *(float4 *)dst = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        #pragma unroll
        for (int j = 0; j < 4; j++) if (r0 + j < ncol) dst[j] = v[j];
    }
}
void k_im2col(const float *x, int N, int C, int H, int W, int HH, int WW,
              int ph, int pw, int sh, int sw, int Ho, int Wo, float *col) {
    const long ncol = (long)N * Ho * Wo;
    const int kc = C * HH * WW;
    const long total = ncol * kc;
    dim3 grid((unsigned)((ncol + 4 * TPB - 1) / (4 * TPB)), (unsigned)kc);
    tt_trace_begin(TTB_K_SPATIAL);
    LAUNCH(im2col_kernel, grid, TPB, 0, x, N, C, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo, col);
    tt_trace_end(TTB_K_SPATIAL, 4.0 * ((double)total + (double)N * C * H * W));
}

/* Adjoint of im2col (src/autograd.c:406-434), as a gather: the element
 * x[n,ci,h,w] receives col[(ci,kh,kw),(n,ho,wo)] for every (kh,kw) with
 * ho*sh-ph+kh == h and wo*sw-pw+kw == w.  The reference adds them with
 * (kh,kw) ascending (its outer loop is c = (ci,kh,kw)); so does this. */
template <bool UNIT_STRIDE>
__global__ void __launch_bounds__(TPB) col2im_kernel(const float *__restrict__ col, int N, int C, int H, int W,
                                                      int HH, int WW, int ph, int pw, int sh, int sw,
                                                      int Ho, int Wo, float *__restrict__ x) {
    const long sp = (long)Ho * Wo, ncol = (long)N * sp;
    const long total = (long)N * C * H * W;
    const long stride = (long)gridDim.x * blockDim.x;
    const int HW = H * W;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long plane = i / HW;                      /* n*C + ci */
        const int pix = (int)(i - plane * HW);
        const int h = pix / W, w = pix - h * W;
        const int n = (int)(plane / C), ci = (int)(plane - (long)n * C);
        const float *src = col + ((long)ci * HH * WW) * ncol + (long)n * sp;
        float acc = 0.0f;
        for (int kh = 0; kh < HH; kh++) {
            int ho = h + ph - kh;
            if (!UNIT_STRIDE) { if (ho < 0 || ho % sh) continue; ho /= sh; }
            if (ho < 0 || ho >= Ho) continue;
            for (int kw = 0; kw < WW; kw++) {
                int wo = w + pw - kw;
                if (!UNIT_STRIDE) { if (wo < 0 || wo % sw) continue; wo /= sw; }
                if (wo < 0 || wo >= Wo) continue;
                acc = acc + src[(long)(kh * WW + kw) * ncol + (long)ho * Wo + wo];
            }
        }
        x[i] = acc;
    }
}
void k_col2im(const float *col, int N, int C, int H, int W, int HH, int WW,
              int ph, int pw, int sh, int sw, int Ho, int Wo, float *x) {
    long total = (long)N * C * H * W;
    tt_trace_begin(TTB_K_SPATIAL);
    if (sh == 1 && sw == 1)
        LAUNCH(col2im_kernel<true>, grid_for(total), TPB, 0, col, N, C, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo, x);
    else
        LAUNCH(col2im_kernel<false>, grid_for(total), TPB, 0, col, N, C, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo, x);
    tt_trace_end(TTB_K_SPATIAL, 4.0 * ((double)total + (double)C * HH * WW * N * Ho * Wo));
}

/* The two permutes around the convolution GEMMs move whole planes of sp floats:
 *   unpermute: out[n,f,:] = om[f, n*sp : (n+1)*sp] + bias[f]   (src/ops_spatial.c:105-119)
 *   permute:   gp[f, n*sp : (n+1)*sp] = g[n,f,:]               (src/autograd.c:494-501)
 * blockIdx.y is the plane (n*F + f); threads run along the plane, 128 bits at a time. */
template <bool TO_NCHW>
__global__ void __launch_bounds__(TPB) conv_plane_kernel(const float *__restrict__ src, const float *__restrict__ bias,
                                                          int N, int F, int sp, float *__restrict__ dst) {
    const int plane = blockIdx.y;
    const int n = plane / F, f = plane - n * F;
    const long nchw = (long)plane * sp, fnhw = ((long)f * N + n) * sp;
    const float *in = src + (TO_NCHW ? fnhw : nchw);
    float *out = dst + (TO_NCHW ? nchw : fnhw);
    const float b = (TO_NCHW && bias) ? bias[f] : 0.0f;
    const bool vec = ((sp & 3) == 0) && ((((uintptr_t)src) & 15u) == 0) && ((((uintptr_t)dst) & 15u) == 0);
    if (vec) {
        for (int i = (blockIdx.x * TPB + threadIdx.x) * 4; i < sp; i += gridDim.x * TPB * 4) {
            float4 v = *(const float4 *)(in + i);
            if (TO_NCHW) { v.x = v.x + b; v.y = v.y + b; v.z = v.z + b; v.w = v.w + b; }
            *(float4 *)(out + i) = v;
        }
    } else {
        for (int i = blockIdx.x * TPB + threadIdx.x; i < sp; i += gridDim.x * TPB)
            out[i] = TO_NCHW ? in[i] + b : in[i];
    }
}
static dim3 plane_grid(int N, int F, long sp) {
    long bx = (sp + 4 * TPB - 1) / (4 * TPB);
    if (bx > 64) bx = 64;
    return dim3((unsigned)bx, (unsigned)(N * F));
}
void k_conv_unpermute_bias(const float *om, const float *bias, int N, int F, long sp, float *out) {
    tt_trace_begin(TTB_K_SPATIAL);
    LAUNCH(conv_plane_kernel<true>, plane_grid(N, F, sp), TPB, 0, om, bias, N, F, (int)sp, out);
    tt_trace_end(TTB_K_SPATIAL, 8.0 * (double)N * F * sp);
}
void k_conv_permute(const float *g, int N, int F, long sp, float *gp) {
    tt_trace_begin(TTB_K_SPATIAL);
    LAUNCH(conv_plane_kernel<false>, plane_grid(N, F, sp), TPB, 0, g, nullptr, N, F, (int)sp, gp);
    tt_trace_end(TTB_K_SPATIAL, 8.0 * (double)N * F * sp);
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
/* Windows that tile the plane exactly (stride == pool, no leftover rows or columns):
 * one thread owns one window, finds its arg-max and writes the whole window -- the
 * gradient at the winner, zero elsewhere.  Same values as the gather above (each
 * element belongs to exactly one window), a quarter of the index arithmetic. */
__global__ void __launch_bounds__(TPB) maxpool_bwd_tiled_kernel(const float *__restrict__ x, const float *__restrict__ g, long NC,
                                                                 int H, int W, int ph, int pw, int Ho, int Wo,
                                                                 float *__restrict__ dx) {
    const long total = NC * Ho * Wo;
    const long stride = (long)gridDim.x * blockDim.x;
    const int sp = Ho * Wo;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long nc = i / sp;
        const int s = (int)(i - nc * sp);
        const int ho = s / Wo, wo = s - ho * Wo;
        const float *plane = x + nc * H * W;
        float best; int bh, bw;
        window_argmax(plane, W, ho * ph, wo * pw, ph, pw, best, bh, bw);
        const float gv = g[i];
        float *out = dx + nc * H * W;
        for (int kh = 0; kh < ph; kh++)
            for (int kw = 0; kw < pw; kw++) {
                const int hh = ho * ph + kh, ww = wo * pw + kw;
                out[(long)hh * W + ww] = (hh == bh && ww == bw) ? 0.0f + gv : 0.0f;
            }
    }
}
void k_maxpool_bwd(const float *x, const float *g, long NC, int H, int W, int ph, int pw,
                   int sh, int sw, int Ho, int Wo, float *dx) {
    long total = NC * H * W;
    tt_trace_begin(TTB_K_SPATIAL);
    if (sh == ph && sw == pw && Ho * ph == H && Wo * pw == W)
        LAUNCH(maxpool_bwd_tiled_kernel, grid_for(NC * Ho * Wo), TPB, 0, x, g, NC, H, W, ph, pw, Ho, Wo, dx);
    else
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
