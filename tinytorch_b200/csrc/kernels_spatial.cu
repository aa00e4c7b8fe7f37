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
#include <stdlib.h>

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
 * Organised by input plane: blockIdx.x is the plane (n, ci), a thread owns one output
 * position (ho, wo) of it and writes that position into the HH*WW rows of col that
 * belong to ci.  The position is decoded once, with 32-bit arithmetic; each of the
 * HH*WW steps is then a bounds test, one load (the plane is a few KB and is re-read
 * from L1) and one store, and a warp's stores are 128 consecutive bytes of one col row.
 * KH, KW > 0 fix the window at compile time so that the loops unroll. */
template <int KH, int KW>
__global__ void __launch_bounds__(TPB) im2col_kernel(const float *__restrict__ x, int C, int H, int W,
                                                      int HHr, int WWr, int ph, int pw, int sh, int sw,
                                                      int Ho, int Wo, long ncol, int planes, int tpp,
                                                      float *__restrict__ col) {
    const int HH = KH > 0 ? KH : HHr, WW = KW > 0 ? KW : WWr;
    /* tpp threads per plane: a block covers TPB / tpp small planes */
    const int sub = threadIdx.x / tpp, t = threadIdx.x - sub * tpp;
    const int ppb = TPB / tpp;
    const int sp = Ho * Wo;
    for (int plane = blockIdx.x * ppb + sub; plane < planes; plane += gridDim.x * ppb) {
    const int n = plane / C, ci = plane - n * C;
    const float *src = x + (long)plane * H * W;
    float *dst0 = col + (long)ci * HH * WW * ncol + (long)n * sp;
    for (int s = blockIdx.y * tpp + t; s < sp; s += gridDim.y * tpp) {
        const int ho = s / Wo, wo = s - ho * Wo;
        const int r0 = ho * sh - ph, q0 = wo * sw - pw;
        float *dst = dst0 + s;
        #pragma unroll
        for (int kh = 0; kh < HH; kh++) {
            const int row = r0 + kh;
            const bool row_ok = row >= 0 && row < H;
            #pragma unroll
            for (int kw = 0; kw < WW; kw++) {
                const int q = q0 + kw;
                float v = 0.0f;
                if (row_ok && q >= 0 && q < W) v = src[row * W + q];
                *dst = v;
                dst += ncol;
            }
        }
    }
    }
}
/* The common convolution -- 3x3 window, stride 1, padding 1, so Ho = H and Wo = W -- with
 * W in {4, 8, 16, 32, 64, 128}: a thread owns four neighbouring positions of one image
 * row.  It reads them with one aligned 128-bit load per window row; the two values the
 * window needs from beyond its four come from the neighbouring lanes by shuffle (W / 4
 * divides the warp, so an image row never straddles two warps, and the lanes at the row
 * ends substitute the zero padding).  Each window row then leaves as three 128-bit stores.
 * About 1.3 instructions per element written against 24 for the general kernel. */
__global__ void __launch_bounds__(TPB) im2col_3x3p1_kernel(const float *__restrict__ x, int C, int H, int W,
                                                            long ncol, int planes, int tpp, float *__restrict__ col) {
    const int sub = threadIdx.x / tpp, t = threadIdx.x - sub * tpp;
    const int ppb = TPB / tpp;
    const int W4 = W >> 2, groups = H * W4, sp = H * W;
    const int groups_up = (groups + 31) & ~31;
    for (int plane = blockIdx.x * ppb + sub; plane < planes; plane += gridDim.x * ppb) {
        const int n = plane / C, ci = plane - n * C;
        const float *src = x + (long)plane * sp;
        float *dst0 = col + (long)ci * 9 * ncol + (long)n * sp;
        for (int g = blockIdx.y * tpp + t; g < groups_up; g += gridDim.y * tpp) {
            const bool live = g < groups;
            const int ho = g / W4, w4 = g - ho * W4;
            float *dst = dst0 + (ho * W + w4 * 4);
            #pragma unroll
            for (int kh = 0; kh < 3; kh++) {
                const int row = ho - 1 + kh;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live && row >= 0 && row < H) v = *(const float4 *)(src + row * W + w4 * 4);
                float left = __shfl_up_sync(0xffffffffu, v.w, 1);
                float right = __shfl_down_sync(0xffffffffu, v.x, 1);
                if (w4 == 0) left = 0.0f;
                if (w4 == W4 - 1) right = 0.0f;
                if (live) {
                    *(float4 *)dst = make_float4(left, v.x, v.y, v.z);
                    *(float4 *)(dst + ncol) = v;
                    *(float4 *)(dst + 2 * ncol) = make_float4(v.y, v.z, v.w, right);
                }
                dst += 3 * ncol;
            }
        }
    }
}
/* The adjoint in the same shape: for each of the nine col rows one aligned 128-bit load of the
 * four values at (ho, w..w+3), the shifted neighbours by shuffle, and the additions in
 * (kh, kw) order from 0, skipping the windows that fall outside -- the sums of the general
 * gather, term for term. */
__global__ void __launch_bounds__(TPB) col2im_3x3p1_kernel(const float *__restrict__ col, int C, int H, int W,
                                                            long ncol, int planes, int tpp, float *__restrict__ x) {
    const int sub = threadIdx.x / tpp, t = threadIdx.x - sub * tpp;
    const int ppb = TPB / tpp;
    const int W4 = W >> 2, groups = H * W4, sp = H * W;
    const int groups_up = (groups + 31) & ~31;
    for (int plane = blockIdx.x * ppb + sub; plane < planes; plane += gridDim.x * ppb) {
        const int n = plane / C, ci = plane - n * C;
        const float *src0 = col + (long)ci * 9 * ncol + (long)n * sp;
        float *dst = x + (long)plane * sp;
        for (int g = blockIdx.y * tpp + t; g < groups_up; g += gridDim.y * tpp) {
            const bool live = g < groups;
            const int h = g / W4, w4 = g - h * W4;
            const float *src = src0 + w4 * 4;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            #pragma unroll
            for (int kh = 0; kh < 3; kh++) {
                const int ho = h + 1 - kh;
                const bool h_ok = live && ho >= 0 && ho < H;
                /* all three loads of this window row are issued before any is used */
                float4 v[3];
                #pragma unroll
                for (int kw = 0; kw < 3; kw++) {
                    v[kw] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (h_ok) v[kw] = *(const float4 *)(src + (long)(kh * 3 + kw) * ncol + ho * W);
                }
                /* kw = 0: wo = w + 1 .. w + 4, the last of them from the next lane */
                const float nx = __shfl_down_sync(0xffffffffu, v[0].x, 1);
                /* kw = 2: wo = w - 1 .. w + 2, the first of them from the previous lane */
                const float pv = __shfl_up_sync(0xffffffffu, v[2].w, 1);
                if (h_ok) {
                    acc.x = acc.x + v[0].y; acc.y = acc.y + v[0].z; acc.z = acc.z + v[0].w;
                    if (w4 != W4 - 1) acc.w = acc.w + nx;
                    acc.x = acc.x + v[1].x; acc.y = acc.y + v[1].y; acc.z = acc.z + v[1].z; acc.w = acc.w + v[1].w;
                    if (w4 != 0) acc.x = acc.x + pv;
                    acc.y = acc.y + v[2].x; acc.z = acc.z + v[2].y; acc.w = acc.w + v[2].z;
                }
            }
            if (live) *(float4 *)(dst + h * W + w4 * 4) = acc;
        }
    }
}
static bool conv3x3p1_fast(const void *a, const void *b, int H, int W, int HH, int WW, int ph, int pw, int sh, int sw,
                           int Ho, int Wo) {
    return HH == 3 && WW == 3 && ph == 1 && pw == 1 && sh == 1 && sw == 1 && Ho == H && Wo == W &&
           (W == 4 || W == 8 || W == 16 || W == 32 || W == 64 || W == 128) &&
           (((uintptr_t)a) & 15u) == 0 && (((uintptr_t)b) & 15u) == 0;
}

/* Planes go on grid.x (no 65535 limit), grid.y covers a plane's positions.  A plane smaller
 * than the block shares the block with its neighbours: tpp threads each, a power of two.
 * The kernels loop over planes with stride gridDim.x * (TPB / tpp). */
static dim3 spatial_grid(long planes, long positions, int *tpp_out) {
    int tpp = TPB;
    while (tpp > 32 && tpp / 2 >= positions) tpp /= 2;
    *tpp_out = tpp;
    const int ppb = TPB / tpp;
    long by = (positions + tpp - 1) / tpp;
    if (by > 64) by = 64;
    /* a few blocks per SM, each walking over many planes: blocks that live for one small plane
     * spend a large part of their time being scheduled */
    long bx = (planes + ppb - 1) / ppb;
    const long cap = ((long)g_tt.sm_count * 16 + by - 1) / by;
    if (bx > cap) bx = cap;
    return dim3((unsigned)bx, (unsigned)by);
}
void k_im2col(const float *x, int N, int C, int H, int W, int HH, int WW,
              int ph, int pw, int sh, int sw, int Ho, int Wo, float *col) {
    const long ncol = (long)N * Ho * Wo;
    const int kc = C * HH * WW;
    const long total = ncol * kc;
    if (total <= 0) return;
    int tpp;
    const int planes = N * C;
    const dim3 grid = spatial_grid(planes, (long)Ho * Wo, &tpp);
    tt_trace_begin(TTB_K_SPATIAL);
    if (conv3x3p1_fast(x, col, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo)) {
        int tpp4;
        const dim3 grid4 = spatial_grid(planes, (long)H * W / 4, &tpp4);
        LAUNCH(im2col_3x3p1_kernel, grid4, TPB, 0, x, C, H, W, ncol, planes, tpp4, col);
    } else if (HH == 3 && WW == 3)
        LAUNCH((im2col_kernel<3, 3>), grid, TPB, 0, x, C, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo, ncol, planes, tpp, col);
    else if (HH == 5 && WW == 5)
        LAUNCH((im2col_kernel<5, 5>), grid, TPB, 0, x, C, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo, ncol, planes, tpp, col);
    else
        LAUNCH((im2col_kernel<0, 0>), grid, TPB, 0, x, C, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo, ncol, planes, tpp, col);
    tt_trace_end(TTB_K_SPATIAL, 4.0 * ((double)total + (double)N * C * H * W));
}

/* Adjoint of im2col (src/autograd.c:406-434), as a gather: the element
 * x[n,ci,h,w] receives col[(ci,kh,kw),(n,ho,wo)] for every (kh,kw) with
 * ho*sh-ph+kh == h and wo*sw-pw+kw == w.  The reference adds them with
 * (kh,kw) ascending (its outer loop is c = (ci,kh,kw)); so does this, starting
 * from 0 and skipping the windows that do not reach the element.  Same
 * organisation as im2col: one plane per blockIdx.x, one element per thread,
 * loads issued without branches between them so that all HH*WW are in flight. */
template <int KH, int KW, bool UNIT_STRIDE>
__global__ void __launch_bounds__(TPB) col2im_kernel(const float *__restrict__ col, int C, int H, int W,
                                                      int HHr, int WWr, int ph, int pw, int sh, int sw,
                                                      int Ho, int Wo, long ncol, int planes, int tpp,
                                                      float *__restrict__ x) {
    const int HH = KH > 0 ? KH : HHr, WW = KW > 0 ? KW : WWr;
    const int sub = threadIdx.x / tpp, t = threadIdx.x - sub * tpp;
    const int ppb = TPB / tpp;
    const int sp = Ho * Wo, HW = H * W;
    for (int plane = blockIdx.x * ppb + sub; plane < planes; plane += gridDim.x * ppb) {
    const int n = plane / C, ci = plane - n * C;
    const float *src0 = col + (long)ci * HH * WW * ncol + (long)n * sp;
    float *dst = x + (long)plane * HW;
    for (int pix = blockIdx.y * tpp + t; pix < HW; pix += gridDim.y * tpp) {
        const int h = pix / W, w = pix - h * W;
        const float *src = src0;
        float acc = 0.0f;
        #pragma unroll
        for (int kh = 0; kh < HH; kh++) {
            int ho = h + ph - kh;
            bool h_ok = ho >= 0;
            if (!UNIT_STRIDE) { h_ok = h_ok && (ho % sh == 0); ho /= sh; }
            h_ok = h_ok && ho < Ho;
            #pragma unroll
            for (int kw = 0; kw < WW; kw++) {
                int wo = w + pw - kw;
                bool ok = h_ok && wo >= 0;
                if (!UNIT_STRIDE) { ok = ok && (wo % sw == 0); wo /= sw; }
                ok = ok && wo < Wo;
                float v = 0.0f;
                if (ok) v = src[ho * Wo + wo];
                acc = ok ? acc + v : acc;
                src += ncol;
            }
        }
        dst[pix] = acc;
    }
    }
}
void k_col2im(const float *col, int N, int C, int H, int W, int HH, int WW,
              int ph, int pw, int sh, int sw, int Ho, int Wo, float *x) {
    const long total = (long)N * C * H * W;
    if (total <= 0) return;
    const long ncol = (long)N * Ho * Wo;
    int tpp;
    const int planes = N * C;
    const dim3 grid = spatial_grid(planes, (long)H * W, &tpp);
    tt_trace_begin(TTB_K_SPATIAL);
    if (conv3x3p1_fast(x, col, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo)) {
        int tpp4;
        const dim3 grid4 = spatial_grid(planes, (long)H * W / 4, &tpp4);
        LAUNCH(col2im_3x3p1_kernel, grid4, TPB, 0, col, C, H, W, ncol, planes, tpp4, x);
    } else if (sh == 1 && sw == 1 && HH == 3 && WW == 3)
        LAUNCH((col2im_kernel<3, 3, true>), grid, TPB, 0, col, C, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo, ncol, planes, tpp, x);
    else if (sh == 1 && sw == 1)
        LAUNCH((col2im_kernel<0, 0, true>), grid, TPB, 0, col, C, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo, ncol, planes, tpp, x);
    else
        LAUNCH((col2im_kernel<0, 0, false>), grid, TPB, 0, col, C, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo, ncol, planes, tpp, x);
    tt_trace_end(TTB_K_SPATIAL, 4.0 * ((double)total + (double)C * HH * WW * N * Ho * Wo));
}

/* The two permutes around the convolution GEMMs move whole planes of sp floats:
 *   unpermute: out[n,f,:] = om[f, n*sp : (n+1)*sp] + bias[f]   (src/ops_spatial.c:105-119)
 *   permute:   gp[f, n*sp : (n+1)*sp] = g[n,f,:]               (src/autograd.c:494-501)
 * blockIdx.x is the plane (n*F + f); threads run along the plane, 128 bits at a time. */
template <bool TO_NCHW>
__global__ void __launch_bounds__(TPB) conv_plane_kernel(const float *__restrict__ src, const float *__restrict__ bias,
                                                          int N, int F, int sp, float *__restrict__ dst) {
    const int plane = blockIdx.x;
    const int n = plane / F, f = plane - n * F;
    const long nchw = (long)plane * sp, fnhw = ((long)f * N + n) * sp;
    const float *in = src + (TO_NCHW ? fnhw : nchw);
    float *out = dst + (TO_NCHW ? nchw : fnhw);
    const float b = (TO_NCHW && bias) ? bias[f] : 0.0f;
    const bool vec = ((sp & 3) == 0) && ((((uintptr_t)src) & 15u) == 0) && ((((uintptr_t)dst) & 15u) == 0);
    if (vec) {
        for (int i = (blockIdx.y * TPB + threadIdx.x) * 4; i < sp; i += gridDim.y * TPB * 4) {
            float4 v = *(const float4 *)(in + i);
            if (TO_NCHW) { v.x = v.x + b; v.y = v.y + b; v.z = v.z + b; v.w = v.w + b; }
            *(float4 *)(out + i) = v;
        }
    } else {
        for (int i = blockIdx.y * TPB + threadIdx.x; i < sp; i += gridDim.y * TPB)
            out[i] = TO_NCHW ? in[i] + b : in[i];
    }
}
static dim3 plane_grid(int N, int F, long sp) {
    long by = (sp + 4 * TPB - 1) / (4 * TPB);
    if (by > 64) by = 64;
    return dim3((unsigned)((long)N * F), (unsigned)by);
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
/* 2x2 windows with stride 2 that tile the plane exactly (H = 2 Ho, W = 2 Wo, W a multiple
 * of 4): a thread takes two neighbouring windows -- one 128-bit load from each of the two
 * input rows, one 64-bit store -- and the index decode is one division per thread.
 * Row r of the output (r = (n*C + c)*Ho + ho) reads input rows 2r and 2r+1, so the plane
 * index never has to be separated out.  Scan order and the strict '>' are those of
 * window_argmax. */
__device__ __forceinline__ int scan4(float v0, float v1, float v2, float v3, float &best) {
    best = -INFINITY;
    int k = 0;
    if (v0 > best) { best = v0; k = 0; }
    if (v1 > best) { best = v1; k = 1; }
    if (v2 > best) { best = v2; k = 2; }
    if (v3 > best) { best = v3; k = 3; }
    return k;
}
template <typename IT>
__global__ void __launch_bounds__(TPB) maxpool2x2_kernel(const float4 *__restrict__ x, IT total, int Wq, float2 *__restrict__ out) {
    const IT stride = (IT)gridDim.x * TPB;
    for (IT i = (IT)blockIdx.x * TPB + threadIdx.x; i < total; i += stride) {
        const IT r = i / Wq;
        const int j = (int)(i - r * Wq);
        const float4 a = x[2 * r * Wq + j], b = x[(2 * r + 1) * Wq + j];
        float2 o;
        scan4(a.x, a.y, b.x, b.y, o.x);
        scan4(a.z, a.w, b.z, b.w, o.y);
        out[i] = o;
    }
}
template <typename IT>
__global__ void __launch_bounds__(TPB) maxpool2x2_bwd_kernel(const float4 *__restrict__ x, const float2 *__restrict__ g, IT total,
                                                              int Wq, float4 *__restrict__ dx) {
    const IT stride = (IT)gridDim.x * TPB;
    for (IT i = (IT)blockIdx.x * TPB + threadIdx.x; i < total; i += stride) {
        const IT r = i / Wq;
        const int j = (int)(i - r * Wq);
        const float4 a = x[2 * r * Wq + j], b = x[(2 * r + 1) * Wq + j];
        const float2 gv = g[i];
        float best;
        const int k0 = scan4(a.x, a.y, b.x, b.y, best);
        const int k1 = scan4(a.z, a.w, b.z, b.w, best);
        const float g0 = 0.0f + gv.x, g1 = 0.0f + gv.y;
        dx[2 * r * Wq + j] = make_float4(k0 == 0 ? g0 : 0.0f, k0 == 1 ? g0 : 0.0f, k1 == 0 ? g1 : 0.0f, k1 == 1 ? g1 : 0.0f);
        dx[(2 * r + 1) * Wq + j] = make_float4(k0 == 2 ? g0 : 0.0f, k0 == 3 ? g0 : 0.0f, k1 == 2 ? g1 : 0.0f, k1 == 3 ? g1 : 0.0f);
    }
}
static bool pool2x2_fast(const void *x, const void *small, int H, int W, int ph, int pw, int sh, int sw, int Ho, int Wo) {
    return ph == 2 && pw == 2 && sh == 2 && sw == 2 && H == 2 * Ho && W == 2 * Wo && (W & 3) == 0 &&
           (((uintptr_t)x) & 15u) == 0 && (((uintptr_t)small) & 7u) == 0;
}
void k_maxpool(const float *x, long NC, int H, int W, int ph, int pw, int sh, int sw,
               int Ho, int Wo, float *out) {
    long total = NC * Ho * Wo;
    tt_trace_begin(TTB_K_SPATIAL);
    if (pool2x2_fast(x, out, H, W, ph, pw, sh, sw, Ho, Wo)) {
        const long items = total / 2;
        if (items < 0x7fffffffL / 4)
            LAUNCH(maxpool2x2_kernel<int>, grid_for(items), TPB, 0, (const float4 *)x, (int)items, W / 4, (float2 *)out);
        else
            LAUNCH(maxpool2x2_kernel<long>, grid_for(items), TPB, 0, (const float4 *)x, items, W / 4, (float2 *)out);
    } else
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
    if (pool2x2_fast(x, g, H, W, ph, pw, sh, sw, Ho, Wo) && (((uintptr_t)dx) & 15u) == 0) {
        const long items = NC * Ho * Wo / 2;
        if (items < 0x7fffffffL / 4)
            LAUNCH(maxpool2x2_bwd_kernel<int>, grid_for(items), TPB, 0, (const float4 *)x, (const float2 *)g, (int)items, W / 4, (float4 *)dx);
        else
            LAUNCH(maxpool2x2_bwd_kernel<long>, grid_for(items), TPB, 0, (const float4 *)x, (const float2 *)g, items, W / 4, (float4 *)dx);
    } else if (sh == ph && sw == pw && Ho * ph == H && Wo * pw == W)
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
