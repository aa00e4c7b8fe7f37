/* Implicit-GEMM convolution on the tensor cores: forward, weight gradient and input gradient
 * without a materialised im2col matrix.
 *
 * The reference builds col[C*kh*kw, N*Hout*Wout] with batched_im2col, multiplies, and permutes
 * (tt_conv2d, src/ops_spatial.c:71-127); backward it builds col again for dW, a second matrix
 * d_col for dX and scatters it back with col2im (backward_conv2d, src/autograd.c:456-553).  Here
 * the three products read the image (or the output gradient) directly:
 *
 *   fprop  out[n,f,ho,wo] = b[f] + sum_{c,kh,kw} x[n,c,ho*s-p+kh, wo*s-p+kw] * W[f,c,kh,kw]
 *          rows = output positions (128 per tile), columns = filters, reduction = (c,kh,kw)
 *   dgrad  dX[n,c,h,w]    = sum_{f,kh,kw} g[n,f,h+p-kh, w+p-kw] * W[f,c,kh,kw]      (stride 1)
 *          rows = input positions, columns = channels, reduction = (f,kh,kw)
 *   wgrad  dW[f,(c,kh,kw)] = sum_{n,ho,wo} x[n,c,ho*s-p+kh, wo*s-p+kw] * g[n,f,ho,wo]
 *          rows = (c,kh,kw), columns = filters, reduction = output positions, cut into slices
 *          over the CTAs whose partial tiles a second kernel adds in order
 *
 * One kernel serves all three.  Its operand tiles are not copied by TMA (a window shifted by one
 * pixel starts 4 bytes off the 16-byte boundary a TMA copy needs) but GATHERED: eight producer
 * warps compute the source index of every tile element, load it (neighbouring taps hit L1/L2),
 * and write the raw value AND the lo part of its 3xTF32 split straight into the K-major,
 * 128-byte-swizzled layout the tensor core reads, so there is no separate split pass either.
 * One thread issues tcgen05.mma kind::tf32 (lo*hi, hi*lo, hi*hi per K step of 8), accumulators
 * live in tensor memory (two, so that the epilogue of a tile overlaps the next tile's MMAs),
 * four epilogue warps read them back and store NCHW rows (32 consecutive positions of one
 * filter per warp: full 128-byte lines) with the bias added.
 *
 * Padding and ragged edges are zeros in the tiles.  Every wait is bounded and reports through
 * the same host-visible status word as the GEMM. */
#include "tt_internal.h"
#include "tcgen05_utils.cuh"

#include <stdlib.h>
#include <string.h>

#define CV_BM 128
#define CV_BK 32
#define CV_EPI_WARPS 4
#define CV_PROD_WARPS 8
#define CV_PROD_THREADS (CV_PROD_WARPS * 32)
#define CV_THREADS ((CV_EPI_WARPS + 1 + CV_PROD_WARPS) * 32)      /* warps 0-3 epilogue, 4 MMA, 5-12 producers */
#define CV_MAX_TAPS 2048                                          /* entries of the (channel, kh, kw) table */
#define CV_A_BYTES (CV_BM * CV_BK * 4)

enum { CV_FPROP = 0, CV_DGRAD = 1, CV_WGRAD = 2 };

struct ConvParams {
    int mode;
    int N, C, H, W, F, HH, WW, sh, sw, ph, pw, Ho, Wo;
    const float *x;          /* fprop, wgrad: image [N,C,H,W] */
    const float *w;          /* fprop, dgrad: filters [F,C,HH,WW] */
    const float *g;          /* dgrad, wgrad: output gradient [N,F,Ho,Wo] */
    const float *bias;       /* fprop: [F] or NULL */
    float *out;              /* fprop: [N,F,Ho,Wo]; dgrad: [N,C,H,W]; wgrad: partial tiles [slices][taps][F] */
    int accumulate;          /* dgrad: add into out */
    long rows_a;             /* valid rows of the A operand: positions (fprop, dgrad) or taps (wgrad) */
    int rows_b;              /* valid rows of the B operand: F (fprop, wgrad) or C (dgrad) */
    int bn;                  /* accumulator width: rows_b rounded up to a multiple of 16 */
    long kdim;               /* reduction length: taps (fprop), F*HH*WW (dgrad), positions (wgrad) */
    int num_kb, kb_per_item; /* K blocks in all, and per work item (wgrad slices; otherwise all) */
    int m_tiles, items;
    int taps;                /* table entries: (channel, kh, kw) for every tap index */
    int stages;
    uint32_t tmem_cols;
    uint32_t *status;
};

/* Bounded wait for the warps that have nothing else to do (MMA issuer, epilogue): between polls the
 * thread sleeps, so that the instruction issue slots go to the producer warps, whose index arithmetic
 * is what bounds this kernel. */
__device__ __forceinline__ bool cv_wait_idle(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                             uint32_t *status, uint32_t code) {
    if (mbar_try(bar, parity)) return true;
    long long t0 = clock64();
    for (;;) {
        __nanosleep(100);
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > TC_WAIT_CYCLES) {
            *abort_flag = 1;
            *(volatile uint32_t *)status = code | (blockIdx.x << 8);
            __threadfence_system();
            return false;
        }
    }
}
__device__ __forceinline__ bool cv_wait_idle_warp(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                                  uint32_t *status, uint32_t code) {
    bool got = true;
    if ((threadIdx.x & 31) == 0) got = cv_wait_idle(bar, parity, abort_flag, status, code);
    got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
    if (got) got = mbar_wait(bar, parity, abort_flag, status, code);     /* immediate: the phase is complete */
    return __all_sync(0xffffffffu, got);
}

#ifdef TT_TUNING
__device__ unsigned long long g_cv_dbg[16];
extern "C" int ttb_debug_conv_read(unsigned long long out[16]) {
    cudaStreamSynchronize(g_tt.stream);
    unsigned long long z[16] = {0};
    if (cudaMemcpyFromSymbol(out, g_cv_dbg, sizeof z) != cudaSuccess) return -1;
    cudaMemcpyToSymbol(g_cv_dbg, z, sizeof z);
    return 0;
}
#define CV_STAMP(i, t0) do { if (blockIdx.x == 0 && gt == 0 && grp == 0) { long long now_ = clock64(); atomicAdd(&g_cv_dbg[i], (unsigned long long)(now_ - (t0))); (t0) = now_; } } while (0)
#else
#define CV_STAMP(i, t0) do { } while (0)
#endif

__device__ __forceinline__ uint32_t cv_swz(uint32_t off) { return off ^ (((off >> 7) & 7u) << 4); }

/* Gather arithmetic.  Every element of an operand tile is src[rowbase + tapoff] or zero:
 *   fprop / wgrad   x[n, ch, oh*sh - ph + kh, ow*sw - pw + kw]
 *       rowbase = n*C*H*W + (oh*sh - ph)*W + (ow*sw - pw)      (from the output position)
 *       tapoff  = ch*H*W + kh*W + kw                            (from the tap)
 *       inside the image iff 0 <= (oh*sh - ph) + kh < H and 0 <= (ow*sw - pw) + kw < W
 *   dgrad (stride 1) g[n, f, h + ph - kh, w + pw - kw]
 *       rowbase = n*F*Ho*Wo + (h + ph)*Wo + (w + pw);  tapoff = f*Ho*Wo - kh*Wo - kw
 *       inside iff 0 <= (h + ph) - kh < Ho and 0 <= (w + pw) - kw < Wo
 * Whether tap (kh, kw) falls inside depends on the position only, so each position gets a bit mask
 * over the kh*WW + kw window slots once (the window has at most 31 slots), and the table holds
 * {tapoff, slot} per tap: an element then costs a shift, an and, one address add and the load.
 * Table entries beyond the last tap name slot 31, which no mask has, and read as zero. */
struct CvRow { const float *ptr; uint32_t mask; };
__device__ __forceinline__ float cv_elem(const CvRow &r, int2 tap) {
    return ((r.mask >> tap.y) & 1u) ? __ldg(r.ptr + tap.x) : 0.0f;      /* a predicated load: measured faster than loading a dummy */
}
/* Row descriptor of output position (n, oh, ow) for fprop / wgrad, of input position (n, h, w) for dgrad. */
template <int MODE>
__device__ __forceinline__ CvRow cv_row(const ConvParams &p, int n, int y, int x) {
    CvRow r;
    int y0, x0;
    if (MODE == CV_DGRAD) {
        y0 = y + p.ph; x0 = x + p.pw;
        r.ptr = p.g + (long)n * p.F * p.Ho * p.Wo + (long)y0 * p.Wo + x0;
    } else {
        y0 = y * p.sh - p.ph; x0 = x * p.sw - p.pw;
        r.ptr = p.x + (long)n * p.C * p.H * p.W + (long)y0 * p.W + x0;
    }
    const int ylim = MODE == CV_DGRAD ? p.Ho : p.H, xlim = MODE == CV_DGRAD ? p.Wo : p.W;
    uint32_t xm = 0;
    for (int kw = 0; kw < p.WW; kw++)
        if ((unsigned)(MODE == CV_DGRAD ? x0 - kw : x0 + kw) < (unsigned)xlim) xm |= 1u << kw;
    uint32_t m = 0;
    for (int kh = 0; kh < p.HH; kh++)
        if ((unsigned)(MODE == CV_DGRAD ? y0 - kh : y0 + kh) < (unsigned)ylim) m |= xm << (kh * p.WW);
    r.mask = m;
    return r;
}

__device__ __forceinline__ void cv_put(uint8_t *hi, uint32_t lo_delta, uint32_t off, float4 v) {
    *(float4 *)(hi + off) = v;
    *(float4 *)(hi + lo_delta + off) = make_float4(split_lo(v.x), split_lo(v.y), split_lo(v.z), split_lo(v.w));
}

template <int MODE>
__global__ void __launch_bounds__(CV_THREADS, 1) conv_tc_kernel(ConvParams p) {
    extern __shared__ uint8_t cv_smem_raw[];
    const uint32_t smem_base = (smem_u32(cv_smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = cv_smem_raw + (smem_base - smem_u32(cv_smem_raw));
    const uint32_t b_bytes = (uint32_t)p.bn * CV_BK * 4;
    const uint32_t stage_bytes = 2 * (CV_A_BYTES + b_bytes);          /* A hi, A lo, B hi, B lo */
    int2 *ktab = (int2 *)(smem_gen + (size_t)p.stages * stage_bytes);
    int *wtab = (int *)(ktab + CV_MAX_TAPS);                           /* dgrad: where tap (f,kh,kw) sits in the filter bank, for channel 0 */
    uint64_t *bars = (uint64_t *)(wtab + CV_MAX_TAPS);
    const uint32_t bar_full = smem_u32(bars);                           /* stages */
    const uint32_t bar_empty = bar_full + 8 * p.stages;                 /* stages */
    const uint32_t bar_tfull = bar_empty + 8 * p.stages;                /* 2 */
    const uint32_t bar_tempty = bar_tfull + 16;                         /* 2 */
    uint32_t *tmem_slot = (uint32_t *)(bars + 2 * p.stages + 4);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    float *sbias = (float *)(tmem_slot + 4);                            /* 256: the epilogue reads the bias from here, so its loads
                                                                          * need not be ordered against the stores of the tile */

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bn32 = (p.bn + 31) & ~31;                                 /* accumulator pitch in tensor-memory columns */
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)(CV_BM >> 4) << 24);
    const long sp_out = (long)p.Ho * p.Wo, sp_in = (long)p.H * p.W;

    for (int c = threadIdx.x; c < 256; c += CV_THREADS) sbias[c] = (p.bias && c < p.rows_b) ? p.bias[c] : 0.0f;
    for (int k = threadIdx.x; k < ((p.taps + 31) & ~31); k += CV_THREADS) {
        const int hw = p.HH * p.WW, ch = k / hw, rem = k - ch * hw, kh = rem / p.WW, kw = rem - kh * p.WW;
        if (k >= p.taps) { ktab[k] = make_int2(0, 31); wtab[k] = 0; continue; }
        if (MODE == CV_DGRAD) {
            ktab[k] = make_int2(ch * p.Ho * p.Wo - kh * p.Wo - kw, rem);
            wtab[k] = ch * p.C * hw + kh * p.WW + kw;
        } else {
            ktab[k] = make_int2(ch * p.H * p.W + kh * p.W + kw, rem);
        }
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(bar_full + 8 * s, CV_PROD_WARPS / p.stages);     /* one arrival per warp of the group that fills it */
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, CV_EPI_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == CV_EPI_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    /* work item -> tile of A rows and K-block range */
    auto decode = [&](int it, long &m0, int &kb0, int &kb1, int &slice) {
        const int mt = it % p.m_tiles;
        slice = it / p.m_tiles;
        m0 = (long)mt * CV_BM;
        kb0 = slice * p.kb_per_item;
        kb1 = kb0 + p.kb_per_item < p.num_kb ? kb0 + p.kb_per_item : p.num_kb;
    };

    if (warp > CV_EPI_WARPS) {
        /* ---------------- producers: gather, split, store swizzled ----------------
         * Filling a stage is a chain of dependent latencies (wait, index arithmetic, loads, stores,
         * fence, arrive), so the eight warps work as independent groups, one per stage (2 or 4):
         * group g fills the K blocks whose running number is g modulo the stage count, always into
         * stage g, and all stages are being filled at the same time. */
        const int pt = threadIdx.x - (CV_EPI_WARPS + 1) * 32;          /* 0..255 */
        const int gthreads = CV_PROD_THREADS / p.stages;               /* 64 or 128 */
        const int grp = pt / gthreads, gt = pt % gthreads;
        const uint32_t lo_a = CV_A_BYTES, lo_b = b_bytes;
        const int hw = p.HH * p.WW;
        long seq = 0;                                                   /* running number of the K block in this CTA */
        int zeroed_for = -1;                                            /* wgrad: item for which this group's stage has its unused rows cleared */
        bool ok = true;
        for (int it = blockIdx.x; it < p.items && ok; it += gridDim.x) {
            long m0; int kb0, kb1, slice;
            decode(it, m0, kb0, kb1, slice);
            /* position-major A tiles (fprop, dgrad): this thread fills rows gt (and gt + 64) */
            CvRow arow[2];
            arow[0].ptr = arow[1].ptr = p.x; arow[0].mask = arow[1].mask = 0;      /* mask 0: the row reads as zeros */
            if (MODE != CV_WGRAD) {
                #pragma unroll
                for (int h = 0; h < 2; h++) {
                    const long pa = m0 + gt + h * gthreads;
                    if (gt + h * gthreads < CV_BM && pa < p.rows_a) {
                        const int spp = (int)(MODE == CV_FPROP ? sp_out : sp_in);      /* positions fit 31 bits (checked on the host) */
                        const int wd = MODE == CV_FPROP ? p.Wo : p.W;
                        const int n = (int)pa / spp;
                        const int q = (int)pa - n * spp;
                        const int y = q / wd;
                        arow[h] = cv_row<MODE>(p, n, y, q - y * wd);
                    }
                }
            }
            for (int kb = kb0; kb < kb1; kb++, seq++) {
                const int s = (int)(seq % p.stages);
                if (s != grp) continue;
                const uint32_t ph = (uint32_t)((seq / p.stages) & 1);
                long long tstamp = clock64(); (void)tstamp;
                uint8_t *a_hi = smem_gen + (size_t)s * stage_bytes;
                uint8_t *b_hi = a_hi + 2 * CV_A_BYTES;
                const int k0 = kb * CV_BK;
                /* The stage is still being read by the tensor core while this group comes round again, so
                 * the loads that fit in registers (the first batch of B and of A, 64 values per thread) are
                 * issued BEFORE the wait for the stage: their latency overlaps the wait, and only the
                 * stores (and, for 64-thread groups, the second A row) follow it. */
                if (MODE != CV_WGRAD) {
                    /* A: 128 positions x 32 taps; lanes run along the positions (contiguous in the image).
                     * B: filters (fprop) or channels (dgrad) x 32 taps, eight 16-byte chunks per thread and batch. */
                    const int4 *tab4 = (const int4 *)(ktab + k0);               /* two taps per 16-byte read */
                    auto load_a = [&](int h, float (&v)[32]) {
                        #pragma unroll
                        for (int q = 0; q < 16; q++) {
                            const int4 t2 = tab4[q];
                            v[2 * q] = cv_elem(arow[h], make_int2(t2.x, t2.y));
                            v[2 * q + 1] = cv_elem(arow[h], make_int2(t2.z, t2.w));
                        }
                    };
                    auto put_a = [&](int h, const float (&v)[32]) {
                        const int ra = gt + h * gthreads;
                        #pragma unroll
                        for (int q = 0; q < 8; q++)
                            cv_put(a_hi, lo_a, cv_swz((uint32_t)ra * 128u + (uint32_t)q * 16u),
                                   make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
                    };
                    auto load_b = [&](int t0, float4 (&v)[8]) {
                        #pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const int t = t0 + j * gthreads, r = t >> 3, q = t & 7;
                            float e4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                            if (t < p.bn * 8 && r < p.rows_b) {
                                #pragma unroll
                                for (int e = 0; e < 4; e++) {
                                    const int k = k0 + q * 4 + e;
                                    if (k < p.kdim)
                                        e4[e] = MODE == CV_FPROP ? __ldg(p.w + (long)r * p.kdim + k) : __ldg(p.w + (long)r * hw + wtab[k]);
                                }
                            }
                            v[j] = make_float4(e4[0], e4[1], e4[2], e4[3]);
                        }
                    };
                    auto put_b = [&](int t0, const float4 (&v)[8]) {
                        #pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const int t = t0 + j * gthreads;
                            if (t < p.bn * 8) cv_put(b_hi, lo_b, cv_swz((uint32_t)(t >> 3) * 128u + (uint32_t)(t & 7) * 16u), v[j]);
                        }
                    };
                    float4 vb[8];
                    float va[32];
                    load_b(gt, vb);
                    load_a(0, va);
                    if (!cv_wait_idle_warp(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 0x13)) { ok = false; break; }
                    CV_STAMP(0, tstamp);
                    put_b(gt, vb);
                    put_a(0, va);
                    if (gthreads < CV_BM) {                                    /* 64-thread groups: rows gt + 64 */
                        load_a(1, va);
                        put_a(1, va);
                    }
                    CV_STAMP(1, tstamp);
                    for (int t0 = gt + 8 * gthreads; t0 < p.bn * 8; t0 += 8 * gthreads) {
                        load_b(t0, vb);
                        put_b(t0, vb);
                    }
                } else {
                    /* wgrad.  A: 128 taps x 32 positions; B: filters x 32 positions; lanes run along the
                     * positions.  The four positions of a chunk are decoded one by one (rows may wrap). */
                    const int q = gt & 7;
                    CvRow prow[4]; const float *gptr[4];
                    #pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int pos = kb * CV_BK + q * 4 + e;
                        prow[e].ptr = p.x; prow[e].mask = 0; gptr[e] = nullptr;
                        if (pos < (int)p.kdim) {
                            const int n = pos / (int)sp_out;
                            const int r2 = pos - n * (int)sp_out;
                            const int y = r2 / p.Wo;
                            prow[e] = cv_row<CV_WGRAD>(p, n, y, r2 - y * p.Wo);
                            gptr[e] = p.g + (long)n * p.F * sp_out + r2;
                        }
                    }
                    const int valid_rows = (int)(p.rows_a - m0 < CV_BM ? p.rows_a - m0 : CV_BM);
                    const int rstep = gthreads / 8;
                    /* eight rows' loads (32 per thread) per batch */
                    auto load_a = [&](int r0, float4 (&v)[8]) {
                        #pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const int r = r0 + j * rstep;
                            v[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                            if (r < valid_rows) {
                                const int2 tap = ktab[m0 + r];
                                v[j] = make_float4(cv_elem(prow[0], tap), cv_elem(prow[1], tap), cv_elem(prow[2], tap), cv_elem(prow[3], tap));
                            }
                        }
                    };
                    auto load_b = [&](int r0, float4 (&v)[8]) {
                        #pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const int r = r0 + j * rstep;
                            float e4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                            if (r < p.rows_b) {
                                #pragma unroll
                                for (int e = 0; e < 4; e++)
                                    if (gptr[e]) e4[e] = __ldg(gptr[e] + (long)r * sp_out);
                            }
                            v[j] = make_float4(e4[0], e4[1], e4[2], e4[3]);
                        }
                    };
                    auto put = [&](uint8_t *hi, uint32_t lo_delta, int r0, int limit, const float4 (&v)[8]) {
                        #pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const int r = r0 + j * rstep;
                            if (r < limit) cv_put(hi, lo_delta, cv_swz((uint32_t)r * 128u + (uint32_t)q * 16u), v[j]);
                        }
                    };
                    float4 va[8], vb[8];
                    load_b(gt >> 3, vb);
                    load_a(gt >> 3, va);
                    if (!cv_wait_idle_warp(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 0x13)) { ok = false; break; }
                    CV_STAMP(0, tstamp);
                    /* tile rows beyond the last tap stay zero for the whole item: they are cleared once, the
                     * first time this group fills its stage for the item (3 -> 32 filters have 27 taps: 101
                     * of the 128 rows would otherwise be stored, hi and lo, in every K block) */
                    if (zeroed_for != it) {
                        for (int r = valid_rows + (gt >> 3); r < CV_BM; r += rstep)
                            cv_put(a_hi, lo_a, cv_swz((uint32_t)r * 128u + (uint32_t)q * 16u), make_float4(0.0f, 0.0f, 0.0f, 0.0f));
                        zeroed_for = it;
                    }
                    put(b_hi, lo_b, gt >> 3, p.bn, vb);
                    put(a_hi, lo_a, gt >> 3, valid_rows, va);
                    CV_STAMP(1, tstamp);
                    for (int r0 = (gt >> 3) + 8 * rstep; r0 < valid_rows; r0 += 8 * rstep) {
                        load_a(r0, va);
                        put(a_hi, lo_a, r0, valid_rows, va);
                    }
                    for (int r0 = (gt >> 3) + 8 * rstep; r0 < p.bn; r0 += 8 * rstep) {
                        load_b(r0, vb);
                        put(b_hi, lo_b, r0, p.bn, vb);
                    }
                }
                CV_STAMP(2, tstamp);
                /* generic-proxy writes -> visible to the tensor core's reads; one arrival per warp */
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full + 8 * s);
                CV_STAMP(3, tstamp);
#ifdef TT_TUNING
                if (blockIdx.x == 0 && gt == 0 && grp == 0) atomicAdd(&g_cv_dbg[4], 1ull);
#endif
            }
        }
    } else if (warp == CV_EPI_WARPS) {
        /* ---------------- MMA issuer ----------------
         * One lane runs the loop (measured faster than the whole warp running it with one lane issuing).
         * A K block's 12 instructions take about 1300 cycles to issue whatever the tile's width: the
         * floor under this kernel once the producers keep up. */
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            int acc = 0; uint32_t acc_ph = 0;
            bool ok = true;
#ifdef TT_TUNING
            long long ms = clock64(); const long long kstart = ms;
#define MM_STAMP(i) do { if (blockIdx.x == 0) { long long n_ = clock64(); atomicAdd(&g_cv_dbg[i], (unsigned long long)(n_ - ms)); ms = n_; } } while (0)
#else
#define MM_STAMP(i) do { } while (0)
#endif
            for (int it = blockIdx.x; it < p.items && ok; it += gridDim.x) {
                long m0; int kb0, kb1, slice;
                decode(it, m0, kb0, kb1, slice);
                MM_STAMP(6);
                if (!cv_wait_idle(bar_tempty + 8 * acc, acc_ph ^ 1, abort_flag, p.status, 0x14)) { ok = false; break; }
                MM_STAMP(7);
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(acc * bn32);
                for (int kb = kb0; kb < kb1; kb++) {
                    MM_STAMP(6);
                    if (!cv_wait_idle(bar_full + 8 * s, ph, abort_flag, p.status, 0x12)) { ok = false; break; }
                    MM_STAMP(5);
                    tc_fence_after();
                    const uint32_t a_hi = smem_base + (uint32_t)s * stage_bytes;
                    const uint32_t a_lo = a_hi + CV_A_BYTES;
                    const uint32_t b_hi = a_hi + 2 * CV_A_BYTES;
                    const uint32_t b_lo = b_hi + b_bytes;
                    #pragma unroll
                    for (int ks = 0; ks < CV_BK / 8; ks++) {
                        const uint32_t off = ks * 32;
                        const uint64_t da_hi = make_desc<0, CV_BK>(a_hi + off), db_hi = make_desc<0, CV_BK>(b_hi + off);
                        const uint64_t da_lo = make_desc<0, CV_BK>(a_lo + off), db_lo = make_desc<0, CV_BK>(b_lo + off);
                        tc_mma_tf32(d, da_lo, db_hi, idesc, (kb > kb0 || ks > 0) ? 1u : 0u);
                        tc_mma_tf32(d, da_hi, db_lo, idesc, 1u);
                        tc_mma_tf32(d, da_hi, db_hi, idesc, 1u);
                    }
                    tc_commit(bar_empty + 8 * s);
                    if (++s == p.stages) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                tc_commit(bar_tfull + 8 * acc);
                if (++acc == 2) { acc = 0; acc_ph ^= 1; }
            }
#ifdef TT_TUNING
            if (blockIdx.x == 0) { MM_STAMP(6); atomicAdd(&g_cv_dbg[9], (unsigned long long)(clock64() - kstart)); }
#endif
        }
    } else {
        /* ---------------- epilogue warps: tensor-memory lane quarter `warp` ---------------- */
        const int q = warp;
        int acc = 0; uint32_t acc_ph = 0;
        bool ok = true;
        for (int it = blockIdx.x; it < p.items && ok; it += gridDim.x) {
            long m0; int kb0, kb1, slice;
            decode(it, m0, kb0, kb1, slice);
            const long row = m0 + q * 32 + lane;
            const bool row_ok = row < p.rows_a;
            /* where this row's values go: base address and the distance between consecutive columns */
            float *dst = p.out; long col_stride = 1;
            if (row_ok) {
                if (MODE == CV_WGRAD) {
                    dst = p.out + ((long)slice * p.rows_a + row) * p.rows_b;
                } else {
                    const long spp = MODE == CV_FPROP ? sp_out : sp_in;
                    const int n = (int)(row / spp);
                    dst = p.out + (long)n * p.rows_b * spp + (row - (long)n * spp);
                    col_stride = spp;
                }
            }
            if (!cv_wait_idle_warp(bar_tfull + 8 * acc, acc_ph, abort_flag, p.status, 0x15)) { ok = false; break; }
            tc_fence_after();
            #pragma unroll 1
            for (int c0 = 0; c0 < p.bn; c0 += 32) {
                uint32_t r[32];
                tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * bn32 + c0), r);
                tc_wait_ld();
                if (c0 + 32 >= p.bn) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
                }
                if (row_ok) {
                    #pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int c = c0 + j;
                        if (c < p.rows_b) {
                            float v = __uint_as_float(r[j]);
                            if (p.bias) v += sbias[c];
                            float *o = dst + (long)c * col_stride;
                            *o = p.accumulate ? *o + v : v;
                        }
                    }
                }
            }
            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == CV_EPI_WARPS) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
    }
}

/* dW[f, tap] (+)= sum over slices of partial[slice][tap][f].  One warp per output: lane l adds the
 * slices l, l+32, ... in order and the lanes are combined by a fixed shuffle tree, so the result
 * does not depend on timing. */
__global__ void __launch_bounds__(256) conv_wgrad_reduce_kernel(const float *__restrict__ part, int slices, int taps, int F,
                                                                float *__restrict__ dw, int accumulate) {
    const int total = taps * F, lane = threadIdx.x & 31;
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < total; i += (gridDim.x * blockDim.x) >> 5) {
        const int tap = i / F, f = i - tap * F;
        float s = 0.0f;
        for (int k = lane; k < slices; k += 32) s += part[(long)k * total + i];
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) {
            float *o = dw + (long)f * taps + tap;
            *o = accumulate ? *o + s : s;
        }
    }
}

/* ---- host side ----------------------------------------------------------------*/
static uint32_t *g_cv_status_host = nullptr, *g_cv_status_dev = nullptr;

static int cv_setup(void) {
    if (g_cv_status_host) return 0;
    if (tt_ctx_init() != 0) return -1;
    if (!tt_cuda_ok(cudaHostAlloc((void **)&g_cv_status_host, sizeof(uint32_t), cudaHostAllocMapped), "cudaHostAlloc")) return -1;
    *g_cv_status_host = 0;
    if (!tt_cuda_ok(cudaHostGetDevicePointer((void **)&g_cv_status_dev, g_cv_status_host, 0), "cudaHostGetDevicePointer")) return -1;
    return 0;
}

int conv_tc_poll_status(void) {
    if (!g_cv_status_host) return 0;
    const uint32_t v = *(volatile uint32_t *)g_cv_status_host;
    if (v) {
        tt_set_error("tcgen05 convolution: bounded wait expired (code 0x%x, CTA %u)", v & 0xffu, v >> 8);
        *g_cv_status_host = 0;
        return (int)v;
    }
    return 0;
}

/* Shapes the gathered kernel takes; everything else keeps the im2col + GEMM path. */
int conv_tc_usable(const ConvGeom *g, int need_dgrad) {
    const long kc = (long)g->C * g->HH * g->WW, kback = (long)g->F * g->HH * g->WW;
    if (g->F < 1 || g->F > 256 || g->C < 1 || kc > CV_MAX_TAPS) return 0;
    if (g->HH * g->WW > 31 || g->C > 32767 || g->F > 32767) return 0;       /* one mask bit per window slot */
    if ((long)g->C * g->H * g->W > 0x7fffffffL || (long)g->F * g->Ho * g->Wo > 0x7fffffffL) return 0;   /* 32-bit tap offsets */
    if ((long)g->N * g->Ho * g->Wo > 0x7fffffffL || (long)g->N * g->H * g->W > 0x7fffffffL) return 0;
    if (need_dgrad && (g->sh != 1 || g->sw != 1 || g->C > 256 || kback > CV_MAX_TAPS)) return 0;
    return 1;
}

static int cv_launch(ConvParams &p) {
    if (cv_setup() != 0) return -1;
    p.bn = (p.rows_b + 15) & ~15;
    const int bn32 = (p.bn + 31) & ~31;
    uint32_t cols = 32;
    while (cols < (uint32_t)(2 * bn32)) cols <<= 1;
    p.tmem_cols = cols;
    const size_t stage = 2 * ((size_t)CV_A_BYTES + (size_t)p.bn * CV_BK * 4);
    int stages = (int)((192u << 10) / stage);
    stages = stages >= 4 ? 4 : (stages >= 2 ? 2 : 0);                  /* one producer group per stage: 256 threads divide by it */
    if (stages < 2) { tt_set_error("tcgen05 convolution: tile does not fit shared memory"); return -1; }
    p.stages = stages;
    p.status = g_cv_status_dev;
    const size_t smem = (size_t)stages * stage + CV_MAX_TAPS * (sizeof(int2) + sizeof(int)) + 8 * (2 * stages + 4) + 16 + 256 * sizeof(float) + 1024;
    static size_t configured[3] = {0, 0, 0};
    void (*kern)(ConvParams) = p.mode == CV_FPROP ? conv_tc_kernel<CV_FPROP> : p.mode == CV_DGRAD ? conv_tc_kernel<CV_DGRAD> : conv_tc_kernel<CV_WGRAD>;
    if (smem > configured[p.mode]) {
        if (!tt_cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                        "cudaFuncSetAttribute(smem)")) return -1;
        configured[p.mode] = smem;
    }
    const int grid = p.items < g_tt.sm_count ? p.items : g_tt.sm_count;
    kern<<<grid, CV_THREADS, smem, g_tt.stream>>>(p);
    g_tt.launches++;
    return tt_cuda_ok(cudaGetLastError(), "tcgen05 convolution launch") ? 0 : -1;
}

static void cv_geom(ConvParams &p, const ConvGeom *g) {
    memset(&p, 0, sizeof p);
    p.N = g->N; p.C = g->C; p.H = g->H; p.W = g->W; p.F = g->F; p.HH = g->HH; p.WW = g->WW;
    p.sh = g->sh; p.sw = g->sw; p.ph = g->ph; p.pw = g->pw; p.Ho = g->Ho; p.Wo = g->Wo;
}

int conv_tc_fprop(const ConvGeom *g, const float *x, const float *w, const float *bias, float *out) {
    ConvParams p;
    cv_geom(p, g);
    p.mode = CV_FPROP; p.x = x; p.w = w; p.bias = bias; p.out = out;
    p.rows_a = (long)g->N * g->Ho * g->Wo; p.rows_b = g->F;
    p.kdim = (long)g->C * g->HH * g->WW; p.taps = (int)p.kdim;
    p.num_kb = (int)((p.kdim + CV_BK - 1) / CV_BK); p.kb_per_item = p.num_kb;
    p.m_tiles = (int)((p.rows_a + CV_BM - 1) / CV_BM); p.items = p.m_tiles;
    tt_trace_begin(TTB_K_SPATIAL);
    const int rc = cv_launch(p);
    tt_trace_end(TTB_K_SPATIAL, 2.0 * (double)p.rows_a * g->F * (double)p.kdim);
    return rc;
}

int conv_tc_dgrad(const ConvGeom *g, const float *grad_out, const float *w, float *dx, int accumulate) {
    ConvParams p;
    cv_geom(p, g);
    p.mode = CV_DGRAD; p.g = grad_out; p.w = w; p.out = dx; p.accumulate = accumulate;
    p.rows_a = (long)g->N * g->H * g->W; p.rows_b = g->C;
    p.kdim = (long)g->F * g->HH * g->WW; p.taps = (int)p.kdim;
    p.num_kb = (int)((p.kdim + CV_BK - 1) / CV_BK); p.kb_per_item = p.num_kb;
    p.m_tiles = (int)((p.rows_a + CV_BM - 1) / CV_BM); p.items = p.m_tiles;
    tt_trace_begin(TTB_K_SPATIAL);
    const int rc = cv_launch(p);
    tt_trace_end(TTB_K_SPATIAL, 2.0 * (double)p.rows_a * g->C * (double)p.kdim);
    return rc;
}

int conv_tc_wgrad(const ConvGeom *g, const float *x, const float *grad_out, float *dw, int accumulate) {
    ConvParams p;
    cv_geom(p, g);
    p.mode = CV_WGRAD; p.x = x; p.g = grad_out;
    p.rows_a = (long)g->C * g->HH * g->WW; p.rows_b = g->F; p.taps = (int)p.rows_a;
    p.kdim = (long)g->N * g->Ho * g->Wo;
    p.num_kb = (int)((p.kdim + CV_BK - 1) / CV_BK);
    p.m_tiles = (int)((p.rows_a + CV_BM - 1) / CV_BM);
    /* as many position slices as give every SM one item, of at least eight K blocks each */
    int slices = g_tt.sm_count / p.m_tiles;
    if (slices < 1) slices = 1;
    if (slices > (p.num_kb + 7) / 8) slices = (p.num_kb + 7) / 8;
    p.kb_per_item = (p.num_kb + slices - 1) / slices;
    slices = (p.num_kb + p.kb_per_item - 1) / p.kb_per_item;
    p.items = slices * p.m_tiles;
    float *part = (float *)tt_dev_alloc(sizeof(float) * (size_t)slices * p.rows_a * g->F);
    if (!part) return -1;
    p.out = part;
    tt_trace_begin(TTB_K_SPATIAL);
    int rc = cv_launch(p);
    if (rc == 0) {
        const int total = (int)p.rows_a * g->F;
        int blocks = (total + 7) / 8;                               /* eight warps per block, one output each */
        if (blocks > g_tt.sm_count * 8) blocks = g_tt.sm_count * 8;
        conv_wgrad_reduce_kernel<<<blocks, 256, 0, g_tt.stream>>>(part, slices, (int)p.rows_a, g->F, dw, accumulate);
        g_tt.launches++;
        rc = tt_cuda_ok(cudaGetLastError(), "convolution weight-gradient reduce") ? 0 : -1;
    }
    tt_trace_end(TTB_K_SPATIAL, 2.0 * (double)p.rows_a * g->F * (double)p.kdim);
    tt_dev_free(part);
    return rc;
}
