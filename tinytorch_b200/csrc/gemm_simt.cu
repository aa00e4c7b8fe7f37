/* Exact-fp32 GEMM on the CUDA cores.
 *
 * This is the path for shapes the tensor-core kernel cannot or should not
 * take: tiny problems (the finite-difference gradient checks run thousands
 * of 4x3 products and leave no room for split-precision error), rows whose
 * pitch is not a multiple of 16 bytes, and N = 10 classifier layers.
 *
 * It reproduces the reference's arithmetic per output element, so on this
 * path results are bit-identical to the reference library:
 *   MODE_FWD   forward sgemm (src/gemm.c:569-641): inside the region covered
 *              by the 6x16 register tile one FMA chain per output, k ascending
 *              (later K blocks reload the accumulators from C and carry on,
 *              src/gemm.c:264-280, so the blocking leaves no trace); outside it (rows
 *              past the last multiple of 6, columns past the last multiple of
 *              16, or everything when the matrix is narrower than one tile)
 *              separately rounded multiply and add that skip exact zeros of
 *              A (src/gemm.c:52-62).  `all_edge` selects the second rule for
 *              every element, which is the naive tt_matmul (src/ops.c:84-102).
 *   MODE_DOT   the backward products dA = dC*B^T and dB = A^T*dC
 *              (src/autograd.c:66-103) and the convolution weight gradient
 *              (src/autograd.c:439-454): one accumulator, separately rounded
 *              multiply and add, k ascending.
 * The file is compiled with -fmad=false so that only the explicit fmaf()
 * fuses.
 *
 * A may carry a virtual column (or, transposed, a virtual row) of ones: that
 * is how a padones node feeding a matmul is consumed without materialising
 * [M,K+1] (src/autograd.c:195-212); the ones take part in the chain at the
 * position the reference has them, k = K-1.
 *
 * 64x64x16 tiles, 256 threads, 4x4 outputs per thread; k-major shared tiles
 * so that the inner loop reads are broadcast / conflict-free. */
#include "tt_internal.h"

#define BM 64
#define BN 64
#define BK 16

enum { MODE_FWD = 0, MODE_DOT = 1 };

struct SimtParams {
    int ta, tb, M, N, K;
    const float *A; long lda;
    const float *B; long ldb;
    float *C; long ldc;
    int accumulate;
    int relu;
    const float *mask; long ldmask;
    int a_pad_ones;
    int all_edge;
    int mfull, nfull;      /* extent of the register-tile region (MODE_FWD) */
};

__device__ __forceinline__ float load_a(const SimtParams &p, int i, int k) {
    if (i >= p.M || k >= p.K) return 0.0f;
    if (p.a_pad_ones) {
        if (!p.ta && k == p.K - 1) return 1.0f;
        if (p.ta && i == p.M - 1) return 1.0f;
    }
    return p.ta ? p.A[(long)k * p.lda + i] : p.A[(long)i * p.lda + k];
}
__device__ __forceinline__ float load_b(const SimtParams &p, int k, int j) {
    if (j >= p.N || k >= p.K) return 0.0f;
    return p.tb ? p.B[(long)j * p.ldb + k] : p.B[(long)k * p.ldb + j];
}

template <int MODE>
__global__ void __launch_bounds__(256) gemm_simt_kernel(SimtParams p) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

    float acc[4][4];
    bool fused[4][4];
    #pragma unroll
    for (int i = 0; i < 4; i++)
        #pragma unroll
        for (int j = 0; j < 4; j++) {
            acc[i][j] = 0.0f;
            int gi = m0 + ty * 4 + i, gj = n0 + tx * 4 + j;
            fused[i][j] = (MODE == MODE_FWD) && !p.all_edge && gi < p.mfull && gj < p.nfull;
        }

    /* The K loop is a chain of global-load latencies for the small problems this kernel serves (a
     * 256 x 257 x 10 classifier layer is four blocks of 17 steps): the next step's operands are
     * fetched into registers while the current step is multiplied out of shared memory.  The order
     * of the arithmetic is untouched. */
    float ra[4], rb[4];
    auto fetch = [&](int k0) {
        #pragma unroll
        for (int r = 0; r < 4; r++) {
            const int e = tid + 256 * r;
            int kk, mm, nn;
            if (p.ta) { mm = e % BM; kk = e / BM; } else { kk = e % BK; mm = e / BK; }
            ra[r] = load_a(p, m0 + mm, k0 + kk);
            if (p.tb) { kk = e % BK; nn = e / BK; } else { nn = e % BN; kk = e / BN; }
            rb[r] = load_b(p, k0 + kk, n0 + nn);
        }
    };
    auto stash = [&]() {
        #pragma unroll
        for (int r = 0; r < 4; r++) {
            const int e = tid + 256 * r;
            int kk, mm, nn;
            if (p.ta) { mm = e % BM; kk = e / BM; } else { kk = e % BK; mm = e / BK; }
            As[kk][mm] = ra[r];
            if (p.tb) { kk = e % BK; nn = e / BK; } else { nn = e % BN; kk = e / BN; }
            Bs[kk][nn] = rb[r];
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < p.K; k0 += BK) {
        stash();
        __syncthreads();
        if (k0 + BK < p.K) fetch(k0 + BK);              /* in flight during the multiply below */
        int kmax = p.K - k0 < BK ? p.K - k0 : BK;
        for (int kk = 0; kk < kmax; kk++) {
            float a[4], b[4];
            #pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
            #pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Bs[kk][tx * 4 + j];
            #pragma unroll
            for (int i = 0; i < 4; i++)
                #pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (MODE == MODE_DOT) {
                        acc[i][j] = acc[i][j] + a[i] * b[j];
                    } else {
                        float f = fmaf(a[i], b[j], acc[i][j]);
                        float e = (a[i] == 0.0f) ? acc[i][j] : acc[i][j] + a[i] * b[j];
                        acc[i][j] = fused[i][j] ? f : e;
                    }
                }
        }
        __syncthreads();
    }

    #pragma unroll
    for (int i = 0; i < 4; i++)
        #pragma unroll
        for (int j = 0; j < 4; j++) {
            int gi = m0 + ty * 4 + i, gj = n0 + tx * 4 + j;
            if (gi >= p.M || gj >= p.N) continue;
            float r = acc[i][j];
            if (p.relu) r = r > 0.0f ? r : 0.0f;
            if (p.mask) r = p.mask[(long)gi * p.ldmask + gj] > 0.0f ? r : 0.0f;
            float *c = p.C + (long)gi * p.ldc + gj;
            *c = p.accumulate ? *c + r : r;
        }
}

int gemm_simt(const GemmArgs *g) {
    const int a_pad_ones = g->a_pad_ones, mode_hint = g->rule;
    if (g->M <= 0 || g->N <= 0 || g->K <= 0) { tt_set_error("gemm: empty shape"); return -1; }
    SimtParams p;
    p.ta = g->ta; p.tb = g->tb; p.M = g->M; p.N = g->N; p.K = g->K;
    p.A = g->A; p.lda = g->lda; p.B = g->B; p.ldb = g->ldb; p.C = g->C; p.ldc = g->ldc;
    p.accumulate = g->accumulate;
    p.relu = g->relu; p.mask = g->mask; p.ldmask = g->ldmask;
    p.a_pad_ones = a_pad_ones;
    p.all_edge = (mode_hint == 2);
    p.mfull = (g->M / 6) * 6;
    p.nfull = (g->N / 16) * 16;
    if (p.nfull <= 0 || p.mfull == 0) p.all_edge = 1;   /* src/gemm.c:571-591 */
    dim3 grid((g->N + BN - 1) / BN, (g->M + BM - 1) / BM);
    tt_trace_begin(TTB_K_GEMM_SIMT);
    if (mode_hint == 1) gemm_simt_kernel<MODE_DOT><<<grid, 256, 0, g_tt.stream>>>(p);
    else                gemm_simt_kernel<MODE_FWD><<<grid, 256, 0, g_tt.stream>>>(p);
    g_tt.launches++;
    tt_trace_end(TTB_K_GEMM_SIMT, 2.0 * (double)g->M * g->N * g->K);
    return 0;
}
