/* Tensor-core GEMM for sm_100a: tcgen05.mma kind::tf32 in a 3xTF32 split,
 * TMA-staged operand tiles, accumulators in tensor memory.
 *
 * Replaces the reference's blocked AVX2 sgemm (src/gemm.c:569-641) and its
 * two naive backward products dA = dC*B^T and dB = A^T*dC
 * (src/autograd.c:66-103).  No operand is ever transposed in memory: an
 * operand whose reduction index is not the contiguous one is loaded as an
 * "MN-major" tile and the instruction descriptor says so.
 *
 *   D[M,N] (+)= A_op[M,K] * B_op[K,N] (+ bias[n])
 *
 * Precision.  kind::tf32 reads 32-bit words and uses the top 19 bits.  Each
 * fp32 operand x is therefore split as hi = x with the low 13 mantissa bits
 * cleared (what the instruction sees when it is handed x itself) and
 * lo = x - hi (exact in fp32; the instruction keeps its top 19 bits), and every K step issues
 *   D += A_lo*B_hi;  D += A_hi*B_lo;  D += A_hi*B_hi
 * into one fp32 accumulator.  The dropped A_lo*B_lo term is below 2^-20
 * relative, so products carry about 21 bits, which is what "fp32-grade"
 * means for this kernel.
 *
 * Structure of one CTA (persistent, one per SM, 448 threads):
 *   warp 0      TMA producer: cp.async.bulk.tensor loads, each CTA fetching its own tiles, of
 *               the raw A and B tiles of a K block into a ring of stages, and
 *               L2 prefetches a few K blocks ahead so that those loads hit L2.
 *   warps 2-9   split: read the raw tiles from shared memory, write the lo
 *               tiles next to them at the same (swizzled) offsets.
 *   warp 1      one thread issues the tcgen05.mma triples and commits to
 *               mbarriers; owns the tensor-memory allocation.
 *   warps 10-13 epilogue: tcgen05.ld the finished accumulator (one of two,
 *               so the next tile's MMAs overlap), add bias / old C, store.
 * Tiles 128x256 (two stages) or 128x128 (three stages), K blocks of 32.
 *
 * Every wait is bounded: a wait that exceeds its cycle budget records a code
 * in a host-visible status word, raises a CTA-wide abort flag that all other
 * waits poll, and the CTA drains, frees its tensor memory and exits. */
#include "tt_internal.h"

#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#define TC_BM 128
/* K block of a stage: 32 fp32 (128-byte rows) or 16 (64-byte rows, twice the stages) -- template parameter BK */
#define TC_THREADS 448
#define TC_SPLIT_THREADS 256
#define TC_EPI_THREADS 128
#define TC2_THREADS (TC_THREADS + 64)   /* pair kernel: two more warps, which pass this CTA's "tiles landed" and "lo tiles written" on to the leader */
#ifndef TC2_STAGES
#define TC2_STAGES 4        /* pair kernel: ring of raw (hi) tiles, 32 KB per stage and CTA */
#endif
#ifndef TC2_LO_SLOTS
#define TC2_LO_SLOTS 3      /* pair kernel: slots for the lo tiles, which live only from the split pass to the cross-term MMAs */
#endif

#include "tcgen05_utils.cuh"

/* The one-pass and no-split modes exist for timing experiments only and give wrong or
 * TF32-grade numbers; a default build has neither (compile with -DTT_TUNING to get them,
 * together with the TT_TC_* environment knobs). */
#ifdef TT_TUNING
#define TC_FULL_SPLIT(p) ((p).passes == 3)
#define TC_MAKE_LO(p) ((p).passes == 3 && !(p).nosplit)
#else
#define TC_FULL_SPLIT(p) true
#define TC_MAKE_LO(p) true
#endif

struct TcParams {
    int M, N, K;
    float *C; long ldc;
    const float *bias;
    int accumulate;
    int relu;                /* epilogue: v = v > 0 ? v : 0 after the bias */
    const float *mask; long ldmask;   /* epilogue: v = mask[m, n] > 0 ? v : 0 (gradient mask of a relu, from its output) */
    int passes;              /* 3 = full split; TT_TUNING builds only: 1 = hi*hi only (bring-up aid, TF32-grade numbers) */
    int nosplit;             /* TT_TUNING builds only: issue the three MMAs but skip producing the lo tiles (wrong numbers) */
    int noprefetch;          /* no L2 prefetch ahead of the loads (the pair kernel runs 5-20 % faster without) */
    int a_3d, b_3d;          /* MN-major operand described by a rank-3 map: one TMA per tile instead of one per 32 columns */
    /* Split-K: the reduction is cut into `splits` slices of kb_per_split K blocks; slice s of a tile
     * writes its partial product to partial + s*M*N (row pitch N) and a second kernel adds the slices
     * in order.  splits == 1: the epilogue writes C itself. */
    int splits, kb_per_split;
    float *partial;
    /* Tail split (one-CTA kernel, splits == 1): the first num_tiles - tail_tiles tiles fill whole
     * waves of CTAs and run over the full reduction; each of the last tail_tiles tiles is cut into
     * tail_splits slices of tail_kb K blocks, so that the last, partly filled wave becomes a
     * full wave of shorter items.  Slice s of tail tile j writes a dense 128 x BN block at
     * tail_partial + (s * tail_tiles + j) * 128 * BN; a second kernel adds the slices in order. */
    int tail_tiles, tail_splits, tail_kb;
    float *tail_partial;
    /* Chunked accumulation: an item's reduction runs in chunks of chunk_kb K blocks; after each chunk
     * the accumulator is handed to the epilogue, which adds it into the destination with a rounded
     * fp32 add (the first chunk stores), and the next chunk starts from zero.  The tensor core
     * truncates towards zero whenever it adds into an accumulator, a bias that grows with the
     * number of MMAs times the accumulator's magnitude: sums of same-signed terms (relu outputs
     * times softmax gradients) came out 6e-5 low at K = 8192 in one accumulator, 7e-6 in chunks of
     * 1024.  Only the main accumulator is folded; the cross terms (2^-11 of the result) keep theirs
     * for the whole item and join with the last chunk.  chunk_kb >= the item's length: one chunk. */
    int chunk_kb;
    int group_m;             /* tile rows per rasterisation group (tc_tile_coords) */
    int push_on;             /* send the parts of C other ranks own into their staging areas (PeerPush) */
    PeerPush push;
    /* host-mapped: 0 = fine, else wait code | cta << 8.  Codes name the wait that gave up: 1 split warps on a
     * stage's loads, 2 MMA thread on a lo tile, 3 load thread on a free stage, 4 MMA thread on a drained
     * accumulator, 5 epilogue on a full accumulator; pair kernel also 6 MMA thread on both CTAs' raw tiles,
     * 7 split warps on a free lo slot, 8 / 9 the relay threads on the split warps / on the loads. */
    uint32_t *status;
};

/* Tile number -> tile coordinates.  Tiles are numbered so that the CTAs that run at the same time
 * (consecutive numbers) cover a compact block of the output instead of a full-height stripe:
 * groups of TC_GROUP_M tile rows, walked row-first inside the group.  A wave of 74 pair tiles then
 * shares 8 row blocks of A and about 9 column blocks of B through L2, where a stripe of 32 row
 * blocks streamed all of A from HBM once per wave (measured on 8192x4096x4096: 1.14 GB of DRAM
 * traffic per launch against 335 MB algorithmic). */
#define TC_GROUP_M 8
__host__ __device__ __forceinline__ void tc_tile_coords(int t, int tiles_m, int tiles_n, int group_m, int &tm, int &tn) {
    const int width = group_m * tiles_n;
    const int group = t / width, first_m = group * group_m;
    const int rows = tiles_m - first_m < group_m ? tiles_m - first_m : group_m;
    const int r = t - group * width;
    tm = first_m + r % rows;
    tn = r / rows;
}

/* What an epilogue thread needs to finish one output row: where the row lives, and the
 * elementwise steps fused behind the product (bias, relu, gradient mask, accumulate). */
struct EpiRow {
    float *crow;             /* crow[n] is column n of this thread's row of the destination */
    const float *bias;       /* per column, or NULL */
    const float *mrow;       /* mrow[n] > 0 keeps column n, or NULL */
    int accumulate, relu;
    int partial;             /* the destination holds the sum of this item's earlier chunks: add it BEFORE the fused steps */
    bool vec_ok;             /* destination (and mask) rows allow 128-bit accesses */
};
__device__ __forceinline__ void red_add_v4(float *p, float4 v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
/* Store 32 consecutive columns [gc, gc+32) of one accumulator row.
 * A chunk after the first (e.partial) adds into what the earlier chunks of the same item left in
 * the destination.  Without fused steps that is a fire-and-forget reduction (red.global.add, rounded
 * fp32 add performed at L2): the thread does not wait for the old value, so the accumulator is
 * drained at store speed.  One thread owns a row for all chunks of an item and its accesses to one
 * address take effect in program order, so the sum is ((c0 + c1) + c2) + ... every time.  The last
 * chunk of a product with relu or a mask needs the total: it reads it back (from L2), finishes,
 * and stores. */
__device__ __forceinline__ void epi_store32(const uint32_t (&r)[32], int gc, int N, const EpiRow &e) {
    const bool reduce_only = e.partial && !e.relu && !e.mrow;
    if (e.vec_ok && gc + 32 <= N) {
        #pragma unroll
        for (int j = 0; j < 32; j += 4) {
            float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                   __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            if (reduce_only) { red_add_v4(e.crow + gc + j, v); continue; }
            if (e.partial) {
                const float4 o = __ldcg((const float4 *)(e.crow + gc + j));
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
            }
            if (e.bias) {
                v.x += e.bias[gc + j]; v.y += e.bias[gc + j + 1];
                v.z += e.bias[gc + j + 2]; v.w += e.bias[gc + j + 3];
            }
            if (e.relu) {
                v.x = v.x > 0.0f ? v.x : 0.0f; v.y = v.y > 0.0f ? v.y : 0.0f;
                v.z = v.z > 0.0f ? v.z : 0.0f; v.w = v.w > 0.0f ? v.w : 0.0f;
            }
            if (e.mrow) {
                const float4 k = *(const float4 *)(e.mrow + gc + j);
                v.x = k.x > 0.0f ? v.x : 0.0f; v.y = k.y > 0.0f ? v.y : 0.0f;
                v.z = k.z > 0.0f ? v.z : 0.0f; v.w = k.w > 0.0f ? v.w : 0.0f;
            }
            if (e.accumulate) {
                const float4 o = *(const float4 *)(e.crow + gc + j);
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
            }
            *(float4 *)(e.crow + gc + j) = v;
        }
    } else {
        #pragma unroll
        for (int j = 0; j < 32; j++) {
            if (gc + j < N) {
                float v = __uint_as_float(r[j]);
                if (reduce_only) { atomicAdd(e.crow + gc + j, v); continue; }
                if (e.partial) v += __ldcg(e.crow + gc + j);
                if (e.bias) v += e.bias[gc + j];
                if (e.relu) v = v > 0.0f ? v : 0.0f;
                if (e.mrow) v = e.mrow[gc + j] > 0.0f ? v : 0.0f;
                if (e.accumulate) v += e.crow[gc + j];
                e.crow[gc + j] = v;
            }
        }
    }
}

/* Second half of the last chunk of a chunked product with relu or a mask: the chunk itself was added
 * like the others (so that the accumulator is free again at once); now the thread reads its finished
 * sums back from L2, applies the elementwise step and stores them.  Runs under the next tile's MMAs. */
__device__ __forceinline__ void epi_finish32(int gc, int N, float *crow, int relu, const float *mrow, bool vec_ok) {
    if (vec_ok && gc + 32 <= N) {
        float4 v[8];
        #pragma unroll
        for (int j = 0; j < 8; j++) v[j] = __ldcg((const float4 *)(crow + gc + 4 * j));
        #pragma unroll
        for (int j = 0; j < 8; j++) {
            if (relu) {
                v[j].x = v[j].x > 0.0f ? v[j].x : 0.0f; v[j].y = v[j].y > 0.0f ? v[j].y : 0.0f;
                v[j].z = v[j].z > 0.0f ? v[j].z : 0.0f; v[j].w = v[j].w > 0.0f ? v[j].w : 0.0f;
            }
            if (mrow) {
                const float4 k = *(const float4 *)(mrow + gc + 4 * j);
                v[j].x = k.x > 0.0f ? v[j].x : 0.0f; v[j].y = k.y > 0.0f ? v[j].y : 0.0f;
                v[j].z = k.z > 0.0f ? v[j].z : 0.0f; v[j].w = k.w > 0.0f ? v[j].w : 0.0f;
            }
            *(float4 *)(crow + gc + 4 * j) = v[j];
        }
    } else {
        for (int j = 0; j < 32; j++) {
            if (gc + j < N) {
                float v = __ldcg(crow + gc + j);
                if (relu) v = v > 0.0f ? v : 0.0f;
                if (mrow) v = mrow[gc + j] > 0.0f ? v : 0.0f;
                crow[gc + j] = v;
            }
        }
    }
}

template <int A_MN, int B_MN, int BN, int BK, int STAGES, int SPLIT_ACC>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcParams p) {
    constexpr uint32_t A_BYTES = TC_BM * BK * 4;
    constexpr uint32_t B_BYTES = BN * BK * 4;
    constexpr uint32_t BOX = BK * 128;                        /* one MN-major box: BK k-rows of 128 bytes */
    constexpr uint32_t HI_BYTES = A_BYTES + B_BYTES;         /* raw tiles of one stage */
    constexpr uint32_t STAGE_BYTES = 2 * HI_BYTES;           /* raw + lo */
    constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)A_MN << 15) |
                               ((uint32_t)B_MN << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
    constexpr uint32_t TMEM_COLS = 2 * BN;                   /* two accumulators */
    /* SPLIT_ACC = 0: the two accumulators alternate between tiles, so the epilogue of
     * one tile overlaps the MMAs of the next.  SPLIT_ACC = 1 (long reductions): one
     * holds the hi*hi products, the other the two small cross terms, and the epilogue
     * adds them.  The tensor core truncates when it adds into an accumulator, an
     * error that grows with the number of MMAs into a LARGE accumulator; keeping the
     * cross terms (2^-11 of the result) apart removes two thirds of those. */
    constexpr int NACC = SPLIT_ACC ? 1 : 2;
    constexpr int TC_PREFETCH = STAGES + (BK == 16 ? 8 : 4);   /* K blocks the producer asks L2 for ahead of its loads */

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    /* control block after the stages */
    uint64_t *bars = (uint64_t *)(smem_gen + STAGES * STAGE_BYTES);
    const uint32_t bar_full = smem_u32(bars);                         /* STAGES */
    const uint32_t bar_lo = bar_full + 8 * STAGES;                    /* STAGES */
    const uint32_t bar_empty = bar_lo + 8 * STAGES;                   /* STAGES */
    const uint32_t bar_tfull = bar_empty + 8 * STAGES;                /* 2 */
    const uint32_t bar_tempty = bar_tfull + 16;                       /* 2 */
    uint32_t *tmem_slot = (uint32_t *)(bars + 3 * STAGES + 4);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (p.M + TC_BM - 1) / TC_BM;
    const int tiles_n = (p.N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (p.K + BK - 1) / BK;
    const int full_tiles = num_tiles - p.tail_tiles;     /* tiles that run over the whole reduction */
    const int num_items = p.tail_tiles ? full_tiles + p.tail_tiles * p.tail_splits
                                       : num_tiles * p.splits;          /* work items: (K slice, tile) */
    /* item -> first row, first column, K-block range, slice */
    auto decode = [&](int it, int &m0, int &n0, int &kb0, int &kb1, int &split) {
        int t;
        if (p.tail_tiles) {
            if (it < full_tiles) { t = it; split = 0; kb0 = 0; kb1 = num_kb; }
            else {
                const int j = it - full_tiles;
                split = j / p.tail_tiles;
                t = full_tiles + (j - split * p.tail_tiles);
                kb0 = split * p.tail_kb;
                kb1 = kb0 + p.tail_kb < num_kb ? kb0 + p.tail_kb : num_kb;
            }
        } else {
            split = it / num_tiles;
            t = it - split * num_tiles;
            kb0 = split * p.kb_per_split;
            kb1 = kb0 + p.kb_per_split < num_kb ? kb0 + p.kb_per_split : num_kb;
        }
        int tm, tn;
        tc_tile_coords(t, tiles_m, tiles_n, p.group_m, tm, tn);
        m0 = tm * TC_BM; n0 = tn * BN;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_lo + 8 * s, TC_SPLIT_THREADS / 32);      /* one arrival per split warp */
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, TC_EPI_THREADS / 32);  /* one arrival per epilogue warp */
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        /* ---------------- TMA producer ---------------- */
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            bool ok = true;
            auto prefetch = [&](int m0, int n0, int kb) {
                if (p.noprefetch) return;
                const int k0 = kb * BK;
                if (A_MN && p.a_3d) {
                    tma_prefetch_3d(&map_a, 0, k0, m0 / 32);
                } else if (A_MN) {
                    #pragma unroll
                    for (int b = 0; b < TC_BM / 32; b++) tma_prefetch_2d(&map_a, m0 + 32 * b, k0);
                } else {
                    tma_prefetch_2d(&map_a, k0, m0);
                }
                if (B_MN && p.b_3d) {
                    tma_prefetch_3d(&map_b, 0, k0, n0 / 32);
                } else if (B_MN) {
                    #pragma unroll
                    for (int b = 0; b < BN / 32; b++) tma_prefetch_2d(&map_b, n0 + 32 * b, k0);
                } else {
                    tma_prefetch_2d(&map_b, k0, n0);
                }
            };
            for (int it = blockIdx.x; it < num_items && ok; it += gridDim.x) {
                int m0, n0, kb0, kb1, split;
                decode(it, m0, n0, kb0, kb1, split);
                if (it == (int)blockIdx.x)
                    for (int kb = kb0 + STAGES; kb < kb0 + TC_PREFETCH && kb < kb1; kb++) prefetch(m0, n0, kb);
                for (int kb = kb0; kb < kb1; kb++) {
                    /* keep L2 TC_PREFETCH K blocks ahead, running on into this CTA's next item */
                    const int pk = kb + TC_PREFETCH;
                    if (pk < kb1) {
                        prefetch(m0, n0, pk);
                    } else if (it + (int)gridDim.x < num_items) {
                        int m2, n2, kb2, kb3, s2;
                        decode(it + gridDim.x, m2, n2, kb2, kb3, s2);
                        if (kb2 + (pk - kb1) < kb3) prefetch(m2, n2, kb2 + (pk - kb1));
                    }
                    if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 3)) { ok = false; break; }
                    const uint32_t st = smem_base + s * STAGE_BYTES;
                    const uint32_t full = bar_full + 8 * s;
                    const int k0 = kb * BK;
                    mbar_expect_tx(full, HI_BYTES);
                    if (A_MN && p.a_3d) {
                        tma_load_3d(st, &map_a, full, 0, k0, m0 / 32);
                    } else if (A_MN) {
                        #pragma unroll
                        for (int b = 0; b < TC_BM / 32; b++) tma_load_2d(st + b * BOX, &map_a, full, m0 + 32 * b, k0);
                    } else {
                        tma_load_2d(st, &map_a, full, k0, m0);
                    }
                    if (B_MN && p.b_3d) {
                        tma_load_3d(st + A_BYTES, &map_b, full, 0, k0, n0 / 32);
                    } else if (B_MN) {
                        #pragma unroll
                        for (int b = 0; b < BN / 32; b++) tma_load_2d(st + A_BYTES + b * BOX, &map_b, full, n0 + 32 * b, k0);
                    } else {
                        tma_load_2d(st + A_BYTES, &map_b, full, k0, n0);
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
            if (!ok) {
                /* give loads already in flight time to land before the CTA exits */
                long long t0 = clock64();
                while (clock64() - t0 < 200000) { }
            }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issuer ---------------- */
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            int acc = 0; uint32_t acc_ph = 0;
            bool ok = true;
            for (int it = blockIdx.x; it < num_items && ok; it += gridDim.x) {
                int m0, n0, kb0, kb1, split;
                decode(it, m0, n0, kb0, kb1, split);
                if (!mbar_wait(bar_tempty + 8 * acc, acc_ph ^ 1, abort_flag, p.status, 4)) { ok = false; break; }
                tc_fence_after();
                uint32_t d_main = tmem_base + (uint32_t)(SPLIT_ACC ? 0 : acc * BN);
                uint32_t d_corr = SPLIT_ACC ? tmem_base + (uint32_t)BN : d_main;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (kb > kb0 && (kb - kb0) % p.chunk_kb == 0) {
                        /* chunk boundary: hand the accumulator over, start the next chunk from zero */
                        tc_commit(bar_tfull + 8 * acc);
                        if (++acc == NACC) { acc = 0; acc_ph ^= 1; }
                        if (!mbar_wait(bar_tempty + 8 * acc, acc_ph ^ 1, abort_flag, p.status, 4)) { ok = false; break; }
                        tc_fence_after();
                        d_main = tmem_base + (uint32_t)(SPLIT_ACC ? 0 : acc * BN);
                        d_corr = SPLIT_ACC ? tmem_base + (uint32_t)BN : d_main;
                    }
                    if (!mbar_wait(bar_lo + 8 * s, ph, abort_flag, p.status, 2) ||
                        !mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 2)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_hi = smem_base + s * STAGE_BYTES;
                    const uint32_t b_hi = a_hi + A_BYTES;
                    const uint32_t a_lo = a_hi + HI_BYTES;
                    const uint32_t b_lo = b_hi + HI_BYTES;
                    #pragma unroll
                    for (int ks = 0; ks < BK / 8; ks++) {
                        const uint32_t a_off = A_MN ? ks * 1024 : ks * 32;
                        const uint32_t b_off = B_MN ? ks * 1024 : ks * 32;
                        const uint64_t da_hi = make_desc<A_MN, BK>(a_hi + a_off);
                        const uint64_t db_hi = make_desc<B_MN, BK>(b_hi + b_off);
                        const uint32_t first = ((kb - kb0) % p.chunk_kb != 0 || ks > 0) ? 1u : 0u;      /* main: restarts with every chunk */
                        const uint32_t first_corr = SPLIT_ACC ? ((kb > kb0 || ks > 0) ? 1u : 0u) : first;   /* cross terms: run over the whole item */
                        if (TC_FULL_SPLIT(p)) {
                            const uint64_t da_lo = make_desc<A_MN, BK>(a_lo + a_off);
                            const uint64_t db_lo = make_desc<B_MN, BK>(b_lo + b_off);
                            tc_mma_tf32(d_corr, da_lo, db_hi, IDESC, first_corr);
                            tc_mma_tf32(d_corr, da_hi, db_lo, IDESC, 1u);
                            tc_mma_tf32(d_main, da_hi, db_hi, IDESC, SPLIT_ACC ? first : 1u);
                        } else {
                            tc_mma_tf32(d_main, da_hi, db_hi, IDESC, first);
                        }
                    }
                    tc_commit(bar_empty + 8 * s);      /* stage reusable once these MMAs have read it */
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                tc_commit(bar_tfull + 8 * acc);        /* accumulator complete */
                if (++acc == NACC) { acc = 0; acc_ph ^= 1; }
            }
        }
    } else if (warp < 2 + TC_SPLIT_THREADS / 32) {
        /* ---------------- split warps: lo = x - trunc19(x) ---------------- */
        const int st_tid = threadIdx.x - 64;
        int s = 0; uint32_t ph = 0;
        bool ok = true;
        for (int it = blockIdx.x; it < num_items && ok; it += gridDim.x) {
            int m0, n0, kb0, kb1, split;
            decode(it, m0, n0, kb0, kb1, split);
            for (int kb = kb0; kb < kb1; kb++) {
                if (!mbar_wait_warp(bar_full + 8 * s, ph, abort_flag, p.status, 1)) { ok = false; break; }
                if (TC_MAKE_LO(p)) {
                    const uint8_t *hi = smem_gen + s * STAGE_BYTES;
                    #pragma unroll 4
                    for (uint32_t c = st_tid; c < HI_BYTES / 16; c += TC_SPLIT_THREADS) {
                        float4 v = *(const float4 *)(hi + c * 16);
                        float4 w = make_float4(split_lo(v.x), split_lo(v.y), split_lo(v.z), split_lo(v.w));
                        *(float4 *)(hi + HI_BYTES + c * 16) = w;
                    }
                    /* make the generic-proxy writes visible to the tensor core's reads */
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                /* every lane has fenced its own writes; the warp barrier orders them before the one arrival
                 * (256 per-thread arrivals on one barrier word cost more shared-memory time than the split) */
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_lo + 8 * s);
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
        }
    } else {
        /* ---------------- epilogue warps ---------------- */
        const int q = warp & 3;                       /* tensor-memory lane quarter this warp may read */
        int acc = 0; uint32_t acc_ph = 0;
        bool ok = true;
        for (int it = blockIdx.x; it < num_items && ok; it += gridDim.x) {
            int m0, n0, kb0, kb1, split;
            decode(it, m0, n0, kb0, kb1, split);
            const bool tail = p.tail_tiles && it >= full_tiles;
            const bool sliced = tail || p.splits > 1;
            const long ldc = tail ? (long)BN : (sliced ? (long)p.N : p.ldc);
            const int row = m0 + q * 32 + lane;
            float *cbase;
            EpiRow e;
            const float *mrow = (sliced || !p.mask) ? nullptr : p.mask + (long)row * p.ldmask;
            if (tail) {
                const int j = it - full_tiles - split * p.tail_tiles;
                cbase = p.tail_partial + ((long)split * p.tail_tiles + j) * (TC_BM * BN);
                e.crow = cbase + (long)(q * 32 + lane) * BN - n0;
            } else {
                cbase = sliced ? p.partial + (long)split * p.M * p.N : p.C;
                e.crow = cbase + (long)row * ldc;
            }
            e.vec_ok = ((ldc & 3) == 0) && ((((uintptr_t)cbase) & 15u) == 0) &&
                       (!mrow || (((p.ldmask & 3) == 0) && ((((uintptr_t)p.mask) & 15u) == 0)));
            for (int c0k = kb0; c0k < kb1 && ok; c0k += p.chunk_kb) {
                /* one accumulator hand-over per chunk: the first chunk stores (bias, caller's accumulate),
                 * later ones add to what the earlier ones left, the last one applies the fused steps */
                const bool first_chunk = c0k == kb0, last_chunk = c0k + p.chunk_kb >= kb1;
                e.partial = first_chunk ? 0 : 1;
                e.bias = (sliced || !first_chunk) ? nullptr : p.bias;
                e.accumulate = (sliced || !first_chunk) ? 0 : p.accumulate;
                e.relu = (sliced || !last_chunk) ? 0 : p.relu;
                e.mrow = last_chunk ? mrow : nullptr;
                /* a later chunk that must also apply relu / a mask: add it like the others first, finish after
                 * the accumulator has been handed back */
                const bool finish_after = e.partial && (e.relu || e.mrow);
                const int fin_relu = e.relu; const float *fin_mrow = e.mrow;
                if (finish_after) { e.relu = 0; e.mrow = nullptr; }
                if (!mbar_wait_warp(bar_tfull + 8 * acc, acc_ph, abort_flag, p.status, 5)) { ok = false; break; }   /* tcgen05.ld needs the whole warp */
                tc_fence_after();
                #pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t r[32];
                    tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0), r);
                    if (SPLIT_ACC && TC_FULL_SPLIT(p) && last_chunk) {      /* the small cross terms join with the last chunk */
                        uint32_t r2[32];
                        tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(BN + c0), r2);
                        tc_wait_ld();
                        #pragma unroll
                        for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
                    }
                    tc_wait_ld();
                    if (c0 + 32 >= BN) {
                        /* last read of this accumulator: hand it back before the stores */
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
                    }
                    const int gc = n0 + c0;
                    if (row < p.M && gc < p.N) {
                        if (p.push_on) {
                            /* fused reduce-scatter: this 32-float block of the flat gradient belongs to chunk c;
                             * a foreign chunk's block goes into this rank's slot of its owner's staging area */
                            const long flat = (long)row * p.ldc + gc;
                            const int c = (int)(flat / p.push.chunk_floats);
                            EpiRow ep = e;
                            if (c != p.push.rank)
                                ep.crow = p.push.stage[c] + (long)p.push.rank * p.push.slot_floats + (flat - (long)c * p.push.chunk_floats) - gc;
                            epi_store32(r, gc, p.N, ep);
                        } else {
                            epi_store32(r, gc, p.N, e);
                        }
                    }
                }
                if (finish_after && row < p.M) {
                    #pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 32)
                        if (n0 + c0 < p.N) epi_finish32(n0 + c0, p.N, e.crow, fin_relu, fin_mrow, e.vec_ok);
                }
                if (++acc == NACC) { acc = 0; acc_ph ^= 1; }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

/* ======================================================================================
 * CTA-pair variant: tcgen05.mma.cta_group::2, tile 256x256 over two SMs.
 *
 * The one-CTA kernel is bound by shared-memory bandwidth: per K block of 32 the tensor core
 * reads 144 KB of operands (three MMAs per K step, A and B each time), the split pass moves
 * 96 KB and TMA writes 48 KB -- more than one SM's shared memory delivers in the 1536 cycles
 * the MMAs take.  In a pair each CTA stages its own 128 rows of A and HALF of B (128 of the
 * 256 columns); the pair's tensor cores share the B halves, so per SM the MMAs read 96 KB,
 * the split pass moves 64 KB and TMA writes 32 KB.  Loads carry no multicast: each CTA
 * fetches its own tiles.
 *
 * Shared memory holds two rings per CTA: TC2_STAGES stages of raw tiles (A rows + B half,
 * 32 KB), which TMA fills far ahead, and TC2_LO_SLOTS slots of lo tiles (32 KB), which live only
 * from the split pass to the cross-term MMAs.  hi*hi needs the raw tiles only and is issued as
 * soon as both CTAs' loads have landed; lo*hi and hi*lo follow when the slot is written.
 *
 * Protocol (rank 0 of the cluster is the leader and issues every MMA):
 *   full[s]     local : each CTA's TMA bytes for stage s (own A rows, own B half)
 *   hi[s]       leader: 2 arrivals, one per CTA, from its "landed" relay thread
 *   pass[l]     local : 8 arrivals, one per split warp: lo slot l is written
 *   lo[l]       leader: 2 arrivals, one per CTA, from its "written" relay thread
 *   empty[s]    both  : tcgen05.commit multicast when the MMAs have read stage s
 *   loempty[l]  both  : tcgen05.commit multicast when the cross-term MMAs have read slot l
 *   tfull[a]    both  : tcgen05.commit multicast when accumulator a is complete
 *   tempty[a]   leader: 2 x 4 arrivals, one per epilogue warp of both CTAs
 * An arrival at the other CTA's barrier carries a cluster-scope release and blocks the arriving
 * thread for 1000-1500 cycles (measured with clock stamps): done by the split warps themselves
 * it was what set the kernel's pace, hence the two relay threads (own warps), which turn the
 * cheap local arrivals into one remote arrival per CTA; the leader's own relays arrive locally.
 * Every CTA runs its own producer, split and epilogue warps on its own half of the tile. */
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                                  uint32_t *status, uint32_t code) {
    if (mbar_try_cluster(bar, parity)) return true;
    long long t0 = clock64();
    for (;;) {
        #pragma unroll 1
        for (int i = 0; i < 16; i++)
            if (mbar_try_cluster(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > TC_WAIT_CYCLES) {
            *abort_flag = 1;
            *(volatile uint32_t *)status = code | (blockIdx.x << 8);
            __threadfence_system();
            return false;
        }
    }
}
/* The same for a whole warp (see mbar_wait_warp). */
__device__ __forceinline__ bool mbar_wait_warp_cluster(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                                       uint32_t *status, uint32_t code) {
    bool got = true;
    if ((threadIdx.x & 31) == 0) got = mbar_wait_cluster(bar, parity, abort_flag, status, code);
    got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
    if (got) got = mbar_wait_cluster(bar, parity, abort_flag, status, code);     /* immediate: the phase is complete */
    return __all_sync(0xffffffffu, got);
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc2_commit_both(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc2_mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

#ifdef TT_TUNING
__device__ unsigned long long g_tc_dbg[24];
extern "C" int ttb_debug_gemm_read(unsigned long long out[24]) {
    cudaStreamSynchronize(g_tt.stream);
    unsigned long long z[24] = {0};
    if (cudaMemcpyFromSymbol(out, g_tc_dbg, sizeof z) != cudaSuccess) return -1;
    cudaMemcpyToSymbol(g_tc_dbg, z, sizeof z);
    return 0;
}
/* phase times are summed in registers and written once when the role ends: a global atomic per stamp
 * would sit in front of every release fence the role executes */
#define TC_STAMP(i) do { long long n_ = clock64(); dl[(i) & 3] += (unsigned long long)(n_ - tstamp); tstamp = n_; } while (0)
__device__ long long g_tc_trace[8 * 12];
extern "C" int ttb_debug_gemm_trace(long long out[96]) {
    cudaStreamSynchronize(g_tt.stream);
    return cudaMemcpyFromSymbol(out, g_tc_trace, sizeof(long long) * 96) == cudaSuccess ? 0 : -1;
}
/* absolute clock of event ev for K blocks 40..47 of CTA 0's first item */
#define TC_TRACE(ev) do { if (blockIdx.x == 0 && it == pair && kb >= 40 && kb < 48) g_tc_trace[(kb - 40) * 12 + (ev)] = clock64(); } while (0)
#define TC_STAMP_INIT long long tstamp = clock64(); unsigned long long dl[4] = {0, 0, 0, 0}; (void)tstamp
#define TC_STAMP_FLUSH(base, n) do { if (blockIdx.x == 0) for (int j_ = 0; j_ < (n); j_++) atomicAdd(&g_tc_dbg[(base) + j_], dl[j_]); } while (0)
#else
#define TC_STAMP(i) do { } while (0)
#define TC_TRACE(ev) do { } while (0)
#define TC_STAMP_INIT do { } while (0)
#define TC_STAMP_FLUSH(base, n) do { } while (0)
#endif

template <int A_MN, int B_MN, int SPLIT_ACC>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC2_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcParams p) {
    constexpr int BK = 32, STAGES = TC2_STAGES, LO_SLOTS = TC2_LO_SLOTS;
    constexpr int BN = 256, BNH = 128;                       /* pair tile is 256 wide, each CTA stages 128 columns of B */
    constexpr uint32_t A_BYTES = TC_BM * BK * 4;              /* 16 KB: this CTA's 128 rows */
    constexpr uint32_t B_BYTES = BNH * BK * 4;                /* 16 KB: this CTA's half of B */
    constexpr uint32_t BOX = BK * 128;
    constexpr uint32_t HI_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t LO_BASE = STAGES * HI_BYTES;           /* the lo slots follow the ring of raw tiles */
    /* M = 256 across the pair, N = 256 */
    constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)A_MN << 15) |
                               ((uint32_t)B_MN << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
    constexpr uint32_t TMEM_COLS = 2 * BN;
    constexpr int NACC = SPLIT_ACC ? 1 : 2;
    constexpr int TC_PREFETCH = STAGES + 4;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    uint64_t *bars = (uint64_t *)(smem_gen + (STAGES + LO_SLOTS) * HI_BYTES);
    const uint32_t bar_full = smem_u32(bars);
    const uint32_t bar_hi = bar_full + 8 * STAGES;
    const uint32_t bar_empty = bar_hi + 8 * STAGES;
    const uint32_t bar_lo = bar_empty + 8 * STAGES;
    const uint32_t bar_loempty = bar_lo + 8 * LO_SLOTS;
    const uint32_t bar_pass = bar_loempty + 8 * LO_SLOTS;      /* local: the split warps are done with a slot */
    const uint32_t bar_tfull = bar_pass + 8 * LO_SLOTS;
    const uint32_t bar_tempty = bar_tfull + 16;
    uint32_t *tmem_slot = (uint32_t *)(bars + 3 * STAGES + 3 * LO_SLOTS + 4);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int tiles_m = (p.M + 255) / 256;
    const int tiles_n = (p.N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (p.K + BK - 1) / BK;
    const int full_tiles = num_tiles - p.tail_tiles;     /* see TcParams: only the last wave's tiles are cut along K */
    const int num_items = p.tail_tiles ? full_tiles + p.tail_tiles * p.tail_splits : num_tiles * p.splits;
    auto decode = [&](int it, int &m0, int &n0, int &kb0, int &kb1, int &split) {
        int t;
        if (p.tail_tiles) {
            if (it < full_tiles) { t = it; split = 0; kb0 = 0; kb1 = num_kb; }
            else {
                const int j = it - full_tiles;
                split = j / p.tail_tiles;
                t = full_tiles + (j - split * p.tail_tiles);
                kb0 = split * p.tail_kb;
                kb1 = kb0 + p.tail_kb < num_kb ? kb0 + p.tail_kb : num_kb;
            }
        } else {
            split = it / num_tiles;
            t = it - split * num_tiles;
            kb0 = split * p.kb_per_split;
            kb1 = kb0 + p.kb_per_split < num_kb ? kb0 + p.kb_per_split : num_kb;
        }
        int tm, tn;
        tc_tile_coords(t, tiles_m, tiles_n, p.group_m, tm, tn);
        m0 = tm * 256; n0 = tn * BN;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_hi + 8 * s, 2);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int l = 0; l < LO_SLOTS; l++) {
            mbar_init(bar_lo + 8 * l, 2);
            mbar_init(bar_loempty + 8 * l, 1);
            mbar_init(bar_pass + 8 * l, TC_SPLIT_THREADS / 32);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, 2 * TC_EPI_THREADS / 32);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                       /* both CTAs' barriers exist before anybody signals across */
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    /* the leader's copies of the barriers everybody arrives on */
    const uint32_t lead_hi = map_to_cta(bar_hi, 0);
    const uint32_t lead_lo = map_to_cta(bar_lo, 0);
    const uint32_t lead_tempty = map_to_cta(bar_tempty, 0);

    if (warp == 0) {
        /* ---------------- TMA producer: own A rows, own half of B ---------------- */
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            bool ok = true;
            TC_STAMP_INIT;
            auto coords = [&](int m0, int n0, int &ma, int &nb) { ma = m0 + (int)rank * TC_BM; nb = n0 + (int)rank * BNH; };
            auto prefetch = [&](int m0, int n0, int kb) {
                if (p.noprefetch) return;
                int ma, nb; coords(m0, n0, ma, nb);
                const int k0 = kb * BK;
                if (A_MN && p.a_3d) tma_prefetch_3d(&map_a, 0, k0, ma / 32);
                else if (A_MN) { for (int b = 0; b < TC_BM / 32; b++) tma_prefetch_2d(&map_a, ma + 32 * b, k0); }
                else tma_prefetch_2d(&map_a, k0, ma);
                if (B_MN && p.b_3d) tma_prefetch_3d(&map_b, 0, k0, nb / 32);
                else if (B_MN) { for (int b = 0; b < BNH / 32; b++) tma_prefetch_2d(&map_b, nb + 32 * b, k0); }
                else tma_prefetch_2d(&map_b, k0, nb);
            };
            for (int it = pair; it < num_items && ok; it += num_pairs) {
                int m0, n0, kb0, kb1, split;
                decode(it, m0, n0, kb0, kb1, split);
                int ma, nb; coords(m0, n0, ma, nb);
                if (it == pair)
                    for (int kb = kb0 + STAGES; kb < kb0 + TC_PREFETCH && kb < kb1; kb++) prefetch(m0, n0, kb);
                for (int kb = kb0; kb < kb1; kb++) {
                    const int pk = kb + TC_PREFETCH;
                    if (pk < kb1) {
                        prefetch(m0, n0, pk);
                    } else if (it + num_pairs < num_items) {
                        int m2, n2, kb2, kb3, s2;
                        decode(it + num_pairs, m2, n2, kb2, kb3, s2);
                        if (kb2 + (pk - kb1) < kb3) prefetch(m2, n2, kb2 + (pk - kb1));
                    }
                    TC_STAMP(0);
                    if (!mbar_wait_cluster(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 3)) { ok = false; break; }
                    TC_STAMP(1);
                    TC_TRACE(0);
                    const uint32_t st = smem_base + s * HI_BYTES;
                    const uint32_t full = bar_full + 8 * s;
                    const int k0 = kb * BK;
                    mbar_expect_tx(full, HI_BYTES);
                    if (A_MN && p.a_3d) tma_load_3d(st, &map_a, full, 0, k0, ma / 32);
                    else if (A_MN) { for (int b = 0; b < TC_BM / 32; b++) tma_load_2d(st + b * BOX, &map_a, full, ma + 32 * b, k0); }
                    else tma_load_2d(st, &map_a, full, k0, ma);
                    if (B_MN && p.b_3d) tma_load_3d(st + A_BYTES, &map_b, full, 0, k0, nb / 32);
                    else if (B_MN) { for (int b = 0; b < BNH / 32; b++) tma_load_2d(st + A_BYTES + b * BOX, &map_b, full, nb + 32 * b, k0); }
                    else tma_load_2d(st + A_BYTES, &map_b, full, k0, nb);
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
            TC_STAMP_FLUSH(0, 2);
            if (!ok) { long long t0 = clock64(); while (clock64() - t0 < 200000) { } }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issuer: the leader CTA only ---------------- */
        if (lane == 0 && rank == 0) {
            int s = 0; uint32_t ph = 0;
            int l = 0; uint32_t lph = 0;
            int acc = 0; uint32_t acc_ph = 0;
            bool ok = true;
            TC_STAMP_INIT;
#ifdef TT_TUNING
            unsigned long long kcount = 0;
#endif
            for (int it = pair; it < num_items && ok; it += num_pairs) {
                int m0, n0, kb0, kb1, split;
                decode(it, m0, n0, kb0, kb1, split);
                TC_STAMP(0);
                if (!mbar_wait_cluster(bar_tempty + 8 * acc, acc_ph ^ 1, abort_flag, p.status, 4)) { ok = false; break; }
                TC_STAMP(3);
                tc_fence_after();
                uint32_t d_main = tmem_base + (uint32_t)(SPLIT_ACC ? 0 : acc * BN);
                uint32_t d_corr = SPLIT_ACC ? tmem_base + (uint32_t)BN : d_main;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (kb > kb0 && (kb - kb0) % p.chunk_kb == 0) {
                        tc2_commit_both(bar_tfull + 8 * acc);
                        if (++acc == NACC) { acc = 0; acc_ph ^= 1; }
                        TC_STAMP(0);
                        if (!mbar_wait_cluster(bar_tempty + 8 * acc, acc_ph ^ 1, abort_flag, p.status, 4)) { ok = false; break; }
                        TC_STAMP(3);
                        tc_fence_after();
                        d_main = tmem_base + (uint32_t)(SPLIT_ACC ? 0 : acc * BN);
                        d_corr = SPLIT_ACC ? tmem_base + (uint32_t)BN : d_main;
                    }
                    /* the raw tiles are enough for hi*hi: those four MMAs are issued as soon as both CTAs'
                     * loads have landed, while the split warps still produce the lo tiles */
                    TC_STAMP(0);
                    if (!mbar_wait_cluster(bar_hi + 8 * s, ph, abort_flag, p.status, 6)) { ok = false; break; }
                    TC_STAMP(1);
                    TC_TRACE(2);
                    tc_fence_after();
                    const uint32_t a_hi = smem_base + s * HI_BYTES;
                    const uint32_t b_hi = a_hi + A_BYTES;
                    const uint32_t a_lo = smem_base + LO_BASE + l * HI_BYTES;
                    const uint32_t b_lo = a_lo + A_BYTES;
                    const bool cross = TC_FULL_SPLIT(p);
                    if (SPLIT_ACC || !cross) {
                        #pragma unroll
                        for (int ks = 0; ks < BK / 8; ks++) {
                            const uint32_t first = ((kb - kb0) % p.chunk_kb != 0 || ks > 0) ? 1u : 0u;      /* main: restarts with every chunk */
                            tc2_mma_tf32(d_main, make_desc<A_MN, BK>(a_hi + (A_MN ? ks * 1024 : ks * 32)),
                                         make_desc<B_MN, BK>(b_hi + (B_MN ? ks * 1024 : ks * 32)), IDESC, first);
                        }
                    }
                    TC_STAMP(0);
                    TC_TRACE(3);
                    if (!mbar_wait_cluster(bar_lo + 8 * l, lph, abort_flag, p.status, 2)) { ok = false; break; }
                    TC_STAMP(2);
                    TC_TRACE(4);
#ifdef TT_TUNING
                    kcount++;
#endif
                    tc_fence_after();
                    if (cross) {
                        #pragma unroll
                        for (int ks = 0; ks < BK / 8; ks++) {
                            const uint32_t a_off = A_MN ? ks * 1024 : ks * 32;
                            const uint32_t b_off = B_MN ? ks * 1024 : ks * 32;
                            const uint64_t da_hi = make_desc<A_MN, BK>(a_hi + a_off);
                            const uint64_t db_hi = make_desc<B_MN, BK>(b_hi + b_off);
                            const uint64_t da_lo = make_desc<A_MN, BK>(a_lo + a_off);
                            const uint64_t db_lo = make_desc<B_MN, BK>(b_lo + b_off);
                            /* cross terms: with their own accumulator they run over the whole item */
                            const uint32_t first_corr = (kb > kb0 || ks > 0) ? 1u : 0u;
                            tc2_mma_tf32(d_corr, da_lo, db_hi, IDESC, first_corr);
                            tc2_mma_tf32(d_corr, da_hi, db_lo, IDESC, 1u);
                            if (!SPLIT_ACC) tc2_mma_tf32(d_main, da_hi, db_hi, IDESC, 1u);
                        }
                    }
                    tc2_commit_both(bar_empty + 8 * s);
                    tc2_commit_both(bar_loempty + 8 * l);
                    TC_TRACE(5);
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                    if (++l == LO_SLOTS) { l = 0; lph ^= 1; }
                }
                if (!ok) break;
                tc2_commit_both(bar_tfull + 8 * acc);
                if (++acc == NACC) { acc = 0; acc_ph ^= 1; }
            }
            TC_STAMP_FLUSH(4, 4);
#ifdef TT_TUNING
            if (blockIdx.x == 0) atomicAdd(&g_tc_dbg[12], kcount);
#endif
        }
    } else if (warp < 2 + TC_SPLIT_THREADS / 32) {
        /* ---------------- split warps: own tiles, report to the leader ---------------- */
        const int st_tid = threadIdx.x - 64;
        int s = 0; uint32_t ph = 0;
        int l = 0; uint32_t lph = 0;
        bool ok = true;
        TC_STAMP_INIT;
#ifdef TT_TUNING
#define SP_STAMP(i) do { if (st_tid == 0) TC_STAMP(i); } while (0)
#else
#define SP_STAMP(i) do { } while (0)
#endif
        for (int it = pair; it < num_items && ok; it += num_pairs) {
            int m0, n0, kb0, kb1, split;
            decode(it, m0, n0, kb0, kb1, split);
            for (int kb = kb0; kb < kb1; kb++) {
                SP_STAMP(0);
                if (!mbar_wait_warp(bar_full + 8 * s, ph, abort_flag, p.status, 1)) { ok = false; break; }
                SP_STAMP(1);
                if (st_tid == 0) TC_TRACE(6);
                /* the lo slot is free once the cross terms of two K blocks ago have been read */
                if (!mbar_wait_warp_cluster(bar_loempty + 8 * l, lph ^ 1, abort_flag, p.status, 7)) { ok = false; break; }
                SP_STAMP(2);
                if (st_tid == 0) TC_TRACE(7);
                if (TC_MAKE_LO(p)) {
                    const uint8_t *hi = smem_gen + s * HI_BYTES;
                    uint8_t *lo = smem_gen + LO_BASE + l * HI_BYTES;
                    #pragma unroll 4
                    for (uint32_t c = st_tid; c < HI_BYTES / 16; c += TC_SPLIT_THREADS) {
                        float4 v = *(const float4 *)(hi + c * 16);
                        float4 w = make_float4(split_lo(v.x), split_lo(v.y), split_lo(v.z), split_lo(v.w));
                        *(float4 *)(lo + c * 16) = w;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                SP_STAMP(3);
                if (st_tid == 0) TC_TRACE(8);
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_pass + 8 * l);      /* local and cheap; the relay warp tells the leader */
                if (++s == STAGES) { s = 0; ph ^= 1; }
                if (++l == LO_SLOTS) { l = 0; lph ^= 1; }
            }
        }
        if (st_tid == 0) TC_STAMP_FLUSH(8, 4);
    } else if (warp == TC_THREADS / 32) {
        /* ---------------- relay: split warps done with a lo slot -> one arrival at the leader ----------------
         * The arrival at another CTA's barrier carries a cluster-scope release, which costs the arriving
         * thread about a thousand cycles; here it costs the split warps nothing. */
        if (lane == 0) {
            int l = 0; uint32_t lph = 0;
            bool ok = true;
            for (int it = pair; it < num_items && ok; it += num_pairs) {
                int m0, n0, kb0, kb1, split;
                decode(it, m0, n0, kb0, kb1, split);
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(bar_pass + 8 * l, lph, abort_flag, p.status, 8)) { ok = false; break; }
                    TC_TRACE(9);
                    if (rank == 0) mbar_arrive(bar_lo + 8 * l); else mbar_arrive_cluster(lead_lo + 8 * l);
                    TC_TRACE(10);
                    if (++l == LO_SLOTS) { l = 0; lph ^= 1; }
                }
            }
        }
    } else if (warp == TC_THREADS / 32 + 1) {
        /* ---------------- relay: this CTA's raw tiles have landed -> one arrival at the leader ---------------- */
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            bool ok = true;
            for (int it = pair; it < num_items && ok; it += num_pairs) {
                int m0, n0, kb0, kb1, split;
                decode(it, m0, n0, kb0, kb1, split);
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 9)) { ok = false; break; }
                    if (rank == 0) mbar_arrive(bar_hi + 8 * s); else mbar_arrive_cluster(lead_hi + 8 * s);
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
        }
    } else {
        /* ---------------- epilogue warps: this CTA's 128 rows, all 256 columns ---------------- */
        const int q = warp & 3;
        int acc = 0; uint32_t acc_ph = 0;
        bool ok = true;
        TC_STAMP_INIT;
#ifdef TT_TUNING
        unsigned long long drains = 0;
#define EP_STAMP(i) do { if (warp == 10 && lane == 0) TC_STAMP(i); } while (0)
#else
#define EP_STAMP(i) do { } while (0)
#endif
        for (int it = pair; it < num_items && ok; it += num_pairs) {
            int m0, n0, kb0, kb1, split;
            decode(it, m0, n0, kb0, kb1, split);
            const bool tail = p.tail_tiles && it >= full_tiles;
            const bool sliced = tail || p.splits > 1;
            const long ldc = tail ? (long)BN : (sliced ? (long)p.N : p.ldc);
            const int row = m0 + (int)rank * TC_BM + q * 32 + lane;
            float *cbase;
            EpiRow e;
            const float *mrow = (sliced || !p.mask) ? nullptr : p.mask + (long)row * p.ldmask;
            if (tail) {
                const int j = it - full_tiles - split * p.tail_tiles;
                cbase = p.tail_partial + ((long)split * p.tail_tiles + j) * (256 * BN);
                e.crow = cbase + (long)((int)rank * TC_BM + q * 32 + lane) * BN - n0;
            } else {
                cbase = sliced ? p.partial + (long)split * p.M * p.N : p.C;
                e.crow = cbase + (long)row * ldc;
            }
            e.vec_ok = ((ldc & 3) == 0) && ((((uintptr_t)cbase) & 15u) == 0) &&
                       (!mrow || (((p.ldmask & 3) == 0) && ((((uintptr_t)p.mask) & 15u) == 0)));
            for (int c0k = kb0; c0k < kb1 && ok; c0k += p.chunk_kb) {
                const bool first_chunk = c0k == kb0, last_chunk = c0k + p.chunk_kb >= kb1;
                e.partial = first_chunk ? 0 : 1;
                e.bias = (sliced || !first_chunk) ? nullptr : p.bias;
                e.accumulate = (sliced || !first_chunk) ? 0 : p.accumulate;
                e.relu = (sliced || !last_chunk) ? 0 : p.relu;
                e.mrow = last_chunk ? mrow : nullptr;
                /* a later chunk that must also apply relu / a mask: add it like the others first, finish after
                 * the accumulator has been handed back */
                const bool finish_after = e.partial && (e.relu || e.mrow);
                const int fin_relu = e.relu; const float *fin_mrow = e.mrow;
                if (finish_after) { e.relu = 0; e.mrow = nullptr; }
                EP_STAMP(3);
                if (!mbar_wait_warp(bar_tfull + 8 * acc, acc_ph, abort_flag, p.status, 5)) { ok = false; break; }
                EP_STAMP(0);
#ifdef TT_TUNING
                drains++;
#endif
                tc_fence_after();
                #pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t r[32];
                    tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0), r);
                    if (SPLIT_ACC && TC_FULL_SPLIT(p) && last_chunk) {      /* the small cross terms join with the last chunk */
                        uint32_t r2[32];
                        tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(BN + c0), r2);
                        tc_wait_ld();
                        #pragma unroll
                        for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
                    }
                    tc_wait_ld();
                    if (c0 + 32 >= BN) {
                        tc_fence_before();
                        __syncwarp();
                        EP_STAMP(1);
                        if (lane == 0) mbar_arrive_cluster(lead_tempty + 8 * acc);
                        EP_STAMP(2);
                    }
                    const int gc = n0 + c0;
                    if (row < p.M && gc < p.N) {
                        if (p.push_on) {
                            /* fused reduce-scatter: this 32-float block of the flat gradient belongs to chunk c;
                             * a foreign chunk's block goes into this rank's slot of its owner's staging area */
                            const long flat = (long)row * p.ldc + gc;
                            const int c = (int)(flat / p.push.chunk_floats);
                            EpiRow ep = e;
                            if (c != p.push.rank)
                                ep.crow = p.push.stage[c] + (long)p.push.rank * p.push.slot_floats + (flat - (long)c * p.push.chunk_floats) - gc;
                            epi_store32(r, gc, p.N, ep);
                        } else {
                            epi_store32(r, gc, p.N, e);
                        }
                    }
                }
                if (finish_after && row < p.M) {
                    #pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 32)
                        if (n0 + c0 < p.N) epi_finish32(n0 + c0, p.N, e.crow, fin_relu, fin_mrow, e.vec_ok);
                }
                if (++acc == NACC) { acc = 0; acc_ph ^= 1; }
            }
        }
#ifdef TT_TUNING
        if (warp == 10 && lane == 0) { EP_STAMP(3); TC_STAMP_FLUSH(16, 4); if (blockIdx.x == 0) atomicAdd(&g_tc_dbg[20], drains); }
#endif
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                       /* no CTA leaves while its peer may still signal it or read its tiles */
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

/* The elementwise steps fused behind a product, for the kernels that finish a sliced one. */
struct EpiFused { const float *bias; int accumulate, relu; const float *mask; long ldmask; };

/* Second phase of split-K: C[m,n] (+)= f(bias[n] + sum over slices), slices added in order. */
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ partial, int splits, int M, int N,
                                                             float *__restrict__ C, long ldc, EpiFused f) {
    const float *__restrict__ bias = f.bias;
    const int accumulate = f.accumulate;
    const long total = (long)M * N;
    const long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int m = (int)(i / N), n = (int)(i - (long)m * N);
        float s = 0.0f;
        for (int k = 0; k < splits; k++) s += partial[(long)k * total + i];
        if (bias) s += bias[n];
        if (f.relu) s = s > 0.0f ? s : 0.0f;
        if (f.mask) s = f.mask[(long)m * f.ldmask + n] > 0.0f ? s : 0.0f;
        float *c = C + (long)m * ldc + n;
        *c = accumulate ? *c + s : s;
    }
}

/* Second phase of the tail split: for each tail tile, C (+)= f(bias + slices in order). */
__global__ void __launch_bounds__(256) tail_reduce_kernel(const float *__restrict__ partial, int splits, int tail_tiles,
                                                           int first_tile, int tiles_m, int tiles_n, int group_m, int BM, int BN, int M, int N,
                                                           float *__restrict__ C, long ldc, EpiFused f) {
    const float *__restrict__ bias = f.bias;
    const int accumulate = f.accumulate;
    const int tile4 = BM * BN / 4, bn4 = BN / 4;
    const long total4 = (long)tail_tiles * tile4;
    const long stride = (long)gridDim.x * blockDim.x;
    const bool vec_c = ((ldc & 3) == 0) && ((((uintptr_t)C) & 15u) == 0) &&
                       (!f.mask || (((f.ldmask & 3) == 0) && ((((uintptr_t)f.mask) & 15u) == 0)));
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += stride) {
        const int tj = (int)(i / tile4);
        const int rem = (int)(i - (long)tj * tile4);
        const int r = rem / bn4, c = (rem - r * bn4) * 4;
        const int t = first_tile + tj;
        int tm, tn;
        tc_tile_coords(t, tiles_m, tiles_n, group_m, tm, tn);
        const int m = tm * BM + r, n = tn * BN + c;
        if (m >= M || n >= N) continue;
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < splits; k++) {
            const float4 v = *(const float4 *)(partial + ((long)k * tail_tiles + tj) * ((long)BM * BN) + (long)rem * 4);
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        float *cp = C + (long)m * ldc + n;
        if (vec_c && n + 3 < N) {
            if (bias) { s.x += bias[n]; s.y += bias[n + 1]; s.z += bias[n + 2]; s.w += bias[n + 3]; }
            if (f.relu) {
                s.x = s.x > 0.0f ? s.x : 0.0f; s.y = s.y > 0.0f ? s.y : 0.0f;
                s.z = s.z > 0.0f ? s.z : 0.0f; s.w = s.w > 0.0f ? s.w : 0.0f;
            }
            if (f.mask) {
                const float4 k = *(const float4 *)(f.mask + (long)m * f.ldmask + n);
                s.x = k.x > 0.0f ? s.x : 0.0f; s.y = k.y > 0.0f ? s.y : 0.0f;
                s.z = k.z > 0.0f ? s.z : 0.0f; s.w = k.w > 0.0f ? s.w : 0.0f;
            }
            if (accumulate) { const float4 o = *(const float4 *)cp; s.x = o.x + s.x; s.y = o.y + s.y; s.z = o.z + s.z; s.w = o.w + s.w; }
            *(float4 *)cp = s;
        } else {
            const float sv[4] = {s.x, s.y, s.z, s.w};
            for (int j = 0; j < 4 && n + j < N; j++) {
                float v = sv[j];
                if (bias) v += bias[n + j];
                if (f.relu) v = v > 0.0f ? v : 0.0f;
                if (f.mask) v = f.mask[(long)m * f.ldmask + n + j] > 0.0f ? v : 0.0f;
                cp[j] = accumulate ? cp[j] + v : v;
            }
        }
    }
}

/* ---- host side ----------------------------------------------------------------*/
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;
static uint32_t *g_status_host = nullptr;     /* mapped pinned word the kernel reports into */
static uint32_t *g_status_dev = nullptr;
static int g_tc_passes = 3;
static int g_tc_nosplit = 0;
static int g_tc_prefetch = -1;       /* TT_TC_PREFETCH: L2 prefetch ahead of the loads; -1 = one-CTA kernel yes, pair kernel no (measured) */
static int g_tc_2cta = 1;            /* TT_TC_2CTA=0: tuning aid, one-CTA kernel for every shape */
static int g_tc_force_bk = 0;        /* TT_TC_BK: tuning aid, 0 = by tile shape */
static int g_tc_force_bn = 0;        /* TT_TC_BN: tuning aid, 0 = choose by tile count */
static int g_tc_splitk = 1;          /* TT_TC_SPLITK=0: tuning aid, never cut the reduction across CTAs */
static int g_tc_tail = 1;            /* TT_TC_TAIL=0: tuning aid, never cut only the last wave's tiles */
static int g_tc_fit = 1;             /* TT_TC_FIT=0: data-parallel jobs use every SM for every GEMM */
static int g_tc_fit_world = 4;       /* from this many ranks on (on two GPUs the collective is light and the fit costs more than it frees) */
static int g_tc_mn3d = 1;            /* TT_TC_MN3D=0: tuning aid, one TMA per 32 columns for MN-major tiles */
static int g_tc_split_k = 1024;      /* reductions longer than this keep the cross terms in their own accumulator */
static int g_tc_group_m = TC_GROUP_M; /* TT_TC_GROUP_M: tile rows per rasterisation group (a huge value = full-height stripes) */
static int g_tc_chunk_k = 2048;      /* reductions of twice this and more fold the main accumulator into the destination every this many K (TT_TC_CHUNK_K) */

/* Tuning knobs from the environment (no GPU needed).  Only a -DTT_TUNING build reads them: several
 * (one pass, no split) make the kernel produce wrong numbers and none belongs in a product build. */
static void tc_read_env(void) {
#ifdef TT_TUNING
    static bool done = false;
    if (done) return;
    done = true;
    const char *e = getenv("TT_TC_PASSES");
    if (e && atoi(e) == 1) g_tc_passes = 1;
    e = getenv("TT_TC_PREFETCH");
    if (e && *e) g_tc_prefetch = atoi(e);
    e = getenv("TT_TC_NOSPLIT");
    if (e && atoi(e) == 1) g_tc_nosplit = 1;
    e = getenv("TT_TC_SPLITK");
    if (e && *e) g_tc_splitk = atoi(e);
    e = getenv("TT_TC_FIT");
    if (e && *e) g_tc_fit = atoi(e);
    e = getenv("TT_TC_FIT_WORLD");
    if (e && *e) g_tc_fit_world = atoi(e);
    e = getenv("TT_TC_TAIL");
    if (e && *e) g_tc_tail = atoi(e);
    e = getenv("TT_TC_MN3D");
    if (e && *e) g_tc_mn3d = atoi(e);
    e = getenv("TT_TC_2CTA");
    if (e && *e) g_tc_2cta = atoi(e);
    e = getenv("TT_TC_BK");
    if (e && *e) g_tc_force_bk = atoi(e);
    e = getenv("TT_TC_BN");
    if (e && *e) g_tc_force_bn = atoi(e);
    e = getenv("TT_TC_SPLIT_K");
    if (e && *e) g_tc_split_k = atoi(e);
    e = getenv("TT_TC_GROUP_M");
    if (e && *e && atoi(e) >= 1) g_tc_group_m = atoi(e);
    e = getenv("TT_TC_CHUNK_K");
    if (e && *e && atoi(e) >= 256) g_tc_chunk_k = atoi(e) / 32 * 32;
#endif
}

static int tc_setup(void) {
    if (g_encode && g_status_host) return 0;
    if (tt_ctx_init() != 0) return -1;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (!tt_cuda_ok(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres), "cudaGetDriverEntryPoint") ||
        qres != cudaDriverEntryPointSuccess || !fn) {
        tt_set_error("cuTensorMapEncodeTiled is not available from this driver");
        return -1;
    }
    g_encode = (EncodeTiledFn)fn;
    if (!tt_cuda_ok(cudaHostAlloc((void **)&g_status_host, sizeof(uint32_t), cudaHostAllocMapped), "cudaHostAlloc")) return -1;
    *g_status_host = 0;
    if (!tt_cuda_ok(cudaHostGetDevicePointer((void **)&g_status_dev, g_status_host, 0), "cudaHostGetDevicePointer")) return -1;
    tc_read_env();
    return 0;
}

/* Non-zero when a tensor-core kernel gave up on a wait since the last call. */
int gemm_tc_poll_status(void) {
    const int conv = conv_tc_poll_status();          /* the convolution kernel reports the same way */
    if (conv) return conv;
    if (!g_status_host) return 0;
    uint32_t v = *(volatile uint32_t *)g_status_host;
    if (v) {
        tt_set_error("tcgen05 GEMM: bounded wait expired (code %u, CTA %u)", v & 0xffu, v >> 8);
        *g_status_host = 0;
        return (int)v;
    }
    return 0;
}

/* Encoded tensor maps are kept: a training loop presents the same few (address, shape, pitch, box)
 * combinations every step (the pool hands a layer's activations the same block each time), and an
 * encode is a driver call.  Direct-mapped, 256 slots, keyed by everything that goes into the map. */
struct MapKey { const float *base; long d0, d1, pitch; int b0, b1, b2, kind; };
struct MapSlot { MapKey key; CUtensorMap map; bool used; };
static MapSlot g_maps[256];
static bool map_key_eq(const MapKey &a, const MapKey &b) {
    return a.base == b.base && a.d0 == b.d0 && a.d1 == b.d1 && a.pitch == b.pitch && a.b0 == b.b0 && a.b1 == b.b1 &&
           a.b2 == b.b2 && a.kind == b.kind;
}
static MapSlot *map_slot(const MapKey &k, bool *hit) {
    uint64_t h = (uint64_t)(uintptr_t)k.base * 0x9E3779B97F4A7C15ull;
    h ^= (uint64_t)k.d0 * 0xC2B2AE3D27D4EB4Full + (uint64_t)k.d1 * 0x165667B19E3779F9ull + (uint64_t)k.pitch * 31 +
         (uint64_t)(k.b0 * 131 + k.b1 * 17 + k.b2 * 7 + k.kind);
    MapSlot *s = &g_maps[(h >> 32) & 255];
    *hit = s->used && map_key_eq(s->key, k);
    return s;
}

/* inner = contiguous extent, outer = number of rows, pitch in floats */
static int encode_map(CUtensorMap *map, const float *base, long inner, long outer, long pitch, int box_inner, int box_outer,
                      int mn_major) {
    const MapKey key = {base, inner, outer, pitch, box_inner, box_outer, 0, mn_major ? 1 : 0};
    bool hit;
    MapSlot *slot = map_slot(key, &hit);
    if (hit) { *map = slot->map; return 0; }
    /* K-major boxes are box_inner*4 bytes wide: 128 -> SWIZZLE_128B, 64 -> SWIZZLE_64B */
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * sizeof(float)};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)base, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                   : (box_inner == 16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B),
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { tt_set_error("cuTensorMapEncodeTiled failed (%d)", (int)r); return -1; }
    slot->key = key; slot->map = *map; slot->used = true;
    return 0;
}

/* MN-major operand stored [K rows][MN] with MN a multiple of 32, seen as a rank-3 tensor
 * {32 values, K rows, MN/32 column groups} with strides {4, pitch*4, 128} bytes.  A box
 * {32, 32, groups} then lands in shared memory group after group, 32 k-rows of 128 bytes
 * each -- the layout the kernel's MN-major descriptors expect -- with ONE copy per tile. */
static int encode_map_mn3d(CUtensorMap *map, const float *base, long mn, long k, long pitch, int groups, int bk) {
    const MapKey key = {base, mn, k, pitch, 32, bk, groups, 2};
    bool hit;
    MapSlot *slot = map_slot(key, &hit);
    if (hit) { *map = slot->map; return 0; }
    cuuint64_t dims[3] = {32, (cuuint64_t)k, (cuuint64_t)(mn / 32)};
    cuuint64_t strides[2] = {(cuuint64_t)pitch * sizeof(float), 128};
    cuuint32_t box[3] = {32, (cuuint32_t)bk, (cuuint32_t)groups};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void *)base, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -1;
    slot->key = key; slot->map = *map; slot->used = true;
    return 0;
}

int gemm_tc_usable(const GemmArgs *g) {
    if (g->a_pad_ones) return 0;
    if (g->M <= 0 || g->N <= 0 || g->K <= 0) return 0;
    if ((((uintptr_t)g->A) & 15u) || (((uintptr_t)g->B) & 15u)) return 0;
    if ((g->lda & 3) || (g->ldb & 3)) return 0;
    if (g->lda >= (1l << 36) || g->ldb >= (1l << 36)) return 0;
    return 1;
}

/* Split-K plan of the launch being prepared (host side, single caller thread). */
static struct { int splits, kb_per_split; float *partial; int tail_tiles, tail_splits, tail_kb; float *tail_partial; int units; int chunk_kb; int push_on; } g_plan = {1, 0, nullptr, 0, 0, 0, nullptr, 0, 1 << 30, 0};

template <int A_MN, int B_MN, int BN, int BK, int STAGES, int SPLIT_ACC>
static int launch_tc(const GemmArgs *g, const CUtensorMap &ma, const CUtensorMap &mb, int a_3d, int b_3d) {
    constexpr size_t smem = (size_t)STAGES * 2 * (TC_BM * BK * 4 + BN * BK * 4) + 1024 + 8 * (3 * STAGES + 4) + 16;
    static bool configured = false;
    auto kern = gemm_tc_kernel<A_MN, B_MN, BN, BK, STAGES, SPLIT_ACC>;
    if (!configured) {
        if (!tt_cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                        "cudaFuncSetAttribute(smem)")) return -1;
        configured = true;
    }
    TcParams p;
    p.M = g->M; p.N = g->N; p.K = g->K; p.C = g->C; p.ldc = g->ldc; p.bias = g->bias;
    p.accumulate = g->accumulate; p.passes = g_tc_passes; p.status = g_status_dev; p.nosplit = g_tc_nosplit; p.noprefetch = g_tc_prefetch == 0;
    p.a_3d = a_3d; p.b_3d = b_3d;
    p.relu = g->relu; p.mask = g->mask; p.ldmask = g->ldmask;
    p.chunk_kb = g_plan.chunk_kb;
    p.group_m = g_tc_group_m;
    p.push_on = g_plan.push_on;
    if (g_plan.push_on) p.push = *g->push;
    const EpiFused fused = {g->bias, g->accumulate, g->relu, g->mask, g->ldmask};
    p.splits = g_plan.splits; p.kb_per_split = g_plan.kb_per_split; p.partial = g_plan.partial;
    p.tail_tiles = g_plan.tail_tiles; p.tail_splits = g_plan.tail_splits; p.tail_kb = g_plan.tail_kb;
    p.tail_partial = g_plan.tail_partial;
    const int tiles_m = (g->M + TC_BM - 1) / TC_BM;
    const int plain_tiles = tiles_m * ((g->N + BN - 1) / BN);
    int tiles = p.tail_tiles ? plain_tiles - p.tail_tiles + p.tail_tiles * p.tail_splits : plain_tiles * p.splits;
    const int max_ctas = g_plan.units > 0 ? g_plan.units : g_tt.gemm_sms;
    int grid = tiles < max_ctas ? tiles : max_ctas;
    tt_trace_begin(TTB_K_GEMM_TC);
    kern<<<grid, TC_THREADS, smem, g_tt.stream>>>(ma, mb, p);
    g_tt.launches++;
    if (p.tail_tiles) {
        long total4 = (long)p.tail_tiles * TC_BM * BN / 4;
        long blocks = (total4 + 255) / 256, cap = (long)g_tt.sm_count * 8;
        tail_reduce_kernel<<<(int)(blocks < cap ? blocks : cap), 256, 0, g_tt.stream>>>(
            p.tail_partial, p.tail_splits, p.tail_tiles, plain_tiles - p.tail_tiles, tiles_m, (g->N + BN - 1) / BN, p.group_m, TC_BM, BN, g->M, g->N,
            g->C, g->ldc, fused);
        g_tt.launches++;
    } else if (p.splits > 1) {
        long total = (long)g->M * g->N;
        long blocks = (total + 255) / 256, cap = (long)g_tt.sm_count * 8;
        splitk_reduce_kernel<<<(int)(blocks < cap ? blocks : cap), 256, 0, g_tt.stream>>>(
            p.partial, p.splits, g->M, g->N, g->C, g->ldc, fused);
        g_tt.launches++;
    }
    tt_trace_end(TTB_K_GEMM_TC, 2.0 * (double)g->M * g->N * g->K);
    return tt_cuda_ok(cudaGetLastError(), "tcgen05 GEMM launch") ? 0 : -1;
}

template <int A_MN, int B_MN, int SPLIT_ACC>
static int launch_tc2_inst(const GemmArgs *g, const CUtensorMap &ma, const CUtensorMap &mb, int a_3d, int b_3d) {
    constexpr size_t smem = (size_t)(TC2_STAGES + TC2_LO_SLOTS) * (TC_BM * 32 * 4 + 128 * 32 * 4) + 1024 + 8 * (3 * TC2_STAGES + 3 * TC2_LO_SLOTS + 4) + 16;
    static bool configured = false;
    auto kern = gemm_tc2_kernel<A_MN, B_MN, SPLIT_ACC>;
    if (!configured) {
        if (!tt_cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                        "cudaFuncSetAttribute(smem)")) return -1;
        configured = true;
    }
    TcParams p;
    p.M = g->M; p.N = g->N; p.K = g->K; p.C = g->C; p.ldc = g->ldc; p.bias = g->bias;
    p.accumulate = g->accumulate; p.passes = g_tc_passes; p.status = g_status_dev; p.nosplit = g_tc_nosplit; p.noprefetch = g_tc_prefetch != 1;
    p.a_3d = a_3d; p.b_3d = b_3d;
    p.relu = g->relu; p.mask = g->mask; p.ldmask = g->ldmask;
    p.chunk_kb = g_plan.chunk_kb;
    p.group_m = g_tc_group_m;
    p.push_on = g_plan.push_on;
    if (g_plan.push_on) p.push = *g->push;
    const EpiFused fused = {g->bias, g->accumulate, g->relu, g->mask, g->ldmask};
    p.splits = g_plan.splits; p.kb_per_split = g_plan.kb_per_split; p.partial = g_plan.partial;
    p.tail_tiles = g_plan.tail_tiles; p.tail_splits = g_plan.tail_splits; p.tail_kb = g_plan.tail_kb;
    p.tail_partial = g_plan.tail_partial;
    const int tiles_m = (g->M + 255) / 256;
    const long plain_tiles = (long)tiles_m * ((g->N + 255) / 256);
    long items = p.tail_tiles ? plain_tiles - p.tail_tiles + (long)p.tail_tiles * p.tail_splits : plain_tiles * p.splits;
    long pairs = g_plan.units > 0 ? g_plan.units : g_tt.gemm_sms / 2;
    if (items < pairs) pairs = items;
    tt_trace_begin(TTB_K_GEMM_TC);
    kern<<<(int)(2 * pairs), TC2_THREADS, smem, g_tt.stream>>>(ma, mb, p);
    g_tt.launches++;
    if (p.tail_tiles) {
        long total4 = (long)p.tail_tiles * 256 * 256 / 4;
        long blocks = (total4 + 255) / 256, cap = (long)g_tt.sm_count * 8;
        tail_reduce_kernel<<<(int)(blocks < cap ? blocks : cap), 256, 0, g_tt.stream>>>(
            p.tail_partial, p.tail_splits, p.tail_tiles, (int)plain_tiles - p.tail_tiles, tiles_m, (g->N + 255) / 256, p.group_m, 256, 256, g->M, g->N,
            g->C, g->ldc, fused);
        g_tt.launches++;
    } else if (p.splits > 1) {
        long total = (long)g->M * g->N;
        long blocks = (total + 255) / 256, cap = (long)g_tt.sm_count * 8;
        splitk_reduce_kernel<<<(int)(blocks < cap ? blocks : cap), 256, 0, g_tt.stream>>>(
            p.partial, p.splits, g->M, g->N, g->C, g->ldc, fused);
        g_tt.launches++;
    }
    tt_trace_end(TTB_K_GEMM_TC, 2.0 * (double)g->M * g->N * g->K);
    return tt_cuda_ok(cudaGetLastError(), "tcgen05 pair GEMM launch") ? 0 : -1;
}
static int launch_tc2(const GemmArgs *g, const CUtensorMap &ma, const CUtensorMap &mb, int a_3d, int b_3d, bool split_acc) {
    const int a_mn = g->ta ? 1 : 0, b_mn = g->tb ? 0 : 1;
    if (split_acc) {
        if (!a_mn && !b_mn) return launch_tc2_inst<0, 0, 1>(g, ma, mb, a_3d, b_3d);
        if (!a_mn && b_mn)  return launch_tc2_inst<0, 1, 1>(g, ma, mb, a_3d, b_3d);
        if (a_mn && !b_mn)  return launch_tc2_inst<1, 0, 1>(g, ma, mb, a_3d, b_3d);
        return launch_tc2_inst<1, 1, 1>(g, ma, mb, a_3d, b_3d);
    }
    if (!a_mn && !b_mn) return launch_tc2_inst<0, 0, 0>(g, ma, mb, a_3d, b_3d);
    if (!a_mn && b_mn)  return launch_tc2_inst<0, 1, 0>(g, ma, mb, a_3d, b_3d);
    if (a_mn && !b_mn)  return launch_tc2_inst<1, 0, 0>(g, ma, mb, a_3d, b_3d);
    return launch_tc2_inst<1, 1, 0>(g, ma, mb, a_3d, b_3d);
}

template <int BN, int BK, int STAGES, int SPLIT_ACC>
static int launch_tc_major(const GemmArgs *g, const CUtensorMap &ma, const CUtensorMap &mb, int a_3d, int b_3d) {
    const int a_mn = g->ta ? 1 : 0, b_mn = g->tb ? 0 : 1;
    if (!a_mn && !b_mn) return launch_tc<0, 0, BN, BK, STAGES, SPLIT_ACC>(g, ma, mb, a_3d, b_3d);
    if (!a_mn && b_mn)  return launch_tc<0, 1, BN, BK, STAGES, SPLIT_ACC>(g, ma, mb, a_3d, b_3d);
    if (a_mn && !b_mn)  return launch_tc<1, 0, BN, BK, STAGES, SPLIT_ACC>(g, ma, mb, a_3d, b_3d);
    return launch_tc<1, 1, BN, BK, STAGES, SPLIT_ACC>(g, ma, mb, a_3d, b_3d);
}

/* What the host decides for one product, from its shape alone: tile width, one-CTA or pair kernel,
 * how many CTAs (or pairs) take tiles, and how the reduction is cut.  Pure: no GPU, no allocation. */
struct TcShapePlan {
    int bn, pair, bk, units;
    long tiles;
    int splits, kb_per_split;                /* uniform split-K: every tile in `splits` slices */
    int tail_tiles, tail_splits, tail_kb;    /* tail split: only the last wave's tiles */
    int split_acc;
};
static void tc_plan_shape(int M, int N, int K, int gemm_sms, int world, TcShapePlan *o) {
    tc_read_env();
    /* 128x256 tiles unless that leaves most SMs idle */
    const long tiles256 = (long)((M + TC_BM - 1) / TC_BM) * ((N + 255) / 256);
    int bn = (tiles256 * 10 < (long)gemm_sms * 7 || N <= 128) ? 128 : 256;
    if (g_tc_force_bn == 128 || g_tc_force_bn == 256) bn = g_tc_force_bn;
    /* CTA pairs (256x256 tile over two SMs) for the big shapes */
    const bool pair = g_tc_2cta && bn == 256 && M >= 256 && gemm_sms >= 2;
    /* K blocks of 32.  TT_TC_BK=16 selects 64-byte rows with twice the stages in the one-CTA kernel;
     * measured equal there and slower in the pair kernel, so it stays a tuning aid. */
    int bk = 32;
    if (!pair && (g_tc_force_bk == 16 || g_tc_force_bk == 32)) bk = g_tc_force_bk;
    const int num_kb = (K + bk - 1) / bk;
    const long tiles = (long)((M + (pair ? 255 : TC_BM - 1)) / (pair ? 256 : TC_BM)) * ((N + bn - 1) / bn);
    int units = pair ? gemm_sms / 2 : gemm_sms;                      /* CTAs, or CTA pairs, that take tiles */
    /* While gradients are being reduced on the other stream, a GEMM takes no more SMs than its wave
     * count needs: 64 pair tiles run as one wave on 64 pairs as fast as on 74, and the ten SM pairs
     * left over are where the collective's CTAs run instead of displacing GEMM CTAs (a GEMM CTA fills
     * an SM's shared memory, so the two never share an SM).  8 GPUs, large MLP: GEMM time per step
     * 2.07 -> 1.71 ms.  Shapes with few tiles keep every SM: they are cut along K instead. */
    if (g_tc_fit && world >= g_tc_fit_world && world > 1 && tiles * 2 > units) {
        const long waves = (tiles + units - 1) / units;
        const long fit = (tiles + waves - 1) / waves;
        if (fit < units) units = (int)fit;
    }
    o->bn = bn; o->pair = pair; o->bk = bk; o->units = units; o->tiles = tiles;
    o->splits = 1; o->kb_per_split = num_kb;
    o->tail_tiles = 0; o->tail_splits = 0; o->tail_kb = 0;
    /* Split-K when the tiles alone leave most SMs idle and the reduction is long enough to cut:
     * slices of at least four K blocks, as many as fill the machine, partials in pool scratch. */
    long want = 1;
    long tail_s = 0;                                   /* > 1: cut only the tiles of the last wave */
    if (g_tc_splitk && tiles * 2 <= units && num_kb >= 2 * (128 / bk)) {
        /* few tiles: as many slices as fill the machine */
        want = units / tiles;
        if (want > num_kb / (128 / bk)) want = num_kb / (128 / bk);      /* slices of at least 128 along K */
    } else if (g_tc_splitk && (long)num_kb * bk >= 1024) {
        /* many tiles: the last wave may be mostly empty (512 tiles on 148 SMs run as 4 waves of
         * work worth 3.46).  Either every tile is cut into two to four slices, or only the
         * tiles of the last wave are (the earlier waves are full already, and the partial
         * products to write and re-read are a fraction).  Each candidate is priced as waves
         * of MMA time plus the traffic of its partial products; the cheapest wins. */
        const double sms = (double)units;
        /* one tile on one SM (a pair tile keeps two SMs busy for as long), 75 % of the pipe */
        const double tile_us = 6.0 * 128.0 * bn * (double)K / (4096.0 * 1.8e3 * 0.75);
        double best = 1e30;
        for (long sp = 1; sp <= 4; sp++) {
            if ((long)(num_kb / sp) * bk < 512) break;
            const double items = (double)tiles * sp;
            const double waves = (double)((long)((items + sms - 1) / sms));
            const double extra_us = sp > 1 ? (2.0 * sp + 1.0) * M * (double)N * 4.0 / 5.0e6 + 6.0 : 0.0;
            const double t = tile_us * waves / sp + extra_us;
            if (t < best * 0.98) { best = t; want = sp; }
        }
        const long full_waves = tiles / units, rest = tiles - full_waves * units;
        if (g_tc_tail && full_waves >= 1 && rest > 0) {
            for (long sp = 2; sp <= 8; sp++) {
                if ((long)(num_kb / sp) * bk < 256) break;
                const double waves = (double)((rest * sp + units - 1) / units);
                const double extra_us = (2.0 * sp + 1.0) * rest * (pair ? 256.0 : 128.0) * bn * 4.0 / 5.0e6 + 6.0;
                const double t = tile_us * ((double)full_waves + waves / sp) + extra_us;
                if (t < best * 0.98) { best = t; want = 1; tail_s = sp; }
            }
        }
    }
    if (want >= 2) {
        const long max_by_mem = (512l << 20) / ((long)M * N * 4 + 1);
        if (want > max_by_mem) want = max_by_mem;
    }
    if (want >= 2) {
        const int per = (int)((num_kb + want - 1) / want);
        o->splits = (num_kb + per - 1) / per; o->kb_per_split = per;
    } else if (tail_s >= 2) {
        const int per = (int)((num_kb + tail_s - 1) / tail_s);
        o->tail_tiles = (int)(tiles % units); o->tail_splits = (num_kb + per - 1) / per; o->tail_kb = per;
    }
    /* long reductions keep the cross terms in their own accumulator (see the kernel) */
    o->split_acc = (long)o->kb_per_split * bk > g_tc_split_k;
}

/* The plan for a shape as ten integers {bn, pair, bk, units, tiles, splits, kb_per_split, tail_tiles,
 * tail_splits, tail_kb}: lets tests check the planner on a machine without a GPU. */
extern "C" int ttb_gemm_plan(int M, int N, int K, int sms, int world, int out[10]) {
    if (!out || M <= 0 || N <= 0 || K <= 0 || sms < 1 || world < 1) return -1;
    TcShapePlan pl;
    tc_plan_shape(M, N, K, sms, world, &pl);
    out[0] = pl.bn; out[1] = pl.pair; out[2] = pl.bk; out[3] = pl.units; out[4] = (int)pl.tiles;
    out[5] = pl.splits; out[6] = pl.kb_per_split; out[7] = pl.tail_tiles; out[8] = pl.tail_splits; out[9] = pl.tail_kb;
    return 0;
}

int gemm_tc(const GemmArgs *g) {
    if (!gemm_tc_usable(g)) { tt_set_error("tcgen05 GEMM: operands are not 16-byte aligned with 16-byte row pitch"); return -1; }
    if (tc_setup() != 0) return -1;
    TcShapePlan pl;
    tc_plan_shape(g->M, g->N, g->K, g_tt.gemm_sms, tt_dist_active() ? ttb_dist_world() : 1, &pl);
    /* A product that pushes its output to other ranks is finished by its own epilogue everywhere: no
     * K slices (their partial tiles would be finished by another kernel), no folding into C. */
    const bool push = g->push && !g->accumulate && !g->bias && !g->relu && !g->mask && g->ldc == g->N && (g->N & 31) == 0;
    if (push) { pl.splits = 1; pl.kb_per_split = (g->K + pl.bk - 1) / pl.bk; pl.tail_tiles = 0; pl.tail_splits = 0; pl.tail_kb = 0;
                pl.split_acc = (long)pl.kb_per_split * pl.bk > g_tc_split_k; }
    const int bn = pl.bn, bk = pl.bk;
    const bool pair = pl.pair != 0;
    CUtensorMap ma, mb;
    const int b_box = pair ? 128 : bn;                 /* in a pair each CTA stages half of B's columns */
    int a_3d = 0, b_3d = 0;
    if (g->ta) {
        if (g_tc_mn3d && g->M % 32 == 0 && encode_map_mn3d(&ma, g->A, g->M, g->K, g->lda, TC_BM / 32, bk) == 0) a_3d = 1;
        else if (encode_map(&ma, g->A, g->M, g->K, g->lda, 32, bk, 1)) return -1;
    } else if (encode_map(&ma, g->A, g->K, g->M, g->lda, bk, TC_BM, 0)) return -1;
    if (g->tb) {
        if (encode_map(&mb, g->B, g->K, g->N, g->ldb, bk, b_box, 0)) return -1;
    } else if (g_tc_mn3d && g->N % 32 == 0 && encode_map_mn3d(&mb, g->B, g->N, g->K, g->ldb, b_box / 32, bk) == 0) b_3d = 1;
    else if (encode_map(&mb, g->B, g->N, g->K, g->ldb, 32, bk, 1)) return -1;
    g_plan.units = pl.units;
    /* long reductions accumulate in chunks (see TcParams::chunk_kb).  A caller's own accumulate cannot
     * be combined with it (the destination holds the chunk sums meanwhile): such a call keeps one chunk. */
    /* Forward products fold from K = 4096 on: their error passes through every later layer and is
     * amplified by the softmax (a logit off by d changes its probability by d, relative), so it decides
     * the accuracy of every gradient.  Backward products are consumed linearly and fold from K = 8192
     * on.  Measured on the benchmark MLP at batch 8192: worst gradient entry 1.6e-4 off (relative to
     * the largest) without folding, 6.8e-5 with. */
    const long k_slice = (long)pl.kb_per_split * bk;
    const bool fold = pl.split_acc && !g->accumulate && k_slice >= (g->rule == 1 ? 4l : 2l) * g_tc_chunk_k;
    g_plan.chunk_kb = (fold && !push) ? g_tc_chunk_k / bk : (1 << 30);
    g_plan.push_on = push ? 1 : 0;
    g_tt.gemm_pushed_floats = push ? (long)g->M * g->N : 0;
    g_plan.splits = pl.splits; g_plan.kb_per_split = pl.kb_per_split; g_plan.partial = nullptr;
    g_plan.tail_tiles = pl.tail_tiles; g_plan.tail_splits = pl.tail_splits; g_plan.tail_kb = pl.tail_kb; g_plan.tail_partial = nullptr;
    if (pl.splits > 1) {
        g_plan.partial = (float *)tt_dev_alloc(sizeof(float) * (size_t)pl.splits * g->M * g->N);
        if (!g_plan.partial) return -1;
    } else if (pl.tail_tiles > 0) {
        g_plan.tail_partial = (float *)tt_dev_alloc(sizeof(float) * (size_t)pl.tail_splits * pl.tail_tiles * (pair ? 256 : TC_BM) * bn);
        if (!g_plan.tail_partial) return -1;
    }
    const bool split_acc = pl.split_acc != 0;
    int rc;
    if (pair) rc = launch_tc2(g, ma, mb, a_3d, b_3d, split_acc);
    else if (bn == 256 && bk == 16) rc = split_acc ? launch_tc_major<256, 16, 4, 1>(g, ma, mb, a_3d, b_3d) : launch_tc_major<256, 16, 4, 0>(g, ma, mb, a_3d, b_3d);
    else if (bn == 256)        rc = split_acc ? launch_tc_major<256, 32, 2, 1>(g, ma, mb, a_3d, b_3d) : launch_tc_major<256, 32, 2, 0>(g, ma, mb, a_3d, b_3d);
    else if (bk == 16)         rc = split_acc ? launch_tc_major<128, 16, 6, 1>(g, ma, mb, a_3d, b_3d) : launch_tc_major<128, 16, 6, 0>(g, ma, mb, a_3d, b_3d);
    else                       rc = split_acc ? launch_tc_major<128, 32, 3, 1>(g, ma, mb, a_3d, b_3d) : launch_tc_major<128, 32, 3, 0>(g, ma, mb, a_3d, b_3d);
    if (g_plan.partial) tt_dev_free(g_plan.partial);
    if (g_plan.tail_partial) tt_dev_free(g_plan.tail_partial);
    g_plan.splits = 1; g_plan.partial = nullptr;
    g_plan.tail_tiles = 0; g_plan.tail_partial = nullptr; g_plan.units = 0; g_plan.chunk_kb = 1 << 30; g_plan.push_on = 0;
    return rc;
}
