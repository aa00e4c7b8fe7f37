/* tcgen05 / TMA / mbarrier building blocks shared by the tensor-core kernels of this library
 * (the GEMM in gemm_tc.cu and the implicit-GEMM convolution in conv_tc.cu): thin inline-PTX
 * wrappers, bounded waits that report through a host-visible status word instead of spinning
 * for ever, the shared-memory matrix descriptor and the lo part of the 3xTF32 split. */
#ifndef TT_TCGEN05_UTILS_CUH
#define TT_TCGEN05_UTILS_CUH

#include <cuda.h>
#include <stdint.h>

#define TC_WAIT_CYCLES (1ll << 30)

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
/* Bounded wait.  Returns false when the budget ran out here or elsewhere in the CTA. */
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          uint32_t *status, uint32_t code) {
    if (mbar_try(bar, parity)) return true;
    long long t0 = clock64();
    for (;;) {
        #pragma unroll 1
        for (int i = 0; i < 16; i++)
            if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > TC_WAIT_CYCLES) {
            *abort_flag = 1;
            *(volatile uint32_t *)status = code | (blockIdx.x << 8);   /* plain store: the word lives in host memory */
            __threadfence_system();
            return false;
        }
    }
}
/* The same for a whole warp: one lane spins (381 spinning threads would spend shared-memory
 * bandwidth the tensor core needs), then every lane checks once so that each thread has
 * observed the phase itself.  Returns the same value in all lanes. */
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                               uint32_t *status, uint32_t code) {
    bool got = true;
    if ((threadIdx.x & 31) == 0) got = mbar_wait(bar, parity, abort_flag, status, code);
    got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
    if (got) got = mbar_wait(bar, parity, abort_flag, status, code);     /* immediate: the phase is complete */
    return __all_sync(0xffffffffu, got);
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap *map, int x, int y, int z) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
                 ::"l"(map), "r"(x), "r"(y), "r"(z) : "memory");
}
/* Ask L2 for a tile without taking shared memory: the loads that follow hit L2. */
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap *map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                 ::"l"(map), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

/* Shared-memory matrix descriptor (64 bit): start address, leading and stride
 * byte offsets in 16-byte units, version 1, swizzle mode in the top bits.
 *   K-major tile  : rows of 128 bytes (32 values along K), 16-byte chunks
 *                   swizzled over 8 rows (mode 2, SWIZZLE_128B; TMA mode
 *                   SWIZZLE_128B); 8-row groups 1024 bytes apart (stride
 *                   offset); a K step of 8 fp32 advances the start by 32 bytes.
 *   MN-major tile : built from boxes of 32 k-rows x 128 bytes (32 values along
 *                   M or N).  For 32-bit operands the only MN-major layout the
 *                   tensor core accepts swizzles 32-byte chunks over 4 rows
 *                   (mode 1; TMA mode SWIZZLE_128B_ATOM_32B): 4-row groups 512
 *                   bytes apart (stride offset), boxes 4096 bytes apart (leading
 *                   offset); a K step of 8 rows advances the start by 1024 bytes. */
template <int MN_MAJOR, int BK>
__device__ __forceinline__ uint64_t make_desc(uint32_t addr) {
    /* K-major rows are BK*4 bytes: 128-byte rows swizzle over 8 rows of 128 (mode 2), 64-byte rows over
     * 8 rows of 64 (mode 4, TMA SWIZZLE_64B).  MN-major boxes hold BK k-rows of 128 bytes. */
    constexpr uint32_t lbo_bytes = MN_MAJOR ? BK * 128 : 16;
    constexpr uint32_t sbo_bytes = MN_MAJOR ? 512 : 8 * BK * 4;
    constexpr uint64_t mode = MN_MAJOR ? 1 : (BK == 32 ? 2 : 4);
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;            /* descriptor version for sm_100 */
    d |= mode << 61;
    return d;
}

/* lo part of the 3xTF32 split: x minus its 19-bit truncation (exact in fp32; the
 * instruction reads its top 19 bits). */
__device__ __forceinline__ float split_lo(float x) {
    float hi = __uint_as_float(__float_as_uint(x) & 0xffffe000u);
    float lo = x - hi;
    return fabsf(x) == INFINITY ? 0.0f : lo;   /* keep Inf an Inf instead of Inf - Inf */
}


#endif
