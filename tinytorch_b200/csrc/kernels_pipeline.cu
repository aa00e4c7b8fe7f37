/* The two ends of a training loop that the reference keeps in NumPy inside its gate scripts:
 *
 *   input   normalise + gather: xb = ((pixels / 255) - mean) / std of the rows a shuffled
 *           index picks (tests/gate_mnist_mlp.py:86-90,107-111; tests/gate_cifar_cnn.py:162-163).
 *           Here the raw 8-bit dataset is uploaded ONCE and stays in HBM (MNIST 47 MB, CIFAR-10
 *           154 MB of 180 GB); per step only the batch's indices cross PCIe, and one kernel reads
 *           the picked rows as bytes and writes the normalised fp32 batch tensor the first GEMM or
 *           convolution consumes: 1 byte read + 4 bytes written per value, nothing re-read.
 *   output  evaluation: pred = argmax(logits, axis 1); correct += (pred == y).sum()
 *           (tests/gate_mnist_mlp.py:74-80, tests/gate_cifar_cnn.py:114-122): one warp per row,
 *           shuffle reduction, a device counter, four bytes back to the host instead of all logits.
 *
 * Both are HBM-bound streaming kernels (128-bit stores, four values per thread); the file is
 * compiled without multiply-add contraction and the divisions are IEEE (__fdiv_rn), so the
 * normalised values are bit-identical to NumPy's float32 arithmetic. */
#include "tt_internal.h"

#include <stdlib.h>
#include <string.h>

#define PL_MAX_CHANNELS 16
#define PL_TPB 256

struct NormParams {
    float mean[PL_MAX_CHANNELS], std[PL_MAX_CHANNELS];
    int channels;
    long plane;          /* values per channel of one sample */
    long row;            /* values per sample = channels * plane */
};

/* dst[i, c, p] = ((float)src[idx[i], c, p] / 255 - mean[c]) / std[c].  One thread per four values
 * (row % 4 == 0 and plane % 4 == 0 on the vector path, so four values share a channel). */
__global__ void __launch_bounds__(PL_TPB) gather_normalize_u8_v4(float4 *__restrict__ dst, const uint8_t *__restrict__ src,
                                                                 const int *__restrict__ idx, long b, NormParams np) {
    const long row4 = np.row / 4, total4 = b * row4;
    const long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += stride) {
        const long s = i / row4, e = (i - s * row4) * 4;
        const int c = (int)(e / np.plane);
        const uchar4 v = *(const uchar4 *)(src + (long)idx[s] * np.row + e);
        const float m = np.mean[c], d = np.std[c];
        float4 o;
        o.x = __fdiv_rn(__fdiv_rn((float)v.x, 255.0f) - m, d);
        o.y = __fdiv_rn(__fdiv_rn((float)v.y, 255.0f) - m, d);
        o.z = __fdiv_rn(__fdiv_rn((float)v.z, 255.0f) - m, d);
        o.w = __fdiv_rn(__fdiv_rn((float)v.w, 255.0f) - m, d);
        dst[i] = o;
    }
}
__global__ void __launch_bounds__(PL_TPB) gather_normalize_u8_s(float *__restrict__ dst, const uint8_t *__restrict__ src,
                                                                const int *__restrict__ idx, long b, NormParams np) {
    const long total = b * np.row;
    const long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long s = i / np.row, e = i - s * np.row;
        const int c = (int)(e / np.plane);
        const float v = (float)src[(long)idx[s] * np.row + e];
        dst[i] = __fdiv_rn(__fdiv_rn(v, 255.0f) - np.mean[c], np.std[c]);
    }
}

/* ---- resident byte buffers (the raw dataset) --------------------------------------------*/
extern "C" void *ttb_bytes_upload(const void *host, size_t nbytes) {
    if (!host || nbytes == 0) { tt_set_error("ttb_bytes_upload: nothing to upload"); return nullptr; }
    if (tt_ctx_init() != 0) return nullptr;
    void *d = nullptr;
    /* a plain allocation, outside the tensor pool: it lives for the whole run */
    if (!tt_cuda_ok(cudaMalloc(&d, (nbytes + 15) & ~(size_t)15), "cudaMalloc(dataset)")) return nullptr;
    if (!tt_cuda_ok(cudaMemcpyAsync(d, host, nbytes, cudaMemcpyHostToDevice, g_tt.stream), "cudaMemcpyAsync(dataset)") ||
        !tt_cuda_ok(cudaStreamSynchronize(g_tt.stream), "cudaStreamSynchronize")) {
        cudaFree(d);
        return nullptr;
    }
    return d;
}
extern "C" void ttb_bytes_free(void *dev) {
    if (!dev || g_tt.ready != 1) return;
    cudaStreamSynchronize(g_tt.stream);
    cudaFree(dev);
}

extern "C" int ttb_gather_normalize_u8(Tensor *dst, const void *src_dev, long n_rows, const int *idx, long b,
                                       int channels, const float *mean, const float *std) {
    if (!dst || !src_dev || !idx || !mean || !std || b <= 0 || n_rows <= 0 || channels < 1 || channels > PL_MAX_CHANNELS ||
        dst->numel % b != 0 || (dst->numel / b) % channels != 0) {
        tt_set_error("ttb_gather_normalize_u8: bad arguments (1..%d channels, batch must divide the tensor)", PL_MAX_CHANNELS);
        return -1;
    }
    for (long i = 0; i < b; i++)
        if (idx[i] < 0 || idx[i] >= n_rows) { tt_set_error("ttb_gather_normalize_u8: index %d out of range", idx[i]); return -1; }
    NormParams np;
    memset(&np, 0, sizeof np);
    np.channels = channels;
    np.row = dst->numel / b;
    np.plane = np.row / channels;
    for (int c = 0; c < channels; c++) { np.mean[c] = mean[c]; np.std[c] = std[c]; }
    float *pd = tt_dev_rw(dst);
    if (!pd) return -1;
    int *didx = (int *)tt_dev_alloc(sizeof(int) * (size_t)b);
    if (!didx) return -1;
    /* pageable source: the call returns once the indices are staged, so the caller may reuse idx */
    if (!tt_cuda_ok(cudaMemcpyAsync(didx, idx, sizeof(int) * (size_t)b, cudaMemcpyHostToDevice, g_tt.stream),
                    "cudaMemcpyAsync(indices)")) { tt_dev_free(didx); return -1; }
    const bool vec = (np.row % 4 == 0) && (np.plane % 4 == 0) && ((((uintptr_t)src_dev) & 3u) == 0) && ((((uintptr_t)pd) & 15u) == 0);
    const long items = vec ? b * np.row / 4 : b * np.row;
    long blocks = (items + PL_TPB - 1) / PL_TPB, cap = (long)g_tt.sm_count * 8;
    if (blocks > cap) blocks = cap;
    tt_trace_begin(TTB_K_ELEMENTWISE);
    if (vec) gather_normalize_u8_v4<<<(int)blocks, PL_TPB, 0, g_tt.stream>>>((float4 *)pd, (const uint8_t *)src_dev, didx, b, np);
    else     gather_normalize_u8_s<<<(int)blocks, PL_TPB, 0, g_tt.stream>>>(pd, (const uint8_t *)src_dev, didx, b, np);
    g_tt.launches++;
    tt_trace_end(TTB_K_ELEMENTWISE, 5.0 * (double)b * np.row);
    tt_dev_free(didx);
    return tt_cuda_ok(cudaGetLastError(), "gather_normalize launch") ? 0 : -1;
}

/* ---- evaluation: argmax per row, and how many rows hit their label ----------------------
 * NumPy's argmax: the first maximum; a NaN counts as the maximum (the first NaN wins). */
__device__ __forceinline__ bool am_better(float v, int i, float bv, int bi) {
    const bool vn = v != v, bn = bv != bv;
    if (bn) return vn && i < bi;
    if (vn) return true;
    return v > bv || (v == bv && i < bi);
}
__global__ void __launch_bounds__(PL_TPB) argmax_rows_kernel(const float *__restrict__ x, long rows, int N,
                                                             const float *__restrict__ labels, float *__restrict__ pred,
                                                             unsigned long long *__restrict__ correct) {
    const int lane = threadIdx.x & 31;
    const long warp0 = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((long)gridDim.x * blockDim.x) >> 5;
    unsigned hits = 0;
    for (long r = warp0; r < rows; r += nwarps) {
        const float *xr = x + r * N;
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int j = lane; j < N; j += 32) {
            const float v = xr[j];
            if (bi == 0x7fffffff || am_better(v, j, bv, bi)) { bv = v; bi = j; }
        }
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || am_better(ov, oi, bv, bi))) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            if (pred) pred[r] = (float)bi;
            if (labels && (float)bi == labels[r]) hits++;
        }
    }
    if (correct && lane == 0 && hits) atomicAdd(correct, (unsigned long long)hits);
}

static int argmax_launch(const Tensor *logits, const Tensor *labels, float *pred, unsigned long long *counter) {
    const long rows = logits->shape[0];
    const int N = (int)logits->shape[1];
    const float *px = tt_dev_ro(logits), *py = labels ? tt_dev_ro(labels) : nullptr;
    if (!px || (labels && !py)) return -1;
    long blocks = (rows * 32 + PL_TPB - 1) / PL_TPB, cap = (long)g_tt.sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    tt_trace_begin(TTB_K_REDUCE);
    argmax_rows_kernel<<<(int)blocks, PL_TPB, 0, g_tt.stream>>>(px, rows, N, py, pred, counter);
    g_tt.launches++;
    tt_trace_end(TTB_K_REDUCE, 4.0 * (double)rows * N);
    return tt_cuda_ok(cudaGetLastError(), "argmax launch") ? 0 : -1;
}

extern "C" Tensor *ttb_argmax(const Tensor *logits) {
    if (!logits || logits->ndim != 2 || logits->shape[1] > 0x7fffffffL) return nullptr;
    long shp[1] = {logits->shape[0]};
    Tensor *out = tt_new_uninit(shp, 1);
    if (!out) return nullptr;
    if (argmax_launch(logits, nullptr, TT(out)->dev, nullptr) != 0) { tt_release(out); return nullptr; }
    return out;
}

extern "C" long ttb_argmax_correct(const Tensor *logits, const Tensor *labels) {
    if (!logits || !labels || logits->ndim != 2 || logits->shape[1] > 0x7fffffffL || labels->numel != logits->shape[0]) {
        tt_set_error("ttb_argmax_correct: logits must be [rows, classes] and labels hold one class per row");
        return -1;
    }
    unsigned long long *counter = (unsigned long long *)tt_dev_alloc(sizeof(unsigned long long));
    if (!counter) return -1;
    unsigned long long host = 0;
    int ok = tt_cuda_ok(cudaMemsetAsync(counter, 0, sizeof(unsigned long long), g_tt.stream), "cudaMemsetAsync") &&
             argmax_launch(logits, labels, nullptr, counter) == 0 &&
             tt_cuda_ok(cudaMemcpyAsync(&host, counter, sizeof host, cudaMemcpyDeviceToHost, g_tt.stream), "cudaMemcpyAsync(D2H)") &&
             tt_cuda_ok(cudaStreamSynchronize(g_tt.stream), "cudaStreamSynchronize");
    tt_dev_free(counter);
    if (!ok || gemm_tc_poll_status()) return -1;
    return (long)host;
}
