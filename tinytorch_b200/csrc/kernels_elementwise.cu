/* Memory-bound kernels of the hot path: elementwise operators, relu and its
 * gradient, padones and its adjoint, softmax forward/backward, the fused
 * softmax-cross-entropy gradient, column sums, optimiser steps, transpose.
 *
 * All of them are HBM-bound streaming kernels: 128-bit loads and stores where
 * the pointers allow it, several independent loads in flight per thread, a
 * grid of a whole number of waves (blocks = SMs x resident blocks per SM)
 * walked with a grid-stride loop, and warp-shuffle reductions for the row
 * operators.  Each kernel names the reference loop it replaces. */
#include "tt_internal.h"

#include <stdlib.h>

#include <math.h>

#define TPB 256

static inline int grid_for(long items, int per_sm = 8) {
    long want = (items + TPB - 1) / TPB;
    long cap = (long)g_tt.sm_count * per_sm;
    if (want < 1) want = 1;
    return (int)(want < cap ? want : cap);
}

static inline bool aligned16(const void *p) { return (((uintptr_t)p) & 15u) == 0; }

#define LAUNCH(kern, grid, block, smem, ...)                         \
    do {                                                             \
        kern<<<(grid), (block), (smem), g_tt.stream>>>(__VA_ARGS__); \
        g_tt.launches++;                                             \
    } while (0)

/* ---- generic streaming maps ----------------------------------------------
 * OP is a functor over scalars; the vector body handles four at a time and
 * keeps two float4 loads per operand in flight. */
template <class OP>
__global__ void __launch_bounds__(TPB) map1_v4(float4 *o, const float4 *a, long n4, OP op) {
    long stride = (long)gridDim.x * blockDim.x;
    long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + stride < n4; i += 2 * stride) {
        float4 x = a[i], y = a[i + stride];
        o[i] = make_float4(op(x.x), op(x.y), op(x.z), op(x.w));
        o[i + stride] = make_float4(op(y.x), op(y.y), op(y.z), op(y.w));
    }
    if (i < n4) {
        float4 x = a[i];
        o[i] = make_float4(op(x.x), op(x.y), op(x.z), op(x.w));
    }
}
template <class OP>
__global__ void __launch_bounds__(TPB) map1_s(float *o, const float *a, long lo, long n, OP op) {
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = lo + (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) o[i] = op(a[i]);
}
template <class OP>
__global__ void __launch_bounds__(TPB) map2_v4(float4 *o, const float4 *a,
                                                const float4 *__restrict__ b, long n4, OP op) {
    long stride = (long)gridDim.x * blockDim.x;
    long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + stride < n4; i += 2 * stride) {
        float4 x = a[i], y = b[i], x2 = a[i + stride], y2 = b[i + stride];
        o[i] = make_float4(op(x.x, y.x), op(x.y, y.y), op(x.z, y.z), op(x.w, y.w));
        o[i + stride] = make_float4(op(x2.x, y2.x), op(x2.y, y2.y), op(x2.z, y2.z), op(x2.w, y2.w));
    }
    if (i < n4) {
        float4 x = a[i], y = b[i];
        o[i] = make_float4(op(x.x, y.x), op(x.y, y.y), op(x.z, y.z), op(x.w, y.w));
    }
}
template <class OP>
__global__ void __launch_bounds__(TPB) map2_s(float *o, const float *a,
                                               const float *__restrict__ b, long lo, long n, OP op) {
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = lo + (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) o[i] = op(a[i], b[i]);
}
template <class OP>
__global__ void __launch_bounds__(TPB) map3_v4(float4 *o, const float4 *a,
                                                const float4 *__restrict__ b, const float4 *__restrict__ c,
                                                long n4, OP op) {
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 x = a[i], y = b[i], z = c[i];
        o[i] = make_float4(op(x.x, y.x, z.x), op(x.y, y.y, z.y), op(x.z, y.z, z.z), op(x.w, y.w, z.w));
    }
}
template <class OP>
__global__ void __launch_bounds__(TPB) map3_s(float *o, const float *a,
                                               const float *__restrict__ b, const float *__restrict__ c,
                                               long lo, long n, OP op) {
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = lo + (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) o[i] = op(a[i], b[i], c[i]);
}

template <class OP>
static void run_map1(float *o, const float *a, long n, OP op) {
    if (n <= 0) return;
    tt_trace_begin(TTB_K_ELEMENTWISE);
    long n4 = (aligned16(o) && aligned16(a)) ? n / 4 : 0;
    if (n4 > 0) LAUNCH((map1_v4<OP>), grid_for((n4 + 1) / 2), TPB, 0, (float4 *)o, (const float4 *)a, n4, op);
    if (n4 * 4 < n) LAUNCH((map1_s<OP>), grid_for(n - n4 * 4), TPB, 0, o, a, n4 * 4, n, op);
    tt_trace_end(TTB_K_ELEMENTWISE, 8.0 * (double)n);
}
template <class OP>
static void run_map2(float *o, const float *a, const float *b, long n, OP op) {
    if (n <= 0) return;
    tt_trace_begin(TTB_K_ELEMENTWISE);
    long n4 = (aligned16(o) && aligned16(a) && aligned16(b)) ? n / 4 : 0;
    if (n4 > 0) LAUNCH((map2_v4<OP>), grid_for((n4 + 1) / 2), TPB, 0, (float4 *)o, (const float4 *)a, (const float4 *)b, n4, op);
    if (n4 * 4 < n) LAUNCH((map2_s<OP>), grid_for(n - n4 * 4), TPB, 0, o, a, b, n4 * 4, n, op);
    tt_trace_end(TTB_K_ELEMENTWISE, 12.0 * (double)n);
}
template <class OP>
static void run_map3(float *o, const float *a, const float *b, const float *c, long n, OP op) {
    if (n <= 0) return;
    tt_trace_begin(TTB_K_ELEMENTWISE);
    long n4 = (aligned16(o) && aligned16(a) && aligned16(b) && aligned16(c)) ? n / 4 : 0;
    if (n4 > 0) LAUNCH((map3_v4<OP>), grid_for(n4), TPB, 0, (float4 *)o, (const float4 *)a, (const float4 *)b, (const float4 *)c, n4, op);
    if (n4 * 4 < n) LAUNCH((map3_s<OP>), grid_for(n - n4 * 4), TPB, 0, o, a, b, c, n4 * 4, n, op);
    tt_trace_end(TTB_K_ELEMENTWISE, 16.0 * (double)n);
}

/* ---- functors -------------------------------------------------------------*/
struct OpFill    { float v; __device__ float operator()(float) const { return v; } };
struct OpCopy    { __device__ float operator()(float x) const { return x; } };
struct OpAddS    { float s; __device__ float operator()(float x) const { return x + s; } };
struct OpMulS    { float s; __device__ float operator()(float x) const { return x * s; } };
/* x > 0 ? x : 0 -- a NaN compares false and becomes 0, as in src/ops.c:104 */
struct OpRelu    { __device__ float operator()(float x) const { return x > 0.0f ? x : 0.0f; } };
struct OpAdd     { __device__ float operator()(float x, float y) const { return x + y; } };
struct OpMul     { __device__ float operator()(float x, float y) const { return x * y; } };
/* mask from the forward input, src/autograd.c:323-324 */
struct OpReluBwd { __device__ float operator()(float x, float g) const { return x > 0.0f ? g : 0.0f; } };
struct OpReluBwdAcc { __device__ float operator()(float d, float x, float g) const { return d + (x > 0.0f ? g : 0.0f); } };
struct OpSgd     { float lr; __device__ float operator()(float w, float g) const { return w - lr * g; } };

__global__ void __launch_bounds__(TPB) fill_kernel(float *__restrict__ p, long n, float v) {
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = v;
}

void k_fill(float *p, long n, float v) {
    if (n <= 0) return;
    LAUNCH(fill_kernel, grid_for(n), TPB, 0, p, n, v);
}
void k_copy(float *dst, const float *src, long n) {
    if (n <= 0) return;
    cudaMemcpyAsync(dst, src, sizeof(float) * (size_t)n, cudaMemcpyDeviceToDevice, g_tt.stream);
}
/* src/ops.c:26-53 (the per-element index walk of the reference is the
 * identity on contiguous tensors, which is all it ever creates) */
void k_add(float *o, const float *a, const float *b, long n) { run_map2(o, a, b, n, OpAdd()); }
void k_mul(float *o, const float *a, const float *b, long n) { run_map2(o, a, b, n, OpMul()); }
/* src/ops.c:71-82 */
void k_addscalar(float *o, const float *a, float s, long n) { OpAddS f; f.s = s; run_map1(o, a, n, f); }
void k_mulscalar(float *o, const float *a, float s, long n) { OpMulS f; f.s = s; run_map1(o, a, n, f); }
/* src/autograd.c:52-54 */
void k_accum(float *dst, const float *src, long n) { run_map2(dst, dst, src, n, OpAdd()); }
/* src/ops.c:55-69,104-106 */
void k_relu(float *o, const float *x, long n) { run_map1(o, x, n, OpRelu()); }
/* src/autograd.c:318-327, optionally fused with the += of accum (:56-63) */
void k_relu_bwd(float *dx, const float *x, const float *g, long n, int accumulate) {
    if (accumulate) run_map3(dx, dx, x, g, n, OpReluBwdAcc());
    else run_map2(dx, x, g, n, OpReluBwd());
}
void k_sgd(float *w, const float *g, float lr, long n) {
    OpSgd f; f.lr = lr;
    tt_trace_begin(TTB_K_OPTIM);
    int was = g_tt.trace; g_tt.trace = 0;
    run_map2(w, w, g, n, f);
    g_tt.trace = was;
    tt_trace_end(TTB_K_OPTIM, 12.0 * (double)n);
}

__global__ void __launch_bounds__(TPB) sgd_momentum_kernel(float *__restrict__ w, float *__restrict__ v,
                                                            const float *__restrict__ g, float lr, float mu, long n) {
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float nv = mu * v[i] - lr * g[i];
        v[i] = nv;
        w[i] = w[i] + nv;
    }
}
void k_sgd_momentum(float *w, float *v, const float *g, float lr, float mu, long n) {
    if (n <= 0) return;
    tt_trace_begin(TTB_K_OPTIM);
    LAUNCH(sgd_momentum_kernel, grid_for(n), TPB, 0, w, v, g, lr, mu, n);
    tt_trace_end(TTB_K_OPTIM, 20.0 * (double)n);
}

/* Adam exactly as tests/gate_cifar_cnn.py:92-98 writes it:
 *   m = b1*m + (1-b1)*g ; v = b2*v + (1-b2)*g*g ; w -= lr_t * m / (sqrt(v) + eps)
 * with lr_t = lr*sqrt(1-b2^t)/(1-b1^t) and the (1-b) factors formed on the host. */
__global__ void __launch_bounds__(TPB) adam_kernel(float *__restrict__ w, float *__restrict__ m, float *__restrict__ v,
                                                    const float *__restrict__ g, float lr_t, float b1, float b2,
                                                    float omb1, float omb2, float eps, long n) {
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float gi = g[i];
        float mi = b1 * m[i] + omb1 * gi;
        float vi = b2 * v[i] + omb2 * (gi * gi);
        m[i] = mi; v[i] = vi;
        w[i] = w[i] - lr_t * mi / (sqrtf(vi) + eps);
    }
}
void k_adam(float *w, float *m, float *v, const float *g, float lr_t, float b1, float b2,
            float omb1, float omb2, float eps, long n) {
    if (n <= 0) return;
    tt_trace_begin(TTB_K_OPTIM);
    LAUNCH(adam_kernel, grid_for(n), TPB, 0, w, m, v, g, lr_t, b1, b2, omb1, omb2, eps, n);
    tt_trace_end(TTB_K_OPTIM, 28.0 * (double)n);
}

/* ---- padones and its adjoint (src/autograd.c:195-212, 348-359) ------------
 * One thread per output element; consecutive threads write consecutive
 * addresses, reads are contiguous runs of K. */
__global__ void __launch_bounds__(TPB) padones_kernel(float *o, const float *__restrict__ x, int M, int K) {
    long n = (long)M * (K + 1);
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        long m = i / (K + 1);
        int k = (int)(i - m * (K + 1));
        o[i] = k < K ? x[m * K + k] : 1.0f;
    }
}
void k_padones(float *o, const float *x, int M, int K) {
    tt_trace_begin(TTB_K_ELEMENTWISE);
    LAUNCH(padones_kernel, grid_for((long)M * (K + 1)), TPB, 0, o, x, M, K);
    tt_trace_end(TTB_K_ELEMENTWISE, 8.0 * (double)M * K);
}
__global__ void __launch_bounds__(TPB) slice_cols_kernel(float *o, const float *__restrict__ g,
                                                          int M, int K, int ldg, int accumulate) {
    long n = (long)M * K;
    long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        long m = i / K;
        int k = (int)(i - m * K);
        float v = g[m * ldg + k];
        o[i] = accumulate ? o[i] + v : v;
    }
}
void k_slice_cols(float *o, const float *g, int M, int K, int ldg, int accumulate) {
    tt_trace_begin(TTB_K_ELEMENTWISE);
    LAUNCH(slice_cols_kernel, grid_for((long)M * K), TPB, 0, o, g, M, K, ldg, accumulate);
    tt_trace_end(TTB_K_ELEMENTWISE, (accumulate ? 12.0 : 8.0) * (double)M * K);
}

/* ---- row reductions --------------------------------------------------------*/
__device__ __forceinline__ float warp_max(float v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) { float u = __shfl_xor_sync(0xffffffffu, v, o); v = u > v ? u : v; }
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

/* Softmax over the last axis (src/ops.c:108-145): one warp per row, the row
 * is read once per pass from L1/L2-resident lines; a row whose maximum is
 * -Inf becomes uniform.  NaN never wins the max, as in the reference. */
#define SM_WARPS 8
#define SM_REG 32            /* values a lane keeps in registers: rows of up to 1024 are read from memory once */

/* Element index of register slot i for this lane.  Vector form: the lane owns four
 * consecutive values per 128-bit access (slots 4q..4q+3 hold elements 4*(lane+32q)..);
 * scalar form: slot i holds element lane + 32*i. */
__device__ __forceinline__ int sm_index(int i, int lane, bool vec) {
    return vec ? 4 * (lane + 32 * (i >> 2)) + (i & 3) : lane + 32 * i;
}

/* Row statistics shared by softmax and the fused loss: loads the row (into registers
 * when it fits), returns max and the sum of exp(x - max), leaves the exponentials in
 * v[].  NaN never wins the max, as in the reference (src/ops.c:120-124). */
__device__ __forceinline__ void softmax_row(const float *__restrict__ xr, int N, int lane, float (&v)[SM_REG],
                                            bool in_regs, bool vec, float &mx, float &sum) {
    mx = -INFINITY;
    if (in_regs && vec) {
        #pragma unroll
        for (int q = 0; q < SM_REG / 4; q++) {
            const int j = 4 * (lane + 32 * q);
            float4 t = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            if (j < N) t = *(const float4 *)(xr + j);
            v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
        }
    } else if (in_regs) {
        #pragma unroll
        for (int i = 0; i < SM_REG; i++) { const int j = lane + 32 * i; v[i] = j < N ? xr[j] : -INFINITY; }
    }
    if (in_regs) {
        #pragma unroll
        for (int i = 0; i < SM_REG; i++) if (v[i] > mx) mx = v[i];
    } else {
        for (int j = lane; j < N; j += 32) { float t = xr[j]; if (t > mx) mx = t; }
    }
    mx = warp_max(mx);
    sum = 0.0f;
    if (mx == -INFINITY) return;
    if (in_regs) {
        #pragma unroll
        for (int i = 0; i < SM_REG; i++) {
            v[i] = expf(v[i] - mx);          /* slots past the row hold -Inf and become 0 */
            sum += v[i];
        }
    } else {
        for (int j = lane; j < N; j += 32) sum += expf(xr[j] - mx);
    }
    sum = warp_sum(sum);
}

/* Store the register-resident row: o[j] = f(v, j). */
template <class F>
__device__ __forceinline__ void sm_store(float *__restrict__ orow, int N, int lane, const float (&v)[SM_REG], bool vec, F f) {
    if (vec) {
        #pragma unroll
        for (int q = 0; q < SM_REG / 4; q++) {
            const int j = 4 * (lane + 32 * q);
            if (j < N)
                *(float4 *)(orow + j) = make_float4(f(v[4 * q], j), f(v[4 * q + 1], j + 1), f(v[4 * q + 2], j + 2), f(v[4 * q + 3], j + 3));
        }
    } else {
        #pragma unroll
        for (int i = 0; i < SM_REG; i++) { const int j = lane + 32 * i; if (j < N) orow[j] = f(v[i], j); }
    }
}

__global__ void __launch_bounds__(SM_WARPS * 32) softmax_kernel(float *__restrict__ o, const float *__restrict__ x,
                                                                  long rows, int N) {
    int lane = threadIdx.x & 31;
    long row = (long)blockIdx.x * SM_WARPS + (threadIdx.x >> 5);
    long rstride = (long)gridDim.x * SM_WARPS;
    const bool in_regs = N <= 32 * SM_REG;
    const bool vec = in_regs && ((N & 3) == 0) && (((((uintptr_t)x) | ((uintptr_t)o)) & 15u) == 0);
    for (; row < rows; row += rstride) {
        const float *xr = x + row * N;
        float *orow = o + row * N;
        float v[SM_REG], mx, sum;
        softmax_row(xr, N, lane, v, in_regs, vec, mx, sum);
        if (mx == -INFINITY) {
            float u = 1.0f / (float)N;
            for (int j = lane; j < N; j += 32) orow[j] = u;
            continue;
        }
        if (in_regs) {
            /* one division per row, then a multiply per element: within 1.5 ulp of e / sum, and the
             * kernel stays under the time the row's bytes take (a per-element division does not) */
            const float inv = 1.0f / sum;
            sm_store(orow, N, lane, v, vec, [inv](float e, int) { return e * inv; });
        } else {
            for (int j = lane; j < N; j += 32) orow[j] = expf(xr[j] - mx) / sum;
        }
    }
}
void k_softmax(float *o, const float *x, long rows, int N) {
    if (rows <= 0) return;
    long blocks = (rows + SM_WARPS - 1) / SM_WARPS;
    long cap = (long)g_tt.sm_count * 8;
    tt_trace_begin(TTB_K_SOFTMAX);
    LAUNCH(softmax_kernel, (int)(blocks < cap ? blocks : cap), SM_WARPS * 32, 0, o, x, rows, N);
    tt_trace_end(TTB_K_SOFTMAX, 8.0 * (double)rows * N);
}

/* dx = s * (g - sum_j g_j s_j) (src/autograd.c:329-346) */
__global__ void __launch_bounds__(SM_WARPS * 32) softmax_bwd_kernel(float *__restrict__ dx, const float *__restrict__ s,
                                                                      const float *__restrict__ g, long rows, int N) {
    int lane = threadIdx.x & 31;
    long row = (long)blockIdx.x * SM_WARPS + (threadIdx.x >> 5);
    long rstride = (long)gridDim.x * SM_WARPS;
    for (; row < rows; row += rstride) {
        const float *sr = s + row * N, *gr = g + row * N;
        float dot = 0.0f;
        for (int j = lane; j < N; j += 32) dot += gr[j] * sr[j];
        dot = warp_sum(dot);
        for (int j = lane; j < N; j += 32) dx[row * N + j] = sr[j] * (gr[j] - dot);
    }
}
void k_softmax_bwd(float *dx, const float *s, const float *g, long rows, int N) {
    if (rows <= 0) return;
    long blocks = (rows + SM_WARPS - 1) / SM_WARPS;
    long cap = (long)g_tt.sm_count * 8;
    tt_trace_begin(TTB_K_SOFTMAX);
    LAUNCH(softmax_bwd_kernel, (int)(blocks < cap ? blocks : cap), SM_WARPS * 32, 0, dx, s, g, rows, N);
    tt_trace_end(TTB_K_SOFTMAX, 12.0 * (double)rows * N);
}

/* Fused softmax + cross-entropy + gradient.  Replaces softmax on the device
 * followed by the NumPy lines of tests/gate_mnist_mlp.py:112-119:
 *   p = softmax(z); loss_r = -log(max(p[y_r], 1e-12)); dz = (p - onehot) * scale.
 * One pass over the logits, one write of dz, 4 bytes of loss per row. */
__global__ void __launch_bounds__(SM_WARPS * 32, 3) softmax_xent_kernel(const float *__restrict__ z, const float *__restrict__ labels,
                                                                       long rows, int N, float scale,
                                                                       float *__restrict__ dz, float *__restrict__ row_loss) {
    int lane = threadIdx.x & 31;
    long row = (long)blockIdx.x * SM_WARPS + (threadIdx.x >> 5);
    long rstride = (long)gridDim.x * SM_WARPS;
    const bool in_regs = N <= 32 * SM_REG;
    const bool vec = in_regs && ((N & 3) == 0) && (((((uintptr_t)z) | ((uintptr_t)dz)) & 15u) == 0);
    for (; row < rows; row += rstride) {
        const float *zr = z + row * N;
        float *drow = dz + row * N;
        const int y = (int)labels[row];
        float v[SM_REG], mx, sum;
        softmax_row(zr, N, lane, v, in_regs, vec, mx, sum);
        float py;
        if (mx == -INFINITY) {
            float u = 1.0f / (float)N;
            for (int j = lane; j < N; j += 32) drow[j] = (u - (j == y ? 1.0f : 0.0f)) * scale;
            py = u;
        } else {
            if (in_regs) {
                /* the label's probability: every lane recomputes it from the (cached) logit with the
                 * operations the stored row uses, so it equals the stored value plus the one-hot */
                const float inv = 1.0f / sum;
                const bool y_ok = y >= 0 && y < N;
                py = y_ok ? expf(zr[y] - mx) * inv : 0.0f;
                /* the row goes out as p * scale; the one element that carries the one-hot is then
                 * rewritten by lane 0 (ordered after the row's stores by the warp barrier) */
                sm_store(drow, N, lane, v, vec, [inv, scale](float e, int) { return (e * inv) * scale; });
                __syncwarp();
                if (lane == 0 && y_ok) drow[y] = (py - 1.0f) * scale;
            } else {
                float mine = 0.0f;
                for (int j = lane; j < N; j += 32) {
                    float p = expf(zr[j] - mx) / sum;
                    if (j == y) mine = p;
                    drow[j] = (p - (j == y ? 1.0f : 0.0f)) * scale;
                }
                py = warp_sum(mine);
            }
        }
        if (lane == 0) row_loss[row] = -logf(fmaxf(py, 1e-12f));
    }
}
void k_softmax_xent(const float *logits, const float *labels, long rows, int N, float scale,
                    float *dlogits, float *row_loss) {
    if (rows <= 0) return;
    long blocks = (rows + SM_WARPS - 1) / SM_WARPS;
    long cap = (long)g_tt.sm_count * 8;
    tt_trace_begin(TTB_K_SOFTMAX);
    LAUNCH(softmax_xent_kernel, (int)(blocks < cap ? blocks : cap), SM_WARPS * 32, 0, logits, labels, rows, N, scale, dlogits, row_loss);
    tt_trace_end(TTB_K_SOFTMAX, 8.0 * (double)rows * N);
}

/* out[0] = sum(x) / n with a fixed summation tree (one block). */
__global__ void __launch_bounds__(1024) mean_kernel(const float *__restrict__ x, long n, float *__restrict__ out) {
    __shared__ float part[32];
    float s = 0.0f;
    for (long i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
        s = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.0f;
        s = warp_sum(s);
        if (threadIdx.x == 0) out[0] = s / (float)n;
    }
}
void k_mean(const float *x, long n, float *out) {
    tt_trace_begin(TTB_K_REDUCE);
    LAUNCH(mean_kernel, 1, 1024, 0, x, n, out);
    tt_trace_end(TTB_K_REDUCE, 4.0 * (double)n);
}

/* ---- column sums: out[n] (+)= sum_m g[m, n] --------------------------------
 * The bias row of dW when padones is folded into the GEMM (the reference gets
 * it as the last row of A^T * dC, src/autograd.c:87-103).  Two deterministic
 * phases: each block sums a slab of rows for 128 columns into a partial row,
 * then one pass adds the partial rows in slab order. */
#define CS_COLS 128
#define CS_ROWS 8
__global__ void __launch_bounds__(CS_COLS * CS_ROWS / 4) colsum_partial_kernel(const float *__restrict__ g, int M, int N, int ldg,
                                                                                 int rows_per_slab, float *__restrict__ part) {
    /* 32 lanes x 4 columns wide, CS_ROWS row lanes */
    __shared__ float4 sh[CS_ROWS][32];
    int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    int col = blockIdx.x * CS_COLS + cx * 4;
    int r0 = blockIdx.y * rows_per_slab;
    int r1 = r0 + rows_per_slab < M ? r0 + rows_per_slab : M;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    bool vec = ((ldg & 3) == 0) && ((((uintptr_t)g) & 15u) == 0) && (col + 3 < N);
    int r = r0 + ry;
    if (vec) {
        /* four independent 128-bit loads in flight per thread */
        for (; r + 3 * CS_ROWS < r1; r += 4 * CS_ROWS) {
            const float *row = g + (long)r * ldg + col;
            float4 a = *(const float4 *)row, b = *(const float4 *)(row + (long)CS_ROWS * ldg);
            float4 c = *(const float4 *)(row + 2l * CS_ROWS * ldg), d = *(const float4 *)(row + 3l * CS_ROWS * ldg);
            acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
            acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
            acc.x += c.x; acc.y += c.y; acc.z += c.z; acc.w += c.w;
            acc.x += d.x; acc.y += d.y; acc.z += d.z; acc.w += d.w;
        }
    }
    for (; r < r1; r += CS_ROWS) {
        const float *row = g + (long)r * ldg;
        if (vec) {
            float4 v = *(const float4 *)(row + col);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        } else {
            if (col < N) acc.x += row[col];
            if (col + 1 < N) acc.y += row[col + 1];
            if (col + 2 < N) acc.z += row[col + 2];
            if (col + 3 < N) acc.w += row[col + 3];
        }
    }
    sh[ry][cx] = acc;
    __syncthreads();
    if (ry == 0) {
        #pragma unroll
        for (int k = 1; k < CS_ROWS; k++) {
            float4 v = sh[k][cx];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        float *p = part + (long)blockIdx.y * N;
        if (col < N) p[col] = acc.x;
        if (col + 1 < N) p[col + 1] = acc.y;
        if (col + 2 < N) p[col + 2] = acc.z;
        if (col + 3 < N) p[col + 3] = acc.w;
    }
}
__global__ void __launch_bounds__(TPB) colsum_final_kernel(const float *__restrict__ part, int slabs, int N,
                                                            float *__restrict__ out, int accumulate) {
    int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float s = 0.0f;
    for (int k = 0; k < slabs; k++) s += part[(long)k * N + n];
    out[n] = accumulate ? out[n] + s : s;
}
/* One-launch form for the pooled path: the block that finishes last among the row slabs of a
 * column block (a ticket counter per column block, reset by its last user) adds the partial
 * rows -- slab k goes to row lane k % 8, the eight lanes are then added in order, so the sum
 * has one fixed shape whatever the arrival order -- and writes the result.  Saves the second
 * launch, which for a 134 MB gradient is a fifth of the time. */
#define CS_MAX_COL_BLOCKS 2048
static __device__ unsigned int g_colsum_tickets[CS_MAX_COL_BLOCKS];
/* CT threads across (four columns each), RT row lanes; CT * RT = 256 */
template <int CT, int RT>
__global__ void __launch_bounds__(256) colsum_fused_kernel(const float *__restrict__ g, int M, int N, int ldg,
                                                                               int rows_per_slab, float *__restrict__ part,
                                                                               float *__restrict__ out, int accumulate) {
    __shared__ float4 sh[RT][CT];
    __shared__ unsigned int ticket;
    const int cx = threadIdx.x % CT, ry = threadIdx.x / CT;
    const int col = blockIdx.x * (CT * 4) + cx * 4;
    const int r0 = blockIdx.y * rows_per_slab;
    const int r1 = r0 + rows_per_slab < M ? r0 + rows_per_slab : M;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const bool vec = ((ldg & 3) == 0) && ((((uintptr_t)g) & 15u) == 0) && (col + 3 < N);
    int r = r0 + ry;
    if (vec) {
        for (; r + 3 * RT < r1; r += 4 * RT) {
            const float *row = g + (long)r * ldg + col;
            float4 a = *(const float4 *)row, b = *(const float4 *)(row + (long)RT * ldg);
            float4 c = *(const float4 *)(row + 2l * RT * ldg), d = *(const float4 *)(row + 3l * RT * ldg);
            acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
            acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
            acc.x += c.x; acc.y += c.y; acc.z += c.z; acc.w += c.w;
            acc.x += d.x; acc.y += d.y; acc.z += d.z; acc.w += d.w;
        }
    }
    for (; r < r1; r += RT) {
        const float *row = g + (long)r * ldg;
        if (vec) {
            float4 v = *(const float4 *)(row + col);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        } else {
            if (col < N) acc.x += row[col];
            if (col + 1 < N) acc.y += row[col + 1];
            if (col + 2 < N) acc.z += row[col + 2];
            if (col + 3 < N) acc.w += row[col + 3];
        }
    }
    sh[ry][cx] = acc;
    __syncthreads();
    /* the partial rows are padded to whole column blocks, so every block stores four floats */
    const int NP = gridDim.x * (CT * 4);
    if (ry == 0) {
        #pragma unroll
        for (int k = 1; k < RT; k++) {
            float4 v = sh[k][cx];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        *(float4 *)(part + (long)blockIdx.y * NP + col) = acc;
        __threadfence();
    }
    __syncthreads();
    if (threadIdx.x == 0) ticket = atomicAdd(&g_colsum_tickets[blockIdx.x], 1u);
    __syncthreads();
    if (ticket != gridDim.y - 1) return;
    __threadfence();
    const int slabs = gridDim.y;
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = ry; k < slabs; k += RT) {
        float4 v = __ldcg((const float4 *)(part + (long)k * NP + col));
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    sh[ry][cx] = acc;
    __syncthreads();
    if (ry == 0) {
        #pragma unroll
        for (int k = 1; k < RT; k++) {
            float4 v = sh[k][cx];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if (col < N) out[col] = accumulate ? out[col] + acc.x : acc.x;
        if (col + 1 < N) out[col + 1] = accumulate ? out[col + 1] + acc.y : acc.y;
        if (col + 2 < N) out[col + 2] = accumulate ? out[col + 2] + acc.z : acc.z;
        if (col + 3 < N) out[col + 3] = accumulate ? out[col + 3] + acc.w : acc.w;
    }
    if (threadIdx.x == 0) g_colsum_tickets[blockIdx.x] = 0;      /* ready for the next launch */
}
int k_colsum(const float *g, int M, int N, int ldg, float *out, int accumulate) {
    /* as many row slabs as give every SM its full set of resident blocks exactly once: a second,
     * nearly empty wave of blocks costs as much time as the first */
    static int per_sm = 0;
    if (!per_sm) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, colsum_fused_kernel<32, 8>, 256, 0) != cudaSuccess || per_sm < 1)
            per_sm = 4;
    }
    const int cols_per_block = CS_COLS;      /* 512 bytes of a row per warp; 2 KB wide blocks measured slower */
    const int col_blocks = (N + cols_per_block - 1) / cols_per_block;
    int slabs = (g_tt.sm_count * per_sm) / col_blocks;
    if (slabs > (M + 31) / 32) slabs = (M + 31) / 32;
    if (slabs < 1) slabs = 1;
    int rows_per_slab = (M + slabs - 1) / slabs;
    slabs = (M + rows_per_slab - 1) / rows_per_slab;
    const bool fused = col_blocks <= CS_MAX_COL_BLOCKS;
    const long part_cols = fused ? (long)col_blocks * cols_per_block : N;
    /* the partial rows live in a buffer that is kept between calls (about 0.6 MB for 4096 columns):
     * a stream-ordered allocation and release around a 20 microsecond kernel showed in its time */
    static float *scratch = nullptr;
    static size_t scratch_floats = 0;
    const size_t need = (size_t)slabs * part_cols;
    if (need > scratch_floats) {
        if (scratch) tt_dev_free(scratch);
        scratch = (float *)tt_dev_alloc(sizeof(float) * need);
        scratch_floats = scratch ? need : 0;
    }
    float *part = scratch;
    if (!part) { tt_set_error("column sum: no scratch memory for %zu partial sums", need); return -1; }
    tt_trace_begin(TTB_K_REDUCE);
    dim3 grid(col_blocks, slabs);
    if (fused) {
        LAUNCH((colsum_fused_kernel<32, 8>), grid, 256, 0, g, M, N, ldg, rows_per_slab, part, out, accumulate);
    } else {
        LAUNCH(colsum_partial_kernel, grid, CS_COLS * CS_ROWS / 4, 0, g, M, N, ldg, rows_per_slab, part);
        LAUNCH(colsum_final_kernel, (N + TPB - 1) / TPB, TPB, 0, part, slabs, N, out, accumulate);
    }
    tt_trace_end(TTB_K_REDUCE, 4.0 * (double)M * N);
    return 0;
}

/* ---- column sums for callers that must not allocate ----------------------------
 * Some hosts of this library cannot reach the device allocator when they need a
 * bias gradient: a process that handed every byte of device memory to its own
 * arena at start-up and forbids any other allocation afterwards, or a
 * latency-bound loop in which an allocator call is not acceptable.  For them the
 * partial sums live in a fixed array inside the library image instead of in pool
 * memory.  Every GPU that loads the library carries the array
 * (TTB_COLSUM_STATIC_SLABS x TTB_COLSUM_STATIC_MAX_COLS floats = 2 MiB) until
 * the process exits.
 *
 * The array's name is only a stand-in on the host; what a kernel can use is the
 * address cudaGetSymbolAddress returns for it on the current device.  That
 * lookup is done here on the first call, for the one device the library runs on
 * and with that device current (the launch goes to the library's stream, which
 * belongs to that device, so a call made while another device is current is
 * refused) -- make the first call before any stream capture is begun.
 * All calls share the one array.  Each call overwrites every partial it later
 * reads, so nothing has to be cleared; but two calls that run on the GPU at the
 * same time (different streams, or different host threads) would trample each
 * other's partials.  Calls made through the library's single stream are safe. */
#define TTB_COLSUM_STATIC_SLABS 32
#define TTB_COLSUM_STATIC_MAX_COLS 16384
static __device__ __align__(256) float g_colsum_static[TTB_COLSUM_STATIC_SLABS * TTB_COLSUM_STATIC_MAX_COLS];
static float *g_colsum_static_addr = nullptr;  /* device address of the array on the library's device */

extern "C" int ttb_colsum_static(const float *g_dev, int rows, int cols, long ldg, float *out_dev, int accumulate) {
    if (!g_dev || !out_dev || rows <= 0 || cols <= 0 || ldg < cols || ldg > 0x7fffffffL) {
        tt_set_error("ttb_colsum_static: bad arguments");
        return -1;
    }
    if (cols > TTB_COLSUM_STATIC_MAX_COLS) {
        tt_set_error("ttb_colsum_static: %d columns exceed the built-in scratch (%d); use ttb_colsum",
                     cols, TTB_COLSUM_STATIC_MAX_COLS);
        return -1;
    }
    if (tt_ctx_init() != 0) return -1;
    int dev = -1;
    if (!tt_cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return -1;
    if (dev != g_tt.device) {
        tt_set_error("ttb_colsum_static: device %d is current but the library runs on device %d", dev, g_tt.device);
        return -1;
    }
    if (!g_colsum_static_addr) {
        float *addr = nullptr;
        if (!tt_cuda_ok(cudaGetSymbolAddress((void **)&addr, g_colsum_static), "cudaGetSymbolAddress") || !addr) return -1;
        g_colsum_static_addr = addr;
    }
    float *part = g_colsum_static_addr;
    int slabs = (rows + 63) / 64;
    if (slabs > TTB_COLSUM_STATIC_SLABS) slabs = TTB_COLSUM_STATIC_SLABS;
    int rows_per_slab = (rows + slabs - 1) / slabs;
    slabs = (rows + rows_per_slab - 1) / rows_per_slab;
    dim3 grid((cols + CS_COLS - 1) / CS_COLS, slabs);
    LAUNCH(colsum_partial_kernel, grid, CS_COLS * CS_ROWS / 4, 0, g_dev, rows, cols, (int)ldg, rows_per_slab, part);
    LAUNCH(colsum_final_kernel, (cols + TPB - 1) / TPB, TPB, 0, part, slabs, cols, out_dev, accumulate);
    return tt_cuda_ok(cudaGetLastError(), "ttb_colsum_static launch") ? 0 : -1;
}

/* ---- transpose: o[C,R] = x[R,C]^T through a padded 32x32 tile ---------------*/
__global__ void __launch_bounds__(256) transpose_kernel(float *o, const float *__restrict__ x, int R, int C) {
    __shared__ float tile[32][33];
    int bx = blockIdx.x * 32, by = blockIdx.y * 32;
    int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int j = ty; j < 32; j += 8) {
        int r = by + j, c = bx + tx;
        if (r < R && c < C) tile[j][tx] = x[(long)r * C + c];
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
        int c = bx + j, r = by + tx;
        if (r < R && c < C) o[(long)c * R + r] = tile[tx][j];
    }
}
void k_transpose(float *o, const float *x, int R, int C) {
    dim3 grid((C + 31) / 32, (R + 31) / 32);
    tt_trace_begin(TTB_K_ELEMENTWISE);
    LAUNCH(transpose_kernel, grid, 256, 0, o, x, R, C);
    tt_trace_end(TTB_K_ELEMENTWISE, 8.0 * (double)R * C);
}
