/* tinytorch tensor C ABI, served by the B200 (sm_100a) library.
 *
 * Drop-in for the reference header include/tensor.h: the same struct (first
 * six fields, same order and types), the same 22 entry points with the same
 * argument meaning, ownership and error convention (NULL on any invalid
 * argument or shape).  A program written against the reference header
 * compiles and links against this one unchanged.
 *
 * What differs is where the payload lives.  Every tensor owns a buffer in
 * GPU memory; all operators run as CUDA kernels on one stream and return as
 * soon as the work is enqueued.  `data` is a host MIRROR of that buffer: it
 * is NULL until tt_data() is called, and tt_data() is the synchronisation
 * point (it waits for the stream and copies device -> host when the mirror is
 * stale).  After tt_data() the caller may also write through the pointer; the
 * library uploads the mirror again before the tensor's next use on the
 * device.  Callers that poke `t->data` directly must therefore call
 * tt_data(t) first.
 */
#ifndef TINYTORCH_H
#define TINYTORCH_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Public tensor record (reference: include/tensor.h:10-17).  Tensors are
 * always contiguous row-major fp32; `strides` is informational.  The library
 * allocates a larger private record whose first bytes are this struct. */
typedef struct Tensor {
    float *data;      /* host mirror of the device payload; see tt_data() */
    long  *shape;     /* ndim extents */
    long  *strides;   /* ndim element strides (contiguous row-major) */
    int    ndim;      /* 1..8 */
    long   numel;     /* product of extents, <= 2^40 */
    int    refcount;
} Tensor;

/* ---- lifecycle (reference: include/tensor.h:20-23, src/tensor.c:10-61) ---- */
/* Zero-filled tensor.  NULL when ndim is outside 1..8, an extent is <= 0, the
 * element count overflows or exceeds 2^40, or device memory is exhausted. */
Tensor *tt_new(const long *shape, int ndim);
/* Copies numel floats from host memory (one host->device transfer).  The
 * shape is validated before `data` is touched. */
Tensor *tt_fromdata(const float *data, const long *shape, int ndim);
Tensor *tt_retain(Tensor *t);      /* refcount+1, returns t (NULL-safe) */
void    tt_release(Tensor *t);     /* refcount-1, frees at zero (NULL-safe) */

/* ---- accessors (reference: include/tensor.h:26-30, src/tensor.c:63-75) ---- */
float  *tt_data(const Tensor *t);  /* waits for the GPU, refreshes and returns the host mirror */
long    tt_numel(const Tensor *t);
int     tt_ndim(const Tensor *t);
void    tt_shape(const Tensor *t, long *out);
void    tt_strides(const Tensor *t, long *out);

/* ---- operators: fresh output, NULL on shape/argument error ----
 * reference: include/tensor.h:33-41, src/ops.c:26-145, src/gemm.c:644-671 */
Tensor *tt_add(const Tensor *a, const Tensor *b);
Tensor *tt_mul(const Tensor *a, const Tensor *b);
Tensor *tt_addscalar(const Tensor *a, float s);
Tensor *tt_mulscalar(const Tensor *a, float s);
/* The three matmuls of the reference (naive / AVX2 one thread / AVX2 OpenMP)
 * are one GPU GEMM here: the tcgen05 3xTF32 kernel for large aligned shapes,
 * the exact-fp32 kernel otherwise.  `nthreads` is accepted and ignored. */
Tensor *tt_matmul(const Tensor *a, const Tensor *b);
Tensor *tt_matmul_fast(const Tensor *a, const Tensor *b);
Tensor *tt_matmul_omp(const Tensor *a, const Tensor *b, int nthreads);
Tensor *tt_relu(const Tensor *a);
Tensor *tt_softmax(const Tensor *a);   /* last axis; an all -Inf row becomes uniform */

/* ---- spatial and shape operators ----
 * reference: include/tensor.h:44-50, src/ops_spatial.c:22-201 */
Tensor *tt_reshape(const Tensor *a, const long *new_shape, int new_ndim);  /* a copy, never a view */
Tensor *tt_conv2d(const Tensor *a, const Tensor *w, const Tensor *b,
                  int stride_h, int stride_w, int pad_h, int pad_w);
Tensor *tt_maxpool2d(const Tensor *a, int pool_h, int pool_w,
                     int stride_h, int stride_w);
Tensor *tt_avgpool2d(const Tensor *a, int pool_h, int pool_w,
                     int stride_h, int stride_w);

/* Host-pointer sgemm exported by the reference library (src/gemm.c:569):
 * C[M,N] = A[M,K] * B[K,N], row-major host arrays; C is overwritten.
 * Returns 0, or -1 on failure.  `nthreads` is ignored. */
int tt_sgemm_rowmajor(int M, int N, int K, const float *A, const float *B,
                      float *C, int nthreads);

#ifdef __cplusplus
}
#endif
#endif
