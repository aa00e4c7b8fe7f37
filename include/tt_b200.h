/* Additive entry points of the B200 tinytorch library.
 *
 * Nothing here is needed by a program written against the reference headers;
 * tensor.h and autograd.h alone are the drop-in surface.  These calls expose
 * what the reference keeps in its Python gate scripts or does not have at
 * all: device control, the backward kernels as stand-alone operators (so
 * that each can be checked and timed on its own), a fused loss, on-device
 * optimiser steps, persistent parameters, and data-parallel gradient
 * reduction over NCCL.  Each comment names the reference code the call
 * stands in for (file:line inside the reference project).
 */
#ifndef TINYTORCH_B200_H
#define TINYTORCH_B200_H

#include "tensor.h"
#include "autograd.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- device, stream, errors ---------------------------------------------- */
/* Number of CUDA devices visible to the process (0 when there is none). */
int         ttb_device_count(void);
/* Select the GPU for this process before the first tensor is created.
 * Without this call the library uses $TT_DEVICE, else $LOCAL_RANK, else 0.
 * Returns 0, or -1 (see ttb_last_error) when the device cannot be used. */
int         ttb_init(int device);
/* Text of the most recent failure ("" when none).  Every entry point that
 * returns NULL or -1 because of CUDA or NCCL leaves its reason here. */
const char *ttb_last_error(void);
/* Wait until everything enqueued so far has finished.  Returns 0 or -1. */
int         ttb_sync(void);
/* Kernel launches enqueued by this library since load. */
long        ttb_launch_count(void);
/* Device address of a tensor's payload (uploads a pending host write first). */
float      *ttb_device_ptr(Tensor *t);
/* {free bytes on the GPU, bytes the library's memory pool holds from the driver, bytes of the pool in
 * use}: lets a caller (and the tests) see whether a call allocated anything.  Returns 0 or -1. */
int         ttb_mem_info(unsigned long long out[3]);

/* Page-locked host memory, so that tt_fromdata / ag_backward_from copy from it
 * with a true asynchronous DMA instead of staging through the driver. */
void       *ttb_pinned_alloc(size_t bytes);
void        ttb_pinned_free(void *p);

/* Input pipeline.  Overwrite an existing tensor with `src` (numel floats, best from
 * ttb_pinned_alloc) on a separate copy stream: the transfer runs under whatever
 * kernels are executing, is ordered after all work enqueued before the call, and
 * the tensor's next use waits for it.  With two tensors used in turn, the upload
 * of batch i+1 hides behind the step on batch i.  Stands in for the per-step
 * normalise/gather/upload of the gate scripts (tests/gate_mnist_mlp.py:107-111).
 * `src` must stay untouched until the tensor has been used.  Returns 0 or -1. */
int         ttb_upload_async(Tensor *dst, const float *src);
/* The other direction: copy src's payload to dst (pinned host memory) on the copy stream, after the compute
 * work enqueued so far; ttb_download_wait() blocks until all such copies have landed.  Lets a loop enqueue
 * step i+1 before it reads step i's loss.  src may be released right after the call (its memory is not
 * reused before the copy has run); dst must stay valid until ttb_download_wait.  No reference counterpart
 * (tt_data is the blocking read). */
int         ttb_download_async(const Tensor *src, float *dst);
int         ttb_download_wait(void);

/* Normalise + gather, the first stage of the gate scripts' input pipeline
 * (tests/gate_mnist_mlp.py:86-90,107-111; tests/gate_cifar_cnn.py:162-163):
 *     xb = ((pixels[idx] / 255) - mean) / std
 * The raw 8-bit dataset [n_rows, channels, plane] is uploaded once (ttb_bytes_upload returns its
 * device address, ttb_bytes_free releases it) and stays resident; every step
 * ttb_gather_normalize_u8 fills `dst` (b * channels * plane floats, any shape) with the b rows
 * idx[0..b) picks, normalised per channel, bit-identical to NumPy's float32 arithmetic.  idx, mean
 * and std are host arrays (mean/std: one value per channel, at most 16 channels); idx may be reused
 * as soon as the call returns.  Returns 0, or -1 on bad arguments or an index outside [0, n_rows). */
void       *ttb_bytes_upload(const void *host, size_t nbytes);
void        ttb_bytes_free(void *dev);
int         ttb_gather_normalize_u8(Tensor *dst, const void *src_dev, long n_rows, const int *idx, long b,
                                    int channels, const float *mean, const float *std);

/* CUDA-event timing on the library's own stream. */
void       *ttb_event_create(void);
void        ttb_event_record(void *ev);
float       ttb_event_elapsed_ms(void *start, void *stop);   /* waits for `stop` */
void        ttb_event_destroy(void *ev);

/* Per-kernel-class timing.  While enabled, every launch of the classes below
 * is bracketed by an event pair; ttb_trace_read waits for the stream and
 * returns the sums since the last ttb_trace_reset. */
enum { TTB_K_GEMM_TC = 0, TTB_K_GEMM_SIMT = 1, TTB_K_ELEMENTWISE = 2,
       TTB_K_SOFTMAX = 3, TTB_K_SPATIAL = 4, TTB_K_REDUCE = 5, TTB_K_OPTIM = 6,
       TTB_K_COUNT = 7 };
void        ttb_trace_enable(int on);
void        ttb_trace_reset(void);
int         ttb_trace_read(int kind, double *total_ms, long *launches, double *work);

/* ---- GEMM ------------------------------------------------------------------
 * 0 = choose by shape, 1 = always the tcgen05 3xTF32 kernel (fails when the
 * shape cannot be fed by TMA), 2 = always the exact-fp32 kernel. */
void    ttb_set_gemm_path(int path);
/* How the tensor-core GEMM would run a product of this shape on `sms` SMs in a job of `world` ranks, as
 * ten integers {tile width, pair kernel?, K block, CTAs or pairs used, tiles, uniform K slices, K blocks
 * per slice, tail tiles, tail K slices, K blocks per tail slice}.  Needs no GPU; for tests and tuning.
 * No reference counterpart. */
int     ttb_gemm_plan(int M, int N, int K, int sms, int world, int out[10]);
/* Stand-alone forms of the two backward GEMMs the reference keeps private:
 *   ttb_matmul_nt: R[M,N] = X[M,K] * Y[N,K]^T   (src/autograd.c:66-84)
 *   ttb_matmul_tn: R[M,N] = X[K,M]^T * Y[K,N]   (src/autograd.c:87-103) */
Tensor *ttb_matmul_nt(const Tensor *x, const Tensor *y);
Tensor *ttb_matmul_tn(const Tensor *x, const Tensor *y);

/* ---- backward kernels as operators ----------------------------------------
 * relu: dx = x > 0 ? g : 0                      (src/autograd.c:318-327)
 * softmax: dx = s * (g - sum(g*s)) per row      (src/autograd.c:329-346) */
Tensor *ttb_relu_bwd(const Tensor *x, const Tensor *g);
Tensor *ttb_softmax_bwd(const Tensor *s, const Tensor *g);
/* Column sums of a 2-D tensor: out[n] = sum over rows of g[m, n].  This is the
 * bias row of a weight gradient, which the reference obtains as the last row of
 * A^T * dC with A carrying a ones column (src/autograd.c:87-103, 195-212). */
Tensor *ttb_colsum(const Tensor *g);
/* The same column sums for a caller that may not allocate device memory at the
 * moment of the call: an application whose own arena owns all of the GPU's
 * memory, or a loop that cannot afford an allocator call.  The partial sums go
 * to a 2 MiB array built into the library instead of pool memory, so the call
 * itself performs no allocation.  g_dev is [rows, cols] with row pitch ldg
 * (floats), out_dev holds cols floats; both are device addresses
 * (ttb_device_ptr) on the library's GPU, and the work is queued on the
 * library's own compute stream (the one every other entry point uses), not on a
 * stream of the caller's.  accumulate != 0 adds into out_dev.  At most 16384
 * columns; more is refused with -1 and a message, and so is a call made while a
 * GPU other than the library's is current.  The first call looks the array's
 * address up (cudaGetSymbolAddress); make that call before any stream capture
 * is begun in the process.  All calls share the array: do not let two of them
 * overlap on the GPU.  There is no counterpart in the reference, which is host
 * code over malloc. */
int     ttb_colsum_static(const float *g_dev, int rows, int cols, long ldg, float *out_dev, int accumulate);
/* Batched im2col and its adjoint (src/ops_spatial.c:37-69,
 * src/autograd.c:406-434).  x is [N,C,H,W]; col is [C*kh*kw, N*Hout*Wout]. */
Tensor *ttb_im2col(const Tensor *x, int kh, int kw, int stride_h, int stride_w,
                   int pad_h, int pad_w);
Tensor *ttb_col2im(const Tensor *col, int N, int C, int H, int W, int kh, int kw,
                   int stride_h, int stride_w, int pad_h, int pad_w);
/* Max-pool gradient routing (src/autograd.c:555-594).  ttb_maxpool_argmax
 * writes, for every output element, the flat offset into x that receives its
 * gradient (host array of Hout*Wout*N*C longs). */
Tensor *ttb_maxpool_bwd(const Tensor *x, const Tensor *g, int pool_h, int pool_w,
                        int stride_h, int stride_w);
int     ttb_maxpool_argmax(const Tensor *x, int pool_h, int pool_w,
                           int stride_h, int stride_w, long *idx_out);
Tensor *ttb_avgpool_bwd(const Tensor *g, int N, int C, int H, int W, int pool_h,
                        int pool_w, int stride_h, int stride_w);

/* ---- fused loss -----------------------------------------------------------
 * Softmax + cross-entropy + gradient in one pass over the logits.  Stands in
 * for softmax on the device followed by the NumPy lines of the gate scripts
 * (tests/gate_mnist_mlp.py:112-119): p = softmax(logits),
 * loss = mean(-log max(p[y], 1e-12)), dlogits = (p - onehot(y)) * scale.
 * labels holds the class index of every row as fp32.  *dlogits receives a new
 * tensor shaped like logits; the return value is a 1-element tensor holding
 * the mean loss.  NULL on shape errors. */
Tensor *ttb_softmax_xent(const Tensor *logits, const Tensor *labels, float scale,
                         Tensor **dlogits);

/* ---- evaluation -----------------------------------------------------------
 * pred = logits.argmax(axis=1); correct = (pred == y).sum()
 * (tests/gate_mnist_mlp.py:74-80, tests/gate_cifar_cnn.py:114-122) without moving the logits to
 * the host.  ttb_argmax returns the [rows] tensor of class indices (as fp32; first maximum, a NaN
 * counts as the maximum, like NumPy); ttb_argmax_correct returns how many rows' argmax equals the
 * label (labels: one class index per row as fp32), or -1.  It waits for the GPU (four bytes back). */
Tensor *ttb_argmax(const Tensor *logits);
long    ttb_argmax_correct(const Tensor *logits, const Tensor *labels);
/* Forward-only mode for evaluation batches: while off, the ag_* builders compute values but record
 * no graph (a node keeps no reference to its parents and requires no gradient), so an activation
 * is freed as soon as the caller releases its node, and a matmul followed by relu never stores
 * its pre-activation.  On by default; ttb_grad_enabled reads the setting. */
void    ttb_set_grad_enabled(int on);
int     ttb_grad_enabled(void);

/* ---- autograd extras ------------------------------------------------------
 * ag_backward_from with the seed already on the device: same contract, no
 * host round trip.  Returns 0, or -1 when the element counts differ.  When
 * `out` is an operator node without a gradient yet, the seed tensor is SHARED
 * as its gradient (retained, not copied): leave its contents alone while the
 * node lives; a later pass with another seed replaces it. */
int     ag_backward_from_tensor(AGNode *out, const Tensor *seed);
/* Drop a node's accumulated gradient so that the next pass starts from zero.
 * Needed once a parameter leaf outlives a step; the reference scripts build
 * new leaves every step instead (tests/gate_mnist_mlp.py:108-110). */
void    ag_zero_grad(AGNode *n);

/* ---- optimiser steps on the device ----------------------------------------
 * In-place forms of the NumPy updates in the gate scripts:
 *   sgd:       w -= lr * g
 *   momentum:  v = mu*v - lr*g ; w += v          (tests/gate_mnist_mlp.py:121-124)
 *   adam:      the update of tests/gate_cifar_cnn.py:81-98, step count t >= 1;
 *              scalars are doubles because the script's are Python floats
 * All return 0, or -1 on a shape mismatch. */
int     ttb_sgd_step(Tensor *w, const Tensor *g, float lr);
int     ttb_sgd_momentum_step(Tensor *w, Tensor *v, const Tensor *g, float lr, float mu);
int     ttb_adam_step(Tensor *w, Tensor *m, Tensor *v, const Tensor *g, double lr,
                      double beta1, double beta2, double eps, int t);

/* ---- data parallel training ----------------------------------------------
 * One process per GPU.  Rank 0 makes an id with ttb_dist_unique_id, the
 * launcher hands its 128 bytes to every rank, every rank calls
 * ttb_dist_init.  A leaf marked with ag_mark_param has its gradient summed
 * over all ranks (fp32 NCCL all-reduce on a second stream) as soon as the
 * backward pass has finished accumulating into it, so the reduction overlaps
 * the rest of the pass; ttb_dist_join makes the compute stream wait for all
 * reductions in flight.  The reference has no counterpart: it is a
 * single-process library. */
int     ttb_dist_unique_id(char id_out[128]);
int     ttb_dist_init(int rank, int world, const char id[128]);
int     ttb_dist_world(void);                        /* 1 when not initialised */
void    ag_mark_param(AGNode *leaf, int on);
/* Fuse plain SGD into the backward pass: as soon as the gradient of `leaf` is final (and,
 * for a marked parameter, summed over the ranks) the library applies value -= lr * grad,
 * on the communication stream when there is one, so the update of layer L runs under the
 * backward kernels of the layers below it.  lr <= 0 switches it off.  Same arithmetic as
 * ttb_sgd_step; call ttb_dist_join before the next forward pass. */
void    ag_param_sgd(AGNode *leaf, float lr);
int     ttb_dist_allreduce(Tensor *t);               /* sum over ranks, in place, async */
int     ttb_dist_join(void);
/* Lifetime rule for everything that runs beside the compute stream (ttb_dist_allreduce, the
 * reductions and fused updates of marked parameters, ttb_download_async): the tensor may be
 * released at any time after the call -- the library orders the reuse of its memory after the
 * work in flight -- but its CONTENTS are final only after ttb_dist_join / ttb_download_wait. */
/* Timing of the collectives while ttb_trace_enable is on, summed since ttb_trace_reset:
 * out = {collectives, bytes reduced, ms inside collectives (event pairs on the communication
 * stream), joins, exposed ms (communication stream's tail minus compute stream's tail at each
 * ttb_dist_join, when positive), longest collective in ms}.  Returns 0 or -1. */
int     ttb_dist_comm_read(double out[6]);
/* Ends the job's communication: frees this rank's peer-memory block (if any) and destroys the
 * NCCL communicator.  ORDER when the peer-memory path is in use: all ranks rendezvous, every
 * rank calls ttb_dist_peer_close, all ranks rendezvous again, then every rank calls
 * ttb_dist_finalize -- a block must not be freed while another process still has it open, and
 * no rank may exit in between.  tinytorch_b200.dist.finalize() does exactly that. */
void    ttb_dist_finalize(void);
/* Optional: reduce gradients with this library's own peer-memory kernel (plain NVLink loads and stores
 * from CTAs that share SMs with the GEMM) instead of ncclAllReduce.  After ttb_dist_init every rank calls
 * ttb_dist_peer_export (allocates its block for gradients of up to max_floats values, returns a 64-byte
 * cudaIpc handle), the handles travel to all ranks by the same side channel as the NCCL id, and every
 * rank calls ttb_dist_peer_import with the world x 64 bytes in rank order.  Gradients that are larger,
 * not a multiple of four values or not 16-byte aligned still go through NCCL.  No reference counterpart. */
int     ttb_dist_peer_export(size_t max_floats, int world, char handle_out[64]);
int     ttb_dist_peer_import(int rank, int world, const char *handles);
int     ttb_dist_peer_active(void);
/* First half of the tear-down: close the other ranks' blocks and switch the peer kernel off
 * (see ttb_dist_finalize for the order). */
void    ttb_dist_peer_close(void);
/* Limit of the peer kernel's device-side waits on other ranks, in milliseconds (default about
 * 2000).  When a wait runs out the kernel stops waiting, ttb_dist_join returns -1 with the phase
 * and the rank it waited for, the failure is passed on to every peer (their next wait or launch
 * reports it too) and this process refuses further peer reductions.  Returns 0 or -1. */
int     ttb_dist_set_wait_limit_ms(int ms);

#ifdef __cplusplus
}
#endif
#endif
