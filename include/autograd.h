/* tinytorch reverse-mode autograd C ABI, served by the B200 library.
 *
 * Drop-in for the reference header include/autograd.h: the same 20 entry
 * points, opaque node type, ownership and error rules.  The graph itself
 * (nodes, refcounts, topological order, dispatch) is host code exactly as in
 * the reference (src/autograd.c:107-125, 630-745); every numeric loop behind
 * a builder or a backward rule is a CUDA kernel on the library's stream.
 */
#ifndef TINYTORCH_AUTOGRAD_H
#define TINYTORCH_AUTOGRAD_H

#include "tensor.h"
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct AGNode AGNode;     /* opaque, refcounted */

/* ---- builders: run the forward operator and record the edge ----
 * reference: include/autograd.h:14-31, src/autograd.c:127-275.
 * Each returns a node with refcount 1 that retains its parents, or NULL when
 * an argument is NULL or the forward operator rejects the shapes. */
AGNode *ag_leaf(Tensor *t, int requires_grad);     /* retains t */
AGNode *ag_add(AGNode *a, AGNode *b);
AGNode *ag_mul(AGNode *a, AGNode *b);
AGNode *ag_addscalar(AGNode *a, float s);
AGNode *ag_mulscalar(AGNode *a, float s);
AGNode *ag_matmul(AGNode *a, AGNode *b);           /* 2-D x 2-D */
AGNode *ag_relu(AGNode *a);
AGNode *ag_softmax(AGNode *a);                     /* last axis */
AGNode *ag_padones(AGNode *a);                     /* [M,K] -> [M,K+1], last column = 1 */
AGNode *ag_reshape(AGNode *a, const long *new_shape, int new_ndim);
AGNode *ag_conv2d(AGNode *a, AGNode *w, AGNode *b, /* b may be NULL */
                  int stride_h, int stride_w, int pad_h, int pad_w);
AGNode *ag_maxpool2d(AGNode *a, int pool_h, int pool_w,
                     int stride_h, int stride_w);
AGNode *ag_avgpool2d(AGNode *a, int pool_h, int pool_w,
                     int stride_h, int stride_w);

/* ---- accessors (reference: include/autograd.h:34-36); borrowed pointers ---- */
Tensor *ag_value(const AGNode *n);
Tensor *ag_grad(const AGNode *n);                  /* NULL until a backward pass reached n */
int     ag_requires_grad(const AGNode *n);

/* ---- reverse pass (reference: include/autograd.h:38-45, src/autograd.c:682-727) ----
 * ag_backward seeds d(out) with ones.  ag_backward_from copies `seed`
 * (seed_numel host floats) into d(out); seed_numel must equal the element
 * count of out, otherwise the call returns without touching anything, and the
 * caller has to surface that as an error.  d(out) is overwritten by the seed,
 * every other node accumulates, and gradients stay on their nodes, so a
 * second pass over the same graph adds to the first. */
void    ag_backward(AGNode *out);
void    ag_backward_from(AGNode *out, const float *seed, size_t seed_numel);

/* ---- node lifetime (reference: include/autograd.h:47-48, src/autograd.c:731-745) ---- */
void    ag_release(AGNode *n);
AGNode *ag_retain(AGNode *n);

#ifdef __cplusplus
}
#endif
#endif
