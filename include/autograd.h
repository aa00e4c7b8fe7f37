/* Reverse-mode autograd over device-resident tensors: the C ABI of the B200 library.
 *
 * A program written against the reference's include/autograd.h compiles against this
 * header unchanged: the same twenty entry points, an opaque node type, the same
 * ownership and error rules.  What differs is behind the calls.  The graph itself --
 * nodes, reference counts, ordering, dispatch -- is host code, as in the reference
 * (src/autograd.c:107-125, 630-745); every numeric loop of a builder or of a backward
 * rule is a CUDA kernel enqueued on the library's stream, and nothing waits for the
 * GPU until the caller asks for host data with tt_data().
 */
#ifndef TT_B200_AUTOGRAD_ABI_H
#define TT_B200_AUTOGRAD_ABI_H

#include <stddef.h>

#include "tensor.h"

#ifdef __cplusplus
extern "C" {
#endif

/* A vertex of the recorded graph.  Opaque and reference counted; it owns one reference
 * to its value tensor and to each of its inputs. */
struct AGNode;
typedef struct AGNode AGNode;

/* ------------------------------------------------------------------------------------
 * Life cycle (reference: include/autograd.h:14,47-48; src/autograd.c:127-133, 731-745)
 * ---------------------------------------------------------------------------------- */

/* Wrap an existing tensor as an input of the graph.  The node takes its own reference
 * to `value`; the caller keeps (and later releases) the one it holds.  NULL in, NULL out. */
AGNode *ag_leaf(Tensor *value, int requires_grad);

/* One more / one fewer reference.  Dropping the last one releases the node's tensors
 * and then its inputs, iteratively, so that a chain of any depth unwinds without
 * recursion on the C stack. */
AGNode *ag_retain(AGNode *node);
void    ag_release(AGNode *node);

/* ------------------------------------------------------------------------------------
 * What a node holds (reference: include/autograd.h:34-36; src/autograd.c:277-281).
 * The pointers are borrowed: valid while the node lives, not to be released.
 * ---------------------------------------------------------------------------------- */
Tensor *ag_value(const AGNode *node);
Tensor *ag_grad(const AGNode *node);              /* NULL until a reverse pass has reached the node */
int     ag_requires_grad(const AGNode *node);

/* ------------------------------------------------------------------------------------
 * Builders (reference: include/autograd.h:15-31; src/autograd.c:135-275).
 * Each runs the forward operator on the GPU, records the edge and returns a node with
 * one reference, or NULL when an argument is NULL or the operator rejects the shapes
 * (the rules are those of the tt_* operator of the same name in tensor.h).
 * ---------------------------------------------------------------------------------- */

/* element by element, equal shapes */
AGNode *ag_add(AGNode *lhs, AGNode *rhs);
AGNode *ag_mul(AGNode *lhs, AGNode *rhs);
AGNode *ag_addscalar(AGNode *x, float c);
AGNode *ag_mulscalar(AGNode *x, float c);
AGNode *ag_relu(AGNode *x);

/* [M,K] times [K,N]; on this library a tcgen05 3xTF32 product, or the exact fp32 kernel
 * for small shapes */
AGNode *ag_matmul(AGNode *lhs, AGNode *rhs);

/* softmax along the last axis */
AGNode *ag_softmax(AGNode *x);

/* [M,K] -> [M,K+1] with a last column of ones: the reference's way of carrying a bias
 * as one more row of the weight matrix.  Feeding a matmul, the column is never written
 * here: the bias row is added in the product's epilogue. */
AGNode *ag_padones(AGNode *x);

/* same elements, new shape (dims[0..ndim-1], product unchanged) */
AGNode *ag_reshape(AGNode *x, const long *dims, int ndim);

/* NCHW convolution with filters [F,C,HH,WW] and an optional bias [F] (bias may be NULL) */
AGNode *ag_conv2d(AGNode *x, AGNode *filters, AGNode *bias, int stride_h, int stride_w, int pad_h, int pad_w);

/* pooling over windows window_h x window_w without padding */
AGNode *ag_maxpool2d(AGNode *x, int window_h, int window_w, int stride_h, int stride_w);
AGNode *ag_avgpool2d(AGNode *x, int window_h, int window_w, int stride_h, int stride_w);

/* ------------------------------------------------------------------------------------
 * Reverse pass (reference: include/autograd.h:38-45; src/autograd.c:682-727).
 *
 * ag_backward starts from d(root) = 1 everywhere.  ag_backward_from starts from `seed`,
 * `count` floats in host memory; `count` has to equal the number of elements of the
 * root's value -- when it does not, or when the root does not require a gradient, the
 * call returns having changed nothing, and it is the caller's job to notice (the Python
 * wrappers compare the sizes first and raise).
 *
 * d(root) is overwritten by the seed; every other node ADDS what arrives to the gradient
 * it already holds, and gradients stay on their nodes afterwards.  A second pass over the
 * same graph therefore adds to the first (the reference's tests pin the resulting values,
 * tests/test_grad.py:293-313, and so do this repository's).
 * ---------------------------------------------------------------------------------- */
void ag_backward(AGNode *root);
void ag_backward_from(AGNode *root, const float *seed, size_t count);

#ifdef __cplusplus
}
#endif
#endif /* TT_B200_AUTOGRAD_ABI_H */
