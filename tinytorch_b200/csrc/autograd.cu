/* Reverse-mode autograd: the graph lives on the host, the numbers on the GPU.
 *
 * Same observable behaviour as the reference's src/autograd.c: builders run
 * the forward operator and retain their parents (:107-275), the reverse pass
 * orders nodes by an iterative depth-first post-order (:650-680), overwrites
 * d(out) with the seed and lets every other node accumulate (:704-725), and
 * gradients stay on their nodes between passes.  Every backward rule launches
 * CUDA kernels on the library stream instead of looping on the host, and the
 * pass doubles as the sequencer for data-parallel training: when the last
 * consumer of a marked parameter leaf has been processed, its gradient is
 * handed to the NCCL stream while the rest of the pass keeps running.
 *
 * One deliberate difference: a padones node that feeds a matmul is folded
 * into that GEMM (ones column -> bias row in the forward epilogue, column sum
 * in the weight gradient), its [M,K+1] value is produced only if somebody
 * asks for it, and the matmul's input gradient goes straight to the padones
 * node's parent.  Leaf gradients are unchanged; ag_grad() of such a padones
 * node stays NULL.  TT_FUSE_PADONES=0 restores the literal behaviour.
 *
 * A second one, for the relu that follows a matmul (TT_FUSE_RELU=0 restores the literal
 * behaviour): ag_matmul does not launch its product at once but leaves its value deferred.
 * If the next builder to touch the node is ag_relu, ONE GEMM runs whose epilogue writes
 * max(x*w + b, 0) as the relu node's value, and the pre-activation is never stored; anybody
 * who does read it later (ag_value + tt_data, another builder, the root of a backward pass)
 * gets it from a plain GEMM launched at that moment -- from the operands as they are then.
 * Backward, the relu's mask is taken from its OUTPUT (y > 0 exactly when x > 0, NaN and the
 * infinities included), and when a matmul's input gradient is the only contribution to a relu
 * node it is masked in that GEMM's epilogue and written straight into the gradient of the
 * relu's parent; ag_grad() of such a relu node stays NULL, every other gradient is unchanged. */
#include "tt_internal.h"

#include <stdlib.h>
#include <string.h>

enum OpKind {
    OP_LEAF = 0, OP_ADD, OP_MUL, OP_ADDSCALAR, OP_MULSCALAR, OP_MATMUL, OP_RELU,
    OP_SOFTMAX, OP_PADONES, OP_RESHAPE, OP_CONV2D, OP_MAXPOOL2D, OP_AVGPOOL2D
};

struct AGNode {
    Tensor *val;
    Tensor *grad;
    AGNode *parents[3];
    int     nparents;
    int     kind;
    float   scalar;
    int     params[4];
    int     requires_grad;
    int     refcount;
    int     mark;          /* depth-first state during ordering */
    int     pending;       /* consumers not yet processed in the running pass */
    int     is_param;      /* gradient is all-reduced across ranks when final */
    int     fused_pad;     /* matmul that consumed its padones parent virtually */
    float   sgd_lr;        /* > 0: value -= sgd_lr * grad as soon as the gradient is final */
    int     reduced_in_rule;   /* the rule that produced the gradient already: 1 reduced and applied it (in chunks), 2 started its reduction */
    int     grad_is_seed;      /* grad is the caller's seed tensor, shared: replace, never write */
};

/* ---- construction ----------------------------------------------------------*/
static AGNode *node_make(Tensor *val, int requires_grad, int kind) {
    if (!val) return nullptr;
    AGNode *n = (AGNode *)calloc(1, sizeof(AGNode));
    if (!n) { tt_release(val); return nullptr; }
    n->val = val;
    n->requires_grad = requires_grad;
    n->kind = kind;
    n->refcount = 1;
    return n;
}
/* Forward-only mode (ttb_set_grad_enabled(0), the evaluation batches of
 * tests/gate_mnist_mlp.py:74-80): a node keeps no link to its parents and asks for no gradient,
 * so every activation is freed the moment the caller releases its node. */
static void node_link(AGNode *n, AGNode *p) {
    if (!g_tt.grad_enabled) { n->requires_grad = 0; return; }
    n->parents[n->nparents++] = ag_retain(p);
}
extern "C" void ttb_set_grad_enabled(int on) { g_tt.grad_enabled = on ? 1 : 0; }
extern "C" int ttb_grad_enabled(void) { return g_tt.grad_enabled; }

extern "C" AGNode *ag_leaf(Tensor *t, int requires_grad) {
    if (!t) return nullptr;
    return node_make(tt_retain(t), requires_grad, OP_LEAF);
}

static AGNode *unary_node(AGNode *a, Tensor *val, int kind) {
    AGNode *n = node_make(val, a->requires_grad, kind);
    if (n) node_link(n, a);
    return n;
}
static AGNode *binary_node(AGNode *a, AGNode *b, Tensor *val, int kind) {
    AGNode *n = node_make(val, a->requires_grad || b->requires_grad, kind);
    if (n) { node_link(n, a); node_link(n, b); }
    return n;
}

extern "C" AGNode *ag_add(AGNode *a, AGNode *b) {
    if (!a || !b) return nullptr;
    return binary_node(a, b, tt_add(a->val, b->val), OP_ADD);
}
extern "C" AGNode *ag_mul(AGNode *a, AGNode *b) {
    if (!a || !b) return nullptr;
    return binary_node(a, b, tt_mul(a->val, b->val), OP_MUL);
}
extern "C" AGNode *ag_addscalar(AGNode *a, float s) {
    if (!a) return nullptr;
    AGNode *n = unary_node(a, tt_addscalar(a->val, s), OP_ADDSCALAR);
    if (n) n->scalar = s;
    return n;
}
extern "C" AGNode *ag_mulscalar(AGNode *a, float s) {
    if (!a) return nullptr;
    AGNode *n = unary_node(a, tt_mulscalar(a->val, s), OP_MULSCALAR);
    if (n) n->scalar = s;
    return n;
}
extern "C" AGNode *ag_relu(AGNode *a) {
    if (!a) return nullptr;
    if (a->kind == OP_MATMUL && tt_is_deferred_matmul(a->val))      /* one GEMM, relu in its epilogue */
        return unary_node(a, tt_deferred_matmul_relu(a->val), OP_RELU);
    return unary_node(a, tt_relu(a->val), OP_RELU);
}
extern "C" AGNode *ag_softmax(AGNode *a) {
    if (!a) return nullptr;
    return unary_node(a, tt_softmax(a->val), OP_SOFTMAX);
}

extern "C" AGNode *ag_padones(AGNode *a) {
    if (!a || a->val->ndim != 2) return nullptr;
    Tensor *v;
    if (g_tt.fuse_padones) {
        v = tt_new_lazy_padones(a->val);
    } else {
        const float *px = tt_dev_ro(a->val);
        if (!px) return nullptr;
        long shp[2] = {a->val->shape[0], a->val->shape[1] + 1};
        v = tt_new_uninit(shp, 2);
        if (v) k_padones(TT(v)->dev, px, (int)a->val->shape[0], (int)a->val->shape[1]);
    }
    return unary_node(a, v, OP_PADONES);
}

static int matmul_shapes_ok(const Tensor *av, const Tensor *bv) {
    return av->ndim == 2 && bv->ndim == 2 && av->shape[1] == bv->shape[0] && av->shape[0] <= 0x7fffffffL &&
           bv->shape[0] <= 0x7fffffffL && bv->shape[1] <= 0x7fffffffL;
}

extern "C" AGNode *ag_matmul(AGNode *a, AGNode *b) {
    if (!a || !b) return nullptr;
    const Tensor *av = a->val, *bv = b->val;
    if (a->kind == OP_PADONES && g_tt.fuse_padones && TT(av)->lazy_kind == TT_LAZY_PADONES && matmul_shapes_ok(av, bv)) {
        /* x.padones().matmul(w) = x * w[:K] + w[K]   (src/autograd.c:195-212 then :168-171); x is the
         * source the deferred padones value holds (the node has no parent link in forward-only mode) */
        Tensor *xv = &TT(av)->lazy_src->pub;
        Tensor *out;
        if (g_tt.fuse_relu) {
            out = tt_new_lazy_matmul(xv, b->val, 1);          /* launched by whoever consumes it */
        } else {
            const float *px = tt_dev_ro(xv), *pw = tt_dev_ro(bv);
            if (!px || !pw) return nullptr;
            long shp[2] = {av->shape[0], bv->shape[1]};
            out = tt_new_uninit(shp, 2);
            if (!out) return nullptr;
            GemmArgs g;
            memset(&g, 0, sizeof g);
            g.M = (int)shp[0]; g.N = (int)shp[1]; g.K = (int)av->shape[1];
            g.A = px; g.lda = xv->shape[1]; g.a_pad_ones = 1;
            g.B = pw; g.ldb = g.N; g.C = TT(out)->dev; g.ldc = g.N;
            if (tt_gemm(&g) != 0) { tt_release(out); return nullptr; }
        }
        AGNode *n = binary_node(a, b, out, OP_MATMUL);
        if (n) n->fused_pad = 1;
        return n;
    }
    if (g_tt.fuse_relu && matmul_shapes_ok(av, bv))
        return binary_node(a, b, tt_new_lazy_matmul(a->val, b->val, 0), OP_MATMUL);
    return binary_node(a, b, tt_matmul_omp(av, bv, 12), OP_MATMUL);
}

extern "C" AGNode *ag_reshape(AGNode *a, const long *new_shape, int new_ndim) {
    if (!a) return nullptr;
    return unary_node(a, tt_reshape(a->val, new_shape, new_ndim), OP_RESHAPE);
}

extern "C" AGNode *ag_conv2d(AGNode *a, AGNode *w, AGNode *b, int stride_h, int stride_w, int pad_h, int pad_w) {
    if (!a || !w) return nullptr;
    Tensor *v = tt_conv2d(a->val, w->val, b ? b->val : nullptr, stride_h, stride_w, pad_h, pad_w);
    int req = a->requires_grad || w->requires_grad || (b && b->requires_grad);
    AGNode *n = node_make(v, req, OP_CONV2D);
    if (!n) return nullptr;
    node_link(n, a); node_link(n, w);
    if (b) node_link(n, b);
    n->params[0] = stride_h; n->params[1] = stride_w; n->params[2] = pad_h; n->params[3] = pad_w;
    return n;
}

static AGNode *pool_node(AGNode *a, Tensor *v, int kind, int ph, int pw, int sh, int sw) {
    AGNode *n = unary_node(a, v, kind);
    if (n) { n->params[0] = ph; n->params[1] = pw; n->params[2] = sh; n->params[3] = sw; }
    return n;
}
extern "C" AGNode *ag_maxpool2d(AGNode *a, int pool_h, int pool_w, int stride_h, int stride_w) {
    if (!a) return nullptr;
    return pool_node(a, tt_maxpool2d(a->val, pool_h, pool_w, stride_h, stride_w), OP_MAXPOOL2D,
                     pool_h, pool_w, stride_h, stride_w);
}
extern "C" AGNode *ag_avgpool2d(AGNode *a, int pool_h, int pool_w, int stride_h, int stride_w) {
    if (!a) return nullptr;
    return pool_node(a, tt_avgpool2d(a->val, pool_h, pool_w, stride_h, stride_w), OP_AVGPOOL2D,
                     pool_h, pool_w, stride_h, stride_w);
}

extern "C" Tensor *ag_value(const AGNode *n) { return n ? n->val : nullptr; }
extern "C" Tensor *ag_grad(const AGNode *n) { return n ? n->grad : nullptr; }
extern "C" int ag_requires_grad(const AGNode *n) { return n ? n->requires_grad : 0; }
extern "C" void ag_mark_param(AGNode *leaf, int on) { if (leaf) leaf->is_param = on ? 1 : 0; }
extern "C" void ag_param_sgd(AGNode *leaf, float lr) { if (leaf) leaf->sgd_lr = lr > 0.0f ? lr : 0.0f; }
extern "C" void ag_zero_grad(AGNode *n) {
    if (!n || !n->grad) return;
    tt_release(n->grad);
    n->grad = nullptr;
    n->grad_is_seed = 0;
}

/* ---- gradient accumulation (src/autograd.c:44-63) ---------------------------
 * give(): the contribution lives in another node's gradient, so the first one
 *         is copied.  take(): the contribution is a fresh temporary whose
 *         reference passes to the node, which saves the copy. */
static void give(AGNode *p, const Tensor *g) {
    if (!p || !p->requires_grad || !g) return;
    const float *pg = tt_dev_ro(g);
    if (!pg) return;
    if (!p->grad) {
        Tensor *c = tt_new_like(g, 0);
        if (!c) return;
        k_copy(TT(c)->dev, pg, g->numel);
        p->grad = c;
        return;
    }
    float *pd = tt_dev_rw(p->grad);
    if (pd) k_accum(pd, pg, g->numel);
}
static void take(AGNode *p, Tensor *t) {
    if (!t) return;
    if (!p || !p->requires_grad) { tt_release(t); return; }
    if (!p->grad) { p->grad = t; return; }
    float *pd = tt_dev_rw(p->grad);
    const float *ps = tt_dev_ro(t);
    if (pd && ps) k_accum(pd, ps, t->numel);
    tt_release(t);
}
/* Destination for a kernel that can write or add in place: the node's
 * gradient when it exists (accumulate), else a new tensor shaped like val. */
static float *grad_target(AGNode *p, int *accumulate) {
    if (p->grad) { *accumulate = 1; return tt_dev_rw(p->grad); }
    Tensor *t = tt_new_like(p->val, 0);
    if (!t) return nullptr;
    p->grad = t;
    *accumulate = 0;
    return TT(t)->dev;
}

/* Elements [off, off+count) of a parameter's gradient are final.  Two steps, which may be issued
 * together or apart:
 *   reduce  sum them over the ranks (marked parameters, communicator present) on the communication
 *           stream, ordered after the kernel that produced them;
 *   update  for a parameter with a fused optimiser, w -= lr * g behind the reduction on the same
 *           stream.  The update overwrites the WEIGHTS, which the input-gradient product of the same
 *           layer still reads: it is ordered after everything enqueued on the compute stream so far,
 *           so it has to be issued once that product has been enqueued.
 * With a communicator both run on the communication stream, under the backward kernels still to
 * come; ttb_dist_join orders the compute stream after them. */
void tt_dist_note_comm_work(void);
int tt_dist_comm_after_compute(void);
enum { PARAM_REDUCE = 1, PARAM_UPDATE = 2 };
enum { PARAM_TAIL = 4 };      /* the reduction has nothing left to hide behind: it may use every SM */
static void param_grad_ready(AGNode *p, long off, long count, int steps) {
    if (!p->grad || count <= 0) return;
    const int dist = tt_dist_active() && p->is_param;
    if (!dist && p->sgd_lr <= 0.0f) return;
    float *g = tt_dev_rw(p->grad);
    if (!g) return;
    if (dist && (steps & PARAM_REDUCE)) {
        if (steps & PARAM_TAIL) tt_dist_allreduce_tail(g + off, (size_t)count);
        else tt_dist_allreduce_range(g + off, (size_t)count);
    }
    if (p->sgd_lr > 0.0f && (steps & PARAM_UPDATE)) {
        float *w = tt_dev_rw(p->val);
        if (!w) return;
        cudaStream_t keep = g_tt.stream;
        if (dist) {
            if (!(steps & PARAM_REDUCE)) tt_dist_comm_after_compute();      /* the reduction was issued earlier: order after the readers of w */
            g_tt.stream = g_tt.comm_stream;
        }
        k_sgd(w + off, g + off, p->sgd_lr, count);
        g_tt.stream = keep;
        if (dist) tt_dist_note_comm_work();
    }
    if (dist) {
        /* the communication stream is still working on both payloads: a release before
         * ttb_dist_join (ag_zero_grad, ag_release) must not recycle their blocks under it */
        tt_mark_busy(p->grad, g_tt.comm_stream);
        if (p->sgd_lr > 0.0f && (steps & PARAM_UPDATE)) tt_mark_busy(p->val, g_tt.comm_stream);
    }
}

/* ---- backward rules ----------------------------------------------------------*/
static void bw_mul(AGNode *n) {              /* src/autograd.c:290-298 */
    take(n->parents[0], tt_mul(n->grad, n->parents[1]->val));
    take(n->parents[1], tt_mul(n->grad, n->parents[0]->val));
}

/* dA = dC * B^T and dB = A^T * dC (src/autograd.c:308-316, 66-103).  The
 * products go straight into the parents' gradients; a parent that needs no
 * gradient is skipped (the reference computes and discards it). */
static void bw_matmul(AGNode *n) {
    AGNode *a = n->parents[0], *b = n->parents[1];
    const float *pg = tt_dev_ro(n->grad);
    if (!pg) return;
    const int M = (int)n->val->shape[0], N = (int)n->val->shape[1];
    GemmArgs g;
    if (n->fused_pad) {
        AGNode *x = a->parents[0];
        const int Kr = (int)x->val->shape[1];
        /* the weight gradient first: its all-reduce (data parallel) then starts one product earlier and
         * runs under the input-gradient product; the two are independent */
        if (b->requires_grad) {               /* dW = [X 1]^T * dC */
            const float *px = tt_dev_ro(x->val);
            int acc;
            float *dst = px ? grad_target(b, &acc) : nullptr;
            static int dp_chunks = -1;
            if (dp_chunks < 0) { const char *e = getenv("TT_DP_CHUNKS"); dp_chunks = e && *e ? atoi(e) : 2; if (dp_chunks < 1) dp_chunks = 1; }
            /* Data parallel with the peer-memory reduction: the product's epilogue delivers every block of
             * the gradient that another rank owns straight into that rank's staging area (reduce-scatter
             * fused into the GEMM); the reduction kernel that follows only has to move the bias row. */
            PeerPush pp;
            const bool fuse_push = dst && !acc && tt_dist_active() && b->is_param && b->pending == 1 && (N & 31) == 0 &&
                                   tt_peer_push_plan(dst, (size_t)b->grad->numel, &pp);
            if (fuse_push) {
                memset(&g, 0, sizeof g);
                g.ta = 1; g.a_pad_ones = 1; g.M = Kr + 1; g.N = N; g.K = M;
                g.A = px; g.lda = Kr; g.B = pg; g.ldb = N; g.C = dst; g.ldc = N;
                g.rule = 1; g.push = &pp;
                if (tt_gemm(&g) == 0) {
                    tt_dist_allreduce_pushed(dst, (size_t)b->grad->numel, (size_t)g_tt.gemm_pushed_floats);
                    tt_mark_busy(b->grad, g_tt.comm_stream);
                    b->reduced_in_rule = 2;               /* the update follows once the dX product has been enqueued */
                }
            } else if (dst && dp_chunks > 1 && tt_dist_active() && b->is_param && b->pending == 1 && Kr >= 2048 &&
                !x->requires_grad) {
                /* Data parallel, first layer (its input needs no gradient, so this is the last GEMM
                 * of the pass and nothing is left to hide its all-reduce behind): produce the
                 * gradient in row blocks (TT_DP_CHUNKS, default two) and hand each to the all-reduce
                 * as soon as it exists; only the last block's reduction is exposed.  Measured on the
                 * per-GPU shapes of the 8-GPU job: 2.38 -> 2.26 ms per step with two blocks, slower
                 * with four (more, smaller collectives). */
                const int rows_per = ((Kr / dp_chunks + 127) / 128) * 128;
                for (int r0 = 0; r0 < Kr; r0 += rows_per) {
                    const int r1 = r0 + rows_per < Kr ? r0 + rows_per : Kr;
                    const int last = (r1 == Kr);
                    memset(&g, 0, sizeof g);
                    g.ta = 1; g.a_pad_ones = last; g.M = r1 - r0 + last; g.N = N; g.K = M;
                    g.A = px + r0; g.lda = Kr; g.B = pg; g.ldb = N; g.C = dst + (long)r0 * N; g.ldc = N;
                    g.accumulate = acc; g.rule = 1;
                    if (tt_gemm(&g) != 0) break;
                    param_grad_ready(b, (long)r0 * N, (long)(r1 - r0 + last) * N, PARAM_REDUCE | PARAM_UPDATE | (last ? PARAM_TAIL : 0));
                }
                b->reduced_in_rule = 1;
            } else if (dst) {
                memset(&g, 0, sizeof g);
                g.ta = 1; g.a_pad_ones = 1; g.M = Kr + 1; g.N = N; g.K = M;
                g.A = px; g.lda = Kr; g.B = pg; g.ldb = N; g.C = dst; g.ldc = N;
                g.accumulate = acc; g.rule = 1;
                if (tt_gemm(&g) == 0 && b->pending == 1 && (b->is_param || b->sgd_lr > 0.0f)) {
                    /* this was the parameter's last consumer: start its reduction now, under the
                     * input-gradient product below; the update follows once that product (which reads
                     * the weights) has been enqueued */
                    param_grad_ready(b, 0, b->grad->numel, PARAM_REDUCE);
                    b->reduced_in_rule = 2;
                }
            }
        }
        if (x->requires_grad) {               /* dX = dC * W[:K]^T, bypassing the padones node */
            const float *pw = tt_dev_ro(b->val);
            /* x is a relu node and this product is all of its gradient: mask it here (the relu's
             * output is the mask) and hand it to the relu's parent; the relu node's own rule then
             * finds no gradient and does nothing (src/autograd.c:318-327 folded into :308-316) */
            AGNode *z = (g_tt.fuse_relu && x->kind == OP_RELU && !x->grad && x->pending == 1 && a->pending == 1 &&
                         x->nparents == 1 && x->parents[0]->requires_grad) ? x->parents[0] : nullptr;
            const float *pm = z ? tt_dev_ro(x->val) : nullptr;
            if (z && !pm) z = nullptr;
            int acc;
            float *dst = pw ? grad_target(z ? z : x, &acc) : nullptr;
            if (dst) {
                memset(&g, 0, sizeof g);
                g.tb = 1; g.M = M; g.N = Kr; g.K = N;
                g.A = pg; g.lda = N; g.B = pw; g.ldb = N; g.C = dst; g.ldc = Kr;
                g.accumulate = acc; g.rule = 1;
                if (z) { g.mask = pm; g.ldmask = Kr; }
                tt_gemm(&g);
            }
        }
        return;
    }
    const int K = (int)a->val->shape[1];
    if (a->requires_grad) {
        const float *pb = tt_dev_ro(b->val);
        int acc;
        float *dst = pb ? grad_target(a, &acc) : nullptr;
        if (dst) {
            memset(&g, 0, sizeof g);
            g.tb = 1; g.M = M; g.N = K; g.K = N;
            g.A = pg; g.lda = N; g.B = pb; g.ldb = N; g.C = dst; g.ldc = K;
            g.accumulate = acc; g.rule = 1;
            tt_gemm(&g);
        }
    }
    if (b->requires_grad) {
        const float *pa = tt_dev_ro(a->val);
        int acc;
        float *dst = pa ? grad_target(b, &acc) : nullptr;
        if (dst) {
            memset(&g, 0, sizeof g);
            g.ta = 1; g.M = K; g.N = N; g.K = M;
            g.A = pa; g.lda = K; g.B = pg; g.ldb = N; g.C = dst; g.ldc = N;
            g.accumulate = acc; g.rule = 1;
            tt_gemm(&g);
        }
    }
}

static void bw_relu(AGNode *n) {             /* src/autograd.c:318-327, fused with the += */
    AGNode *p = n->parents[0];
    if (!p->requires_grad) return;
    /* x > 0 exactly when relu(x) > 0: a pre-activation that was never stored is not produced for this */
    const Tensor *m = tt_is_deferred_matmul(p->val) ? n->val : p->val;
    const float *px = tt_dev_ro(m), *pg = tt_dev_ro(n->grad);
    if (!px || !pg) return;
    int acc;
    float *dst = grad_target(p, &acc);
    if (dst) k_relu_bwd(dst, px, pg, p->val->numel, acc);
}

static void bw_softmax(AGNode *n) {          /* src/autograd.c:329-346 */
    take(n->parents[0], ttb_softmax_bwd(n->val, n->grad));
}

static void bw_padones(AGNode *n) {          /* src/autograd.c:348-359 */
    AGNode *p = n->parents[0];
    if (!p->requires_grad) return;
    const float *pg = tt_dev_ro(n->grad);
    if (!pg) return;
    int acc;
    float *dst = grad_target(p, &acc);
    const int M = (int)p->val->shape[0], K = (int)p->val->shape[1];
    if (dst) k_slice_cols(dst, pg, M, K, K + 1, acc);
}

static void bw_reshape(AGNode *n) {          /* src/autograd.c:361-369 */
    AGNode *p = n->parents[0];
    if (!p->requires_grad) return;
    take(p, tt_reshape(n->grad, p->val->shape, p->val->ndim));
}

/* Convolution backward (src/autograd.c:456-553):
 *   db = sum of g over n, ho, wo
 *   dW = g_perm[F, N*sp] * col^T               (dot-product rule, :439-454)
 *   dX = col2im( W^T[kc,F] * g_perm )           (forward-sgemm rule, :538-541)
 * Each part is skipped when its parent needs no gradient. */
static void bw_conv2d(AGNode *n) {
    AGNode *a = n->parents[0], *w = n->parents[1];
    AGNode *b = n->nparents > 2 ? n->parents[2] : nullptr;
    const int sh = n->params[0], sw = n->params[1], ph = n->params[2], pw = n->params[3];
    const Tensor *g = n->grad;
    const int N = (int)a->val->shape[0], C = (int)a->val->shape[1], H = (int)a->val->shape[2], W = (int)a->val->shape[3];
    const int F = (int)w->val->shape[0], HH = (int)w->val->shape[2], WW = (int)w->val->shape[3];
    if (HH <= 0 || WW <= 0 || sh <= 0 || sw <= 0 || ph < 0 || pw < 0) return;
    const int Ho = (int)g->shape[2], Wo = (int)g->shape[3];
    const long sp = (long)Ho * Wo, ncol = (long)N * sp;
    const int kc = C * HH * WW;
    const float *pg = tt_dev_ro(g);
    if (!pg) return;

    if (b && b->requires_grad) {
        long shp[1] = {F};
        Tensor *gb = tt_new_uninit(shp, 1);
        if (gb) { k_conv_bias_grad(pg, N, F, sp, TT(gb)->dev); take(b, gb); }
    }
    if (!w->requires_grad && !a->requires_grad) return;

    /* implicit GEMMs where the forward pass would have used one: dW and dX straight from the image
     * and the output gradient, no col, d_col or permuted copy of g */
    const ConvGeom cg = {N, C, H, W, F, HH, WW, sh, sw, ph, pw, Ho, Wo};
    const bool implicit = g_tt.conv_implicit && g_tt.gemm_path != 2 && (double)ncol * F * kc >= (double)(1l << 21);
    bool dw_done = !w->requires_grad, dx_done = !a->requires_grad;
    if (implicit && !dw_done && conv_tc_usable(&cg, 0)) {
        const float *px = tt_dev_ro(a->val);
        int acc;
        float *dst = px ? grad_target(w, &acc) : nullptr;
        if (dst) { conv_tc_wgrad(&cg, px, pg, dst, acc); dw_done = true; }      /* a failed launch is reported, not retried another way */
    }
    if (implicit && !dx_done && conv_tc_usable(&cg, 1)) {
        const float *pwt = tt_dev_ro(w->val);
        int acc;
        float *dst = pwt ? grad_target(a, &acc) : nullptr;
        if (dst) { conv_tc_dgrad(&cg, pg, pwt, dst, acc); dx_done = true; }
    }
    if (dw_done && dx_done) return;

    float *gp = (float *)tt_dev_alloc(sizeof(float) * (size_t)F * ncol);
    if (!gp) return;
    k_conv_permute(pg, N, F, sp, gp);
    GemmArgs m;

    if (!dw_done) {
        const float *px = tt_dev_ro(a->val);
        float *col = px ? (float *)tt_dev_alloc(sizeof(float) * (size_t)kc * ncol) : nullptr;
        Tensor *gw = col ? tt_new_like(w->val, 0) : nullptr;
        if (gw) {
            k_im2col(px, N, C, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo, col);
            memset(&m, 0, sizeof m);
            m.tb = 1; m.M = F; m.N = kc; m.K = (int)ncol;
            m.A = gp; m.lda = ncol; m.B = col; m.ldb = ncol; m.C = TT(gw)->dev; m.ldc = kc;
            m.rule = 1;
            if (tt_gemm(&m) == 0) take(w, gw); else tt_release(gw);
        }
        tt_dev_free(col);
    }
    if (!dx_done) {
        const float *pwt = tt_dev_ro(w->val);
        float *dcol = pwt ? (float *)tt_dev_alloc(sizeof(float) * (size_t)kc * ncol) : nullptr;
        Tensor *ga = dcol ? tt_new_like(a->val, 0) : nullptr;
        if (ga) {
            memset(&m, 0, sizeof m);
            m.ta = 1; m.M = kc; m.N = (int)ncol; m.K = F;
            m.A = pwt; m.lda = kc; m.B = gp; m.ldb = ncol; m.C = dcol; m.ldc = ncol;
            m.rule = 0;
            if (tt_gemm(&m) == 0) {
                k_col2im(dcol, N, C, H, W, HH, WW, ph, pw, sh, sw, Ho, Wo, TT(ga)->dev);
                take(a, ga);
            } else {
                tt_release(ga);
            }
        }
        tt_dev_free(dcol);
    }
    tt_dev_free(gp);
}

static void bw_maxpool(AGNode *n) {          /* src/autograd.c:555-594 */
    AGNode *a = n->parents[0];
    if (!a->requires_grad) return;
    take(a, ttb_maxpool_bwd(a->val, n->grad, n->params[0], n->params[1], n->params[2], n->params[3]));
}
static void bw_avgpool(AGNode *n) {          /* src/autograd.c:596-628 */
    AGNode *a = n->parents[0];
    if (!a->requires_grad) return;
    const Tensor *v = a->val;
    take(a, ttb_avgpool_bwd(n->grad, (int)v->shape[0], (int)v->shape[1], (int)v->shape[2], (int)v->shape[3],
                            n->params[0], n->params[1], n->params[2], n->params[3]));
}

static void backward_rule(AGNode *n) {
    switch (n->kind) {
        case OP_ADD:       give(n->parents[0], n->grad); give(n->parents[1], n->grad); break;
        case OP_MUL:       bw_mul(n); break;
        case OP_ADDSCALAR: give(n->parents[0], n->grad); break;
        case OP_MULSCALAR: take(n->parents[0], tt_mulscalar(n->grad, n->scalar)); break;
        case OP_MATMUL:    bw_matmul(n); break;
        case OP_RELU:      bw_relu(n); break;
        case OP_SOFTMAX:   bw_softmax(n); break;
        case OP_PADONES:   bw_padones(n); break;
        case OP_RESHAPE:   bw_reshape(n); break;
        case OP_CONV2D:    bw_conv2d(n); break;
        case OP_MAXPOOL2D: bw_maxpool(n); break;
        case OP_AVGPOOL2D: bw_avgpool(n); break;
        default: break;
    }
}

/* ---- ordering and the pass -----------------------------------------------------
 * Post-order by an explicit stack, so a 1000-node chain does not recurse
 * (src/autograd.c:650-680; tests/test_grad.py:271-290). */
typedef struct Order { AGNode **v; size_t n, cap; } Order;
typedef struct Frame { AGNode *node; int next; } Frame;

static int order_push(Order *o, AGNode *x) {
    if (o->n == o->cap) {
        size_t nc = o->cap ? o->cap * 2 : 64;
        AGNode **nv = (AGNode **)realloc(o->v, nc * sizeof(AGNode *));
        if (!nv) return 0;
        o->v = nv; o->cap = nc;
    }
    o->v[o->n++] = x;
    return 1;
}

static int post_order(AGNode *root, Order *out) {
    size_t cap = 64, top = 0;
    Frame *st = (Frame *)malloc(cap * sizeof(Frame));
    if (!st) return 0;
    st[top].node = root; st[top].next = 0; top++;
    root->mark = 1;
    while (top) {
        Frame *f = &st[top - 1];
        if (f->next < f->node->nparents) {
            AGNode *p = f->node->parents[f->next++];
            if (p->mark) continue;
            if (top == cap) {
                Frame *ns = (Frame *)realloc(st, 2 * cap * sizeof(Frame));
                if (!ns) { free(st); return 0; }
                st = ns; cap *= 2;
            }
            p->mark = 1;
            st[top].node = p; st[top].next = 0; top++;
        } else {
            if (!order_push(out, f->node)) { free(st); return 0; }
            top--;
        }
    }
    free(st);
    return 1;
}

/* seed_host / seed_dev: at most one is set; neither means ones. */
static void run_backward(AGNode *out, const float *seed_host, const Tensor *seed_dev) {
    Order ord = {nullptr, 0, 0};
    if (!post_order(out, &ord)) {
        for (size_t i = 0; i < ord.n; i++) ord.v[i]->mark = 0;
        free(ord.v);
        return;
    }
    /* the root's value is observable once the pass has run: a product still deferred is launched now */
    if (tt_is_deferred_matmul(out->val)) tt_dev_ro(out->val);
    /* d(out) is OVERWRITTEN by the seed (src/autograd.c:711-719).  A seed that already is a device
     * tensor is shared instead of copied: nothing ever adds into the root's gradient (it has no
     * consumer in its own graph), and a later pass replaces the shared tensor instead of writing it. */
    if (out->grad && out->grad_is_seed) { tt_release(out->grad); out->grad = nullptr; out->grad_is_seed = 0; }
    float *pd = nullptr;
    if (seed_dev && !out->grad && out->nparents > 0 && !out->is_param && out->sgd_lr <= 0.0f && tt_dev_ro(seed_dev)) {
        out->grad = tt_retain((Tensor *)seed_dev);
        out->grad_is_seed = 1;
    } else {
        if (!out->grad) out->grad = tt_new_like(out->val, 0);
        pd = out->grad ? tt_dev_rw(out->grad) : nullptr;
    }
    if (pd || out->grad_is_seed) {
        const long numel = out->val->numel;
        int seeded = 1;
        if (out->grad_is_seed) {
            /* shared */
        } else if (seed_host) {
            seeded = tt_cuda_ok(cudaMemcpyAsync(pd, seed_host, sizeof(float) * (size_t)numel,
                                                cudaMemcpyHostToDevice, g_tt.stream), "cudaMemcpyAsync(seed)");
        } else if (seed_dev) {
            const float *ps = tt_dev_ro(seed_dev);
            if (ps) k_copy(pd, ps, numel); else seeded = 0;
        } else {
            k_fill(pd, numel, 1.0f);
        }
        if (seeded) {
            for (size_t i = 0; i < ord.n; i++) { ord.v[i]->pending = 0; ord.v[i]->reduced_in_rule = 0; }
            for (size_t i = 0; i < ord.n; i++)
                for (int k = 0; k < ord.v[i]->nparents; k++) ord.v[i]->parents[k]->pending++;
            for (size_t i = ord.n; i-- > 0;) {
                AGNode *n = ord.v[i];
                if (n->grad && n->nparents > 0) backward_rule(n);
                for (int k = 0; k < n->nparents; k++) {
                    AGNode *p = n->parents[k];
                    if (--p->pending == 0 && p->grad && p->reduced_in_rule != 1 && (p->is_param || p->sgd_lr > 0.0f))
                        param_grad_ready(p, 0, p->grad->numel, p->reduced_in_rule == 2 ? PARAM_UPDATE : PARAM_REDUCE | PARAM_UPDATE);
                }
            }
        }
    }
    for (size_t i = 0; i < ord.n; i++) ord.v[i]->mark = 0;
    free(ord.v);
}

extern "C" void ag_backward_from(AGNode *out, const float *seed, size_t seed_numel) {
    if (!out || !out->requires_grad) return;
    if (seed && (!out->val || seed_numel != (size_t)out->val->numel)) return;
    run_backward(out, seed, nullptr);
}
extern "C" void ag_backward(AGNode *out) { ag_backward_from(out, nullptr, 0); }

extern "C" int ag_backward_from_tensor(AGNode *out, const Tensor *seed) {
    if (!out || !seed || !out->val || seed->numel != out->val->numel) {
        tt_set_error("ag_backward_from_tensor: seed does not match the node");
        return -1;
    }
    if (!out->requires_grad) return 0;
    run_backward(out, nullptr, seed);
    return 0;
}

/* ---- lifetime (src/autograd.c:731-745), without recursion -------------------*/
extern "C" AGNode *ag_retain(AGNode *n) {
    if (!n) return nullptr;
    n->refcount++;
    return n;
}

extern "C" void ag_release(AGNode *n) {
    if (!n) return;
    size_t cap = 16, top = 0;
    AGNode **st = (AGNode **)malloc(cap * sizeof(AGNode *));
    if (!st) return;
    st[top++] = n;
    while (top) {
        AGNode *x = st[--top];
        if (--x->refcount > 0) continue;
        tt_release(x->val);
        tt_release(x->grad);
        for (int i = 0; i < x->nparents; i++) {
            if (top == cap) {
                AGNode **ns = (AGNode **)realloc(st, 2 * cap * sizeof(AGNode *));
                if (!ns) { free(st); return; }
                st = ns; cap *= 2;
            }
            st[top++] = x->parents[i];
        }
        free(x);
    }
    free(st);
}
