"""NumPy-facing view of the CPU oracle (oracle/tt_oracle.c) plus the two
training steps composed from it.

TEST INFRASTRUCTURE ONLY: the checker for the CUDA path.  Nothing under
``tinytorch_b200/`` imports this module; the test-suite, the smoke check and the
CPU-baseline leg of the benchmark do.

``load_ref()`` returns the reference's own library (compiled from its sources
by oracle/Makefile into oracle/_ref/) bound through the same ctypes wrapper the
product uses, or None when that build is not present.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liboracle.so")
REF_PATH = os.path.join(HERE, "_ref", "libtinytorch_ref.so")

F32P = ctypes.POINTER(ctypes.c_float)
I64P = ctypes.POINTER(ctypes.c_long)
CI, CL, CF = ctypes.c_int, ctypes.c_long, ctypes.c_float
_lib = None


def build():
    """Compile liboracle.so (and oracle/_ref when the reference sources exist)."""
    subprocess.run(["make", "-s", "-C", HERE], check=True)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        _lib = ctypes.CDLL(LIB_PATH)
    return _lib


def load_ref():
    if not os.path.exists(REF_PATH):
        return None
    from tinytorch_b200 import api
    return api.bind(REF_PATH)


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(F32P)


def sgemm(a, b):
    a, b = _f(a), _f(b)
    m, k = a.shape
    n = b.shape[1]
    c = np.zeros((m, n), np.float32)
    lib().orc_sgemm(CI(m), CI(n), CI(k), _p(a), _p(b), _p(c))
    return c


def matmul_naive(a, b):
    a, b = _f(a), _f(b)
    m, k = a.shape
    n = b.shape[1]
    c = np.zeros((m, n), np.float32)
    lib().orc_matmul_naive(CI(m), CI(n), CI(k), _p(a), _p(b), _p(c))
    return c


def matmul_nt(x, y):
    x, y = _f(x), _f(y)
    m, k = x.shape
    n = y.shape[0]
    r = np.zeros((m, n), np.float32)
    lib().orc_matmul_nt(CI(m), CI(n), CL(k), _p(x), _p(y), _p(r))
    return r


def matmul_tn(x, y):
    x, y = _f(x), _f(y)
    k, m = x.shape
    n = y.shape[1]
    r = np.zeros((m, n), np.float32)
    lib().orc_matmul_tn(CI(m), CI(n), CI(k), _p(x), _p(y), _p(r))
    return r


def _map2(name, a, b):
    a, b = _f(a), _f(b)
    o = np.empty_like(a)
    getattr(lib(), name)(CL(a.size), _p(a), _p(b), _p(o))
    return o


def add(a, b):
    return _map2("orc_add", a, b)


def mul(a, b):
    return _map2("orc_mul", a, b)


def addscalar(a, s):
    a = _f(a); o = np.empty_like(a)
    lib().orc_addscalar(CL(a.size), _p(a), CF(s), _p(o))
    return o


def mulscalar(a, s):
    a = _f(a); o = np.empty_like(a)
    lib().orc_mulscalar(CL(a.size), _p(a), CF(s), _p(o))
    return o


def relu(a):
    a = _f(a); o = np.empty_like(a)
    lib().orc_relu(CL(a.size), _p(a), _p(o))
    return o


def relu_bwd(x, g):
    x, g = _f(x), _f(g)
    o = np.empty_like(x)
    lib().orc_relu_bwd(CL(x.size), _p(x), _p(g), _p(o))
    return o


def softmax(x):
    x = _f(x); o = np.empty_like(x)
    n = x.shape[-1]
    lib().orc_softmax(CL(x.size // n), CI(n), _p(x), _p(o))
    return o


def softmax_bwd(s, g):
    s, g = _f(s), _f(g)
    o = np.empty_like(s)
    n = s.shape[-1]
    lib().orc_softmax_bwd(CL(s.size // n), CI(n), _p(s), _p(g), _p(o))
    return o


def padones(x):
    x = _f(x)
    m, k = x.shape
    o = np.empty((m, k + 1), np.float32)
    lib().orc_padones(CI(m), CI(k), _p(x), _p(o))
    return o


def padones_bwd(g):
    g = _f(g)
    m, k1 = g.shape
    o = np.empty((m, k1 - 1), np.float32)
    lib().orc_padones_bwd(CI(m), CI(k1 - 1), _p(g), _p(o))
    return o


def _out_hw(h, w, kh, kw, sh, sw, ph, pw):
    return (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1


def im2col(x, kh, kw, sh, sw, ph, pw):
    x = _f(x)
    n, c, h, w = x.shape
    ho, wo = _out_hw(h, w, kh, kw, sh, sw, ph, pw)
    col = np.empty((c * kh * kw, n * ho * wo), np.float32)
    lib().orc_im2col(_p(x), CI(n), CI(c), CI(h), CI(w), CI(kh), CI(kw), CI(ph), CI(pw), CI(sh), CI(sw), _p(col))
    return col


def col2im(col, n, c, h, w, kh, kw, sh, sw, ph, pw):
    col = _f(col)
    x = np.empty((n, c, h, w), np.float32)
    lib().orc_col2im(_p(col), CI(n), CI(c), CI(h), CI(w), CI(kh), CI(kw), CI(ph), CI(pw), CI(sh), CI(sw), _p(x))
    return x


def conv2d(x, w, b, sh, sw, ph, pw):
    x, w = _f(x), _f(w)
    n, c, h, wi = x.shape
    f, _, kh, kw = w.shape
    ho, wo = _out_hw(h, wi, kh, kw, sh, sw, ph, pw)
    out = np.empty((n, f, ho, wo), np.float32)
    bp = _p(_f(b)) if b is not None else None
    rc = lib().orc_conv2d(_p(x), _p(w), bp, CI(n), CI(c), CI(h), CI(wi), CI(f), CI(kh), CI(kw),
                          CI(sh), CI(sw), CI(ph), CI(pw), _p(out))
    if rc != 0:
        raise MemoryError("orc_conv2d")
    return out


def conv2d_bwd(x, w, g, sh, sw, ph, pw, need_dx=True):
    x, w, g = _f(x), _f(w), _f(g)
    n, c, h, wi = x.shape
    f, _, kh, kw = w.shape
    dx = np.empty_like(x) if need_dx else None
    dw = np.empty_like(w)
    db = np.empty((f,), np.float32)
    rc = lib().orc_conv2d_bwd(_p(x), _p(w), _p(g), CI(n), CI(c), CI(h), CI(wi), CI(f), CI(kh), CI(kw),
                              CI(sh), CI(sw), CI(ph), CI(pw), _p(dx) if need_dx else None, _p(dw), _p(db))
    if rc != 0:
        raise MemoryError("orc_conv2d_bwd")
    return dx, dw, db


def maxpool(x, ph, pw, sh, sw):
    x = _f(x)
    n, c, h, w = x.shape
    ho, wo = (h - ph) // sh + 1, (w - pw) // sw + 1
    o = np.empty((n, c, ho, wo), np.float32)
    lib().orc_maxpool(_p(x), CI(n), CI(c), CI(h), CI(w), CI(ph), CI(pw), CI(sh), CI(sw), _p(o))
    return o


def maxpool_bwd(x, g, ph, pw, sh, sw):
    """Returns (dx, argmax offsets)."""
    x, g = _f(x), _f(g)
    n, c, h, w = x.shape
    dx = np.empty_like(x)
    idx = np.empty(g.shape, np.int64)
    lib().orc_maxpool_bwd(_p(x), _p(g), CI(n), CI(c), CI(h), CI(w), CI(ph), CI(pw), CI(sh), CI(sw),
                          _p(dx), idx.ctypes.data_as(I64P))
    return dx, idx


def avgpool(x, ph, pw, sh, sw):
    x = _f(x)
    n, c, h, w = x.shape
    ho, wo = (h - ph) // sh + 1, (w - pw) // sw + 1
    o = np.empty((n, c, ho, wo), np.float32)
    lib().orc_avgpool(_p(x), CI(n), CI(c), CI(h), CI(w), CI(ph), CI(pw), CI(sh), CI(sw), _p(o))
    return o


def avgpool_bwd(g, n, c, h, w, ph, pw, sh, sw):
    g = _f(g)
    dx = np.empty((n, c, h, w), np.float32)
    lib().orc_avgpool_bwd(_p(g), CI(n), CI(c), CI(h), CI(w), CI(ph), CI(pw), CI(sh), CI(sw), _p(dx))
    return dx


# ------------------------------------------------------------------ composed steps
def _onehot(y, classes):
    o = np.zeros((y.shape[0], classes), np.float32)
    o[np.arange(y.shape[0]), y] = 1.0
    return o


def mlp_step(x, y, ws, lr=0.1, global_batch=None, relu_masks=None):
    """Forward + backward + SGD of x.padones().matmul(w).relu()... with the
    softmax-cross-entropy seed, as the reference executes it through its
    autograd (tests/gate_mnist_mlp.py:104-126, src/autograd.c:308-359).

    relu_masks (one boolean array per hidden layer) replaces `pre > 0` in the
    backward pass.  A test that compares two implementations whose forward
    values differ in the last bits uses it to take the relu kink out of the
    comparison: a pre-activation within rounding error of zero may land on
    either side, and the derivative jumps there."""
    batch = x.shape[0]
    gb = global_batch or batch
    acts, pre = [], []
    h = _f(x)
    for i, w in enumerate(ws):
        hp = padones(h)
        z = sgemm(hp, w)
        acts.append(hp); pre.append(z)
        h = relu(z) if i + 1 < len(ws) else z
    logits = h
    p = softmax(logits)
    loss = float(-np.log(np.maximum(p[np.arange(batch), y], 1e-12)).mean())
    g = ((p - _onehot(y, p.shape[1])) / gb).astype(np.float32)
    grads = [None] * len(ws)
    for i in reversed(range(len(ws))):
        grads[i] = matmul_tn(acts[i], g)
        if i > 0:
            g = padones_bwd(matmul_nt(g, ws[i]))
            gate = pre[i - 1] if relu_masks is None else np.where(relu_masks[i - 1], 1.0, -1.0).astype(np.float32)
            g = relu_bwd(gate, g)
    new_ws = [w - np.float32(lr) * gw for w, gw in zip(ws, grads)]
    return {"loss": loss, "logits": logits, "probs": p, "grads": grads, "weights": new_ws, "pre": pre[:-1]}


def cnn_step(x, y, params, global_batch=None, forward=None):
    """Forward + backward of the benchmark CNN (graph of tests/gate_cifar_cnn.py:101-111
    with two conv blocks) through the oracle's operators.

    forward (dict with z1, z2, z3, logits) evaluates the BACKWARD pass at somebody
    else's forward values instead of the oracle's own.  relu and max-pool are not
    differentiable where a pre-activation is zero or two window entries tie; two
    implementations whose forward values differ in the last bits take different
    branches there.  A test first shows that the forward values agree, then
    compares gradients at the same point."""
    batch = x.shape[0]
    gb = global_batch or batch
    z1 = conv2d(x, params["w1"], params["b1"], 1, 1, 1, 1)
    a1 = relu(z1)
    p1 = maxpool(a1, 2, 2, 2, 2)
    z2 = conv2d(p1, params["w2"], params["b2"], 1, 1, 1, 1)
    a2 = relu(z2)
    p2 = maxpool(a2, 2, 2, 2, 2)
    flat = p2.reshape(batch, -1)
    f1 = padones(flat)
    z3 = sgemm(f1, params["fc1"])
    a3 = relu(z3)
    f2 = padones(a3)
    logits = sgemm(f2, params["fc2"])
    p = softmax(logits)
    loss = float(-np.log(np.maximum(p[np.arange(batch), y], 1e-12)).mean())
    own = {"z1": z1, "z2": z2, "z3": z3}
    if forward is not None:
        z1, z2, z3 = _f(forward["z1"]), _f(forward["z2"]), _f(forward["z3"])
        a1 = relu(z1); p1 = maxpool(a1, 2, 2, 2, 2)
        a2 = relu(z2); p2 = maxpool(a2, 2, 2, 2, 2)
        f1 = padones(p2.reshape(batch, -1))
        f2 = padones(relu(z3))
        p = softmax(_f(forward["logits"]))
    g = ((p - _onehot(y, p.shape[1])) / gb).astype(np.float32)
    grads = {}
    grads["fc2"] = matmul_tn(f2, g)
    g = relu_bwd(z3, padones_bwd(matmul_nt(g, params["fc2"])))
    grads["fc1"] = matmul_tn(f1, g)
    g = padones_bwd(matmul_nt(g, params["fc1"])).reshape(p2.shape)
    g, _ = maxpool_bwd(a2, g, 2, 2, 2, 2)
    g = relu_bwd(z2, g)
    g, grads["w2"], grads["b2"] = conv2d_bwd(p1, params["w2"], g, 1, 1, 1, 1, need_dx=True)
    g, _ = maxpool_bwd(a1, g, 2, 2, 2, 2)
    g = relu_bwd(z1, g)
    _, grads["w1"], grads["b1"] = conv2d_bwd(x, params["w1"], g, 1, 1, 1, 1, need_dx=False)
    return {"loss": loss, "logits": logits, "grads": grads, "pre": own}


def gemm_fwd_bwd(a, b, dc):
    return {"c": sgemm(a, b), "da": matmul_nt(dc, b), "db": matmul_tn(a, dc)}
