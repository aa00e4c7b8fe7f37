"""Seeded synthetic inputs and training steps for the benchmark configurations.

The reference's own workloads are its gate scripts (tests/gate_mnist_mlp.py,
tests/gate_cifar_cnn.py), which download MNIST / CIFAR-10.  Neither dataset is
available offline, so the inputs here are seeded synthetic tensors with the
same shapes and value ranges; the graphs are the gate scripts' graphs.

Every step function takes the namespace returned by ``api.bind`` and uses only
``Node``/``Tensor``, so the same code drives this library and, in the tests,
a CPU build of the reference.  The ``*_reference_style`` steps follow the gate
scripts literally (softmax value to NumPy, loss and seed in NumPy, gradients
back to NumPy, SGD in NumPy); the trainer classes keep parameters, the loss
and the optimiser on the device and are what the benchmark times.
"""
import math

import numpy as np


# --------------------------------------------------------------------------- inputs
def kaiming_uniform(rng, fan_in, shape):
    """U(-b, b) with b = sqrt(6 / fan_in), drawn in float64 and cast to fp32."""
    b = math.sqrt(6.0 / fan_in)
    return rng.uniform(-b, b, size=shape).astype(np.float32)


def dense_weight(rng, fan_in, fan_out):
    """[fan_in + 1, fan_out]: Kaiming-uniform rows plus a zero bias row (the
    reference folds biases into the weight via a ones column, src/autograd.c:195-212)."""
    w = np.zeros((fan_in + 1, fan_out), dtype=np.float32)
    w[:fan_in] = kaiming_uniform(rng, fan_in, (fan_in, fan_out))
    return w


def config_mlp_small():
    """MLP 784 -> 256 (relu) -> 10, batch 128, seed 0."""
    rng = np.random.default_rng(0)
    x = rng.random((128, 784)).astype(np.float32)
    y = rng.integers(0, 10, size=128)
    ws = [dense_weight(rng, 784, 256), dense_weight(rng, 256, 10)]
    return x, y, ws


def config_gemm(n=1024, seed=1):
    """Isolated GEMM forward + backward: A, B, dC ~ N(0,1), square n."""
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((n, n)).astype(np.float32)
    b = rng.standard_normal((n, n)).astype(np.float32)
    dc = rng.standard_normal((n, n)).astype(np.float32)
    return a, b, dc


def config_gemm_shape(m, k, n, seed=4):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    dc = rng.standard_normal((m, n)).astype(np.float32)
    return a, b, dc


GEMM_SWEEP = [(s, s, s) for s in (256, 512, 1024, 2048, 4096, 8192)] + \
             [(32, 4096, 4096), (64, 4096, 4096), (128, 4096, 4096), (256, 16384, 16384)]


def config_cnn(batch=256):
    """CNN of the benchmark: conv3x3 3->32 p1, relu, pool2, conv3x3 32->64 p1,
    relu, pool2, flatten 4096, fc 4096->256 relu, fc 256->10; seed 2."""
    rng = np.random.default_rng(2)
    x = rng.standard_normal((batch, 3, 32, 32)).astype(np.float32)
    y = rng.integers(0, 10, size=batch)
    p = {
        "w1": kaiming_uniform(rng, 27, (32, 3, 3, 3)), "b1": np.zeros(32, np.float32),
        "w2": kaiming_uniform(rng, 288, (64, 32, 3, 3)), "b2": np.zeros(64, np.float32),
        "fc1": dense_weight(rng, 4096, 256), "fc2": dense_weight(rng, 256, 10),
    }
    return x, y, p


MLP_LARGE_DIMS = (4096, 4096, 4096, 4096, 1000)


def config_mlp_large(batch=8192, dims=MLP_LARGE_DIMS, seed=3):
    """Large data-parallel MLP 4096 -> 4096 -> 4096 -> 4096 -> 1000, global batch 8192."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((batch, dims[0])).astype(np.float32)
    y = rng.integers(0, dims[-1], size=batch)
    ws = [dense_weight(rng, dims[i], dims[i + 1]) for i in range(len(dims) - 1)]
    return x, y, ws


def mlp_flops_per_sample(dims, observable=True):
    """Algorithmic fwd+bwd FLOPs per sample (2 per multiply-add).  Forward and dW
    for every layer; dX for every layer but the first, whose input needs no
    gradient (the reference computes and discards it, src/autograd.c:308-316)."""
    total = 0
    for i in range(len(dims) - 1):
        k, n = dims[i] + 1, dims[i + 1]
        total += 2 * k * n * 2
        if i > 0 or not observable:
            total += 2 * k * n
    return total


def onehot(y, classes):
    o = np.zeros((y.shape[0], classes), dtype=np.float32)
    o[np.arange(y.shape[0]), y] = 1.0
    return o


# ----------------------------------------------------------------- gate-script style
def mlp_step_reference_style(ns, x, y, ws, lr=0.1, global_batch=None, return_pre=False):
    """One forward + backward + SGD step exactly as tests/gate_mnist_mlp.py:104-126
    runs it (plain SGD instead of momentum).  Returns loss, gradients, new weights;
    with return_pre also the pre-activations of the hidden layers."""
    Node = ns.Node
    batch = x.shape[0]
    gb = global_batch or batch
    nodes = []

    def keep(n):
        nodes.append(n)
        return n

    wn = [keep(Node.leaf(w, True)) for w in ws]
    h = keep(Node.leaf(x, False))
    pre_nodes = []
    for i, w in enumerate(wn):
        h = keep(keep(h.padones()).matmul(w))
        if i + 1 < len(wn):
            pre_nodes.append(h)
            h = keep(h.relu())
    logits = h
    probs = keep(logits.softmax())
    p = probs.value()
    loss = float(-np.log(np.maximum(p[np.arange(batch), y], 1e-12)).mean())
    logits.backward((p - onehot(y, p.shape[1])) / gb)
    grads = [w.grad() for w in wn]
    logits_v = logits.value()
    pre = [n.value() for n in pre_nodes] if return_pre else None
    for n in nodes:
        n.release()
    new_ws = [w - np.float32(lr) * g for w, g in zip(ws, grads)]
    return {"loss": loss, "logits": logits_v, "probs": p, "grads": grads, "weights": new_ws, "pre": pre}


def cnn_forward(ns, keep, xn, pn, pre=None):
    h = keep(xn.conv2d(pn["w1"], pn["b1"], stride=1, pad=1))
    if pre is not None:
        pre["z1"] = h
    h = keep(h.relu())
    h = keep(h.maxpool2d(2, 2))
    h = keep(h.conv2d(pn["w2"], pn["b2"], stride=1, pad=1))
    if pre is not None:
        pre["z2"] = h
    h = keep(h.relu())
    return keep(h.maxpool2d(2, 2))


def cnn_step_reference_style(ns, x, y, params, global_batch=None, return_pre=False):
    """One forward + backward of the benchmark CNN in the style of
    tests/gate_cifar_cnn.py:101-111,160-185.  Returns loss, logits and the
    gradient of every parameter; with return_pre also the three pre-activations."""
    Node = ns.Node
    batch = x.shape[0]
    gb = global_batch or batch
    nodes = []

    def keep(n):
        nodes.append(n)
        return n

    pn = {k: keep(Node.leaf(v, True)) for k, v in params.items()}
    xn = keep(Node.leaf(x, False))
    pre_nodes = {} if return_pre else None
    h = cnn_forward(ns, keep, xn, pn, pre_nodes)
    h = keep(h.reshape((batch, int(np.prod(h.value_tensor().shape[1:])))))
    h = keep(keep(h.padones()).matmul(pn["fc1"]))
    if return_pre:
        pre_nodes["z3"] = h
    h = keep(h.relu())
    logits = keep(keep(h.padones()).matmul(pn["fc2"]))
    probs = keep(logits.softmax())
    p = probs.value()
    loss = float(-np.log(np.maximum(p[np.arange(batch), y], 1e-12)).mean())
    logits.backward((p - onehot(y, p.shape[1])) / gb)
    grads = {k: n.grad() for k, n in pn.items()}
    logits_v = logits.value()
    pre = {k: n.value() for k, n in pre_nodes.items()} if return_pre else None
    for n in nodes:
        n.release()
    return {"loss": loss, "logits": logits_v, "grads": grads, "pre": pre}


def gemm_fwd_bwd(ns, a, b, dc):
    """C = A*B through the autograd path, then dA = dC*B^T and dB = A^T*dC
    (src/autograd.c:168-171, 308-316)."""
    Node = ns.Node
    an, bn = Node.leaf(a, True), Node.leaf(b, True)
    c = an.matmul(bn)
    c.backward(dc)
    out = {"c": c.value(), "da": an.grad(), "db": bn.grad()}
    for n in (c, an, bn):
        n.release()
    return out


# ----------------------------------------------------------------- device-resident
class MLPTrainer:
    """Data-parallel MLP training with everything on the device: persistent
    parameter leaves, fused softmax-cross-entropy seed, SGD kernel, and (when the
    library has a communicator) gradient all-reduce overlapped with backward.

    Needs the additive entry points, i.e. this library, not the reference."""

    def __init__(self, ns, ws, lr=0.1, global_batch=None, fused_sgd=True):
        if not ns.has_ext:
            raise RuntimeError("MLPTrainer needs the ttb_* entry points")
        self.ns = ns
        self.lr = float(lr)
        self.global_batch = global_batch
        self.fused_sgd = fused_sgd
        self.params = []
        for w in ws:
            n = ns.Node.leaf(w, True)
            n.mark_param(True)
            if fused_sgd:
                n.param_sgd(lr)       # the update rides behind each gradient's all-reduce
            self.params.append(n)
        self.dims = tuple([ws[0].shape[0] - 1] + [w.shape[1] for w in ws])

    def step(self, x_t, y_t):
        """x_t: Tensor [b, d0]; y_t: Tensor [b] of class indices as fp32.
        Returns the 1-element loss Tensor (still on the device)."""
        ns = self.ns
        batch = x_t.shape[0]
        gb = self.global_batch or batch
        nodes = []
        h = ns.Node.from_tensor(x_t, False)
        nodes.append(h)
        for i, w in enumerate(self.params):
            p = h.padones(); nodes.append(p)
            h = p.matmul(w); nodes.append(h)
            if i + 1 < len(self.params):
                h = h.relu(); nodes.append(h)
        loss, dlogits = ns.softmax_xent(h.value_tensor(), y_t, 1.0 / gb)
        h.backward(dlogits)
        ns.status(ns.LIB.ttb_dist_join(), "ttb_dist_join")
        for w in self.params:
            if not self.fused_sgd:
                ns.sgd_step(w.value_tensor(), w.grad_tensor(), self.lr)
            w.zero_grad()
        dlogits.release()
        for n in nodes:
            n.release()
        return loss

    def evaluate(self, x_t, y_t):
        """How many rows of the batch the model classifies as their label: the forward graph of
        step() in forward-only mode (no graph recorded, every activation freed as soon as the next
        layer has consumed it, relu inside the GEMM epilogues) and the arg-max / hit count on the
        device -- evaluate() of tests/gate_mnist_mlp.py:74-80 without the logits leaving the GPU."""
        ns = self.ns
        with ns.no_grad():
            h = ns.Node.from_tensor(x_t, False)
            for i, w in enumerate(self.params):
                p = h.padones()
                z = p.matmul(w)
                h.release(); p.release()
                if i + 1 < len(self.params):
                    h = z.relu()
                    z.release()
                else:
                    h = z
            correct = ns.argmax_correct(h.value_tensor(), y_t)
            h.release()
        return correct

    def weights(self):
        return [w.value() for w in self.params]

    def close(self):
        for w in self.params:
            w.release()
        self.params = []


class CNNTrainer:
    """The benchmark CNN with everything on the device: persistent parameter leaves, the
    convolutions, pools and dense layers of cnn_step_reference_style, fused
    softmax-cross-entropy seed and SGD kernels.  Same arithmetic as the host-fed step; what
    it leaves out is the per-step upload of every parameter and download of every gradient
    that the reference's CIFAR gate does (tests/gate_cifar_cnn.py:160-185)."""

    ORDER = ("w1", "b1", "w2", "b2", "fc1", "fc2")

    def __init__(self, ns, params, lr=0.01, global_batch=None):
        if not ns.has_ext:
            raise RuntimeError("CNNTrainer needs the ttb_* entry points")
        self.ns = ns
        self.lr = float(lr)
        self.global_batch = global_batch
        self.pn = {}
        for k in self.ORDER:
            n = ns.Node.leaf(params[k], True)
            n.mark_param(True)
            self.pn[k] = n

    def step(self, x_t, y_t):
        """x_t: Tensor [b, 3, 32, 32]; y_t: Tensor [b] of class indices as fp32.
        Returns the 1-element loss Tensor (still on the device)."""
        ns = self.ns
        batch = x_t.shape[0]
        gb = self.global_batch or batch
        nodes = []

        def keep(n):
            nodes.append(n)
            return n

        xn = keep(ns.Node.from_tensor(x_t, False))
        h = cnn_forward(ns, keep, xn, self.pn)
        h = keep(h.reshape((batch, int(np.prod(h.value_tensor().shape[1:])))))
        h = keep(keep(h.padones()).matmul(self.pn["fc1"]))
        h = keep(h.relu())
        logits = keep(keep(h.padones()).matmul(self.pn["fc2"]))
        loss, dlogits = ns.softmax_xent(logits.value_tensor(), y_t, 1.0 / gb)
        logits.backward(dlogits)
        ns.status(ns.LIB.ttb_dist_join(), "ttb_dist_join")
        for w in self.pn.values():
            ns.sgd_step(w.value_tensor(), w.grad_tensor(), self.lr)
            w.zero_grad()
        dlogits.release()
        for n in nodes:
            n.release()
        return loss

    def grads_after(self, x_t, y_t):
        """Gradients of one step without the update (for tests): dict of arrays."""
        lr, self.lr = self.lr, 0.0
        ns = self.ns
        batch = x_t.shape[0]
        gb = self.global_batch or batch
        nodes = []

        def keep(n):
            nodes.append(n)
            return n

        xn = keep(ns.Node.from_tensor(x_t, False))
        h = cnn_forward(ns, keep, xn, self.pn)
        h = keep(h.reshape((batch, int(np.prod(h.value_tensor().shape[1:])))))
        h = keep(keep(h.padones()).matmul(self.pn["fc1"]))
        h = keep(h.relu())
        logits = keep(keep(h.padones()).matmul(self.pn["fc2"]))
        loss, dlogits = ns.softmax_xent(logits.value_tensor(), y_t, 1.0 / gb)
        logits.backward(dlogits)
        ns.status(ns.LIB.ttb_dist_join(), "ttb_dist_join")
        out = {k: w.grad() for k, w in self.pn.items()}
        out["loss"] = float(loss.to_np()[0])
        for w in self.pn.values():
            w.zero_grad()
        dlogits.release(); loss.release()
        for n in nodes:
            n.release()
        self.lr = lr
        return out

    def weights(self):
        return {k: w.value() for k, w in self.pn.items()}

    def close(self):
        for w in self.pn.values():
            w.release()
        self.pn = {}

