"""What sits either side of the GEMMs in a training step, fused or moved onto the device:
relu and its gradient mask inside the GEMM epilogues (src/ops.c:55-69,104-106 and
src/autograd.c:318-327 of the reference, folded into the products next to them),
forward-only evaluation batches with the arg-max on the device
(tests/gate_mnist_mlp.py:74-80), and the normalise + gather stage of the input pipeline
(tests/gate_mnist_mlp.py:86-90,107-111; tests/gate_cifar_cnn.py:162-163).  Everything here
is elementwise or index work on top of a product, so fused and literal results are compared
bit for bit."""
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import rel_err
from tinytorch_b200 import workloads as W

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _mlp_graph(tt, x, ws, requires_x=False):
    """x -> (padones -> matmul -> relu) x (n-1) -> padones -> matmul; returns (nodes by name, all nodes)."""
    Node = tt.Node
    keep = []
    wn = [Node.leaf(w, True) for w in ws]
    xn = Node.leaf(x, requires_x)
    keep += wn + [xn]
    h, pre, act = xn, [], []
    for i, w in enumerate(wn):
        p = h.padones(); keep.append(p)
        z = p.matmul(w); keep.append(z)
        if i + 1 < len(wn):
            pre.append(z)
            h = z.relu(); keep.append(h); act.append(h)
        else:
            h = z
    return {"w": wn, "x": xn, "pre": pre, "act": act, "out": h}, keep


LITERAL = r"""
import sys, numpy as np
sys.path.insert(0, sys.argv[1])
import tinytorch_b200
from tinytorch_b200 import workloads as W
tt = tinytorch_b200.default()
d = np.load(sys.argv[2])
ws = [d["w0"], d["w1"], d["w2"]]
Node = tt.Node
wn = [Node.leaf(w, True) for w in ws]
xn = Node.leaf(d["x"], True)
h, pre, act = xn, [], []
for i, w in enumerate(wn):
    z = h.padones().matmul(w)
    if i + 1 < len(wn):
        pre.append(z); h = z.relu(); act.append(h)
    else:
        h = z
h.backward(d["seed"])
out = {"out": h.value(), "gx": xn.grad()}
for i, w in enumerate(wn):
    out["g%d" % i] = w.grad()
for i, (z, a) in enumerate(zip(pre, act)):
    out["z%d" % i] = z.value(); out["a%d" % i] = a.value(); out["gz%d" % i] = z.grad(); out["ga%d" % i] = a.grad()
np.savez(sys.argv[3], **out)
"""


@pytest.mark.parametrize("dims,batch", [((384, 512, 256, 40), 256), ((20, 12, 9, 5), 7)],
                         ids=["tensor-core", "exact-path"])
def test_fused_relu_is_bit_identical_to_the_literal_passes(tt, tmp_path, dims, batch):
    """The same graph with the fusion on (this process) and off (TT_FUSE_RELU=0 in a child
    process, which runs relu and its gradient as separate kernels like the reference does):
    values, pre-activations read back afterwards, and every gradient are equal bit for bit."""
    rng = np.random.default_rng(11)
    x = rng.standard_normal((batch, dims[0])).astype(np.float32)
    ws = [W.dense_weight(rng, dims[i], dims[i + 1]) for i in range(3)]
    for w in ws:
        w[-1] = rng.standard_normal(w.shape[1]).astype(np.float32) * 0.1      # non-zero biases
    seed = rng.standard_normal((batch, dims[-1])).astype(np.float32)
    np.savez(tmp_path / "in.npz", x=x, w0=ws[0], w1=ws[1], w2=ws[2], seed=seed)
    script = tmp_path / "literal.py"
    script.write_text(LITERAL)
    env = dict(os.environ, TT_FUSE_RELU="0")
    r = subprocess.run([sys.executable, str(script), ROOT, str(tmp_path / "in.npz"), str(tmp_path / "lit.npz")],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    lit = np.load(tmp_path / "lit.npz")

    l0 = tt.LIB.ttb_launch_count()
    g, keep = _mlp_graph(tt, x, ws, requires_x=True)
    g["out"].backward(seed)
    fused_launches = tt.LIB.ttb_launch_count() - l0
    assert np.array_equal(g["out"].value(), lit["out"])
    assert np.array_equal(g["x"].grad(), lit["gx"])
    for i, w in enumerate(g["w"]):
        assert np.array_equal(w.grad(), lit["g%d" % i]), i
    for i, (z, a) in enumerate(zip(g["pre"], g["act"])):
        assert np.array_equal(a.value(), lit["a%d" % i])
        assert np.array_equal(z.grad(), lit["gz%d" % i])          # masked in the dX epilogue
        assert a.grad() is None                                   # the relu node was bypassed (documented)
        assert lit["ga%d" % i] is not None
        # the pre-activation was never stored; reading it now launches the plain product
        assert np.array_equal(z.value(), lit["z%d" % i])
        assert np.array_equal(np.maximum(z.value(), 0), a.value())
    for n in keep:
        n.release()
    # 3 forward products + 3 dX + 3 dW (+ column sums, seed): no relu / relu_bwd launches at all
    if dims[0] >= 128:
        tt.LIB.ttb_trace_reset(); tt.LIB.ttb_trace_enable(1)
        g, keep = _mlp_graph(tt, x, ws, requires_x=True)
        g["out"].backward(seed)
        ms, n_elementwise, _ = tt.trace_read(2)
        tt.LIB.ttb_trace_enable(0)
        assert n_elementwise == 0, (n_elementwise, fused_launches)
        for n in keep:
            n.release()


def test_relu_with_two_consumers_or_a_literal_parent_falls_back(tt):
    """The mask fusion only applies when the product is ALL of the relu node's gradient; a relu
    output used twice, and a relu of something that is not a matmul, take the literal rule."""
    rng = np.random.default_rng(12)
    x = rng.standard_normal((64, 128)).astype(np.float32)
    w1, w2, w3 = (W.dense_weight(rng, 128, 128) for _ in range(3))
    Node = tt.Node
    xn, a, b, c = Node.leaf(x, True), Node.leaf(w1, True), Node.leaf(w2, True), Node.leaf(w3, True)
    h = xn.padones().matmul(a).relu()
    y = h.padones().matmul(b) + h.padones().matmul(c)            # h feeds two products
    y.backward(np.ones((64, 128), np.float32))
    z = x.astype(np.float64) @ w1[:-1].astype(np.float64) + w1[-1]
    hv = np.maximum(z, 0)
    ones = np.ones((64, 128))
    gh = ones @ w2[:-1].astype(np.float64).T + ones @ w3[:-1].astype(np.float64).T
    gx = (gh * (z > 0)) @ w1[:-1].astype(np.float64).T
    assert rel_err(h.grad(), gh) <= 1e-4
    assert rel_err(xn.grad(), gx) <= 1e-4
    assert rel_err(h.value(), hv) <= 1e-4
    # relu of a non-matmul
    t = (xn * 2.0).relu()
    t.backward()
    assert np.array_equal(t.value(), np.maximum(x * 2.0, 0).astype(np.float32))


def test_nan_and_inf_through_the_fused_relu(tt):
    """relu(NaN) = 0 with zero gradient, relu(+Inf) = Inf with the gradient passed on
    (src/ops.c:104, src/autograd.c:323-324), also when the mask is taken from the output."""
    x = np.zeros((16, 32), np.float32)
    x[0, 0], x[1, 0], x[2, 0], x[3, 0] = np.nan, np.inf, -np.inf, 1.0
    w = np.zeros((33, 8), np.float32)
    w[0, :] = 1.0
    xn, wn = tt.Node.leaf(x, True), tt.Node.leaf(w, True)
    h = xn.padones().matmul(wn).relu()
    w2 = tt.Node.leaf(np.ones((9, 4), np.float32), True)
    out = h.padones().matmul(w2)
    out.backward(np.ones((16, 4), np.float32))
    hv = h.value()
    assert np.all(hv[0] == 0) and np.all(np.isposinf(hv[1])) and np.all(hv[2] == 0) and np.all(hv[3] == 1)
    gz = xn.grad()           # d/dx[r, 0] = sum over the 8 units of mask * 4
    assert gz[0, 0] == 0 and gz[1, 0] == 32 and gz[2, 0] == 0 and gz[3, 0] == 32 and gz[4, 0] == 0


def test_forward_only_mode_and_device_argmax(tt):
    """Evaluation batches: no graph is recorded, the hit count comes from the device, and it equals
    NumPy's on the logits of the training-mode forward pass."""
    rng = np.random.default_rng(13)
    dims, B = (256, 384, 128, 40), 500
    x = rng.standard_normal((B, dims[0])).astype(np.float32)
    ws = [W.dense_weight(rng, dims[i], dims[i + 1]) for i in range(3)]
    g, keep = _mlp_graph(tt, x, ws)
    logits = g["out"].value()
    for n in keep:
        n.release()
    y = logits.argmax(1).astype(np.int64)
    y[::3] = (y[::3] + 1) % dims[-1]                                # a third of the labels made wrong
    tr = W.MLPTrainer(tt, ws, lr=0.1)
    xt, yt = tt.Tensor.from_np(x), tt.Tensor.from_np(y.astype(np.float32))
    assert tr.evaluate(xt, yt) == int((logits.argmax(1) == y).sum())
    # nothing is recorded: a node built in this mode asks for no gradient and backward is a no-op
    with tt.no_grad():
        n = tt.Node.leaf(x, True).padones().matmul(tt.Node.leaf(ws[0], True))
        assert not n.requires_grad()
        n.backward()
        assert n.grad() is None
    assert tt.LIB.ttb_grad_enabled() == 1
    tr.close(); xt.release(); yt.release()
    # arg-max semantics of NumPy: first maximum, a NaN counts as the maximum
    z = rng.standard_normal((300, 1000)).astype(np.float32)
    z[5, 7] = z[5, 900] = 50.0
    z[6, 3] = np.nan; z[6, 4] = np.nan
    z[7, :] = -np.inf
    zt = tt.Tensor.from_np(z)
    pred = tt.argmax(zt)
    assert np.array_equal(pred.to_np().astype(np.int64), z.argmax(1))
    small = tt.Tensor.from_np(z[:, :10]); ps = tt.argmax(small)
    assert np.array_equal(ps.to_np().astype(np.int64), z[:, :10].argmax(1))
    for t in (zt, pred, small, ps):
        t.release()


@pytest.mark.parametrize("shape,mean,std", [((1000, 1, 28, 28), [0.1307], [0.3081]),
                                            ((600, 3, 32, 32), [0.4914, 0.4822, 0.4465], [0.2023, 0.1994, 0.2010]),
                                            ((50, 2, 3, 5), [0.5, 0.25], [0.5, 2.0])],
                         ids=["mnist-shaped", "cifar-shaped", "odd-sizes"])
def test_gather_normalize_is_bit_identical_to_numpy(tt, shape, mean, std):
    rng = np.random.default_rng(14)
    raw = rng.integers(0, 256, size=shape, dtype=np.uint8)
    idx = rng.permutation(shape[0])[:37]
    m = np.asarray(mean, np.float32).reshape(1, -1, 1, 1)
    s = np.asarray(std, np.float32).reshape(1, -1, 1, 1)
    want = (raw.astype(np.float32)[idx] / np.float32(255.0) - m) / s        # the gate scripts' expression
    assert want.dtype == np.float32
    ds = tt.ByteDataset(raw, mean, std)
    out = tt.Tensor.zeros((37,) + shape[1:])
    ds.batch_into(out, idx)
    assert np.array_equal(out.to_np(), want)
    with pytest.raises(RuntimeError):
        ds.batch_into(out, np.full(37, shape[0]))                           # out of range: refused on the host
    ds.free(); out.release()


def test_release_right_after_an_async_download(tt):
    """The source of ttb_download_async may be released at once: its block is not handed to the
    next allocation before the copy has run."""
    n = 1 << 22
    pin = tt.pinned_array((n,))
    a = np.arange(n, dtype=np.float32)
    for _ in range(3):
        t = tt.Tensor.from_np(a)
        tt.download_async(t, pin)
        t.release()
        clobber = [tt.Tensor.zeros((n,)) for _ in range(2)]                 # same size: would reuse the block
        tt.download_wait()
        assert np.array_equal(pin, a)
        for c in clobber:
            c.release()
