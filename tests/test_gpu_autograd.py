"""The reference's autograd gate (its tests/test_grad.py) against the CUDA
library: central-difference gradient checks of every operator, the seed-size
contract, graph stress and accumulation semantics, plus comparison of every
backward rule with the fixtures produced by the reference library."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL, ATOL, H = 1e-4, 1e-5, 1e-2          # tests/test_grad.py:13-15


def gradcheck(tt, build, arrays, atol=ATOL):
    Node = tt.Node
    probe_nodes = [Node.leaf(a.copy(), False) for a in arrays]
    probe = build(*probe_nodes)
    out_shape = probe.value().shape
    probe.release()
    for n in probe_nodes:
        n.release()
    R = np.random.default_rng(7).standard_normal(out_shape).astype(np.float32)

    def forward(arrs):
        nodes = [Node.leaf(a.copy(), True) for a in arrs]
        out = build(*nodes)
        val = float(np.sum(R * out.value(), dtype=np.float64))
        return val, nodes, out

    _, nodes, out = forward(arrays)
    out.backward(R)
    analytic = [n.grad().copy() for n in nodes]
    for n in nodes:
        n.release()
    out.release()
    worst = -np.inf
    for k in range(len(arrays)):
        num = np.zeros(arrays[k].size, np.float64)
        for i in range(arrays[k].size):
            vals = []
            for sign in (+1, -1):
                pert = [x.copy() for x in arrays]
                pert[k].reshape(-1)[i] += sign * H
                v, ns_, o = forward(pert)
                vals.append(v)
                for n in ns_:
                    n.release()
                o.release()
            num[i] = (vals[0] - vals[1]) / (2 * H)
        num = num.reshape(arrays[k].shape)
        viol = np.abs(analytic[k] - num) - RTOL * np.abs(num)
        worst = max(worst, float(viol.max()))
    return worst


def clear(rng, shape):
    """Random values with |x| > 0.05, away from the relu kink (tests/test_grad.py:80-85)."""
    while True:
        x = rng.standard_normal(shape).astype(np.float32)
        if np.abs(x).min() > 0.05:
            return x


CASES = [
    ("add", lambda x, y: x + y, [(4, 3), (4, 3)], ATOL),
    ("mul", lambda x, y: x * y, [(4, 3), (4, 3)], ATOL),
    ("addscalar", lambda x: x + 1.5, [(4, 3)], ATOL),
    ("mulscalar", lambda x: x * (-0.7), [(4, 3)], ATOL),
    ("relu", lambda x: x.relu(), [(4, 3)], ATOL),
    ("matmul", lambda x, w: x.matmul(w), [(4, 3), (3, 5)], ATOL),
    ("softmax", lambda x: x.softmax(), [(4, 5)], ATOL),
    ("padones", lambda x: x.padones(), [(4, 3)], ATOL),
    ("padones_matmul", lambda x, w: x.padones().matmul(w), [(4, 3), (4, 5)], ATOL),
    ("reshape", lambda x: x.reshape((2, 6)), [(3, 4)], ATOL),
    ("conv2d", lambda x, w, b: x.conv2d(w, b, stride=1, pad=1), [(2, 2, 5, 5), (3, 2, 3, 3), (3,)], 2e-4),
    ("maxpool2d", lambda x: x.maxpool2d(pool_size=2, stride=2), [(2, 2, 6, 6)], ATOL),
    ("avgpool2d", lambda x: x.avgpool2d(pool_size=2, stride=2), [(2, 2, 6, 6)], ATOL),
    ("composite", lambda x, w: ((x.matmul(w) * 0.5).relu() + 0.1).softmax(), [(4, 3), (3, 6)], ATOL),
]


@pytest.mark.parametrize("name,build,shapes,atol", CASES, ids=[c[0] for c in CASES])
def test_gradcheck(tt, name, build, shapes, atol):
    import zlib
    rng = np.random.default_rng(zlib.crc32(name.encode()) % 1000)
    arrays = [clear(rng, s) for s in shapes]
    worst = gradcheck(tt, build, arrays, atol)
    assert worst < atol, f"{name}: violation {worst:.3e}"


def _leaf10(tt):
    return tt.Node.leaf(np.arange(1, 11, dtype=np.float32), True)


def test_seed_size_contract(tt):
    """Short and long seeds raise; None seeds ones; other dtypes are coerced
    (tests/test_grad.py:138-268)."""
    x = _leaf10(tt); z = x * 2
    with pytest.raises(ValueError):
        z.backward(np.array([1.0], np.float32))
    with pytest.raises(ValueError):
        z.backward(np.ones(20, np.float32))
    assert x.grad() is None                       # nothing happened
    z.backward(None)
    assert np.all(z.grad() == 1.0) and np.all(x.grad() == 2.0)
    z.release(); x.release()
    for seed in (np.arange(1, 11, dtype=np.float32), np.arange(1, 11, dtype=np.int32),
                 np.arange(1, 11, dtype=np.float64), np.arange(1, 21, dtype=np.float64)[::2]):
        x = _leaf10(tt); z = x * 2
        z.backward(seed)
        assert np.array_equal(x.grad(), 2 * np.asarray(seed, dtype=np.float32))
        z.release(); x.release()
    # the raw C entry point ignores a mismatched seed instead of reading out of bounds
    import ctypes
    x = _leaf10(tt); z = x * 2
    bad = np.ones(3, np.float32)
    tt.LIB.ag_backward_from(z.ptr, bad.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), 3)
    assert x.grad() is None and z.grad() is None
    z.release(); x.release()


def test_deep_chain_does_not_overflow_the_stack(tt):
    v = tt.Node.leaf(np.array([1.0, 2.0], np.float32), True)
    nodes, cur = [v], v
    for _ in range(1000):
        cur = cur + 1.0
        nodes.append(cur)
    cur.backward(None)
    assert np.allclose(v.grad(), 1.0, atol=1e-6)
    assert np.allclose(cur.value(), [1001.0, 1002.0])
    for n in nodes:
        n.release()
    # and releasing only the tail of a long chain unwinds without recursion
    v = tt.Node.leaf(np.array([1.0], np.float32), True)
    cur = v
    for _ in range(20000):
        nxt = cur + 1.0
        cur.release()
        cur = nxt
    cur.release()


def test_second_backward_accumulates_to_three_times(tt, golden_ops):
    x = tt.Node.leaf(np.array([1.0, 2.0, 3.0], np.float32), True)
    y = x * x
    z = y + y
    z.backward(None)
    g1 = x.grad().copy()
    assert np.array_equal(g1, golden_ops["acc_first"]) and np.allclose(g1, [4.0, 8.0, 12.0])
    z.backward(None)
    g2 = x.grad()
    assert np.array_equal(g2, golden_ops["acc_second"]) and np.allclose(g2, 3 * g1)
    for n in (z, y, x):
        n.release()


def test_nan_and_inf_backward(tt):
    x = tt.Node.leaf(np.array([np.nan, 1.0], np.float32), True)
    y = x * x
    y.backward(None)
    assert x.grad().shape == (2,)
    y.release(); x.release()
    x = tt.Node.leaf(np.array([np.inf, -np.inf], np.float32), True)
    r = x.relu()
    r.backward(None)
    assert np.isfinite(x.grad()).all()
    r.release(); x.release()


def test_requires_grad_false_leaves_get_no_gradient(tt):
    a = tt.Node.leaf(np.ones((3, 4), np.float32), False)
    w = tt.Node.leaf(np.ones((4, 2), np.float32), True)
    o = a.matmul(w)
    assert o.requires_grad() and not a.requires_grad()
    o.backward(None)
    assert a.grad() is None and np.all(w.grad() == 3.0)
    q = a.relu()
    q.backward(None)                       # not differentiable: silently nothing
    assert q.grad() is None
    for n in (o, q, a, w):
        n.release()


def _autograd(tt, build, arrays, seed):
    nodes = [tt.Node.leaf(a, True) for a in arrays]
    out = build(*nodes)
    val = out.value()
    out.backward(seed)
    grads = [n.grad() for n in nodes]
    out.release()
    for n in nodes:
        n.release()
    return val, grads


def test_backward_rules_match_reference_fixtures(tt, golden_ops):
    g = golden_ops
    x, y, r = g["ew_x"], g["ew_y"], g["ew_r"]
    v, gr = _autograd(tt, lambda a, b: a + b, [x, y], r)
    assert np.array_equal(v, g["add_out"]) and np.array_equal(gr[0], g["add_gx"]) and np.array_equal(gr[1], g["add_gy"])
    v, gr = _autograd(tt, lambda a, b: a * b, [x, y], r)
    assert np.array_equal(v, g["mul_out"]) and np.array_equal(gr[0], g["mul_gx"]) and np.array_equal(gr[1], g["mul_gy"])
    for name, fn in [("addscalar", lambda a: a + 1.5), ("mulscalar", lambda a: a * (-0.7)), ("relu", lambda a: a.relu()),
                     ("padones", lambda a: a.padones()), ("reshape", lambda a: a.reshape((7, 5)))]:
        v, gr = _autograd(tt, fn, [x], g[f"{name}_seed"])
        assert np.array_equal(v, g[f"{name}_out"]), name
        assert np.array_equal(gr[0], g[f"{name}_gx"]), name
    v, gr = _autograd(tt, lambda a: a.softmax(), [x], g["softmax_seed"])
    assert np.allclose(v, g["softmax_out"], rtol=2e-6, atol=1e-7)
    assert np.allclose(gr[0], g["softmax_gx"], rtol=1e-5, atol=1e-6)
    # matmul forward and both backward products, bit for bit on the exact path
    for i in range(8):
        a, b, s = g[f"mm{i}_a"], g[f"mm{i}_b"], g[f"mm{i}_g"]
        v, gr = _autograd(tt, lambda p, q: p.matmul(q), [a, b], s)
        assert np.array_equal(v, g[f"mm{i}_c"]), i
        assert np.array_equal(gr[0], g[f"mm{i}_da"]), i
        assert np.array_equal(gr[1], g[f"mm{i}_db"]), i


def test_conv_and_pool_rules_match_reference_fixtures(tt, golden_ops):
    g = golden_ops
    for i in range(4):
        n, c, h, w, f, kh, kw, sh, sw, ph, pw = (int(v) for v in g[f"conv{i}_geom"])
        v, gr = _autograd(tt, lambda a, b, c2: a.conv2d(b, c2, stride=(sh, sw), pad=(ph, pw)),
                          [g[f"conv{i}_x"], g[f"conv{i}_w"], g[f"conv{i}_b"]], g[f"conv{i}_g"])
        assert np.array_equal(v, g[f"conv{i}_out"]), i               # exact GEMM chain + bias add
        assert np.array_equal(gr[0], g[f"conv{i}_dx"]), i            # exact GEMM + ordered gather
        assert np.array_equal(gr[1], g[f"conv{i}_dw"]), i            # dot-product rule
        assert np.allclose(gr[2], g[f"conv{i}_db"], rtol=2e-5, atol=1e-5), i   # tree sum vs serial sum
    for i in range(4):
        n, c, h, w, ph, pw, sh, sw = (int(v) for v in g[f"pool{i}_geom"])
        v, gr = _autograd(tt, lambda a: a.maxpool2d((ph, pw), (sh, sw)), [g[f"pool{i}_x"]], g[f"pool{i}_g"])
        assert np.array_equal(v, g[f"pool{i}_max_out"]) and np.array_equal(gr[0], g[f"pool{i}_max_dx"]), i
        v, gr = _autograd(tt, lambda a: a.avgpool2d((ph, pw), (sh, sw)), [g[f"pool{i}_x"]], g[f"pool{i}_g"])
        assert np.array_equal(v, g[f"pool{i}_avg_out"]) and np.array_equal(gr[0], g[f"pool{i}_avg_dx"]), i
    v, gr = _autograd(tt, lambda a: a.maxpool2d(2, 2), [g["pool_nan_x"]], np.ones((1, 1, 2, 2), np.float32))
    assert np.array_equal(v, g["pool_nan_out"]) and np.array_equal(gr[0], g["pool_nan_dx"])


def test_unfused_padones_is_literal(tt, orc):
    """A padones node that is read, or feeds something other than a matmul, is
    materialised and differentiated exactly as the reference does."""
    rng = np.random.default_rng(2)
    x = rng.standard_normal((5, 3)).astype(np.float32)
    seed = rng.standard_normal((5, 4)).astype(np.float32)
    xn = tt.Node.leaf(x, True)
    p = xn.padones()
    assert np.array_equal(p.value(), orc.padones(x))
    q = p * 2.0
    q.backward(seed)
    assert np.array_equal(p.grad(), seed * 2)
    assert np.array_equal(xn.grad(), orc.padones_bwd(seed * 2))
    for n in (q, p, xn):
        n.release()


def test_pybind_module_contract(tt):
    """The pybind11 module keeps the reference's Python surface (src/bindings.cpp:125-150)."""
    import os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "build"))
    try:
        import tinytorch_pybind as m
    except ImportError:
        subprocess.run(["make", "-s", "pybind"], cwd=root, check=True)
        import tinytorch_pybind as m
    a = m.Node.leaf(np.ones((2, 3), np.float32), False)
    b = m.Node.leaf(np.ones((4, 5), np.float32), False)
    with pytest.raises(ValueError):
        a.matmul(b)
    x_np = np.arange(12, dtype=np.float32).reshape(2, 6)
    y = m.Node.leaf(x_np, False).reshape([3, 4])
    assert np.array_equal(np.asarray(y.value()), x_np.reshape(3, 4))
    w = m.Node.leaf(np.full((3, 2), 0.5, np.float32))
    out = (a.matmul(w)).relu()
    out.backward()
    assert np.allclose(np.asarray(w.grad()), 2.0) and a.grad() is None
    c = m.Node.leaf(np.ones((1, 1, 4, 4), np.float32)).conv2d(m.Node.leaf(np.ones((1, 1, 3, 3), np.float32)), pad_h=1, pad_w=1)
    assert np.asarray(c.maxpool2d().value()).shape == (1, 1, 2, 2)
    with pytest.raises(ValueError):
        out.backward(np.ones(5, np.float32))
