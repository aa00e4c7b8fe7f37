"""Parity of every CUDA kernel with the CPU oracle, called through the C ABI.

Bit-exact for copies, index work, elementwise arithmetic and for the exact-fp32
GEMM (which reproduces the reference's accumulation order); a stated tolerance
where the GPU orders a floating-point reduction differently or uses its own
expf.  The golden fixtures (outputs of the reference library itself) are
checked alongside the live oracle."""
import ctypes
import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu

# softmax: CUDA expf (2 ulp) and a tree reduction instead of a sequential sum
SOFT = dict(rtol=2e-6, atol=1e-7)
# reductions in a different order over n terms of size ~1: a few ulp * sqrt(n)
REDUCE = dict(rtol=2e-5, atol=1e-5)
# stated tolerance for fp32 results of the tensor-core path, reduction length <= 8192
TC_TOL = 1e-4


def T(tt, a):
    return tt.Tensor.from_np(a)


def run1(tt, name, a, *args):
    t = T(tt, a)
    o = tt.Tensor(tt.checked(getattr(tt.LIB, name)(t.ptr, *args), name))
    out = o.to_np()
    t.release(); o.release()
    return out


def run2(tt, name, a, b, *args):
    ta, tb = T(tt, a), T(tt, b)
    o = tt.Tensor(tt.checked(getattr(tt.LIB, name)(ta.ptr, tb.ptr, *args), name))
    out = o.to_np()
    ta.release(); tb.release(); o.release()
    return out


SIZES = [(1,), (7,), (8,), (3, 4), (2, 3, 4), (1023,), (4096,), (1 << 20,), (3, 1000, 333), (2, 3, 4, 5, 2, 3)]


@pytest.mark.parametrize("shape", SIZES)
def test_elementwise_bit_exact(tt, orc, shape):
    rng = np.random.default_rng(42)
    x = rng.standard_normal(shape).astype(np.float32)
    y = rng.standard_normal(shape).astype(np.float32)
    assert np.array_equal(run2(tt, "tt_add", x, y), orc.add(x, y).reshape(shape))
    assert np.array_equal(run2(tt, "tt_mul", x, y), orc.mul(x, y).reshape(shape))
    assert np.array_equal(run1(tt, "tt_addscalar", x, 2.5), orc.addscalar(x, 2.5).reshape(shape))
    assert np.array_equal(run1(tt, "tt_mulscalar", x, -0.5), orc.mulscalar(x, -0.5).reshape(shape))
    assert np.array_equal(run1(tt, "tt_relu", x), orc.relu(x).reshape(shape))
    assert np.array_equal(run2(tt, "ttb_relu_bwd", x, y), orc.relu_bwd(x, y).reshape(shape))


def test_elementwise_edge_values(tt, orc):
    x = np.array([np.nan, np.inf, -np.inf, 0.0, -0.0, 1.5, -2.0, 1e-45], np.float32)
    g = np.arange(8, dtype=np.float32) + 1
    assert np.array_equal(run1(tt, "tt_relu", x), orc.relu(x), equal_nan=True)
    got = run2(tt, "ttb_relu_bwd", x, g)
    assert np.array_equal(got, orc.relu_bwd(x, g))
    assert np.isfinite(got).all()                       # relu(NaN / +-Inf) has a finite gradient
    assert np.array_equal(run2(tt, "tt_add", x, x), orc.add(x, x), equal_nan=True)
    assert np.array_equal(run2(tt, "tt_mul", x, x), orc.mul(x, x), equal_nan=True)


def test_shape_errors_return_null(tt):
    a, b, c = T(tt, np.ones((3, 4), np.float32)), T(tt, np.ones((5, 6), np.float32)), T(tt, np.ones((2, 3), np.float32))
    assert not tt.LIB.tt_matmul(a.ptr, b.ptr)
    assert not tt.LIB.tt_matmul_fast(a.ptr, b.ptr)
    assert not tt.LIB.tt_add(a.ptr, c.ptr)
    assert not tt.LIB.tt_mul(a.ptr, c.ptr)
    for t in (a, b, c):
        t.release()


def test_metadata_and_lifecycle(tt):
    import ctypes
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    t = T(tt, x)
    shp, st = (ctypes.c_long * 3)(), (ctypes.c_long * 3)()
    tt.LIB.tt_shape(t.ptr, shp); tt.LIB.tt_strides(t.ptr, st)
    assert list(shp) == [2, 3, 4] and list(st) == [12, 4, 1]
    assert tt.LIB.tt_ndim(t.ptr) == 3 and tt.LIB.tt_numel(t.ptr) == 24
    for _ in range(10000):
        u = tt.LIB.tt_retain(t.ptr)
        assert u
        tt.LIB.tt_release(u)
    z = tt.Tensor.zeros((3, 5))
    assert np.array_equal(z.to_np(), np.zeros((3, 5), np.float32))
    # a reshape is a copy with its own storage and contiguous strides
    r = tt.Tensor(tt.checked(tt.LIB.tt_reshape(t.ptr, (ctypes.c_long * 2)(6, 4), 2), "tt_reshape"))
    assert np.array_equal(r.to_np(), x.reshape(6, 4))
    pa = ctypes.cast(tt.LIB.tt_data(t.ptr), ctypes.c_void_p).value
    pr = ctypes.cast(tt.LIB.tt_data(r.ptr), ctypes.c_void_p).value
    assert pa != pr
    assert tt.LIB.ttb_device_ptr(t.ptr) != tt.LIB.ttb_device_ptr(r.ptr)
    assert not tt.LIB.tt_reshape(t.ptr, (ctypes.c_long * 2)(5, 5), 2)
    for q in (t, z, r):
        q.release()


def test_host_writes_through_tt_data_are_seen(tt):
    """tt_data hands out the mirror; a write through it reaches the next device use."""
    import ctypes
    t = tt.Tensor.zeros((4, 4))
    p = tt.LIB.tt_data(t.ptr)
    host = np.ctypeslib.as_array(p, shape=(16,))
    host[:] = np.arange(16, dtype=np.float32)
    o = tt.Tensor(tt.checked(tt.LIB.tt_mulscalar(t.ptr, 2.0), "tt_mulscalar"))
    assert np.array_equal(o.to_np().reshape(-1), 2 * np.arange(16, dtype=np.float32))
    t.release(); o.release()


def test_async_upload_is_ordered_with_compute(tt):
    """ttb_upload_async overwrites a tensor on the copy stream: work enqueued before the call
    still sees the old contents, work enqueued after sees the new ones."""
    n = 1 << 22
    a = np.full(n, 1.0, np.float32)
    pin = tt.pinned_array((n,))
    t = tt.Tensor.from_np(a)
    outs = []
    for k in range(4):
        before = tt.Tensor(tt.checked(tt.LIB.tt_mulscalar(t.ptr, 2.0), "tt_mulscalar"))   # reads the old payload
        pin[...] = float(k + 10)
        tt.upload_async(t, pin)
        after = tt.Tensor(tt.checked(tt.LIB.tt_mulscalar(t.ptr, 2.0), "tt_mulscalar"))    # must wait for the copy
        want_before = 2.0 if k == 0 else 2.0 * (k + 9)
        assert np.all(before.to_np() == want_before), k
        assert np.all(after.to_np() == 2.0 * (k + 10)), k
        assert np.all(t.to_np() == float(k + 10))
        before.release(); after.release()
    t.release()


@pytest.mark.parametrize("shape", [(5,), (3, 6), (2, 3, 4), (128, 10), (64, 1000), (7, 1031), (4, 5000)])
def test_softmax_forward_backward(tt, orc, shape):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(shape) * 3).astype(np.float32)
    g = rng.standard_normal(shape).astype(np.float32)
    s = run1(tt, "tt_softmax", x)
    want = orc.softmax(x)
    # the reference adds the exponentials one after another, the kernel as a tree:
    # for rows of thousands of terms the two sums drift apart by a few ulp more
    tol = SOFT if shape[-1] <= 1024 else dict(rtol=1e-5, atol=1e-7)
    assert np.allclose(s, want, **tol)
    assert np.allclose(s.sum(-1), 1.0, atol=1e-5)
    assert np.allclose(run2(tt, "ttb_softmax_bwd", want, g), orc.softmax_bwd(want, g), rtol=1e-5, atol=1e-6)


def test_softmax_edges(tt, orc, golden_ops):
    e = golden_ops["softmax_edge_in"]
    got = run1(tt, "tt_softmax", e)
    assert np.all(got[0] == 0.25)                          # all -Inf row -> uniform
    assert np.allclose(got, golden_ops["softmax_edge_out"], **SOFT)
    assert run1(tt, "tt_softmax", np.array([1.0, np.inf, -np.inf, 0.0], np.float32)).shape == (4,)
    big = (np.random.default_rng(1).standard_normal((2, 3, 4)) + 100).astype(np.float32)
    assert np.allclose(run1(tt, "tt_softmax", big), orc.softmax(big), **SOFT)


def test_fused_softmax_xent_matches_the_composite(tt, orc):
    rng = np.random.default_rng(8)
    for rows, n in [(128, 10), (64, 1000), (33, 7)]:
        z = (rng.standard_normal((rows, n)) * 2).astype(np.float32)
        y = rng.integers(0, n, size=rows)
        scale = 1.0 / 256
        p = orc.softmax(z)
        want_loss = float(-np.log(np.maximum(p[np.arange(rows), y], 1e-12)).mean())
        oh = np.zeros_like(p); oh[np.arange(rows), y] = 1
        want_dz = (p - oh) * np.float32(scale)
        zt, yt = T(tt, z), T(tt, y.astype(np.float32))
        loss, dz = tt.softmax_xent(zt, yt, scale)
        assert abs(float(loss.to_np()[0]) - want_loss) < 2e-6 * max(1.0, want_loss)
        assert np.allclose(dz.to_np(), want_dz, rtol=2e-6, atol=1e-9)
        for t in (zt, yt, loss, dz):
            t.release()


GEOMS = [(2, 2, 5, 5, 3, 3, 1, 1, 1, 1), (2, 3, 8, 7, 3, 2, 2, 1, 0, 1), (1, 1, 6, 6, 1, 1, 1, 1, 0, 0),
         (3, 4, 9, 9, 5, 5, 2, 2, 2, 2), (4, 3, 32, 32, 3, 3, 1, 1, 1, 1), (2, 32, 16, 16, 3, 3, 1, 1, 1, 1),
         (1, 2, 7, 5, 2, 3, 3, 1, 4, 0),
         # 3x3 / stride 1 / pad 1 with W in {4, 8, 128}: the shuffle kernels, rows that end inside a warp
         (2, 3, 5, 4, 3, 3, 1, 1, 1, 1), (3, 5, 7, 8, 3, 3, 1, 1, 1, 1), (1, 2, 3, 128, 3, 3, 1, 1, 1, 1),
         (1, 1, 9, 12, 3, 3, 1, 1, 1, 1)]


@pytest.mark.parametrize("geom", GEOMS)
def test_im2col_col2im_bit_exact(tt, orc, geom):
    n, c, h, w, kh, kw, sh, sw, ph, pw = geom
    rng = np.random.default_rng(17)
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    want = orc.im2col(x, kh, kw, sh, sw, ph, pw)
    xt = T(tt, x)
    col = tt.im2col(xt, kh, kw, sh, sw, ph, pw)
    assert np.array_equal(col.to_np(), want)
    d = rng.standard_normal(want.shape).astype(np.float32)
    dt = T(tt, d)
    back = tt.col2im(dt, n, c, h, w, kh, kw, sh, sw, ph, pw)
    assert np.array_equal(back.to_np(), orc.col2im(d, n, c, h, w, kh, kw, sh, sw, ph, pw))
    for t in (xt, col, dt, back):
        t.release()


@pytest.mark.parametrize("shape", [(256, 3, 32, 32), (256, 32, 16, 16)], ids=["conv1", "conv2"])
def test_full_size_im2col_col2im_are_adjoint(tt, shape):
    """The benchmark CNN's two convolutions at batch 256, through properties that need no oracle
    run: im2col only copies (every entry of col is an entry of x or 0, and the centre tap is x
    itself), and col2im is its adjoint: <im2col(x), c> = <x, col2im(c)>."""
    n, c, h, w = shape
    rng = np.random.default_rng(31)
    x = rng.standard_normal(shape).astype(np.float32)
    xt = T(tt, x)
    col_t = tt.im2col(xt, 3, 3, 1, 1, 1, 1)
    col = col_t.to_np()
    assert col.shape == (c * 9, n * h * w)
    centre = col.reshape(c, 9, n, h * w)[:, 4]                              # tap (kh, kw) = (1, 1)
    assert np.array_equal(centre, x.reshape(n, c, h * w).transpose(1, 0, 2))
    corner = col.reshape(c, 9, n, h, w)[:, 0]                               # tap (0, 0): x shifted by one, zero border
    assert np.all(corner[:, :, 0, :] == 0) and np.all(corner[:, :, :, 0] == 0)
    assert np.array_equal(corner[:, :, 1:, 1:], x.transpose(1, 0, 2, 3)[:, :, :-1, :-1])
    d = rng.standard_normal(col.shape).astype(np.float32)
    dt = T(tt, d)
    back = tt.col2im(dt, n, c, h, w, 3, 3, 1, 1, 1, 1).to_np()
    lhs = float(np.dot(col.reshape(-1).astype(np.float64), d.reshape(-1).astype(np.float64)))
    rhs = float(np.dot(x.reshape(-1).astype(np.float64), back.reshape(-1).astype(np.float64)))
    assert abs(lhs - rhs) <= 1e-6 * np.sqrt(col.size)
    # an interior element is the sum of its nine taps, in (kh, kw) order
    d5 = d.reshape(c, 3, 3, n, h, w)
    for (nn, cc, hh, ww) in [(0, 0, 5, 7), (n - 1, c - 1, h - 2, w - 2), (n // 2, c // 2, 1, 1)]:
        acc = np.float32(0)
        for kh in range(3):
            for kw in range(3):
                acc = np.float32(acc + d5[cc, kh, kw, nn, hh + 1 - kh, ww + 1 - kw])
        assert back[nn, cc, hh, ww] == acc
    for t in (xt, col_t, dt):
        t.release()


def test_full_size_maxpool_forward_backward_properties(tt):
    """[256, 32, 32, 32] with 2x2 windows: the forward equals a reshape-max in NumPy exactly; the
    backward puts each window's gradient on the window's (unique) maximum and zero elsewhere."""
    rng = np.random.default_rng(37)
    x = rng.standard_normal((256, 32, 32, 32)).astype(np.float32)
    g = rng.standard_normal((256, 32, 16, 16)).astype(np.float32)
    out = run1(tt, "tt_maxpool2d", x, 2, 2, 2, 2)
    want = x.reshape(256, 32, 16, 2, 16, 2).max(axis=(3, 5))
    assert np.array_equal(out, want)
    xt, gt = T(tt, x), T(tt, g)
    dx = tt.maxpool_bwd(xt, gt, 2, 2, 2, 2).to_np()
    up = lambda a: np.repeat(np.repeat(a, 2, axis=2), 2, axis=3)
    winners = x == up(want)
    assert winners.reshape(256, 32, 16, 2, 16, 2).sum(axis=(3, 5)).max() == 1        # no ties in this draw
    assert np.array_equal(dx, np.where(winners, up(g), np.float32(0)))
    for t in (xt, gt):
        t.release()


def test_full_size_softmax_xent_properties(tt):
    """[8192, 1000] logits of the large MLP: every row of the gradient sums to zero (probabilities
    sum to one, minus the one-hot), the label's entry is the only negative one, the loss equals the
    float64 log-sum-exp form."""
    rng = np.random.default_rng(41)
    z = (rng.standard_normal((8192, 1000)) * 3).astype(np.float32)
    y = rng.integers(0, 1000, size=8192)
    zt, yt = T(tt, z), T(tt, y.astype(np.float32))
    scale = 1.0 / 8192
    loss, dz_t = tt.softmax_xent(zt, yt, scale)
    dz = dz_t.to_np().astype(np.float64)
    assert np.abs(dz.sum(1)).max() <= 5e-6 * scale
    neg = dz < 0
    assert np.array_equal(neg.sum(1), np.ones(8192, dtype=np.int64)) and np.all(neg[np.arange(8192), y])
    z64 = z.astype(np.float64)
    mx = z64.max(1)
    want_loss = float((mx + np.log(np.exp(z64 - mx[:, None]).sum(1)) - z64[np.arange(8192), y]).mean())
    assert abs(float(loss.to_np()[0]) - want_loss) <= 2e-6 * want_loss
    for t in (zt, yt, loss, dz_t):
        t.release()


POOLS = [(2, 2, 6, 6, 2, 2, 2, 2), (2, 3, 7, 9, 3, 2, 1, 2), (1, 2, 5, 5, 3, 3, 1, 1), (2, 2, 8, 8, 2, 2, 3, 3),
         (8, 32, 32, 32, 2, 2, 2, 2), (1, 1, 4, 4, 4, 4, 1, 1), (3, 5, 10, 12, 2, 2, 2, 2)]


@pytest.mark.parametrize("geom", POOLS)
def test_pooling_and_argmax_bit_exact(tt, orc, geom):
    n, c, h, w, ph, pw, sh, sw = geom
    rng = np.random.default_rng(23)
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    x[0, 0, :2, :2] = 0.25                                   # ties
    x.reshape(-1)[::7] = np.round(x.reshape(-1)[::7])        # more ties
    ho, wo = (h - ph) // sh + 1, (w - pw) // sw + 1
    g = rng.standard_normal((n, c, ho, wo)).astype(np.float32)
    assert np.array_equal(run1(tt, "tt_maxpool2d", x, ph, pw, sh, sw), orc.maxpool(x, ph, pw, sh, sw))
    assert np.array_equal(run1(tt, "tt_avgpool2d", x, ph, pw, sh, sw), orc.avgpool(x, ph, pw, sh, sw))
    want_dx, want_idx = orc.maxpool_bwd(x, g, ph, pw, sh, sw)
    xt, gt = T(tt, x), T(tt, g)
    assert np.array_equal(tt.maxpool_argmax(xt, ph, pw, sh, sw), want_idx)
    dx = tt.maxpool_bwd(xt, gt, ph, pw, sh, sw)
    assert np.array_equal(dx.to_np(), want_dx)
    adx = tt.avgpool_bwd(gt, n, c, h, w, ph, pw, sh, sw)
    assert np.array_equal(adx.to_np(), orc.avgpool_bwd(g, n, c, h, w, ph, pw, sh, sw))
    for t in (xt, gt, dx, adx):
        t.release()


def test_maxpool_edge_values(tt):
    """-2e30 and -Inf propagate, an all-NaN window gives -Inf (reference: tests/test_ops.py:551-567)."""
    for fill, want in [(-2e30, np.float32(-2e30)), (-np.inf, -np.inf), (np.nan, -np.inf)]:
        got = run1(tt, "tt_maxpool2d", np.full((1, 1, 4, 4), fill, np.float32), 2, 2, 2, 2)
        assert np.all(got == want)


def test_hostile_spatial_parameters_return_null(tt):
    import ctypes
    from test_abi import CTensor
    a, w = T(tt, np.ones((1, 1, 8, 8), np.float32)), T(tt, np.ones((2, 1, 3, 3), np.float32))
    L = tt.LIB
    assert not L.tt_conv2d(a.ptr, w.ptr, None, 0, 1, 0, 0)
    assert not L.tt_conv2d(a.ptr, w.ptr, None, -1, 1, 0, 0)
    assert not L.tt_conv2d(a.ptr, w.ptr, None, 1, 1, -1, 0)
    mirror = CTensor.from_address(w.ptr)
    assert mirror.ndim == 4 and mirror.shape[2] == 3
    mirror.shape[2] = 0                      # kernel height 0, poked through the public struct
    assert not L.tt_conv2d(a.ptr, w.ptr, None, 1, 1, 0, 0)
    mirror.shape[2] = 3
    assert not L.tt_maxpool2d(a.ptr, 0, 2, 2, 2)
    assert not L.tt_avgpool2d(a.ptr, 2, 2, 0, 2)
    assert not L.tt_maxpool2d(a.ptr, 9, 9, 1, 1)
    bad_bias = T(tt, np.ones((3,), np.float32))
    assert not L.tt_conv2d(a.ptr, w.ptr, bad_bias.ptr, 1, 1, 0, 0)
    for t in (a, w, bad_bias):
        t.release()


MM_SHAPES = [(3, 4, 5), (16, 16, 16), (1, 7, 1), (32, 64, 17), (17, 13, 5), (7, 7, 7), (5, 300, 3), (9, 256, 33),
             (64, 512, 16), (13, 800, 40), (130, 257, 70), (128, 785, 256), (128, 257, 10)]


@pytest.mark.parametrize("shape", MM_SHAPES)
def test_exact_gemm_is_bit_identical_to_the_reference_arithmetic(tt, orc, shape):
    m, k, n = shape
    rng = np.random.default_rng(m * 1000 + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    g = rng.standard_normal((m, n)).astype(np.float32)
    a[0, 0] = 0.0
    tt.LIB.ttb_set_gemm_path(2)
    try:
        assert np.array_equal(run2(tt, "tt_matmul", a, b), orc.matmul_naive(a, b))
        assert np.array_equal(run2(tt, "tt_matmul_fast", a, b), orc.sgemm(a, b))
        assert np.array_equal(run2(tt, "tt_matmul_omp", a, b, 4), orc.sgemm(a, b))
        assert np.array_equal(run2(tt, "ttb_matmul_nt", g, b), orc.matmul_nt(g, b))
        assert np.array_equal(run2(tt, "ttb_matmul_tn", a, g), orc.matmul_tn(a, g))
    finally:
        tt.LIB.ttb_set_gemm_path(0)


def test_exact_gemm_matches_reference_fixtures(tt, golden_ops):
    g = golden_ops
    tt.LIB.ttb_set_gemm_path(2)
    try:
        for i in range(8):
            a, b = g[f"mm{i}_a"], g[f"mm{i}_b"]
            assert np.array_equal(run2(tt, "tt_matmul", a, b), g[f"mm{i}_naive"]), i
            assert np.array_equal(run2(tt, "tt_matmul_fast", a, b), g[f"mm{i}_fast"]), i
            assert np.array_equal(run2(tt, "tt_matmul_omp", a, b, 4), g[f"mm{i}_omp"]), i
    finally:
        tt.LIB.ttb_set_gemm_path(0)


def test_sgemm_rowmajor_host_pointers(tt, orc):
    import ctypes
    rng = np.random.default_rng(4)
    a = rng.standard_normal((20, 33)).astype(np.float32)
    b = rng.standard_normal((33, 18)).astype(np.float32)
    c = np.zeros((20, 18), np.float32)
    F = ctypes.POINTER(ctypes.c_float)
    rc = tt.LIB.tt_sgemm_rowmajor(20, 18, 33, a.ctypes.data_as(F), b.ctypes.data_as(F), c.ctypes.data_as(F), 4)
    assert rc == 0 and np.array_equal(c, orc.sgemm(a, b))


TC_SHAPES = [(128, 128, 128), (128, 256, 64), (256, 256, 256), (1024, 1024, 1024), (384, 512, 1000), (100, 260, 72),
             (129, 36, 260), (640, 4096, 384), (2048, 64, 2048), (300, 8192, 200),
             # more tiles than SMs with a short last wave: only the last wave's tiles are cut along K (ragged edges)
             (1500, 2048, 3500), (2304, 1024, 2560),
             # CTA-pair kernel with reductions shorter than, equal to and just beyond its rings (four raw stages,
             # three lo slots), and several short items per pair (the rings' phases run on across items)
             (512, 32, 512), (512, 96, 768), (768, 160, 512), (4096, 96, 2304)]


@pytest.mark.parametrize("shape", TC_SHAPES)
def test_tensor_core_gemm_all_three_products(tt, shape):
    """C = A*B, dA = G*B^T, dB = A^T*G on the tcgen05 3xTF32 kernel against float64;
    stated tolerance max|err|/max|ref| <= 1e-4 (reduction length <= 8192)."""
    m, k, n = shape
    rng = np.random.default_rng(m + k + n)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    g = rng.standard_normal((m, n)).astype(np.float32)
    a64, b64, g64 = a.astype(np.float64), b.astype(np.float64), g.astype(np.float64)
    tt.LIB.ttb_set_gemm_path(1)
    try:
        errs = {
            "nn": rel_err(run2(tt, "tt_matmul_fast", a, b), a64 @ b64),
            "nt": rel_err(run2(tt, "ttb_matmul_nt", g, b), g64 @ b64.T),
            "tn": rel_err(run2(tt, "ttb_matmul_tn", a, g), a64.T @ g64),
        }
    finally:
        tt.LIB.ttb_set_gemm_path(0)
    tt.sync()
    assert max(errs.values()) <= TC_TOL, errs


def test_tensor_core_gemm_random_shapes(tt):
    """Forty seeded random shapes on the CTA-pair kernel (M >= 256, 256-wide tiles): every count of K blocks
    from 1 to 40 occurs against rings of four and three slots, with ragged M and N edges; same tolerance."""
    rng = np.random.default_rng(2024)
    tt.LIB.ttb_set_gemm_path(1)
    worst = {}
    try:
        for kblocks in range(1, 41):
            m = int(rng.integers(256, 900))
            n = 4 * int(rng.integers(64, 300))                   # rows of C and B stay 16-byte multiples
            k = 32 * kblocks - 4 * int(rng.integers(0, 8))       # the last K block may be partial
            a = rng.standard_normal((m, k)).astype(np.float32)
            b = rng.standard_normal((k, n)).astype(np.float32)
            err = rel_err(run2(tt, "tt_matmul_fast", a, b), a.astype(np.float64) @ b.astype(np.float64))
            if err > TC_TOL:
                worst[(m, k, n)] = err
    finally:
        tt.LIB.ttb_set_gemm_path(0)
    tt.sync()
    assert not worst, worst


def test_tensor_core_gemm_is_no_worse_than_the_reference_arithmetic(tt, orc):
    """Against float64 the 3xTF32 product must be about as accurate as the
    reference's own fp32 chain on the same inputs."""
    rng = np.random.default_rng(99)
    a = rng.standard_normal((256, 2048)).astype(np.float32)
    b = rng.standard_normal((2048, 256)).astype(np.float32)
    exact = a.astype(np.float64) @ b.astype(np.float64)
    tt.LIB.ttb_set_gemm_path(1)
    try:
        got = run2(tt, "tt_matmul_fast", a, b)
    finally:
        tt.LIB.ttb_set_gemm_path(0)
    ours, theirs = rel_err(got, exact), rel_err(orc.sgemm(a, b), exact)
    assert ours <= max(4 * theirs, 2e-6), (ours, theirs)


def test_tensor_core_gemm_rejects_what_tma_cannot_address(tt):
    a, b = T(tt, np.ones((128, 130), np.float32)), T(tt, np.ones((130, 70), np.float32))
    tt.LIB.ttb_set_gemm_path(1)
    try:
        assert not tt.LIB.tt_matmul_fast(a.ptr, b.ptr)     # row pitch 130*4 and 70*4 bytes
        assert b"TMA" in tt.LIB.ttb_last_error()
    finally:
        tt.LIB.ttb_set_gemm_path(0)
    o = tt.Tensor(tt.checked(tt.LIB.tt_matmul_fast(a.ptr, b.ptr), "tt_matmul_fast"))   # auto: exact path
    assert np.all(o.to_np() == 130.0)
    for t in (a, b, o):
        t.release()


@pytest.mark.parametrize("n", [4096])
def test_full_size_gemm_checksum_of_checksums(tt, n):
    """Benchmark-size GEMM checked through a size-independent property: the
    column sums of C equal (column sums of A) * B, and likewise for the two
    backward products; the right-hand sides cost O(n^2) in float64."""
    rng = np.random.default_rng(4)
    a = rng.standard_normal((n, n)).astype(np.float32)
    b = rng.standard_normal((n, n)).astype(np.float32)
    g = rng.standard_normal((n, n)).astype(np.float32)
    a64, b64, g64 = a.astype(np.float64), b.astype(np.float64), g.astype(np.float64)
    c = run2(tt, "tt_matmul_fast", a, b)
    da = run2(tt, "ttb_matmul_nt", g, b)
    db = run2(tt, "ttb_matmul_tn", a, g)
    tt.sync()
    checks = [(c.astype(np.float64).sum(0), a64.sum(0) @ b64), (c.astype(np.float64).sum(1), a64 @ b64.sum(1)),
              (da.astype(np.float64).sum(0), g64.sum(0) @ b64.T), (db.astype(np.float64).sum(1), a64.T @ g64.sum(1))]
    for got, want in checks:
        assert np.abs(got - want).max() / np.abs(want).max() < TC_TOL
    # and a few hundred entries exactly
    idx = rng.integers(0, n, size=(200, 2))
    for i, j in idx[:100]:
        assert abs(c[i, j] - a64[i] @ b64[:, j]) <= 1e-4 * np.abs(c).max()


@pytest.mark.parametrize("shape", [(1, 1), (7, 5), (128, 10), (130, 1000), (1000, 257), (8192, 4096), (3, 5000)])
def test_column_sums(tt, shape):
    """Bias row of a weight gradient: tree sum here, sequential in the reference."""
    g = np.random.default_rng(shape[0]).standard_normal(shape).astype(np.float32)
    gt = T(tt, g)
    out = tt.colsum(gt)
    want = g.astype(np.float64).sum(0)
    assert np.allclose(out.to_np(), want, rtol=2e-5, atol=1e-5 * np.sqrt(shape[0]))
    gt.release(); out.release()


def test_optimizer_steps_match_numpy(tt):
    rng = np.random.default_rng(12)
    w = rng.standard_normal((257, 33)).astype(np.float32)
    g = rng.standard_normal((257, 33)).astype(np.float32)
    wt, gt = T(tt, w), T(tt, g)
    tt.sgd_step(wt, gt, 0.1)
    assert np.array_equal(wt.to_np(), w - np.float32(0.1) * g)
    v = np.zeros_like(w); vt = T(tt, v)
    w2 = wt.to_np().copy()
    for _ in range(3):
        tt.sgd_momentum_step(wt, vt, gt, 0.05, 0.9)
        v = np.float32(0.9) * v - np.float32(0.05) * g
        w2 = w2 + v
    assert np.array_equal(vt.to_np(), v) and np.array_equal(wt.to_np(), w2)
    # Adam exactly as the reference's CIFAR gate writes it
    m, vv = np.zeros_like(w), np.zeros_like(w)
    mt, vt2 = T(tt, m), T(tt, vv)
    p = wt.to_np().copy()
    lr, b1, b2, eps = 0.003, 0.9, 0.999, 1e-8
    for t in range(1, 4):
        tt.adam_step(wt, mt, vt2, gt, lr, b1, b2, eps, t)
        lr_t = lr * (np.sqrt(1.0 - b2 ** t) / (1.0 - b1 ** t))
        m = b1 * m + (1.0 - b1) * g
        vv = b2 * vv + (1.0 - b2) * (g * g)
        p -= lr_t * m / (np.sqrt(vv) + eps)
    assert np.allclose(wt.to_np(), p, rtol=1e-6, atol=1e-7)
    for t in (wt, gt, vt, mt, vt2):
        t.release()


def test_async_download_is_ordered_after_compute(tt):
    """ttb_download_async copies on the copy stream what the compute stream has produced so far;
    after ttb_download_wait the pinned array holds it (here: the result of a chain of kernels)."""
    x = np.random.default_rng(2).standard_normal((512, 1024)).astype(np.float32)
    xt = T(tt, x)
    h = xt
    keep = []
    for _ in range(6):
        h = tt.Tensor(tt.checked(tt.LIB.tt_addscalar(h.ptr, ctypes.c_float(1.0)), "tt_addscalar")); keep.append(h)
    out = tt.pinned_array(x.shape)
    out[...] = 0
    tt.download_async(h, out)
    tt.download_wait()
    want = x.copy()
    for _ in range(6):
        want = want + np.float32(1.0)
    assert np.array_equal(out, want)
    for t in keep + [xt]:
        t.release()
