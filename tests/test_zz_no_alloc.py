"""ttb_colsum_static: the column-sum entry point for callers that cannot allocate.

Some users of the library are not allowed to ask CUDA for memory when they need
a bias gradient -- their own arena owns the whole GPU, or they sit in a loop or
a stream recording where an allocator call is off limits.  The entry point keeps
its partial sums in an array compiled into the library, so the call allocates
nothing; the caller brings input and output buffers it made earlier.

Checked here through the C ABI against the ordinary ttb_colsum, twice in a row
(the array keeps the previous call's contents, which must not leak into the
next result), plus the size limit.  The file name sorts last so that a run that
stops at the first failure has already been through every other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _static_colsum(tt, g_t, out_t, accumulate=0):
    rows, cols = g_t.shape
    rc = tt.LIB.ttb_colsum_static(tt.LIB.ttb_device_ptr(g_t.ptr), rows, cols, cols,
                                  tt.LIB.ttb_device_ptr(out_t.ptr), accumulate)
    return rc


def test_static_column_sums_match_the_allocating_entry_point_twice(tt):
    rng = np.random.default_rng(31)
    # second shape is smaller than the first: stale partials of call one lie beyond what call two may read
    for shape in [(2048, 4096), (300, 1000), (8192, 4096), (5, 7)]:
        g = rng.standard_normal(shape).astype(np.float32)
        g_t = tt.Tensor.from_np(g)
        ref_t = tt.colsum(g_t)
        want = ref_t.to_np()
        out_t = tt.Tensor.zeros((shape[1],))
        for _ in range(2):
            assert _static_colsum(tt, g_t, out_t) == 0, tt.LIB.ttb_last_error()
            tt.sync()
            # a device write the host wrapper did not see: read the buffer through a fresh copy
            got = tt.Tensor(tt.checked(tt.LIB.tt_addscalar(out_t.ptr, 0.0), "tt_addscalar"))
            assert np.allclose(got.to_np(), want, rtol=2e-5, atol=1e-5 * np.sqrt(shape[0]))
            assert np.allclose(got.to_np(), g.astype(np.float64).sum(0), rtol=2e-5, atol=1e-5 * np.sqrt(shape[0]))
            got.release()
        # accumulate adds to what is there
        assert _static_colsum(tt, g_t, out_t, accumulate=1) == 0
        got = tt.Tensor(tt.checked(tt.LIB.tt_addscalar(out_t.ptr, 0.0), "tt_addscalar"))
        assert np.allclose(got.to_np(), 2 * want, rtol=4e-5, atol=2e-5 * np.sqrt(shape[0]))
        for t in (got, g_t, ref_t, out_t):
            t.release()


def _mem(tt):
    import ctypes
    buf = (ctypes.c_ulonglong * 3)()
    assert tt.LIB.ttb_mem_info(buf) == 0
    return tuple(buf)


def test_static_column_sums_allocate_nothing(tt):
    """Free memory on the GPU, what the library's pool holds and what it has handed out are the same
    before and after the calls.  The very first call in a process is the set-up call (it looks the
    array's address up, and with CUDA's lazy module loading the driver loads the kernels' code then),
    so it is made before the first reading."""
    g_t = tt.Tensor.from_np(np.ones((4096, 2048), np.float32))
    out_t = tt.Tensor.zeros((2048,))
    assert _static_colsum(tt, g_t, out_t) == 0, tt.LIB.ttb_last_error()
    tt.sync()
    before = _mem(tt)
    for _ in range(3):
        assert _static_colsum(tt, g_t, out_t) == 0, tt.LIB.ttb_last_error()
    tt.sync()
    assert _mem(tt) == before
    g_t.release(); out_t.release()


def test_static_column_sums_refuse_what_does_not_fit(tt):
    g_t = tt.Tensor.zeros((2, 16385))
    out_t = tt.Tensor.zeros((16385,))
    assert _static_colsum(tt, g_t, out_t) == -1
    assert b"exceed" in tt.LIB.ttb_last_error()
    assert tt.LIB.ttb_colsum_static(None, 2, 2, 2, None, 0) == -1
    g_t.release(); out_t.release()
