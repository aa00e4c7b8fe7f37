"""ctypes view of the tinytorch C ABI: ``Tensor`` and ``Node``.

Mirrors the reference's Python wrapper (tests/torch_py.py:80-203): the same
two classes, method names, argument conventions and error behaviour (a NULL
from C raises ValueError, a seed of the wrong length raises ValueError before
the C call).  ``bind(path)`` builds the classes over any shared object that
exports the tinytorch C ABI, so the very same wrapper drives this library and,
in the test-suite, a CPU build of the reference.

When the library also exports the additive ``ttb_*`` entry points
(include/tt_b200.h) the returned namespace carries them as plain functions.
"""
import ctypes
import types

import numpy as np

from . import _lib

F32P = ctypes.POINTER(ctypes.c_float)
I64P = ctypes.POINTER(ctypes.c_long)
VP = ctypes.c_void_p
CI = ctypes.c_int

# name -> (restype, argtypes); the 43 symbols of the reference ABI
# (include/tensor.h:20-50, include/autograd.h:14-48, src/gemm.c:569)
CORE_ABI = {
    "tt_new": (VP, [I64P, CI]),
    "tt_fromdata": (VP, [F32P, I64P, CI]),
    "tt_retain": (VP, [VP]),
    "tt_release": (None, [VP]),
    "tt_data": (F32P, [VP]),
    "tt_numel": (ctypes.c_long, [VP]),
    "tt_ndim": (CI, [VP]),
    "tt_shape": (None, [VP, I64P]),
    "tt_strides": (None, [VP, I64P]),
    "tt_add": (VP, [VP, VP]),
    "tt_mul": (VP, [VP, VP]),
    "tt_addscalar": (VP, [VP, ctypes.c_float]),
    "tt_mulscalar": (VP, [VP, ctypes.c_float]),
    "tt_matmul": (VP, [VP, VP]),
    "tt_matmul_fast": (VP, [VP, VP]),
    "tt_matmul_omp": (VP, [VP, VP, CI]),
    "tt_relu": (VP, [VP]),
    "tt_softmax": (VP, [VP]),
    "tt_reshape": (VP, [VP, I64P, CI]),
    "tt_conv2d": (VP, [VP, VP, VP, CI, CI, CI, CI]),
    "tt_maxpool2d": (VP, [VP, CI, CI, CI, CI]),
    "tt_avgpool2d": (VP, [VP, CI, CI, CI, CI]),
    "tt_sgemm_rowmajor": (CI, [CI, CI, CI, F32P, F32P, F32P, CI]),
    "ag_leaf": (VP, [VP, CI]),
    "ag_add": (VP, [VP, VP]),
    "ag_mul": (VP, [VP, VP]),
    "ag_addscalar": (VP, [VP, ctypes.c_float]),
    "ag_mulscalar": (VP, [VP, ctypes.c_float]),
    "ag_matmul": (VP, [VP, VP]),
    "ag_relu": (VP, [VP]),
    "ag_softmax": (VP, [VP]),
    "ag_padones": (VP, [VP]),
    "ag_reshape": (VP, [VP, I64P, CI]),
    "ag_conv2d": (VP, [VP, VP, VP, CI, CI, CI, CI]),
    "ag_maxpool2d": (VP, [VP, CI, CI, CI, CI]),
    "ag_avgpool2d": (VP, [VP, CI, CI, CI, CI]),
    "ag_value": (VP, [VP]),
    "ag_grad": (VP, [VP]),
    "ag_requires_grad": (CI, [VP]),
    "ag_backward": (None, [VP]),
    "ag_backward_from": (None, [VP, F32P, ctypes.c_size_t]),
    "ag_release": (None, [VP]),
    "ag_retain": (VP, [VP]),
}

# additive entry points (include/tt_b200.h)
EXT_ABI = {
    "ttb_device_count": (CI, []),
    "ttb_init": (CI, [CI]),
    "ttb_last_error": (ctypes.c_char_p, []),
    "ttb_sync": (CI, []),
    "ttb_launch_count": (ctypes.c_long, []),
    "ttb_device_ptr": (VP, [VP]),
    "ttb_mem_info": (CI, [ctypes.POINTER(ctypes.c_ulonglong)]),
    "ttb_pinned_alloc": (VP, [ctypes.c_size_t]),
    "ttb_pinned_free": (None, [VP]),
    "ttb_upload_async": (CI, [VP, F32P]),
    "ttb_event_create": (VP, []),
    "ttb_event_record": (None, [VP]),
    "ttb_event_elapsed_ms": (ctypes.c_float, [VP, VP]),
    "ttb_event_destroy": (None, [VP]),
    "ttb_trace_enable": (None, [CI]),
    "ttb_trace_reset": (None, []),
    "ttb_trace_read": (CI, [CI, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_long),
                            ctypes.POINTER(ctypes.c_double)]),
    "ttb_set_gemm_path": (None, [CI]),
    "ttb_matmul_nt": (VP, [VP, VP]),
    "ttb_matmul_tn": (VP, [VP, VP]),
    "ttb_relu_bwd": (VP, [VP, VP]),
    "ttb_colsum": (VP, [VP]),
    "ttb_colsum_static": (CI, [VP, CI, CI, ctypes.c_long, VP, CI]),
    "ttb_softmax_bwd": (VP, [VP, VP]),
    "ttb_im2col": (VP, [VP, CI, CI, CI, CI, CI, CI]),
    "ttb_col2im": (VP, [VP, CI, CI, CI, CI, CI, CI, CI, CI, CI, CI]),
    "ttb_maxpool_bwd": (VP, [VP, VP, CI, CI, CI, CI]),
    "ttb_maxpool_argmax": (CI, [VP, CI, CI, CI, CI, I64P]),
    "ttb_avgpool_bwd": (VP, [VP, CI, CI, CI, CI, CI, CI, CI, CI]),
    "ttb_softmax_xent": (VP, [VP, VP, ctypes.c_float, ctypes.POINTER(VP)]),
    "ag_backward_from_tensor": (CI, [VP, VP]),
    "ag_zero_grad": (None, [VP]),
    "ttb_sgd_step": (CI, [VP, VP, ctypes.c_float]),
    "ttb_sgd_momentum_step": (CI, [VP, VP, VP, ctypes.c_float, ctypes.c_float]),
    "ttb_adam_step": (CI, [VP, VP, VP, VP, ctypes.c_double, ctypes.c_double, ctypes.c_double,
                           ctypes.c_double, CI]),
    "ttb_dist_unique_id": (CI, [ctypes.c_char_p]),
    "ttb_dist_init": (CI, [CI, CI, ctypes.c_char_p]),
    "ttb_dist_world": (CI, []),
    "ag_mark_param": (None, [VP, CI]),
    "ag_param_sgd": (None, [VP, ctypes.c_float]),
    "ttb_dist_allreduce": (CI, [VP]),
    "ttb_dist_join": (CI, []),
    "ttb_dist_finalize": (None, []),
    "ttb_download_async": (CI, [VP, ctypes.c_void_p]),
    "ttb_download_wait": (CI, []),
    "ttb_gemm_plan": (CI, [CI, CI, CI, CI, CI, ctypes.POINTER(ctypes.c_int)]),
    "ttb_dist_peer_export": (CI, [ctypes.c_size_t, CI, ctypes.c_char_p]),
    "ttb_dist_peer_import": (CI, [CI, CI, ctypes.c_char_p]),
    "ttb_dist_peer_active": (CI, []),
    "ttb_dist_peer_close": (None, []),
    "ttb_dist_set_wait_limit_ms": (CI, [CI]),
    "ttb_dist_comm_read": (CI, [ctypes.POINTER(ctypes.c_double)]),
    "ttb_bytes_upload": (VP, [VP, ctypes.c_size_t]),
    "ttb_bytes_free": (None, [VP]),
    "ttb_gather_normalize_u8": (CI, [VP, VP, ctypes.c_long, ctypes.POINTER(ctypes.c_int), ctypes.c_long, CI, F32P, F32P]),
    "ttb_argmax": (VP, [VP]),
    "ttb_argmax_correct": (ctypes.c_long, [VP, VP]),
    "ttb_set_grad_enabled": (None, [CI]),
    "ttb_grad_enabled": (CI, []),
}

# kernel classes of ttb_trace_read
K_GEMM_TC, K_GEMM_SIMT, K_ELEMENTWISE, K_SOFTMAX, K_SPATIAL, K_REDUCE, K_OPTIM = range(7)


def _declare(lib, table, required=True):
    ok = True
    for name, (res, args) in table.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            if required:
                raise
            ok = False
            continue
        fn.restype = res
        fn.argtypes = args
    return ok


def bind(path=None):
    """Load a tinytorch shared object and return a namespace with LIB, Tensor, Node."""
    lib = _lib.load(path)
    _declare(lib, CORE_ABI)
    has_ext = _declare(lib, EXT_ABI, required=False)

    def why():
        if has_ext:
            msg = lib.ttb_last_error()
            return (": " + msg.decode()) if msg else ""
        return ""

    def checked(ptr, op):
        if not ptr:
            raise ValueError(f"tinytorch: {op} failed (invalid arguments or shape mismatch){why()}")
        return ptr

    def c_shape(shape):
        return (ctypes.c_long * max(len(shape), 1))(*shape)

    class Tensor:
        """Owns one reference to a C Tensor."""

        def __init__(self, ptr, borrowed=False):
            self.ptr = ptr
            self._borrowed = borrowed

        @classmethod
        def from_np(cls, arr):
            arr = np.ascontiguousarray(arr, dtype=np.float32)
            ptr = lib.tt_fromdata(arr.ctypes.data_as(F32P), c_shape(arr.shape), arr.ndim)
            return cls(checked(ptr, "tt_fromdata"))

        @classmethod
        def zeros(cls, shape):
            return cls(checked(lib.tt_new(c_shape(shape), len(shape)), "tt_new"))

        @property
        def shape(self):
            ndim = int(lib.tt_ndim(self.ptr))
            buf = (ctypes.c_long * max(ndim, 1))()
            lib.tt_shape(self.ptr, buf)
            return tuple(buf)[:ndim]

        def numel(self):
            return int(lib.tt_numel(self.ptr))

        def to_np(self):
            n = self.numel()
            data = lib.tt_data(self.ptr)
            if not data:
                raise RuntimeError(f"tinytorch: tt_data failed{why()}")
            return np.ctypeslib.as_array(data, shape=(max(n, 1),)).copy().reshape(self.shape)

        def release(self):
            if self.ptr and not self._borrowed:
                lib.tt_release(self.ptr)
            self.ptr = None

    class Node:
        """Owns one reference to an AGNode; call release() when done."""

        def __init__(self, ptr):
            self.ptr = ptr

        @classmethod
        def leaf(cls, arr, requires_grad=True):
            t = Tensor.from_np(arr)
            try:
                return cls(checked(lib.ag_leaf(t.ptr, 1 if requires_grad else 0), "ag_leaf"))
            finally:
                t.release()          # the node keeps its own reference

        @classmethod
        def from_tensor(cls, tensor, requires_grad=True):
            return cls(checked(lib.ag_leaf(tensor.ptr, 1 if requires_grad else 0), "ag_leaf"))

        def value_tensor(self):
            return Tensor(lib.ag_value(self.ptr), borrowed=True)

        def grad_tensor(self):
            g = lib.ag_grad(self.ptr)
            return Tensor(g, borrowed=True) if g else None

        def value(self):
            return self.value_tensor().to_np()

        def grad(self):
            g = self.grad_tensor()
            return None if g is None else g.to_np()

        def requires_grad(self):
            return bool(lib.ag_requires_grad(self.ptr))

        def backward(self, seed=None):
            if seed is None:
                lib.ag_backward(self.ptr)
                return
            if isinstance(seed, Tensor):
                if lib.ag_backward_from_tensor(self.ptr, seed.ptr) != 0:
                    raise ValueError(f"tinytorch: seed length mismatch{why()}")
                return
            seed = np.ascontiguousarray(seed, dtype=np.float32)
            need = int(lib.tt_numel(lib.ag_value(self.ptr)))
            if int(seed.size) != need:
                raise ValueError(f"tinytorch: seed length mismatch (got {int(seed.size)}, need {need})")
            lib.ag_backward_from(self.ptr, seed.ctypes.data_as(F32P), int(seed.size))

        def __add__(self, other):
            if isinstance(other, (int, float)):
                return Node(checked(lib.ag_addscalar(self.ptr, float(other)), "ag_addscalar"))
            return Node(checked(lib.ag_add(self.ptr, other.ptr), "ag_add"))

        def __mul__(self, other):
            if isinstance(other, (int, float)):
                return Node(checked(lib.ag_mulscalar(self.ptr, float(other)), "ag_mulscalar"))
            return Node(checked(lib.ag_mul(self.ptr, other.ptr), "ag_mul"))

        __rmul__ = __mul__

        def matmul(self, other):
            return Node(checked(lib.ag_matmul(self.ptr, other.ptr), "ag_matmul"))

        def relu(self):
            return Node(checked(lib.ag_relu(self.ptr), "ag_relu"))

        def softmax(self):
            return Node(checked(lib.ag_softmax(self.ptr), "ag_softmax"))

        def padones(self):
            return Node(checked(lib.ag_padones(self.ptr), "ag_padones"))

        def reshape(self, shape):
            return Node(checked(lib.ag_reshape(self.ptr, c_shape(shape), len(shape)), "ag_reshape"))

        def conv2d(self, w, b=None, stride=1, pad=0):
            sh, sw = (stride, stride) if isinstance(stride, int) else stride
            ph, pw = (pad, pad) if isinstance(pad, int) else pad
            return Node(checked(lib.ag_conv2d(self.ptr, w.ptr, b.ptr if b else None, sh, sw, ph, pw),
                                "ag_conv2d"))

        def maxpool2d(self, pool_size=2, stride=2):
            ph, pw = (pool_size, pool_size) if isinstance(pool_size, int) else pool_size
            sh, sw = (stride, stride) if isinstance(stride, int) else stride
            return Node(checked(lib.ag_maxpool2d(self.ptr, ph, pw, sh, sw), "ag_maxpool2d"))

        def avgpool2d(self, pool_size=2, stride=2):
            ph, pw = (pool_size, pool_size) if isinstance(pool_size, int) else pool_size
            sh, sw = (stride, stride) if isinstance(stride, int) else stride
            return Node(checked(lib.ag_avgpool2d(self.ptr, ph, pw, sh, sw), "ag_avgpool2d"))

        def zero_grad(self):
            lib.ag_zero_grad(self.ptr)

        def mark_param(self, on=True):
            lib.ag_mark_param(self.ptr, 1 if on else 0)

        def param_sgd(self, lr):
            lib.ag_param_sgd(self.ptr, float(lr))

        def release(self):
            if self.ptr:
                lib.ag_release(self.ptr)
                self.ptr = None

    ns = types.SimpleNamespace(LIB=lib, Tensor=Tensor, Node=Node, has_ext=has_ext,
                               checked=checked, why=why, path=path or _lib.LIB_PATH)

    if has_ext:
        def op(name, *args):
            return Tensor(checked(getattr(lib, name)(*args), name))

        def softmax_xent(logits, labels, scale):
            d = VP()
            loss = checked(lib.ttb_softmax_xent(logits.ptr, labels.ptr, scale, ctypes.byref(d)),
                           "ttb_softmax_xent")
            return Tensor(loss), Tensor(d.value)

        def maxpool_argmax(x, ph, pw, sh, sw):
            n, c, h, w = x.shape
            ho, wo = (h - ph) // sh + 1, (w - pw) // sw + 1
            out = np.empty(n * c * ho * wo, dtype=np.int64)
            if lib.ttb_maxpool_argmax(x.ptr, ph, pw, sh, sw, out.ctypes.data_as(I64P)) != 0:
                raise ValueError(f"tinytorch: ttb_maxpool_argmax failed{why()}")
            return out.reshape(n, c, ho, wo)

        def trace_read(kind):
            ms, n, work = ctypes.c_double(), ctypes.c_long(), ctypes.c_double()
            if lib.ttb_trace_read(kind, ctypes.byref(ms), ctypes.byref(n), ctypes.byref(work)) != 0:
                raise RuntimeError(f"tinytorch: ttb_trace_read failed{why()}")
            return ms.value, n.value, work.value

        def sync():
            if lib.ttb_sync() != 0:
                raise RuntimeError(f"tinytorch: device synchronisation failed{why()}")

        def status(rc, name):
            if rc != 0:
                raise RuntimeError(f"tinytorch: {name} failed{why()}")

        def pinned_array(shape, dtype=np.float32):
            """NumPy array over page-locked host memory (freed when the array dies)."""
            nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
            ptr = lib.ttb_pinned_alloc(nbytes)
            if not ptr:
                raise MemoryError(f"tinytorch: ttb_pinned_alloc failed{why()}")
            buf = (ctypes.c_char * nbytes).from_address(ptr)
            arr = np.frombuffer(buf, dtype=dtype).reshape(shape)
            ns._pinned.append(ptr)
            return arr

        def upload_async(tensor, arr):
            """Queue a host -> device copy of `arr` (same element count) into `tensor`."""
            arr = np.ascontiguousarray(arr, dtype=np.float32)
            if arr.size != tensor.numel():
                raise ValueError("tinytorch: ttb_upload_async size mismatch")
            status(lib.ttb_upload_async(tensor.ptr, arr.ctypes.data_as(F32P)), "ttb_upload_async")

        def download_async(tensor, arr):
            """Queue a device -> host copy of `tensor` into `arr` (pinned, same element count);
            the values are there after download_wait()."""
            if arr.dtype != np.float32 or not arr.flags["C_CONTIGUOUS"] or arr.size != tensor.numel():
                raise ValueError("tinytorch: ttb_download_async needs a contiguous float32 array of the tensor's size")
            status(lib.ttb_download_async(tensor.ptr, arr.ctypes.data), "ttb_download_async")

        class ByteDataset:
            """A raw 8-bit dataset [rows, channels, ...] resident on the device, and the
            normalise + gather stage that cuts fp32 batches from it."""

            def __init__(self, arr_u8, mean, std):
                arr = np.ascontiguousarray(arr_u8, dtype=np.uint8)
                self.shape = arr.shape
                self.rows = int(arr.shape[0])
                self.channels = int(arr.shape[1]) if arr.ndim > 2 else 1
                self.mean = np.ascontiguousarray(np.broadcast_to(np.asarray(mean, np.float32).ravel(), (self.channels,)))
                self.std = np.ascontiguousarray(np.broadcast_to(np.asarray(std, np.float32).ravel(), (self.channels,)))
                self.dev = lib.ttb_bytes_upload(arr.ctypes.data, arr.nbytes)
                if not self.dev:
                    raise MemoryError(f"tinytorch: ttb_bytes_upload failed{why()}")

            def batch_into(self, tensor, idx):
                """tensor <- ((rows[idx] / 255) - mean) / std; idx: integer array of the batch's rows."""
                idx = np.ascontiguousarray(idx, dtype=np.int32)
                status(lib.ttb_gather_normalize_u8(tensor.ptr, self.dev, self.rows,
                                                   idx.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), int(idx.size),
                                                   self.channels, self.mean.ctypes.data_as(F32P),
                                                   self.std.ctypes.data_as(F32P)), "ttb_gather_normalize_u8")

            def free(self):
                if self.dev:
                    lib.ttb_bytes_free(self.dev)
                    self.dev = None

        class no_grad:
            """Context manager: forward-only mode (no graph, no saved activations)."""

            def __enter__(self):
                self.prev = lib.ttb_grad_enabled()
                lib.ttb_set_grad_enabled(0)

            def __exit__(self, *exc):
                lib.ttb_set_grad_enabled(self.prev)
                return False

        def argmax_correct(logits, labels):
            n = int(lib.ttb_argmax_correct(logits.ptr, labels.ptr))
            if n < 0:
                raise RuntimeError(f"tinytorch: ttb_argmax_correct failed{why()}")
            return n

        def comm_read():
            buf = (ctypes.c_double * 6)()
            status(lib.ttb_dist_comm_read(buf), "ttb_dist_comm_read")
            return {"collectives": int(buf[0]), "bytes": buf[1], "collective_ms": buf[2], "joins": int(buf[3]),
                    "exposed_ms": buf[4], "longest_collective_ms": buf[5]}

        ns.ByteDataset = ByteDataset
        ns.no_grad = no_grad
        ns.argmax = lambda t: op("ttb_argmax", t.ptr)
        ns.argmax_correct = argmax_correct
        ns.comm_read = comm_read
        ns.upload_async = upload_async
        ns.download_async = download_async
        ns.download_wait = lambda: status(lib.ttb_download_wait(), "ttb_download_wait")
        ns._pinned = []
        ns.pinned_array = pinned_array
        ns.matmul_nt = lambda x, y: op("ttb_matmul_nt", x.ptr, y.ptr)
        ns.matmul_tn = lambda x, y: op("ttb_matmul_tn", x.ptr, y.ptr)
        ns.relu_bwd = lambda x, g: op("ttb_relu_bwd", x.ptr, g.ptr)
        ns.colsum = lambda g: op("ttb_colsum", g.ptr)
        ns.softmax_bwd = lambda s, g: op("ttb_softmax_bwd", s.ptr, g.ptr)
        ns.im2col = lambda x, kh, kw, sh, sw, ph, pw: op("ttb_im2col", x.ptr, kh, kw, sh, sw, ph, pw)
        ns.col2im = lambda col, n, c, h, w, kh, kw, sh, sw, ph, pw: op(
            "ttb_col2im", col.ptr, n, c, h, w, kh, kw, sh, sw, ph, pw)
        ns.maxpool_bwd = lambda x, g, ph, pw, sh, sw: op("ttb_maxpool_bwd", x.ptr, g.ptr, ph, pw, sh, sw)
        ns.avgpool_bwd = lambda g, n, c, h, w, ph, pw, sh, sw: op(
            "ttb_avgpool_bwd", g.ptr, n, c, h, w, ph, pw, sh, sw)
        ns.maxpool_argmax = maxpool_argmax
        ns.softmax_xent = softmax_xent
        ns.sgd_step = lambda w, g, lr: status(lib.ttb_sgd_step(w.ptr, g.ptr, lr), "ttb_sgd_step")
        ns.sgd_momentum_step = lambda w, v, g, lr, mu: status(
            lib.ttb_sgd_momentum_step(w.ptr, v.ptr, g.ptr, lr, mu), "ttb_sgd_momentum_step")
        ns.adam_step = lambda w, m, v, g, lr, b1, b2, eps, t: status(
            lib.ttb_adam_step(w.ptr, m.ptr, v.ptr, g.ptr, lr, b1, b2, eps, t), "ttb_adam_step")
        ns.trace_read = trace_read
        ns.sync = sync
        ns.status = status
        ns.device_count = lambda: int(lib.ttb_device_count())
    return ns
