"""CPU checks of the drop-in boundary: the shared object loads, exports every
symbol the public headers declare, mirrors the reference's struct layout and
rejects hostile arguments on the host before anything touches a GPU.  No
compute entry point is called here."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INCLUDE = os.path.join(ROOT, "include")


def declared_functions(header):
    text = open(os.path.join(INCLUDE, header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b((?:tt|ttb|ag)_[a-z0-9_]+)\s*\(", text))


@pytest.fixture(scope="module")
def ns():
    import tinytorch_b200
    return tinytorch_b200.default()


def test_library_exports_every_declared_symbol(ns):
    names = set()
    for h in ("tensor.h", "autograd.h", "tt_b200.h"):
        names |= declared_functions(h)
    assert len(declared_functions("tensor.h")) == 23          # 22 operators + tt_sgemm_rowmajor
    assert len(declared_functions("autograd.h")) == 20
    missing = [n for n in sorted(names) if not hasattr(ns.LIB, n)]
    assert not missing, missing


def test_shipped_library_is_not_a_tuning_build(ns):
    """The clock-stamp readers and the wrong-numbers-by-design timing modes exist only in a library built
    with -DTT_TUNING; the one in the tree must not be such a build, and the tuning module must say so
    instead of printing figures."""
    for name in ("ttb_debug_gemm_read", "ttb_debug_gemm_trace", "ttb_debug_conv_read"):
        assert not hasattr(ns.LIB, name), name
    from tinytorch_b200 import tuning
    for run in (tuning.gemm_phases, tuning.conv_phases):
        with pytest.raises(SystemExit) as why:
            run()
        assert "TT_TUNING" in str(why.value)


def test_reference_abi_is_a_subset(ns):
    """The 43 symbols of the reference library (nm -D of its build) are all here."""
    from tinytorch_b200 import api
    assert len(api.CORE_ABI) == 43
    for name in api.CORE_ABI:
        assert hasattr(ns.LIB, name), name
    ref = os.path.join(ROOT, "oracle", "_ref", "libtinytorch_ref.so")
    if os.path.exists(ref):
        out = subprocess.run(["nm", "-D", "--defined-only", ref], capture_output=True, text=True, check=True).stdout
        exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
        exported = {s for s in exported if s.startswith(("tt_", "ag_"))}
        assert exported == set(api.CORE_ABI), exported ^ set(api.CORE_ABI)


def test_headers_compile_as_c_and_cxx(tmp_path):
    src = tmp_path / "probe.c"
    src.write_text('#include "tensor.h"\n#include "autograd.h"\n#include "tt_b200.h"\n'
                   "int main(void){ Tensor t; t.data=0; t.shape=0; t.strides=0; t.ndim=0; t.numel=0; t.refcount=0;"
                   " return (int)sizeof(t) - (int)sizeof(Tensor); }\n")
    subprocess.run(["/usr/bin/gcc", "-std=c11", "-fsyntax-only", f"-I{INCLUDE}", str(src)], check=True)
    subprocess.run(["/usr/bin/g++", "-std=c++17", "-x", "c++", "-fsyntax-only", f"-I{INCLUDE}", str(src)], check=True)


class CTensor(ctypes.Structure):
    """Field order and types of the reference struct (include/tensor.h:10-17),
    which its tests poke through a mirror (tests/test_ops.py:232-238)."""
    _fields_ = [("data", ctypes.POINTER(ctypes.c_float)), ("shape", ctypes.POINTER(ctypes.c_long)),
                ("strides", ctypes.POINTER(ctypes.c_long)), ("ndim", ctypes.c_int),
                ("numel", ctypes.c_long), ("refcount", ctypes.c_int)]


def test_struct_layout():
    assert ctypes.sizeof(CTensor) == 48
    assert [getattr(CTensor, f).offset for f, _ in CTensor._fields_] == [0, 8, 16, 24, 32, 40]


def _new(ns, dims):
    arr = (ctypes.c_long * len(dims))(*dims)
    return ns.LIB.tt_new(arr, len(dims))


def test_hostile_allocations_are_rejected_on_the_host(ns):
    """Overflow, over-cap, negative, zero and rank errors return NULL before any
    allocation (reference: src/tensor.c:10-18, tests/test_ops.py:303-332)."""
    assert not _new(ns, (2**40, 2**40))
    assert not _new(ns, (2**62, 2))
    assert not _new(ns, (2**21, 2**21))
    assert not _new(ns, (2**40 + 1,))
    assert not _new(ns, (-3, 4))
    assert not _new(ns, (0, 4))
    assert not ns.LIB.tt_new((ctypes.c_long * 9)(*([1] * 9)), 9)
    assert not ns.LIB.tt_new((ctypes.c_long * 1)(1), 0)
    big = (ctypes.c_long * 2)(2**40, 2**40)
    assert not ns.LIB.tt_fromdata(None, big, 2)


def test_null_arguments_never_crash(ns):
    L = ns.LIB
    assert L.tt_numel(None) == 0 and L.tt_ndim(None) == 0
    assert not L.tt_data(None)
    assert not L.tt_retain(None)
    L.tt_release(None)
    L.tt_shape(None, None)
    for name in ("tt_add", "tt_mul", "tt_matmul", "tt_matmul_fast"):
        assert not getattr(L, name)(None, None)
    assert not L.tt_matmul_omp(None, None, 4)
    assert not L.tt_relu(None) and not L.tt_softmax(None)
    assert not L.tt_conv2d(None, None, None, 1, 1, 0, 0)
    assert not L.tt_maxpool2d(None, 2, 2, 2, 2) and not L.tt_avgpool2d(None, 2, 2, 2, 2)
    assert not L.tt_reshape(None, None, 0)
    assert not L.ag_leaf(None, 1)
    for name in ("ag_add", "ag_mul", "ag_matmul"):
        assert not getattr(L, name)(None, None)
    assert not L.ag_relu(None) and not L.ag_softmax(None) and not L.ag_padones(None)
    assert not L.ag_value(None) and not L.ag_grad(None)
    assert L.ag_requires_grad(None) == 0
    L.ag_backward(None)
    L.ag_backward_from(None, None, 0)
    L.ag_release(None)
    assert not L.ag_retain(None)
    assert L.tt_sgemm_rowmajor(0, 1, 1, None, None, None, 1) == -1


def test_no_gpu_means_a_loud_error_not_a_fallback(ns):
    """Without a device the library refuses to compute and says why."""
    if ns.device_count() > 0:
        pytest.skip("a GPU is visible")
    assert not _new(ns, (2, 3))
    assert b"no CPU path" in ns.LIB.ttb_last_error()
    with pytest.raises(ValueError):
        ns.Tensor.from_np(np.ones((2, 2), np.float32))


def test_missing_shared_object_is_an_import_error(tmp_path):
    from tinytorch_b200 import _lib
    with pytest.raises(ImportError):
        _lib.load(str(tmp_path / "absent.so"))


def test_product_never_touches_the_oracle():
    """Nothing under the package or the C sources may reference oracle/."""
    pkg = os.path.join(ROOT, "tinytorch_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), os.path.join(dirpath, f)
