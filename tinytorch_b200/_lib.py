"""Locate and load libtinytorch.so (the sm_100a build of the tinytorch C ABI).

The library is built in-tree by ``make lib`` (or ``tinytorch_b200.build``).
There is no fallback of any kind: if the shared object is missing the import
fails, and if no B200 is visible every compute entry point returns NULL and
the wrappers raise with the library's own error text.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtinytorch.so")


def load(path=None):
    path = path or LIB_PATH
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `make lib` at the repository root "
            "(needs nvcc with sm_100a support). tinytorch_b200 has no CPU fallback.")
    return ctypes.CDLL(path)
