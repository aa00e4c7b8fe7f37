"""tinytorch_b200: the training hot path of tinytorch on one or more B200 GPUs.

The product is ``libtinytorch.so`` -- a drop-in for the reference's C ABI
(include/tensor.h, include/autograd.h) whose every numeric loop is a
hand-written sm_100a CUDA kernel.  This package is the thin Python side:

  api        ctypes ``Tensor`` / ``Node`` classes, same surface as the
             reference's tests/torch_py.py
  workloads  seeded synthetic inputs and training steps of the benchmark
             configurations
  dist       batch sharding and NCCL bootstrap for data-parallel runs
  build      compiles the shared objects in-tree

Importing the package loads nothing; ``tinytorch_b200.default()`` binds the
in-tree library and fails loudly if it has not been built.
"""
from . import api

_default = None


def default():
    """The namespace (LIB, Tensor, Node, ...) bound to the in-tree libtinytorch.so."""
    global _default
    if _default is None:
        _default = api.bind()
    return _default
