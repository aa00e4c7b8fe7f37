import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; runs the CUDA path through the C ABI")


@pytest.fixture(scope="session")
def golden_ops():
    return np.load(os.path.join(GOLDEN, "ops.npz"))


@pytest.fixture(scope="session")
def golden_steps():
    return np.load(os.path.join(GOLDEN, "steps.npz"))


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (C restatement), built on demand."""
    from oracle import oracle
    oracle.lib()
    return oracle


@pytest.fixture(scope="session")
def ref(orc):
    """The reference's own library, when its build travelled with the repo."""
    r = orc.load_ref()
    if r is None:
        pytest.skip("oracle/_ref/libtinytorch_ref.so not present")
    return r


@pytest.fixture(scope="session")
def tt():
    """The product library on the GPU.  No GPU -> the gpu tests cannot run."""
    import tinytorch_b200
    ns = tinytorch_b200.default()
    if ns.device_count() < 1:
        pytest.fail("gpu test selected but no CUDA device is visible")
    return ns


def rel_err(got, want):
    """max|got - want| / max|want|: the metric of the reference's GEMM gate
    (bench/bench_gemm_opt.py:73-75)."""
    want64 = np.asarray(want, dtype=np.float64)
    denom = max(float(np.abs(want64).max()), 1e-30)
    return float(np.abs(np.asarray(got, dtype=np.float64) - want64).max()) / denom
