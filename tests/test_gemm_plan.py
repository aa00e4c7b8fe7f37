"""The tensor-core GEMM's host-side planner (tile width, kernel, CTA count, how the reduction
is cut), checked through ttb_gemm_plan on a machine without a GPU: the plan must cover every
tile and every K block exactly once, and reproduce the decisions the design rests on."""
import ctypes

import numpy as np
import pytest

from tinytorch_b200 import _lib

NAMES = ("bn", "pair", "bk", "units", "tiles", "splits", "kb_per_split", "tail_tiles", "tail_splits", "tail_kb")


@pytest.fixture(scope="module")
def plan():
    lib = _lib.load()
    lib.ttb_gemm_plan.restype = ctypes.c_int
    lib.ttb_gemm_plan.argtypes = [ctypes.c_int] * 5 + [ctypes.POINTER(ctypes.c_int)]

    def f(m, n, k, sms=148, world=1):
        out = (ctypes.c_int * 10)()
        assert lib.ttb_gemm_plan(m, n, k, sms, world, out) == 0
        return dict(zip(NAMES, list(out)))
    return f


def check_invariants(p, m, n, k):
    bm = 256 if p["pair"] else 128
    assert p["bn"] in (128, 256) and p["bk"] in (16, 32)
    assert p["tiles"] == -(-m // bm) * -(-n // p["bn"])
    num_kb = -(-k // p["bk"])
    assert 1 <= p["units"] <= (74 if p["pair"] else 148)
    assert not (p["splits"] > 1 and p["tail_tiles"] > 0)            # one way of cutting at a time
    # uniform slices: together they cover the reduction, and none is empty
    assert p["splits"] * p["kb_per_split"] >= num_kb
    assert (p["splits"] - 1) * p["kb_per_split"] < num_kb
    if p["tail_tiles"]:
        assert 0 < p["tail_tiles"] < p["units"]
        assert (p["tiles"] - p["tail_tiles"]) % p["units"] == 0       # the earlier waves are full
        assert p["tail_splits"] >= 2
        assert p["tail_splits"] * p["tail_kb"] >= num_kb and (p["tail_splits"] - 1) * p["tail_kb"] < num_kb
        assert p["tail_tiles"] * p["tail_splits"] <= 8 * p["units"]


def test_plans_of_the_benchmark_shapes(plan):
    p = plan(4096, 4096, 4096)                     # 256 pair tiles on 74 pairs: 3.46 waves, the last one cut in two
    assert (p["pair"], p["bn"], p["tiles"], p["units"]) == (1, 256, 256, 74)
    assert (p["splits"], p["tail_tiles"], p["tail_splits"], p["tail_kb"]) == (1, 34, 2, 64)
    p = plan(8192, 4096, 4096)                     # forward GEMM of the large MLP: 6.9 waves, nothing to gain
    assert (p["tiles"], p["splits"], p["tail_tiles"]) == (512, 1, 0)
    p = plan(4096, 4096, 8192)                     # its weight gradient: tail split over the long reduction
    assert (p["tail_tiles"], p["tail_splits"]) == (34, 2)
    p = plan(1024, 1024, 1024)                     # too few 256-wide tiles: 64 tiles of 128x128, each cut in two
    assert (p["pair"], p["bn"], p["tiles"], p["splits"], p["kb_per_split"]) == (0, 128, 64, 2, 16)
    p = plan(256, 10, 256)                         # narrow output: one-CTA kernel, 128-wide tiles
    assert (p["pair"], p["bn"]) == (0, 128)


def test_data_parallel_jobs_leave_sms_to_the_collective(plan):
    for world, units in ((1, 74), (2, 74), (4, 64), (8, 64)):
        p = plan(1024, 4096, 4096, world=world)    # 64 pair tiles: one wave on 64 pairs as on 74
        assert (p["tiles"], p["units"], p["splits"], p["tail_tiles"]) == (64, units, 1, 0), world
    p = plan(4096, 4096, 1024, world=8)            # 256 tiles: exactly four waves on 64 pairs, no tail left
    assert (p["units"], p["tail_tiles"]) == (64, 0)
    p = plan(1024, 1024, 1024, world=8)            # few tiles: keeps every SM and cuts along K instead
    assert (p["units"], p["splits"]) == (148, 2)


def test_every_plan_covers_its_problem(plan):
    rng = np.random.default_rng(7)
    shapes = [(16, 8, 8), (129, 36, 260), (300, 200, 8192), (2048, 2048, 64), (32, 4096, 4096), (256, 16384, 16384),
              (1500, 3500, 2048), (8192, 1000, 4096), (8192, 4096, 1000)]
    shapes += [tuple(int(v) for v in rng.integers(16, 6000, size=3)) for _ in range(300)]
    for m, n, k in shapes:
        for world in (1, 4, 8):
            for sms in (148, 128, 2):
                check_invariants(plan(m, n, k, sms=sms, world=world), m, n, k)
