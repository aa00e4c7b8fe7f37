"""CPU tests of the host side: workload generators, FLOP accounting, batch
sharding, and the data-parallel arithmetic (two gloo ranks on CPU whose summed
shard gradients must equal the single-process gradient)."""
import os
import subprocess
import sys

import numpy as np
import pytest

from tinytorch_b200 import dist as D
from tinytorch_b200 import workloads as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_configs_are_seeded_and_shaped():
    x, y, ws = W.config_mlp_small()
    x2, y2, ws2 = W.config_mlp_small()
    assert np.array_equal(x, x2) and np.array_equal(y, y2) and np.array_equal(ws[0], ws2[0])
    assert x.shape == (128, 784) and x.dtype == np.float32 and 0.0 <= x.min() and x.max() < 1.0
    assert [w.shape for w in ws] == [(785, 256), (257, 10)]
    assert np.all(ws[0][784] == 0) and np.all(ws[1][256] == 0)
    assert np.abs(ws[0][:784]).max() <= np.sqrt(6 / 784)
    a, b, dc = W.config_gemm()
    assert a.shape == b.shape == dc.shape == (1024, 1024)
    x, y, p = W.config_cnn(4)
    assert x.shape == (4, 3, 32, 32) and p["w2"].shape == (64, 32, 3, 3) and p["fc1"].shape == (4097, 256)
    assert len(W.GEMM_SWEEP) == 10


def test_flop_accounting_matches_the_stated_figures():
    dims = W.MLP_LARGE_DIMS
    assert abs(W.mlp_flops_per_sample(dims, observable=True) / 1e6 - 293.1) < 0.1
    assert abs(W.mlp_flops_per_sample(dims, observable=False) / 1e6 - 326.6) < 0.1
    n_params = sum((dims[i] + 1) * dims[i + 1] for i in range(4))
    assert n_params == 54_440_936


def test_shard_rows():
    assert [D.shard_rows(8192, r, 8) for r in range(8)] == [(r * 1024, (r + 1) * 1024) for r in range(8)]
    assert D.shard_rows(10, 0, 1) == (0, 10)
    with pytest.raises(ValueError):
        D.shard_rows(10, 0, 3)
    with pytest.raises(ValueError):
        D.shard_rows(8, 2, 2)


WORKER = r"""
import os, sys
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from tinytorch_b200 import dist as D, workloads as W
from oracle import oracle as O
rank, world, _ = D.init_process_group("gloo")
rng = np.random.default_rng(9)
B = 32
x = rng.standard_normal((B, 24)).astype(np.float32)
y = rng.integers(0, 5, size=B)
ws = [W.dense_weight(rng, 24, 16), W.dense_weight(rng, 16, 5)]
lo, hi = D.shard_rows(B, rank, world)
part = O.mlp_step(x[lo:hi], y[lo:hi], ws, global_batch=B)
summed = []
for g in part["grads"]:
    t = torch.from_numpy(g.copy())
    dist.all_reduce(t)                       # SUM, what the NCCL path does on the device
    summed.append(t.numpy())
loss = torch.tensor([part["loss"] * (hi - lo) / B], dtype=torch.float64)
dist.all_reduce(loss)
full = O.mlp_step(x, y, ws, global_batch=B)
assert D.all_max(float(rank)) == world - 1
for a, b in zip(summed, full["grads"]):
    assert np.allclose(a, b, rtol=1e-5, atol=1e-7), float(np.abs(a - b).max())
assert abs(loss.item() - full["loss"]) < 1e-6
D.barrier()
dist.destroy_process_group()
sys.stdout.write("rank%dok\n" % rank)
"""


def test_two_gloo_ranks_reproduce_the_full_batch_gradient(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29611", str(script), ROOT]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "rank0ok" in out.stdout and "rank1ok" in out.stdout


# The host-side plumbing bench.py relies on at N > 1, on two gloo ranks: the global loss from shard
# means, the replica comparison, and the order of the tear-down calls (observed through a recording
# stand-in for the library; the calls themselves need a GPU).
PLUMBING_WORKER = r"""
import os, sys, time
import numpy as np
sys.path.insert(0, sys.argv[1])
from tinytorch_b200 import dist as D
rank, world, _ = D.init_process_group("gloo")
# global mean loss from per-rank shard means, weighted by rows
rows = [3, 5]
shard_mean = [2.0, 4.0][rank]
total = D.all_sum([shard_mean * rows[rank]])[0] / sum(rows)
assert abs(total - (2.0 * 3 + 4.0 * 5) / 8) < 1e-12
# replicas: identical arrays give 0, a difference on one rank is found on both
w = np.arange(12, dtype=np.float32)
assert D.max_abs_diff_from_rank0(w) == 0.0
w2 = w.copy()
if rank == 1:
    w2[7] += 0.25
assert D.max_abs_diff_from_rank0(w2) == 0.25
# tear-down order: nobody frees its block (finalize) before everybody has closed its imports
log = os.path.join(sys.argv[2], "order.log")
class Lib:
    def ttb_dist_peer_close(self):
        if rank == 1: time.sleep(0.5)            # a slow rank must hold the others back
        with open(log, "a") as f: f.write("close%d\n" % rank)
    def ttb_dist_finalize(self):
        with open(log, "a") as f: f.write("final%d\n" % rank)
class NS: LIB = Lib()
D.finalize(NS)
if rank == 0:
    seq = open(log).read().split()
    assert sorted(seq[:2]) == ["close0", "close1"] and sorted(seq[2:]) == ["final0", "final1"], seq
sys.stdout.write("rank%dok\n" % rank)
"""


def test_two_gloo_ranks_host_plumbing(tmp_path):
    script = tmp_path / "plumbing.py"
    script.write_text(PLUMBING_WORKER)
    env = dict(os.environ, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29613", str(script), ROOT, str(tmp_path)]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "rank0ok" in out.stdout and "rank1ok" in out.stdout
