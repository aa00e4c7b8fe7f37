"""Data-parallel training on two GPUs: per-rank shards, NCCL gradient all-reduce
overlapped with backward, SGD on every replica.  The replicas must stay equal and
match a single-process run of the CPU oracle on the full batch."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys
import numpy as np
sys.path.insert(0, sys.argv[1])
import tinytorch_b200
from tinytorch_b200 import dist as D, workloads as W
from oracle import oracle as O
rank, world, local = D.init_process_group("gloo")
ns = tinytorch_b200.default()
ns.status(ns.LIB.ttb_init(local), "ttb_init")
D.connect(ns, rank, world)
assert ns.LIB.ttb_dist_world() == world
rng = np.random.default_rng(5)
dims, B = (2048, 384, 128, 40), 512      # first layer wide enough for the chunked dW + all-reduce path
x = rng.standard_normal((B, dims[0])).astype(np.float32)
y = rng.integers(0, dims[-1], size=B)
ws = [W.dense_weight(rng, dims[i], dims[i + 1]) for i in range(3)]
lo, hi = D.shard_rows(B, rank, world)
tr = W.MLPTrainer(ns, ws, lr=0.1, global_batch=B)
xt, yt = ns.Tensor.from_np(x[lo:hi]), ns.Tensor.from_np(y[lo:hi].astype(np.float32))
for _ in range(3):
    tr.step(xt, yt).release()
got = tr.weights()
want = [w.copy() for w in ws]
for _ in range(3):
    want = O.mlp_step(x, y, want, lr=0.1, global_batch=B)["weights"]
for a, b in zip(got, want):
    err = float(np.abs(a.astype(np.float64) - b).max() / np.abs(b).max())
    assert err <= 1e-4, err
# replicas identical across ranks
import torch, torch.distributed as dist
for a in got:
    t = torch.from_numpy(a.copy()); t0 = t.clone()
    dist.broadcast(t0, src=0)
    assert torch.equal(t, t0)
tr.close(); ns.LIB.ttb_dist_finalize(); D.barrier()
sys.stdout.write("rank%dok\n" % rank)
"""


def test_two_gpu_data_parallel_matches_full_batch(tt, tmp_path):
    if tt.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29633", str(script), ROOT]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "rank0ok" in out.stdout and "rank1ok" in out.stdout
