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
peer_floats = int(sys.argv[2])
D.connect(ns, rank, world, peer_floats=peer_floats)
assert ns.LIB.ttb_dist_world() == world
assert bool(ns.LIB.ttb_dist_peer_active()) == bool(peer_floats)
# plain all-reduce of tensors every rank can regenerate: sizes that the peer kernel takes (a multiple
# of four values, within the block), one beyond the block and one odd length (both fall back to NCCL)
for n in (4, 1000, 262144 + 8, 2048 * 384, 3 * 2048 * 384, 1001):
    parts = [np.random.default_rng(100 + r).standard_normal(n).astype(np.float32) for r in range(world)]
    t = ns.Tensor.from_np(parts[rank])
    for _ in range(2):                                   # twice: the second launch reuses the staging areas
        ns.status(ns.LIB.ttb_dist_allreduce(t.ptr), "ttb_dist_allreduce")
        ns.status(ns.LIB.ttb_dist_join(), "ttb_dist_join")
    want = parts[0].copy()
    for r in range(1, world):
        want = want + parts[r]                           # rank order
    once = t.to_np()
    # after two reductions every rank holds world * (sum): check through the first one's algebra
    assert np.array_equal(once, want * np.float32(world)), (n, np.abs(once - want * world).max())
    t.release()
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
tr.close(); D.finalize(ns)
sys.stdout.write("rank%dok\n" % rank)
"""

# One rank skips a reduction, so the other's device-side wait on it runs out.  The failure is made on
# the host (a call that is not issued); no kernel traps, faults or spins without a limit.
FAILURE_WORKER = r"""
import os, sys, time
import numpy as np
sys.path.insert(0, sys.argv[1])
import tinytorch_b200
from tinytorch_b200 import dist as D
rank, world, local = D.init_process_group("gloo")
ns = tinytorch_b200.default()
ns.status(ns.LIB.ttb_init(local), "ttb_init")
D.connect(ns, rank, world, peer_floats=1 << 20)
assert ns.LIB.ttb_dist_peer_active()
assert ns.LIB.ttb_dist_set_wait_limit_ms(300) == 0
a = np.full(4096, float(rank + 1), np.float32)
t = ns.Tensor.from_np(a)
# a healthy round first
ns.status(ns.LIB.ttb_dist_allreduce(t.ptr), "ttb_dist_allreduce")
ns.status(ns.LIB.ttb_dist_join(), "ttb_dist_join")
assert np.all(t.to_np() == 3.0)
D.barrier()
if rank == 0:
    # rank 1 never launches this one: the wait on its flag gives up after the shortened limit
    assert ns.LIB.ttb_dist_allreduce(t.ptr) == 0
    t0 = time.time()
    ns.LIB.ttb_sync()
    took = time.time() - t0
    assert ns.LIB.ttb_dist_join() == -1
    msg = ns.LIB.ttb_last_error().decode()
    assert "wait expired" in msg and "rank 1" in msg, msg
    assert took < 5.0, took
    # the failure is sticky: this process launches no further peer reductions
    assert ns.LIB.ttb_dist_allreduce(t.ptr) == -1
D.barrier()
if rank == 1:
    # out of step with rank 0 now; the poison word rank 0 left makes this launch report instead of
    # passing its waits on stale flags
    assert ns.LIB.ttb_dist_allreduce(t.ptr) == 0
    ns.LIB.ttb_sync()
    assert ns.LIB.ttb_dist_join() == -1
    assert "gave up" in ns.LIB.ttb_last_error().decode() or "given up" in ns.LIB.ttb_last_error().decode()
# the device still answers on both ranks
u = ns.Tensor.from_np(a)
assert np.all(u.to_np() == float(rank + 1))
t.release(); u.release()
D.finalize(ns)
sys.stdout.write("rank%dok\n" % rank)
"""


@pytest.mark.parametrize("peer_floats", [0, 2048 * 384 + 384], ids=["nccl", "peer-memory"])
def test_two_gpu_data_parallel_matches_full_batch(tt, tmp_path, peer_floats):
    """Once with every reduction through NCCL, once with the library's own peer-memory kernel for the
    gradients that fit its block (the largest parameter of the model)."""
    if tt.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29633", str(script), ROOT, str(peer_floats)]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "rank0ok" in out.stdout and "rank1ok" in out.stdout


def test_a_peer_that_skips_a_reduction_is_reported_not_waited_for(tt, tmp_path):
    """Bounded device-side waits: with the limit shortened to 0.3 s, a reduction whose partner never
    launches ends with a status the host reads (phase and rank), the other rank learns of it through
    the poison word, both processes keep a working GPU context and tear down in order.  Plain peer
    loads and stores only (NVLS off)."""
    if tt.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "failure_worker.py"
    script.write_text(FAILURE_WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29637", str(script), ROOT]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "rank0ok" in out.stdout and "rank1ok" in out.stdout
