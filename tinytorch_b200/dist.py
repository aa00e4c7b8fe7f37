"""Data-parallel plumbing: which rows a rank owns, and how ranks find each other.

Training shards by batch rows (every operator on the path is independent per
sample; only the weight gradients reduce over the batch, src/autograd.c:87-103).
Rank r of G owns rows [r*B/G, (r+1)*B/G) of the inputs and labels, holds a full
replica of the parameters, and scales its loss seed by 1/B (the GLOBAL batch),
so a SUM all-reduce of the parameter gradients equals the single-process
gradient.  The reference has no counterpart (it is a single-process library).

``torch.distributed`` is used for rendezvous only (passing the NCCL id, barriers,
taking the max of the per-rank timings); the gradient traffic itself is the
library's own NCCL communicator.
"""
import os


def shard_rows(n_rows, rank, world):
    """Half-open row range owned by `rank`.  Rows must divide evenly: the
    benchmark's global batch of 8192 does for 1, 2, 4 and 8 ranks."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    if n_rows % world:
        raise ValueError(f"{n_rows} rows do not split evenly over {world} ranks")
    per = n_rows // world
    return rank * per, (rank + 1) * per


def env_rank_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), \
        int(os.environ.get("LOCAL_RANK", "0"))


def init_process_group(backend="gloo"):
    """Join the torchrun rendezvous (MASTER_ADDR/PORT, RANK, WORLD_SIZE from the
    environment).  Returns (rank, world, local_rank)."""
    import torch.distributed as dist
    rank, world, local = env_rank_world()
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return rank, world, local


def connect(ns, rank, world, peer_floats=0):
    """Create the library's NCCL communicator: rank 0 makes the id, everybody
    receives it through torch.distributed, everybody calls ttb_dist_init.

    peer_floats > 0 also sets up the library's own peer-memory all-reduce for
    gradients of up to that many values: every rank exports its block, the
    64-byte handles are gathered over torch.distributed, every rank opens the
    others'.  Larger or oddly sized gradients keep going through NCCL."""
    import ctypes
    if world == 1:
        return
    import torch
    import torch.distributed as dist
    buf = ctypes.create_string_buffer(128)
    if rank == 0:
        ns.status(ns.LIB.ttb_dist_unique_id(buf), "ttb_dist_unique_id")
    t = torch.tensor(list(buf.raw), dtype=torch.uint8)
    dist.broadcast(t, src=0)
    ident = bytes(t.tolist())
    ns.status(ns.LIB.ttb_dist_init(rank, world, ident), "ttb_dist_init")
    if peer_floats:
        handle = ctypes.create_string_buffer(64)
        ns.status(ns.LIB.ttb_dist_peer_export(ctypes.c_size_t(int(peer_floats)), world, handle), "ttb_dist_peer_export")
        mine = torch.tensor(list(handle.raw), dtype=torch.uint8)
        everybody = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(everybody, mine)
        blob = b"".join(bytes(t.tolist()) for t in everybody)
        ns.status(ns.LIB.ttb_dist_peer_import(rank, world, blob), "ttb_dist_peer_import")


def finalize(ns):
    """End the job's communication on every rank, in the order CUDA requires for memory that
    was exported to other processes: everybody stops using the peer blocks (barrier), everybody
    closes the blocks it imported, a second barrier, and only then does each rank free its own
    block and destroy the communicator.  No rank returns from here before all have freed."""
    barrier()
    ns.LIB.ttb_dist_peer_close()
    barrier()
    ns.LIB.ttb_dist_finalize()
    barrier()


def all_sum(values):
    """Element-wise sum of a list of Python floats over all ranks (float64)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return list(values)
    import torch
    t = torch.tensor(list(values), dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return [float(v) for v in t.tolist()]


def max_abs_diff_from_rank0(arr):
    """max |arr - rank 0's arr| over all elements and ranks (0.0 when the replicas are identical)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return 0.0
    import torch
    mine = torch.from_numpy(arr.reshape(-1).copy())
    ref = mine.clone()
    dist.broadcast(ref, src=0)
    d = (mine.double() - ref.double()).abs().max().reshape(1)
    dist.all_reduce(d, op=dist.ReduceOp.MAX)
    return float(d.item())


def all_max(value):
    """Max of a Python float over all ranks (1-rank: the value itself)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier():
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
