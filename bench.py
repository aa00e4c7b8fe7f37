#!/usr/bin/env python3
"""Benchmark of the tinytorch training hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # N = 1
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N \
        --master-addr 127.0.0.1 --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference --steps K --warmup W     # the reference's CPU path

Workload: the large data-parallel MLP 4096->4096->4096->4096->1000 (relu,
softmax cross-entropy, SGD lr 0.1), fp32, global batch 8192 split evenly over
the ranks, synthetic N(0,1) inputs and Kaiming-uniform weights from seed 3.  A
step is forward + backward + gradient all-reduce + SGD over the whole global
batch; `value` is global samples per second with the inputs resident in HBM.
`e2e` is the same step fed from pinned host buffers through the C ABI with the
loss read back, every step.  One JSON line is printed by rank 0.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from tinytorch_b200 import dist as D                      # noqa: E402
from tinytorch_b200 import workloads as W                 # noqa: E402

GLOBAL_BATCH = 8192
DIMS = W.MLP_LARGE_DIMS
LR = 0.1
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------ clock sampling
class ClockSampler:
    """nvidia-smi polling in a child process for the length of the timed region."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.device_index = device_index
        self.proc = None
        self.path = os.path.join("/tmp", f"tt_clocks_{os.getpid()}.csv")

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "50"], stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    @staticmethod
    def _seconds(stamp):
        """'2026/11/25 05:41:07.123' -> seconds since the epoch (local time)."""
        import datetime
        try:
            return datetime.datetime.strptime(stamp.strip(), "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def stop(self, window=None):
        """window = (t0, t1) in time.time() seconds: only samples inside it count."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                if window is not None:
                    ts = self._seconds(parts[0])
                    if ts is None or ts < window[0] - 0.05 or ts > window[1] + 0.05:
                        continue
                try:
                    sm.append(float(parts[1])); mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, flag in zip(names, parts[5:9]):
                    if flag.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_min_mhz": min(sm), "sm_max_mhz": max(mx), "samples": len(sm),
                "reasons": sorted(reasons)}


# ------------------------------------------------------------------ reference arm
def reference_step_fn():
    """(callable(batch) -> seconds per step, kind, threads) for the reference's own CPU path."""
    from oracle import oracle as O
    ref = O.load_ref()
    cache = {}

    def data(batch):
        if batch not in cache:
            cache[batch] = W.config_mlp_large(batch=batch)
        return cache[batch]

    if ref is not None:
        def step(batch):
            x, y, ws = data(batch)
            t0 = time.perf_counter()
            W.mlp_step_reference_style(ref, x, y, ws, lr=LR, global_batch=GLOBAL_BATCH)
            return time.perf_counter() - t0
        return step, "reference"

    O.lib()

    def step(batch):
        x, y, ws = data(batch)
        t0 = time.perf_counter()
        O.mlp_step(x, y, ws, lr=LR, global_batch=GLOBAL_BATCH)
        return time.perf_counter() - t0
    return step, "port"


def host_threads():
    n = os.environ.get("OMP_NUM_THREADS")
    return int(n) if n else (os.cpu_count() or 1)


def run_reference(args):
    """Times the reference's CPU implementation of the same training step on the
    host cores.  Each step is a bounded sample (a slice of the global batch)."""
    rank, world, _ = D.env_rank_world()
    if rank != 0:
        return
    if world > 1:
        # torch.distributed.run sets OMP_NUM_THREADS=1 for its workers; the reference arm is one
        # process on rank 0 and is to use every host core, as it does at N=1
        n = os.cpu_count() or 1
        os.environ["OMP_NUM_THREADS"] = str(n)
        try:
            ctypes.CDLL("libgomp.so.1").omp_set_num_threads(n)
        except OSError:
            pass
    step, kind = reference_step_fn()
    # Every step is the FULL global batch unless the first one predicts that warm-up + timed steps
    # would not fit the budget; only then is a slice of the batch timed and the line says so.
    step(64)                                             # page in, build the thread pool
    batch, extrapolated, ran_full_probe = GLOBAL_BATCH, False, False
    n_steps = max(args.warmup, 1) + max(args.steps, 1)
    if args.ref_batch:
        batch, extrapolated = args.ref_batch, args.ref_batch != GLOBAL_BATCH
    else:
        per_sample = step(256) / 256                     # probe: over-estimates the full step (fixed costs spread over fewer samples)
        if per_sample * GLOBAL_BATCH * n_steps > args.ref_budget_s:
            first = step(GLOBAL_BATCH) if kind == "reference" and per_sample * GLOBAL_BATCH < args.ref_budget_s / 4 else None
            ran_full_probe = first is not None
            if first is not None and first * n_steps <= args.ref_budget_s:
                pass
            else:
                if first is not None:
                    per_sample = first / GLOBAL_BATCH
                fit = args.ref_budget_s / (n_steps * per_sample)
                batch = min(GLOBAL_BATCH, max(64, 1 << int(np.floor(np.log2(max(fit, 64))))))
                extrapolated = batch != GLOBAL_BATCH
    for _ in range(max(args.warmup, 1) - (1 if ran_full_probe and not extrapolated else 0)):   # the full-batch probe was a warm-up step
        step(batch)
    times = [step(batch) for _ in range(max(args.steps, 1))]
    sec = statistics.median(times)
    value = batch / sec
    sample = (f"{batch} of {GLOBAL_BATCH} samples per step through the reference's autograd C ABI "
              f"(weights re-uploaded as leaves, softmax to NumPy, seed from NumPy, SGD in NumPy), median of {len(times)}; "
              f"the reference caps its forward sgemm at 12 threads")
    line = {
        "impl": "reference", "metric": "train_samples_per_sec", "value": value, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3 * GLOBAL_BATCH / batch,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus), "extrapolated": extrapolated,
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": host_threads(), "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    return {"workload": "large data-parallel MLP 4096-4096-4096-4096-1000, relu, softmax cross-entropy, SGD lr 0.1 "
                        "(BASELINE.json configs[3])",
            "global_batch": GLOBAL_BATCH, "per_gpu_batch": GLOBAL_BATCH // n_gpus, "parallelism": f"dp{n_gpus}",
            "seed": 3, "l2": "inputs larger than L2: each step streams 218 MB of weights, 218 MB of gradients "
                             "and the activations, no flush needed"}


# ------------------------------------------------------------------ our arm
def gemm_block(ns, peaks, cases=((1024, 5), (4096, 5))):
    """Forward + backward GEMM throughput (C = A*B, dA = dC*B^T, dB = A^T*dC).  A case is
    (n, reps) for a square problem or ((M, K, N), reps).  Each timed pass runs over enough
    independent operand sets that the pass as a whole touches more than L2 holds (300 MB),
    back to back, so that small problems are timed on the GPU and not on the host's launch
    path.  Every case is reported against both roofs: tensor (6MNK over the TF32 peak) and
    HBM (12(MK+KN+MN) bytes, each operand read and each result written once per product,
    over the measured copy bandwidth); `bound` names the one that allows less."""
    out = []
    tf32_peak = peaks["bf16_tflops"] / 2.0
    hbm = peaks["hbm_gbs"]
    for shape, reps in cases:
        m, k, n = (shape, shape, shape) if isinstance(shape, int) else shape
        bytes_alg = 12.0 * (m * k + k * n + m * n)
        sets = max(1, -(-300 * 1024 * 1024 // int(bytes_alg / 3)))
        sets = min(sets, 64)
        ops = []
        for i in range(sets):
            if isinstance(shape, int):
                a, b, dc = W.config_gemm(n, 1000 + i) if i else W.config_gemm(n, 1 if n == 1024 else 4)
            else:
                a, b, dc = W.config_gemm_shape(m, k, n, 4 + 1000 * i)
            ops.append((ns.Node.leaf(a, True), ns.Node.leaf(b, True), ns.Tensor.from_np(dc)))
        times = []
        for r in range(reps + 3):
            e0, e1 = ns.LIB.ttb_event_create(), ns.LIB.ttb_event_create()
            ns.LIB.ttb_event_record(e0)
            for an, bn, dct in ops:
                c = an.matmul(bn)
                c.backward(dct)
                c.release(); an.zero_grad(); bn.zero_grad()
            ns.LIB.ttb_event_record(e1)
            ms = ns.LIB.ttb_event_elapsed_ms(e0, e1) / sets
            ns.LIB.ttb_event_destroy(e0); ns.LIB.ttb_event_destroy(e1)
            if r >= 3:
                times.append(ms)
        med = statistics.median(times)
        tflops = 6.0 * m * k * n / (med * 1e-3) / 1e12
        gbs = bytes_alg / (med * 1e-3) / 1e9
        t_tensor, t_hbm = 6.0 * m * k * n / (tf32_peak * 1e12), bytes_alg / (hbm * 1e9)
        out.append({"shape": [m, k, n], "ms": med, "operand_sets_per_pass": sets, "tflops": tflops,
                    "frac_of_tf32_peak": tflops / tf32_peak,
                    "algorithmic_gbs": gbs, "frac_of_hbm_peak": gbs / hbm,
                    "bound": "hbm" if t_hbm > t_tensor else "tensor"})
        for an, bn, dct in ops:
            an.release(); bn.release(); dct.release()
    return out


# dram__bytes_read.sum + dram__bytes_write.sum per tcgen05 GEMM launch, averaged over the launches of
# one step of this workload at N GPUs (ncu, one step captured; see the named summary).  None: not captured.
MLP_GEMM_TRAFFIC = {1: 648.1e6}
MLP_GEMM_TRAFFIC_SOURCE = "profiles/mlp_step_gemm_dram_traffic.md (ncu, the 11 GEMM launches of one step; 331 MB algorithmic per launch)"
# sm__pipe_tensor_cycles_active of the pair kernel, from the ncu capture named here (not an estimate)
TENSOR_PIPE_NCU = {"value": 0.713, "case": "4096^3 forward + backward, gemm_tc2_kernel, sm__pipe_tensor_cycles_active % of elapsed (70.3 / 71.5 / 72.0)",
                   "source": "profiles/gemm_tc2_kernel_square4096.md"}


def weights_checksum(ws, samples_per_param=25):
    """float64 checksums of every parameter plus a few fixed entries: equal (to rounding of the
    different reduction orders) for every number of GPUs after the same number of steps.  The norms
    are the figures to compare across N; a plain sum of zero-mean weights is 5e-4 of their absolute
    sum, so it magnifies the same differences two thousand times and is not reported."""
    rng = np.random.default_rng(12345)
    out = {"abs_sum": [], "l2": [], "samples": [], "replicas_max_abs_diff": 0.0}
    for w in ws:
        w64 = w.astype(np.float64)
        out["abs_sum"].append(float(np.abs(w64).sum()))
        out["l2"].append(float(np.sqrt((w64 * w64).sum())))
        idx = rng.integers(0, w.size, size=samples_per_param)
        out["samples"].extend(float(v) for v in w.reshape(-1)[idx])
        out["replicas_max_abs_diff"] = max(out["replicas_max_abs_diff"], D.max_abs_diff_from_rank0(w))
    out["replicas_identical"] = out["replicas_max_abs_diff"] == 0.0
    return out


def run_ours(args):
    import tinytorch_b200
    rank, world, local = D.init_process_group("gloo") if int(os.environ.get("WORLD_SIZE", "1")) > 1 else (0, 1, 0)
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    ns = tinytorch_b200.default()
    if ns.device_count() < 1:
        raise SystemExit("bench.py: no CUDA device visible; this library has no CPU path")
    ns.status(ns.LIB.ttb_init(local), "ttb_init")
    # TT_DP_PEER=1: gradients go through the library's peer-memory all-reduce instead of ncclAllReduce
    peer_floats = (DIMS[0] + 1) * DIMS[1] if os.environ.get("TT_DP_PEER", "0") == "1" else 0
    D.connect(ns, rank, world, peer_floats=peer_floats)
    peaks, peak_kind = load_peaks()
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()                     # polls for the whole run; only the timed windows are kept

    x, y, ws = W.config_mlp_large(batch=GLOBAL_BATCH)
    lo, hi = D.shard_rows(GLOBAL_BATCH, rank, world)
    b = hi - lo
    xs, ys = np.ascontiguousarray(x[lo:hi]), y[lo:hi].astype(np.float32)
    del x
    trainer = W.MLPTrainer(ns, ws, lr=LR, global_batch=GLOBAL_BATCH, fused_sgd=os.environ.get("TT_FUSED_SGD", "1") != "0")
    x_dev, y_dev = ns.Tensor.from_np(xs), ns.Tensor.from_np(ys)

    def resident_step():
        loss = trainer.step(x_dev, y_dev)
        return loss

    # -------- device-resident timing
    for _ in range(args.warmup):
        resident_step().release()
    ns.sync(); D.barrier()
    # what the host needs to enqueue a step, measured on two steps into an empty launch queue (in the
    # timed loop below the queue fills and the host is paced by the GPU, which says nothing about it)
    host_t0 = time.perf_counter()
    for _ in range(2):
        resident_step().release()
    host_enqueue_ms = (time.perf_counter() - host_t0) * 1e3 / 2
    ns.sync(); D.barrier()
    window0 = time.time()
    ns.LIB.ttb_trace_reset(); ns.LIB.ttb_trace_enable(1)
    launches0 = ns.LIB.ttb_launch_count()
    e0, e1 = ns.LIB.ttb_event_create(), ns.LIB.ttb_event_create()
    ns.LIB.ttb_event_record(e0)
    last = None
    for _ in range(args.steps):
        if last is not None:
            last.release()
        last = resident_step()
    ns.LIB.ttb_event_record(e1)
    ms_total = ns.LIB.ttb_event_elapsed_ms(e0, e1)
    ns.sync(); D.barrier()
    launches = ns.LIB.ttb_launch_count() - launches0
    comm = ns.comm_read() if world > 1 else None
    ns.LIB.ttb_trace_enable(0)
    # the loss of the last timed step over the GLOBAL batch: every rank holds the mean over its own rows
    final_loss = D.all_sum([float(last.to_np()[0]) * b])[0] / GLOBAL_BATCH
    last.release()
    # the parameters after warm-up + 2 + timed steps: float64 checksums (comparable across N: the same
    # number of steps has run on the same global batch) and the largest difference between replicas
    checksum = None if args.no_checksum else weights_checksum(trainer.weights())
    ms_total = D.all_max(float(ms_total))
    ms_step = ms_total / args.steps
    value = GLOBAL_BATCH / (ms_step * 1e-3)
    tc_ms, tc_n, tc_work = ns.trace_read(0)
    simt_ms, simt_n, _ = ns.trace_read(1)
    classes = {}
    for kind, name in enumerate(["gemm_tcgen05", "gemm_exact_fp32", "elementwise", "softmax", "spatial", "reduce", "optimizer"]):
        ms, n, work = ns.trace_read(kind)
        if n:
            classes[name] = {"ms_per_step": ms / args.steps, "launches_per_step": n / args.steps}

    # -------- end to end: pinned host inputs in, loss out, every step.  Two device buffers used in
    # turn: the copy of step i+1's shard runs on the copy stream under step i's kernels (the input
    # pipeline a training loop would run); every step's inputs still cross PCIe inside the timed region.
    x_pin, y_pin = ns.pinned_array(xs.shape), ns.pinned_array(ys.shape)
    x_pin[...] = xs; y_pin[...] = ys
    xbuf = [ns.Tensor.zeros(xs.shape), ns.Tensor.zeros(xs.shape)]
    ybuf = [ns.Tensor.zeros(ys.shape), ns.Tensor.zeros(ys.shape)]

    loss_pin = ns.pinned_array((2,))

    def e2e_run(n):
        """Every step: its inputs cross PCIe on the copy stream under the previous step's kernels, and
        its loss crosses back (4 bytes) on the same stream; the host looks at step i-1's loss after it
        has enqueued step i, so the GPU never waits for the host."""
        ns.upload_async(xbuf[0], x_pin); ns.upload_async(ybuf[0], y_pin)
        v = None
        prev = None                                                  # loss tensor whose copy is in flight
        for i in range(n):
            if i + 1 < n:
                ns.upload_async(xbuf[(i + 1) % 2], x_pin); ns.upload_async(ybuf[(i + 1) % 2], y_pin)
            loss = trainer.step(xbuf[i % 2], ybuf[i % 2])
            if prev is not None:
                ns.download_wait()                                  # step i-1's loss has landed
                v = float(loss_pin[(i - 1) % 2])
                prev.release()
            ns.download_async(loss, loss_pin[i % 2:i % 2 + 1])       # device -> host read of this step's result
            prev = loss
        if prev is not None:
            ns.download_wait()
            v = float(loss_pin[(n - 1) % 2])
            prev.release()
        return v

    e2e_run(min(args.warmup, 3))
    ns.sync(); D.barrier()
    t0 = time.perf_counter()
    ns.LIB.ttb_event_record(e0)
    e2e_run(args.steps)
    ns.LIB.ttb_event_record(e1)
    e2e_ms = ns.LIB.ttb_event_elapsed_ms(e0, e1)
    ns.sync(); D.barrier()
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = D.all_max(float(max(e2e_ms, e2e_wall_ms)))
    clock_info = clocks.stop((window0, time.time())) if rank == 0 else None
    e2e_value = GLOBAL_BATCH / (e2e_ms / args.steps * 1e-3)

    if world > 1:
        # every rank ends communication together (peer blocks are closed by all before any is freed)
        trainer.close()
        D.finalize(ns)
    if rank != 0:
        return

    tf32_peak = peaks["bf16_tflops_sustained"] / 2.0
    achieved = (tc_work / 1e12) / (tc_ms * 1e-3) if tc_ms > 0 else 0.0
    flops_step = W.mlp_flops_per_sample(DIMS, observable=True) * GLOBAL_BATCH
    line = {
        "metric": "train_samples_per_sec", "value": value, "unit": "samples/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(world),
        "fwd_bwd_tflops": flops_step / (ms_step * 1e-3) / 1e12,
        "fwd_bwd_tflops_frac_of_tf32_peak": flops_step / (ms_step * 1e-3) / 1e12 / (tf32_peak * world),
        "final_loss": final_loss, "weights_checksum": checksum,
        "host_enqueue_ms_per_step": host_enqueue_ms,
        "roofline": {
            "kernel": "gemm_tc2_kernel (tcgen05.mma.cta_group::2 kind::tf32 on CTA pairs, 3xTF32 split, TMA-staged)",
            "bound": "tensor", "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s",
            "frac": achieved / tf32_peak if tf32_peak else None, "traffic": MLP_GEMM_TRAFFIC.get(world),
            "launches": tc_n, "avg_launch_ms": tc_ms / tc_n if tc_n else None,
            "peak_source": f"{peak_kind} bf16_tflops_sustained / 2 (no TF32 figure is recorded; TF32 dense is half of bf16)",
            "note": "achieved counts algorithmic FLOPs (2MNK per GEMM); the 3xTF32 split issues three MMAs per "
                    "product, so a kernel whose tensor pipe never idles reads 0.333 here",
            "traffic_source": MLP_GEMM_TRAFFIC_SOURCE if MLP_GEMM_TRAFFIC.get(world) else None,
            "tensor_pipe_active_ncu": TENSOR_PIPE_NCU,
        },
        "kernel_classes": classes,
        "e2e": {"value": e2e_value, "unit": "samples/s", "h2d_bytes_per_step": int(xs.nbytes + ys.nbytes) * world,
                "d2h_bytes_per_step": 4 * world, "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": int(launches),
        "clocks": clock_info,
    }
    if comm is not None and comm["collectives"]:
        # rank 0's view of its collectives: CUDA-event pairs on the communication stream (the wait for
        # the slowest rank is inside them), bus bandwidth 2(G-1)/G * bytes / time, and per step the time
        # the communication stream ran on after the compute stream's last kernel (what was not hidden)
        sec = comm["collective_ms"] * 1e-3
        line["comm"] = {
            "allreduces_per_step": comm["collectives"] / args.steps,
            "bytes_per_step": comm["bytes"] / args.steps,
            "collective_ms_per_step": comm["collective_ms"] / args.steps,
            "longest_collective_ms": comm["longest_collective_ms"],
            "bus_gbs": (2.0 * (world - 1) / world) * comm["bytes"] / sec / 1e9 if sec > 0 else None,
            "exposed_ms": comm["exposed_ms"] / max(comm["joins"], 1),
            "transport": "peer-memory kernel" if peer_floats else "ncclAllReduce",
            "nccl_max_ctas": os.environ.get("NCCL_MAX_CTAS"),
        }
    if world == 1:
        if not args.no_gemm:
            line["gemm_fwd_bwd"] = gemm_block(ns, peaks)
        if not args.no_cpu_baseline:
            step, kind = reference_step_fn()
            batch = args.ref_batch or (GLOBAL_BATCH if kind == "reference" else 256)   # the scalar port is far slower
            step(64)                                     # page in, build thread pool
            sec = step(batch)
            line["cpu_baseline"] = {
                "value": batch / sec, "unit": "samples/s", "cores": host_threads(), "kind": kind,
                "sample": f"one step on {batch} of {GLOBAL_BATCH} samples on the host cores ({sec:.2f} s); "
                          f"the reference caps its forward sgemm at 12 threads"}
        trainer.close()
        ns.LIB.ttb_dist_finalize()
    print(json.dumps(line), flush=True)


def run_gemm(args):
    """Isolated forward + backward GEMM (BASELINE.json configs[1] and the square
    sizes of configs[4]); also the small case the ncu captures run."""
    import tinytorch_b200
    ns = tinytorch_b200.default()
    if ns.device_count() < 1:
        raise SystemExit("bench.py: no CUDA device visible; this library has no CPU path")
    peaks, peak_kind = load_peaks()
    if args.workload == "gemm-sweep":
        # BASELINE.json configs[4]: every shape of the sweep, one line
        rows = gemm_block(ns, peaks, cases=tuple(((m, k, n), 3) for m, k, n in W.GEMM_SWEEP))
        line = {"metric": "gemm_fwd_bwd_tflops", "value": statistics.median([r["tflops"] for r in rows]), "unit": "TFLOP/s",
                "n_gpus": 1, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "GEMM forward + backward shape sweep (BASELINE.json configs[4]); shapes are [M, K, N]",
                           "l2": "independent operand sets per timed pass, more than L2 holds"},
                "peak": {"tf32_tflops": peaks["bf16_tflops"] / 2.0, "hbm_gbs": peaks["hbm_gbs"], "source": peak_kind},
                "shapes": rows, "gpu_launches": int(ns.LIB.ttb_launch_count())}
        print(json.dumps(line), flush=True)
        return
    shape = tuple(int(v) for v in args.gemm_shape.split(",")) if args.gemm_shape else args.gemm_n
    res = gemm_block(ns, peaks, cases=((shape, max(args.steps, 1)),))[0]
    name = "x".join(map(str, res["shape"])) + " (M x K x N)"
    hbm_bound = res["bound"] == "hbm"
    line = {"metric": "gemm_fwd_bwd_tflops", "value": res["tflops"], "unit": "TFLOP/s", "n_gpus": 1,
            "steps": args.steps, "warmup": 3, "ms_per_step": res["ms"], "higher_is_better": True,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"isolated GEMM forward + backward, {name}",
                       "l2": f"{res['operand_sets_per_pass']} independent operand sets per timed pass, more than L2 holds"},
            "roofline": ({"bound": "hbm", "achieved": res["algorithmic_gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                          "frac": res["frac_of_hbm_peak"], "traffic": None,
                          "peak_source": f"{peak_kind} hbm_gbs (copy)"} if hbm_bound else
                         {"bound": "tensor", "achieved": res["tflops"], "peak": peaks["bf16_tflops"] / 2.0, "unit": "TFLOP/s",
                          "frac": res["frac_of_tf32_peak"],
                          # dram__bytes_read.sum + dram__bytes_write.sum per launch, from the ncu capture of this
                          # very case (square 4096); other sizes were not captured
                          "traffic": 383.0e6 if res["shape"] == [4096, 4096, 4096] else None,
                          "algorithmic_bytes": 4.0 * (res["shape"][0] * res["shape"][1] + res["shape"][1] * res["shape"][2] + res["shape"][0] * res["shape"][2]),
                          "peak_source": f"{peak_kind} bf16_tflops / 2 (burst: kernel timed alone)"}),
            "gpu_launches": int(ns.LIB.ttb_launch_count())}
    print(json.dumps(line), flush=True)


def _time_op(ns, fn, reps=10, warm=3):
    """Median CUDA-event time (ms) of fn(), which enqueues work and returns tensors to release."""
    times = []
    for r in range(reps + warm):
        e0, e1 = ns.LIB.ttb_event_create(), ns.LIB.ttb_event_create()
        ns.LIB.ttb_event_record(e0)
        outs = fn()
        ns.LIB.ttb_event_record(e1)
        ms = ns.LIB.ttb_event_elapsed_ms(e0, e1)
        ns.LIB.ttb_event_destroy(e0); ns.LIB.ttb_event_destroy(e1)
        for t in outs:
            t.release()
        if r >= warm:
            times.append(ms)
    return statistics.median(times)


def run_kernels(args):
    """HBM-bound kernels of the path, one by one, at the sizes the CNN and the large
    MLP use them (inputs larger than L2 where the configuration allows): achieved
    algorithmic GB/s against the measured copy bandwidth, and the oracle on one
    host thread beside each."""
    import tinytorch_b200
    from oracle import oracle as O
    ns = tinytorch_b200.default()
    if ns.device_count() < 1:
        raise SystemExit("bench.py: no CUDA device visible; this library has no CPU path")
    peaks, peak_kind = load_peaks()
    hbm = peaks["hbm_gbs"]
    rng = np.random.default_rng(0)
    T = ns.Tensor.from_np
    rows = []

    small = bool(args.small)                      # a quarter of the rows / images, two launches each: the case a profiler captures
    SM_ROWS = 32768 if small else 65536
    B = 512 if small else 2048

    def add(name, nbytes, fn, cpu_fn=None, cpu_scale=1.0):
        ms = _time_op(ns, fn, reps=1, warm=1) if small else _time_op(ns, fn)
        gbs = nbytes / (ms * 1e-3) / 1e9
        row = {"kernel": name, "bytes": int(nbytes), "ms": ms, "gbs": gbs, "frac_of_hbm_peak": gbs / hbm}
        if cpu_fn is not None and not args.no_cpu_baseline:
            t0 = time.perf_counter(); cpu_fn(); dt = time.perf_counter() - t0
            row["cpu_oracle_ms"] = dt * 1e3 * cpu_scale
        rows.append(row)

    # large MLP activations: [8192, 4096] = 134 MB
    x = rng.standard_normal((8192, 4096)).astype(np.float32); g = rng.standard_normal((8192, 4096)).astype(np.float32)
    xt, gt = T(x), T(g)
    part = slice(0, 512)
    add("relu [8192,4096]", 8 * x.size, lambda: [ns.Tensor(ns.LIB.tt_relu(xt.ptr))], lambda: O.relu(x[part]), 16)
    add("relu_bwd [8192,4096]", 12 * x.size, lambda: [ns.relu_bwd(xt, gt)], lambda: O.relu_bwd(x[part], g[part]), 16)
    add("colsum [8192,4096]", 4 * x.size, lambda: [ns.colsum(gt)])
    w = T(x[:4097]); gw = T(g[:4097])
    add("sgd [4097,4096]", 12 * 4097 * 4096, lambda: (ns.sgd_step(w, gw, 0.1), [])[1])
    for t in (xt, gt, w, gw):
        t.release()
    # the spatial and softmax tensors of the configurations are 30-80 MB and take 10-20 us, less than the
    # host needs to enqueue the next launch; they are scaled up eightfold (same row and plane shapes, more
    # rows / images) so that the timing sees the kernel and not the launch path
    z = rng.standard_normal((SM_ROWS, 1000)).astype(np.float32); y = rng.integers(0, 1000, size=SM_ROWS).astype(np.float32)
    zt, yt = T(z), T(y)
    add(f"softmax_xent [{SM_ROWS},1000]", 8 * z.size, lambda: list(ns.softmax_xent(zt, yt, 1.0 / 8192)), lambda: O.softmax(z[part]), SM_ROWS / 512)
    add(f"softmax [{SM_ROWS},1000]", 8 * z.size, lambda: [ns.Tensor(ns.LIB.tt_softmax(zt.ptr))])
    zt.release(); yt.release()
    # CNN tensors, 2048 images
    a1 = rng.standard_normal((B, 32, 32, 32)).astype(np.float32)              # conv1 output
    a1t = T(a1)
    g1 = rng.standard_normal((B, 32, 16, 16)).astype(np.float32); g1t = T(g1)
    add(f"maxpool 2x2 [{B},32,32,32]", 4 * (a1.size + g1.size), lambda: [ns.Tensor(ns.LIB.tt_maxpool2d(a1t.ptr, 2, 2, 2, 2))],
        lambda: O.maxpool(a1[:16], 2, 2, 2, 2), B / 16)
    add(f"maxpool_bwd 2x2 [{B},32,32,32]", 4 * (2 * a1.size + g1.size), lambda: [ns.maxpool_bwd(a1t, g1t, 2, 2, 2, 2)],
        lambda: O.maxpool_bwd(a1[:16], g1[:16], 2, 2, 2, 2), B / 16)
    a1t.release(); del a1
    p1 = g1; p1t = g1t                                                          # conv2 input has the same shape
    col_bytes = 4 * (288 * B * 256)
    add(f"im2col 3x3 p1 [{B},32,16,16]", col_bytes + 4 * p1.size, lambda: [ns.im2col(p1t, 3, 3, 1, 1, 1, 1)],
        lambda: O.im2col(p1[:16], 3, 3, 1, 1, 1, 1), B / 16)
    colt = ns.im2col(p1t, 3, 3, 1, 1, 1, 1)
    add(f"col2im 3x3 p1 [{B},32,16,16]", col_bytes + 4 * p1.size, lambda: [ns.col2im(colt, B, 32, 16, 16, 3, 3, 1, 1, 1, 1)])
    for t in (g1t, colt):
        t.release()
    line = {"metric": "hbm_bound_kernels_gbs", "value": statistics.median([r["gbs"] for r in rows]), "unit": "GB/s",
            "n_gpus": 1, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "memory-bound kernels of the training path, one by one", "l2": "operands 130-700 MB"},
            "peak": {"hbm_gbs": hbm, "source": peak_kind}, "kernels": rows, "gpu_launches": int(ns.LIB.ttb_launch_count())}
    print(json.dumps(line), flush=True)


def run_cnn(args):
    """BASELINE.json configs[2]: the CNN forward + backward at batch 256, driven the
    way the reference's CIFAR gate drives it (leaves from NumPy each step, softmax to
    NumPy, seed from NumPy, gradients back to NumPy), against the reference library
    doing the same on the host cores."""
    import tinytorch_b200
    ns = tinytorch_b200.default()
    if ns.device_count() < 1:
        raise SystemExit("bench.py: no CUDA device visible; this library has no CPU path")
    x, y, p = W.config_cnn(256)
    for _ in range(3):
        W.cnn_step_reference_style(ns, x, y, p)
    ns.sync()
    l0 = ns.LIB.ttb_launch_count()
    times = []
    for _ in range(max(args.steps, 1)):
        t0 = time.perf_counter()
        r = W.cnn_step_reference_style(ns, x, y, p)
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    line = {"metric": "cnn_fwd_bwd_samples_per_sec", "value": 256 / sec, "unit": "samples/s", "n_gpus": 1,
            "steps": args.steps, "warmup": 3, "ms_per_step": sec * 1e3, "higher_is_better": True, "dtype": "f32",
            "data": "synthetic", "loss": r["loss"],
            "config": {"workload": "CNN conv3x3(3->32) relu pool conv3x3(32->64) relu pool fc4096->256 relu fc256->10, "
                                   "batch 256, host arrays in and gradients out every step (BASELINE.json configs[2])"},
            "e2e": {"value": 256 / sec, "unit": "samples/s",
                    "h2d_bytes_per_step": int(x.nbytes + sum(v.nbytes for v in p.values()) + 256 * 10 * 4),
                    "d2h_bytes_per_step": int(sum(v.nbytes for v in p.values()) + 2 * 256 * 10 * 4)},
            "gpu_launches": int(ns.LIB.ttb_launch_count() - l0)}
    # the same step with parameters resident and the loss seed and SGD on the device
    tr = W.CNNTrainer(ns, p, lr=0.01)
    xt, yt = ns.Tensor.from_np(x), ns.Tensor.from_np(y.astype(np.float32))
    for _ in range(3):
        tr.step(xt, yt).release()
    ns.sync()
    e0, e1 = ns.LIB.ttb_event_create(), ns.LIB.ttb_event_create()
    l1 = ns.LIB.ttb_launch_count()
    reps = max(args.steps, 1)
    ns.LIB.ttb_event_record(e0)
    for _ in range(reps):
        tr.step(xt, yt).release()
    ns.LIB.ttb_event_record(e1)
    ms = ns.LIB.ttb_event_elapsed_ms(e0, e1) / reps
    launches_per_step = int(ns.LIB.ttb_launch_count() - l1) // reps
    # where the GPU time of a step goes (a second, traced pass: the event pairs cost host time)
    ns.LIB.ttb_trace_reset(); ns.LIB.ttb_trace_enable(1)
    for _ in range(reps):
        tr.step(xt, yt).release()
    classes = {}
    for kind, name in enumerate(["gemm_tcgen05", "gemm_exact_fp32", "elementwise", "softmax", "spatial", "reduce", "optimizer"]):
        cms, n, _ = ns.trace_read(kind)
        if n:
            classes[name] = {"ms_per_step": cms / reps, "launches_per_step": n / reps}
    ns.LIB.ttb_trace_enable(0)
    line["device_resident"] = {"value": 256 / (ms * 1e-3), "unit": "samples/s", "ms_per_step": ms,
                               "launches_per_step": launches_per_step, "kernel_classes": classes,
                               "what": "parameters stay on the device, fused softmax-cross-entropy seed, SGD kernels; CUDA events"}
    tr.close(); xt.release(); yt.release()
    if not args.no_cpu_baseline:
        from oracle import oracle as O
        ref = O.load_ref()
        xs, ys = x[:64], y[:64]
        t0 = time.perf_counter()
        if ref is not None:
            W.cnn_step_reference_style(ref, xs, ys, p); kind = "reference"
        else:
            O.cnn_step(xs, ys, p); kind = "port"
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": 64 / dt, "unit": "samples/s", "cores": host_threads(), "kind": kind,
                                "sample": "one step on 64 of the 256 samples"}
    print(json.dumps(line), flush=True)


def main():
    global GLOBAL_BATCH
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--ref-batch", type=int, default=0,
                    help="samples per CPU step of the reference arm / CPU baseline; 0 = the full global batch "
                         "(the reference arm falls back to a slice, and says so, only if the run would not fit --ref-budget-s)")
    ap.add_argument("--ref-budget-s", type=float, default=780.0,
                    help="wall-clock the reference arm may spend on warm-up + timed steps")
    ap.add_argument("--global-batch", type=int, default=GLOBAL_BATCH,
                    help="tuning aid: a smaller global batch reproduces the per-GPU shapes of a larger job on fewer GPUs")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gemm", action="store_true")
    ap.add_argument("--no-checksum", action="store_true", help="tuning runs: skip the parameter checksums (218 MB per rank to the host)")
    ap.add_argument("--small", action="store_true",
                    help="kernels workload: a quarter of the rows and images, one warm-up and one timed launch each")
    ap.add_argument("--workload", choices=["mlp", "gemm", "gemm-sweep", "kernels", "cnn"], default="mlp")
    ap.add_argument("--gemm-shape", default="", help="gemm workload: M,K,N instead of the square --gemm-n")
    ap.add_argument("--gemm-n", type=int, default=4096)
    args = ap.parse_args()
    GLOBAL_BATCH = args.global_batch
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in ("gemm", "gemm-sweep"):
        run_gemm(args)
    elif args.workload == "kernels":
        run_kernels(args)
    elif args.workload == "cnn":
        run_cnn(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
