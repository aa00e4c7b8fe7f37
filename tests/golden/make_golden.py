#!/usr/bin/env python3
"""Generate tests/golden/*.npz from the REFERENCE library itself.

Run in a container that has the reference sources:

    make -C oracle REF=<reference checkout>   # builds oracle/_ref/libtinytorch_ref.so from its sources
    python tests/golden/make_golden.py

Every array written here is an output of the reference's own C code
(oracle/_ref/libtinytorch_ref.so, compiled from its unmodified sources with the
flags of its Makefile), driven through its public C ABI.  The fixtures pin the
CPU oracle (tests/test_oracle.py) and the CUDA path (tests/test_gpu_*.py) on
machines where the reference is not available.  Inputs are seeded; they are
stored next to the outputs so that the fixtures do not depend on NumPy's
generator staying bit-stable.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle as O                      # noqa: E402
from tinytorch_b200 import workloads as W           # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def sample_index(shape, count, seed):
    n = int(np.prod(shape))
    rng = np.random.default_rng(seed)
    return np.sort(rng.choice(n, size=min(count, n), replace=False))


def grads_of(ref, build, arrays, seed):
    """Reference autograd: returns (value, [grad per input])."""
    nodes = [ref.Node.leaf(a, True) for a in arrays]
    out = build(*nodes)
    val = out.value()
    out.backward(seed if seed is not None else None)
    gr = [n.grad() for n in nodes]
    out.release()
    for n in nodes:
        n.release()
    return val, gr


def ops_fixture(ref):
    rng = np.random.default_rng(1234)
    d = {}

    def rnd(*shape):
        return rng.standard_normal(shape).astype(np.float32)

    # elementwise + softmax forward / backward through autograd
    x, y = rnd(5, 7), rnd(5, 7)
    r = rnd(5, 7)
    d["ew_x"], d["ew_y"], d["ew_r"] = x, y, r
    for name, fn in [("add", lambda a, b: a + b), ("mul", lambda a, b: a * b)]:
        v, g = grads_of(ref, fn, [x, y], r)
        d[f"{name}_out"], d[f"{name}_gx"], d[f"{name}_gy"] = v, g[0], g[1]
    for name, fn in [("addscalar", lambda a: a + 1.5), ("mulscalar", lambda a: a * (-0.7)),
                     ("relu", lambda a: a.relu()), ("softmax", lambda a: a.softmax()),
                     ("padones", lambda a: a.padones()), ("reshape", lambda a: a.reshape((7, 5)))]:
        seed = r if name not in ("padones", "reshape") else (
            rnd(5, 8) if name == "padones" else rnd(7, 5))
        d[f"{name}_seed"] = seed
        v, g = grads_of(ref, fn, [x], seed)
        d[f"{name}_out"], d[f"{name}_gx"] = v, g[0]
    sm = np.array([[-np.inf] * 4, [1, 2, 3, 4], [100, 101, 99, 100], [-1e9, -1e9, 0, -1e9]], np.float32)
    t = ref.Tensor.from_np(sm)
    o = ref.Tensor(ref.checked(ref.LIB.tt_softmax(t.ptr), "tt_softmax"))
    d["softmax_edge_in"], d["softmax_edge_out"] = sm, o.to_np()
    t.release(); o.release()

    # the three matmuls on edge shapes (M<6, N<16, K>384, ragged everything)
    shapes = [(3, 4, 5), (17, 13, 5), (7, 7, 7), (5, 300, 3), (9, 256, 33), (64, 512, 16), (13, 800, 40), (6, 16, 16)]
    for i, (m, k, n) in enumerate(shapes):
        a, b, g = rnd(m, k), rnd(k, n), rnd(m, n)
        a[0, 0] = 0.0
        d[f"mm{i}_a"], d[f"mm{i}_b"], d[f"mm{i}_g"] = a, b, g
        ta, tb = ref.Tensor.from_np(a), ref.Tensor.from_np(b)
        for tag, call in [("naive", lambda: ref.LIB.tt_matmul(ta.ptr, tb.ptr)),
                          ("fast", lambda: ref.LIB.tt_matmul_fast(ta.ptr, tb.ptr)),
                          ("omp", lambda: ref.LIB.tt_matmul_omp(ta.ptr, tb.ptr, 4))]:
            o = ref.Tensor(ref.checked(call(), tag))
            d[f"mm{i}_{tag}"] = o.to_np()
            o.release()
        ta.release(); tb.release()
        v, gr = grads_of(ref, lambda p, q: p.matmul(q), [a, b], g)
        d[f"mm{i}_c"], d[f"mm{i}_da"], d[f"mm{i}_db"] = v, gr[0], gr[1]

    # conv / pool forward + backward, several geometries
    convs = [(2, 2, 5, 5, 3, 3, 3, 1, 1, 1, 1), (2, 3, 8, 7, 4, 3, 2, 2, 1, 0, 1), (1, 1, 6, 6, 2, 1, 1, 1, 1, 0, 0),
             (3, 4, 9, 9, 5, 5, 5, 2, 2, 2, 2)]
    for i, (n, c, h, w, f, kh, kw, sh, sw, ph, pw) in enumerate(convs):
        xx, ww, bb = rnd(n, c, h, w), rnd(f, c, kh, kw), rnd(f)
        ho, wo = (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
        g = rnd(n, f, ho, wo)
        d[f"conv{i}_geom"] = np.array([n, c, h, w, f, kh, kw, sh, sw, ph, pw])
        d[f"conv{i}_x"], d[f"conv{i}_w"], d[f"conv{i}_b"], d[f"conv{i}_g"] = xx, ww, bb, g
        v, gr = grads_of(ref, lambda a, b2, c2: a.conv2d(b2, c2, stride=(sh, sw), pad=(ph, pw)), [xx, ww, bb], g)
        d[f"conv{i}_out"], d[f"conv{i}_dx"], d[f"conv{i}_dw"], d[f"conv{i}_db"] = v, gr[0], gr[1], gr[2]
    pools = [(2, 2, 6, 6, 2, 2, 2, 2), (2, 3, 7, 9, 3, 2, 1, 2), (1, 2, 5, 5, 3, 3, 1, 1), (2, 2, 8, 8, 2, 2, 3, 3)]
    for i, (n, c, h, w, ph, pw, sh, sw) in enumerate(pools):
        xx = rnd(n, c, h, w)
        xx[0, 0, :2, :2] = 0.25              # ties: first maximum in scan order must win
        ho, wo = (h - ph) // sh + 1, (w - pw) // sw + 1
        g = rnd(n, c, ho, wo)
        d[f"pool{i}_geom"] = np.array([n, c, h, w, ph, pw, sh, sw])
        d[f"pool{i}_x"], d[f"pool{i}_g"] = xx, g
        for tag, fn in [("max", lambda a: a.maxpool2d((ph, pw), (sh, sw))), ("avg", lambda a: a.avgpool2d((ph, pw), (sh, sw)))]:
            v, gr = grads_of(ref, fn, [xx], g)
            d[f"pool{i}_{tag}_out"], d[f"pool{i}_{tag}_dx"] = v, gr[0]
    nanx = np.full((1, 1, 4, 4), np.nan, np.float32)
    nanx[0, 0, 2:, :] = -np.inf
    v, gr = grads_of(ref, lambda a: a.maxpool2d(2, 2), [nanx], np.ones((1, 1, 2, 2), np.float32))
    d["pool_nan_x"], d["pool_nan_out"], d["pool_nan_dx"] = nanx, v, gr[0]

    # accumulation semantics: z = y + y with y = x*x, two passes give 3x
    xv = np.array([1.0, 2.0, 3.0], np.float32)
    xn = ref.Node.leaf(xv, True)
    yn = xn * xn
    zn = yn + yn
    zn.backward(None)
    d["acc_first"] = xn.grad()
    zn.backward(None)
    d["acc_second"] = xn.grad()
    for n in (zn, yn, xn):
        n.release()
    return d


def steps_fixture(ref):
    d = {}
    # tiny MLP and CNN steps, stored in full
    rng = np.random.default_rng(77)
    x = rng.standard_normal((6, 16)).astype(np.float32)
    y = rng.integers(0, 4, size=6)
    ws = [W.dense_weight(rng, 16, 8), W.dense_weight(rng, 8, 4)]
    ws[0][16] = 0.1
    r = W.mlp_step_reference_style(ref, x, y, ws, lr=0.1)
    d["mlp_tiny_x"], d["mlp_tiny_y"], d["mlp_tiny_w0"], d["mlp_tiny_w1"] = x, y, ws[0], ws[1]
    d["mlp_tiny_loss"] = np.float64(r["loss"])
    d["mlp_tiny_logits"], d["mlp_tiny_g0"], d["mlp_tiny_g1"] = r["logits"], r["grads"][0], r["grads"][1]
    d["mlp_tiny_nw0"], d["mlp_tiny_nw1"] = r["weights"][0], r["weights"][1]

    # configuration 1 in full size: outputs sampled
    x, y, ws = W.config_mlp_small()
    r = W.mlp_step_reference_style(ref, x, y, ws, lr=0.1)
    d["cfg1_loss"] = np.float64(r["loss"])
    d["cfg1_logits"] = r["logits"]
    d["cfg1_g1"] = r["grads"][1]
    idx = sample_index(r["grads"][0].shape, 4096, 11)
    d["cfg1_g0_idx"], d["cfg1_g0_val"] = idx, r["grads"][0].reshape(-1)[idx]
    d["cfg1_g0_sum"] = np.float64(r["grads"][0].astype(np.float64).sum())
    d["cfg1_nw0_val"] = r["weights"][0].reshape(-1)[idx]

    # configuration 2: 1024^3 forward + backward, sampled
    a, b, dc = W.config_gemm(1024, 1)
    r = W.gemm_fwd_bwd(ref, a, b, dc)
    idx = sample_index((1024, 1024), 4096, 12)
    d["cfg2_idx"] = idx
    for k in ("c", "da", "db"):
        d[f"cfg2_{k}_val"] = r[k].reshape(-1)[idx]
        d[f"cfg2_{k}_abs_max"] = np.float64(np.abs(r[k]).max())

    # configuration 3 at batch 16 (same layers as the batch-256 benchmark case)
    x, y, p = W.config_cnn(16)
    r = W.cnn_step_reference_style(ref, x, y, p)
    d["cfg3_loss"] = np.float64(r["loss"])
    d["cfg3_logits"] = r["logits"]
    for k in ("w1", "b1", "b2", "fc2"):
        d[f"cfg3_g_{k}"] = r["grads"][k]
    for k in ("w2", "fc1"):
        idx = sample_index(r["grads"][k].shape, 4096, 13)
        d[f"cfg3_g_{k}_idx"], d[f"cfg3_g_{k}_val"] = idx, r["grads"][k].reshape(-1)[idx]

    # configuration 4 scaled to batch 64 with the real layer widths, sampled
    x, y, ws = W.config_mlp_large(batch=64)
    r = W.mlp_step_reference_style(ref, x, y, ws, lr=0.1, global_batch=64)
    d["cfg4_loss"] = np.float64(r["loss"])
    idx = sample_index(r["logits"].shape, 4096, 14)
    d["cfg4_logits_idx"], d["cfg4_logits_val"] = idx, r["logits"].reshape(-1)[idx]
    for i, g in enumerate(r["grads"]):
        idx = sample_index(g.shape, 2048, 20 + i)
        d[f"cfg4_g{i}_idx"], d[f"cfg4_g{i}_val"] = idx, g.reshape(-1)[idx]
        d[f"cfg4_g{i}_abs_max"] = np.float64(np.abs(g).max())
    return d


def main():
    ref = O.load_ref()
    if ref is None:
        sys.exit("oracle/_ref/libtinytorch_ref.so is missing: run `make -C oracle REF=<reference checkout>`")
    np.savez_compressed(os.path.join(HERE, "ops.npz"), **ops_fixture(ref))
    np.savez_compressed(os.path.join(HERE, "steps.npz"), **steps_fixture(ref))
    for f in ("ops.npz", "steps.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
