"""Pins the CPU oracle (oracle/tt_oracle.c): against the fixtures generated from
the reference library, and -- where the reference build travelled with the
repository -- against that library itself on fresh random inputs."""
import numpy as np
import pytest

from tinytorch_b200 import workloads as W

# glibc picks its expf variant by CPU; everything that passes through softmax is
# compared to 1e-6 relative instead of bit for bit.
SOFT = dict(rtol=1e-6, atol=1e-8)


def test_elementwise_and_softmax_match_fixtures(orc, golden_ops):
    g = golden_ops
    x, y, r = g["ew_x"], g["ew_y"], g["ew_r"]
    assert np.array_equal(orc.add(x, y), g["add_out"])
    assert np.array_equal(orc.mul(x, y), g["mul_out"])
    assert np.array_equal(orc.mul(r, y), g["mul_gx"]) and np.array_equal(orc.mul(r, x), g["mul_gy"])
    assert np.array_equal(orc.addscalar(x, 1.5), g["addscalar_out"])
    assert np.array_equal(orc.mulscalar(x, -0.7), g["mulscalar_out"])
    assert np.array_equal(orc.mulscalar(r, -0.7), g["mulscalar_gx"])
    assert np.array_equal(orc.relu(x), g["relu_out"])
    assert np.array_equal(orc.relu_bwd(x, r), g["relu_gx"])
    s = orc.softmax(x)
    assert np.allclose(s, g["softmax_out"], **SOFT)
    assert np.allclose(orc.softmax_bwd(g["softmax_out"], r), g["softmax_gx"], **SOFT)
    assert np.array_equal(orc.padones(x), g["padones_out"])
    assert np.array_equal(orc.padones_bwd(g["padones_seed"]), g["padones_gx"])
    e = orc.softmax(g["softmax_edge_in"])
    assert np.allclose(e, g["softmax_edge_out"], **SOFT)
    assert np.all(e[0] == 0.25)


def test_gemms_match_fixtures_bit_for_bit(orc, golden_ops):
    g = golden_ops
    i = 0
    while f"mm{i}_a" in g:
        a, b, s = g[f"mm{i}_a"], g[f"mm{i}_b"], g[f"mm{i}_g"]
        assert np.array_equal(orc.matmul_naive(a, b), g[f"mm{i}_naive"]), i
        assert np.array_equal(orc.sgemm(a, b), g[f"mm{i}_fast"]), i
        assert np.array_equal(orc.sgemm(a, b), g[f"mm{i}_omp"]), i
        assert np.array_equal(orc.sgemm(a, b), g[f"mm{i}_c"]), i
        assert np.array_equal(orc.matmul_nt(s, b), g[f"mm{i}_da"]), i
        assert np.array_equal(orc.matmul_tn(a, s), g[f"mm{i}_db"]), i
        i += 1
    assert i == 8


def test_conv_and_pool_match_fixtures_bit_for_bit(orc, golden_ops):
    g = golden_ops
    for i in range(4):
        n, c, h, w, f, kh, kw, sh, sw, ph, pw = (int(v) for v in g[f"conv{i}_geom"])
        x, wt, b, s = g[f"conv{i}_x"], g[f"conv{i}_w"], g[f"conv{i}_b"], g[f"conv{i}_g"]
        assert np.array_equal(orc.conv2d(x, wt, b, sh, sw, ph, pw), g[f"conv{i}_out"]), i
        dx, dw, db = orc.conv2d_bwd(x, wt, s, sh, sw, ph, pw)
        assert np.array_equal(dx, g[f"conv{i}_dx"]), i
        assert np.array_equal(dw, g[f"conv{i}_dw"]), i
        assert np.array_equal(db, g[f"conv{i}_db"]), i
        col = orc.im2col(x, kh, kw, sh, sw, ph, pw)
        assert col.shape == (c * kh * kw, n * s.shape[2] * s.shape[3])
    for i in range(4):
        n, c, h, w, ph, pw, sh, sw = (int(v) for v in g[f"pool{i}_geom"])
        x, s = g[f"pool{i}_x"], g[f"pool{i}_g"]
        assert np.array_equal(orc.maxpool(x, ph, pw, sh, sw), g[f"pool{i}_max_out"]), i
        dx, idx = orc.maxpool_bwd(x, s, ph, pw, sh, sw)
        assert np.array_equal(dx, g[f"pool{i}_max_dx"]), i
        assert np.array_equal(orc.avgpool(x, ph, pw, sh, sw), g[f"pool{i}_avg_out"]), i
        assert np.array_equal(orc.avgpool_bwd(s, n, c, h, w, ph, pw, sh, sw), g[f"pool{i}_avg_dx"]), i
    x = g["pool_nan_x"]
    assert np.array_equal(orc.maxpool(x, 2, 2, 2, 2), g["pool_nan_out"])
    dx, idx = orc.maxpool_bwd(x, np.ones((1, 1, 2, 2), np.float32), 2, 2, 2, 2)
    assert np.array_equal(dx, g["pool_nan_dx"])
    assert idx.reshape(-1).tolist() == [0, 2, 8, 10]     # nothing beats -Inf: window origins


def test_training_steps_match_fixtures(orc, golden_steps):
    g = golden_steps
    ws = [g["mlp_tiny_w0"], g["mlp_tiny_w1"]]
    r = orc.mlp_step(g["mlp_tiny_x"], g["mlp_tiny_y"], ws, lr=0.1)
    assert np.array_equal(r["logits"], g["mlp_tiny_logits"])
    assert abs(r["loss"] - float(g["mlp_tiny_loss"])) < 1e-6
    for k, want in (("grads", ("mlp_tiny_g0", "mlp_tiny_g1")), ("weights", ("mlp_tiny_nw0", "mlp_tiny_nw1"))):
        for got, name in zip(r[k], want):
            assert np.allclose(got, g[name], **SOFT), name

    x, y, ws = W.config_mlp_small()
    r = orc.mlp_step(x, y, ws, lr=0.1)
    assert np.array_equal(r["logits"], g["cfg1_logits"])
    assert abs(r["loss"] - float(g["cfg1_loss"])) < 1e-6
    assert np.allclose(r["grads"][1], g["cfg1_g1"], **SOFT)
    assert np.allclose(r["grads"][0].reshape(-1)[g["cfg1_g0_idx"]], g["cfg1_g0_val"], **SOFT)
    assert np.allclose(r["weights"][0].reshape(-1)[g["cfg1_g0_idx"]], g["cfg1_nw0_val"], **SOFT)

    x, y, p = W.config_cnn(16)
    r = orc.cnn_step(x, y, p)
    assert np.array_equal(r["logits"], g["cfg3_logits"])
    assert abs(r["loss"] - float(g["cfg3_loss"])) < 1e-6
    for k in ("w1", "b1", "b2", "fc2"):
        assert np.allclose(r["grads"][k], g[f"cfg3_g_{k}"], rtol=1e-5, atol=1e-7), k
    for k in ("w2", "fc1"):
        assert np.allclose(r["grads"][k].reshape(-1)[g[f"cfg3_g_{k}_idx"]], g[f"cfg3_g_{k}_val"],
                           rtol=1e-5, atol=1e-7), k


def test_large_mlp_scaled_matches_fixture(orc, golden_steps):
    g = golden_steps
    x, y, ws = W.config_mlp_large(batch=64)
    r = orc.mlp_step(x, y, ws, lr=0.1, global_batch=64)
    assert abs(r["loss"] - float(g["cfg4_loss"])) < 1e-6
    assert np.array_equal(r["logits"].reshape(-1)[g["cfg4_logits_idx"]], g["cfg4_logits_val"])
    for i, gw in enumerate(r["grads"]):
        assert np.allclose(gw.reshape(-1)[g[f"cfg4_g{i}_idx"]], g[f"cfg4_g{i}_val"], rtol=1e-5, atol=1e-9), i


def test_oracle_equals_reference_library_live(orc, ref):
    """Fresh random inputs through both: bit-identical where no expf is involved."""
    rng = np.random.default_rng(5)
    for m, k, n in [(1, 1, 1), (6, 16, 16), (7, 385, 17), (50, 770, 48), (12, 384, 32), (130, 60, 200)]:
        a = rng.standard_normal((m, k)).astype(np.float32)
        b = rng.standard_normal((k, n)).astype(np.float32)
        dc = rng.standard_normal((m, n)).astype(np.float32)
        want = W.gemm_fwd_bwd(ref, a, b, dc)
        got = orc.gemm_fwd_bwd(a, b, dc)
        for key in want:
            assert np.array_equal(want[key], got[key]), (m, k, n, key)
    x, y, p = W.config_cnn(4)
    want = W.cnn_step_reference_style(ref, x, y, p)
    got = orc.cnn_step(x, y, p)
    assert np.array_equal(want["logits"], got["logits"])
    for key in p:
        assert np.array_equal(want["grads"][key], got["grads"][key]), key
    x, y, ws = W.config_mlp_small()
    want = W.mlp_step_reference_style(ref, x, y, ws)
    got = orc.mlp_step(x, y, ws)
    assert want["loss"] == got["loss"]
    for a, b in zip(want["grads"] + want["weights"], got["grads"] + got["weights"]):
        assert np.array_equal(a, b)
