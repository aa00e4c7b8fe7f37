"""Implicit-GEMM convolution (forward, weight gradient, input gradient on the tensor cores, no
im2col matrix) against the CPU oracle's literal im2col + GEMM + col2im restatement of
src/ops_spatial.c:71-127 and src/autograd.c:456-553, on geometries chosen to hit every ragged
edge of the gathered tiles: channel counts that are not multiples of 16, tap counts that are not
multiples of 32, position counts that are not multiples of 128, rectangular kernels and images,
strides and paddings other than 1.  Tolerance of the tensor-core path: max|err|/max|ref| <= 1e-4
(reductions up to 8192 terms); weight gradients reduce over N*Hout*Wout positions and are held to
the bar the configuration tests use for such lengths (5e-4)."""
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

#        N   C   H   W   F  kh kw sh sw ph pw
GEOMS = [(16, 3, 32, 32, 32, 3, 3, 1, 1, 1, 1),        # first convolution of the benchmark CNN
         (16, 32, 16, 16, 64, 3, 3, 1, 1, 1, 1),       # second one
         (67, 5, 13, 17, 20, 3, 2, 1, 1, 0, 2),        # ragged everything, stride 1
         (30, 7, 21, 19, 24, 5, 3, 2, 3, 2, 1),        # strides 2 and 3: forward and dW implicit, dX by col2im
         (130, 4, 8, 8, 200, 1, 1, 1, 1, 0, 0)]        # 1x1 kernel, wide filter bank


def _run(tt, x, w, b, g, sh, sw, ph, pw):
    Node = tt.Node
    xn, wn, bn = Node.leaf(x, True), Node.leaf(w, True), Node.leaf(b, True)
    out = xn.conv2d(wn, bn, stride=(sh, sw), pad=(ph, pw))
    out.backward(g)
    res = out.value(), xn.grad(), wn.grad(), bn.grad()
    for n in (out, xn, wn, bn):
        n.release()
    return res


@pytest.mark.parametrize("geom", GEOMS, ids=lambda g: "x".join(map(str, g)))
def test_implicit_conv_matches_the_oracle(tt, orc, geom):
    n, c, h, w_, f, kh, kw, sh, sw, ph, pw = geom
    rng = np.random.default_rng(sum(geom))
    x = rng.standard_normal((n, c, h, w_)).astype(np.float32)
    w = (rng.standard_normal((f, c, kh, kw)) / np.sqrt(c * kh * kw)).astype(np.float32)
    b = rng.standard_normal(f).astype(np.float32)
    want = orc.conv2d(x, w, b, sh, sw, ph, pw)
    g = rng.standard_normal(want.shape).astype(np.float32)
    wdx, wdw, wdb = orc.conv2d_bwd(x, w, g, sh, sw, ph, pw)
    l0 = tt.LIB.ttb_launch_count()
    out, dx, dw, db = _run(tt, x, w, b, g, sh, sw, ph, pw)
    launches = tt.LIB.ttb_launch_count() - l0
    assert rel_err(out, want) <= 1e-4
    assert rel_err(dx, wdx) <= 1e-4
    assert rel_err(dw, wdw) <= 5e-4
    assert rel_err(db, wdb) <= 2e-5
    if sh == 1 and sw == 1:
        # fprop, bias gradient (two kernels), wgrad + its slice reduction, dgrad: no im2col / col2im / permute passes
        assert launches <= 6, launches


def test_implicit_conv_agrees_with_the_im2col_route(tt, tmp_path):
    """The same convolution through the literal route (TT_CONV_IMPLICIT=0 in a child process: im2col,
    tensor-core GEMM, permute; col2im backward): two tensor-core formulations of one sum agree far inside
    the tolerance either has against the reference."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal((32, 32, 16, 16)).astype(np.float32)
    w = (rng.standard_normal((64, 32, 3, 3)) / 17.0).astype(np.float32)
    b = rng.standard_normal(64).astype(np.float32)
    g = rng.standard_normal((32, 64, 16, 16)).astype(np.float32)
    np.savez(tmp_path / "in.npz", x=x, w=w, b=b, g=g)
    script = tmp_path / "literal.py"
    script.write_text(
        "import sys, numpy as np\n"
        "sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + '/tests')\n"
        "import tinytorch_b200\n"
        "from test_gpu_conv import _run\n"
        "d = np.load(sys.argv[2]); tt = tinytorch_b200.default()\n"
        "o, dx, dw, db = _run(tt, d['x'], d['w'], d['b'], d['g'], 1, 1, 1, 1)\n"
        "np.savez(sys.argv[3], o=o, dx=dx, dw=dw, db=db)\n")
    r = subprocess.run([sys.executable, str(script), ROOT, str(tmp_path / "in.npz"), str(tmp_path / "lit.npz")],
                       capture_output=True, text=True, env=dict(os.environ, TT_CONV_IMPLICIT="0"), timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    lit = np.load(tmp_path / "lit.npz")
    out, dx, dw, db = _run(tt, x, w, b, g, 1, 1, 1, 1)
    assert rel_err(out, lit["o"]) <= 2e-5
    assert rel_err(dx, lit["dx"]) <= 2e-5
    assert rel_err(dw, lit["dw"]) <= 2e-5
    assert np.array_equal(db, lit["db"])
