"""Timing aids that exist only in a library built with `make lib EXTRA=-DTT_TUNING`.

    python -m tinytorch_b200.tuning conv-phases

prints, for the two convolutions of the CNN workload (batch 256), the clock-cycle stamps the
implicit-GEMM kernel collects in CTA 0: per K block filled by the first producer group the wait for
the stage, the A tile, the B tile and fence + arrive; for the thread that issues the MMAs the total
wait for full stages, issue time, wait for a drained accumulator and kernel time.  The production
library does not export the symbol: the module says so and stops.
"""
import ctypes
import sys

import numpy as np


def conv_phases():
    import tinytorch_b200
    from tinytorch_b200 import workloads as W
    tt = tinytorch_b200.default()
    try:
        read = tt.LIB.ttb_debug_conv_read
    except AttributeError:
        raise SystemExit("this library was built without -DTT_TUNING: no phase stamps (make lib EXTRA=-DTT_TUNING)")
    read.argtypes = [ctypes.POINTER(ctypes.c_ulonglong)]
    read.restype = ctypes.c_int

    def stamps():
        buf = (ctypes.c_ulonglong * 16)()
        if read(buf) != 0:
            raise RuntimeError("ttb_debug_conv_read failed")
        return list(buf)

    def show(what, d):
        n = max(d[4], 1)
        print("%-28s K blocks %3d | per block: wait %5.0f  A %5.0f  B %5.0f  fence+arrive %4.0f | MMA thread: "
              "wait_full %d issue %d wait_drained %d kernel %d"
              % (what, d[4], d[0] / n, d[1] / n, d[2] / n, d[3] / n, d[5], d[6], d[7], d[9]))

    x, _, p = W.config_cnn(256)
    x2 = np.random.default_rng(0).standard_normal((256, 32, 16, 16)).astype(np.float32)
    for name, xin, w, b in (("conv 3->32 on 32x32", x, p["w1"], p["b1"]), ("conv 32->64 on 16x16", x2, p["w2"], p["b2"])):
        xn, wn, bn = tt.Node.leaf(xin, True), tt.Node.leaf(w, True), tt.Node.leaf(b, True)
        for _ in range(2):                                   # the second round is the warm one
            stamps()
            out = xn.conv2d(wn, bn, stride=1, pad=1)
            out.value_tensor().numel()
            tt.sync()
            show(name + " fprop", stamps())
            out.backward(np.ones(out.value_tensor().shape, np.float32))
            tt.sync()
            show(name + " wgrad+dgrad", stamps())
            out.release(); xn.zero_grad(); wn.zero_grad(); bn.zero_grad()


if __name__ == "__main__":
    if len(sys.argv) != 2 or sys.argv[1] != "conv-phases":
        raise SystemExit(__doc__)
    conv_phases()
