"""Timing aids that exist only in a library built with `make lib EXTRA=-DTT_TUNING`.

    python -m tinytorch_b200.tuning conv-phases
    python -m tinytorch_b200.tuning gemm-phases [N]

The first prints, for the two convolutions of the CNN workload (batch 256), the clock-cycle stamps the
implicit-GEMM kernel collects in CTA 0: per K block filled by the first producer group the wait for
the stage, the A tile, the B tile and fence + arrive; for the thread that issues the MMAs the total
wait for full stages, issue time, wait for a drained accumulator and kernel time.  The second runs
an N x N x N product (default 4096) on the CTA-pair GEMM kernel and prints CTA 0's cycles per K block
by role (load thread, MMA thread, first split thread) and the absolute clock of each hand-over for
eight consecutive K blocks.  The production library does not export the symbols: the module says so
and stops.
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


def gemm_phases(n=4096):
    import tinytorch_b200
    tt = tinytorch_b200.default()
    try:
        read, trace = tt.LIB.ttb_debug_gemm_read, tt.LIB.ttb_debug_gemm_trace
    except AttributeError:
        raise SystemExit("this library was built without -DTT_TUNING: no phase stamps (make lib EXTRA=-DTT_TUNING)")
    read.argtypes = [ctypes.POINTER(ctypes.c_ulonglong)]
    trace.argtypes = [ctypes.POINTER(ctypes.c_longlong)]

    def stamps():
        buf = (ctypes.c_ulonglong * 24)()
        if read(buf) != 0:
            raise RuntimeError("ttb_debug_gemm_read failed")
        return list(buf)

    rng = np.random.default_rng(0)
    a = tt.Node.leaf(rng.standard_normal((n, n)).astype(np.float32), False)
    b = tt.Node.leaf(rng.standard_normal((n, n)).astype(np.float32), False)
    for _ in range(3):
        stamps()
        c = a.matmul(b)
        c.value_tensor().to_np()                              # a deferred product runs when its value is read
        tt.sync()
        d = stamps()
        c.release()
        k = max(d[12], 1)
        print("K blocks %d | per block: load thread other %.0f wait_empty %.0f | MMA thread issue %.0f wait_raw %.0f "
              "wait_lo %.0f wait_drained %.0f | split thread wait_raw %.0f wait_slot %.0f pass %.0f arrive %.0f"
              % (k, d[0] / k, d[1] / k, d[4] / k, d[5] / k, d[6] / k, d[7] / k, d[9] / k, d[10] / k, d[11] / k, d[8] / k))
        n = max(d[20], 1)
        print("    epilogue warp, per accumulator hand-over (%d): wait_full %.0f  loads and first stores %.0f  arrive %.0f  "
              "remaining stores %.0f" % (n, d[16] / n, d[17] / n, d[18] / n, d[19] / n))
    buf = (ctypes.c_longlong * 96)()
    trace(buf)
    t = list(buf)
    names = {0: "load:stage free", 2: "mma:raw tiles seen", 3: "mma:hi*hi issued", 4: "mma:lo slot seen",
             5: "mma:cross terms issued", 6: "split:raw tiles seen", 7: "split:slot free", 8: "split:pass done",
             9: "relay:pass seen", 10: "relay:arrived at the leader"}
    seen = [v for v in t if v > 0]
    if seen:
        base = min(seen)
        for kb in range(8):
            row = t[kb * 12:(kb + 1) * 12]
            print("K block", 40 + kb, "  ".join("%s=%d" % (names[e], row[e] - base) for e in sorted(names)))


if __name__ == "__main__":
    if len(sys.argv) >= 2 and sys.argv[1] == "conv-phases":
        conv_phases()
    elif len(sys.argv) >= 2 and sys.argv[1] == "gemm-phases":
        gemm_phases(int(sys.argv[2]) if len(sys.argv) > 2 else 4096)
    else:
        raise SystemExit(__doc__)
