"""Timing of the memory-bound operators at the ResNet-50 (CIFAR shape) sizes, against the HBM roofline.

    python stream_bench.py [--batch 128] [--reps 10] [--no-flush] [--json out.json]

Every operator is called through the C ABI on tensors of the sizes the training step uses and timed with the
library's launch profiler (CUDA events around every kernel on the launching stream). Between calls a 256 MB buffer
is read so that the operands come from HBM, not from the 126 MB L2 (--no-flush leaves them where the previous call
left them, which is how the training step mostly finds them). Achieved GB/s = compulsory bytes / time, where the
compulsory bytes of a call are: every distinct input read once, every output written once, one more read of a
destination that is accumulated into. Per element (4 B floats):

    relu in place 8          relu grad in place 12        same-shape add 12       its grad (both sides) 24
    batch-norm forward 8     batch-norm backward 16       2x2 max-pool 6 per input element (x, y/4, idx/4)
    max-pool backward 10 per input element                SGD step 16 per parameter
"""
import argparse
import ctypes
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

def shapes(batch):
    """(C, H) of every conv output (batch-norm input) and of every residual sum of ResNet-50, with multiplicities."""
    import bench as mod                  # the workload arithmetic lives beside this file
    bn, add = {}, {}
    for (ci, co, k, s, p, h) in mod.resnet50_convs():
        ho = (h + 2 * p - k) // s + 1
        bn[(co, ho)] = bn.get((co, ho), 0) + 1
    for (c, h, n) in ((256, 16, 3), (512, 8, 4), (1024, 4, 6), (2048, 2, 3)):
        add[(c, h)] = n
    return bn, add


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--json", default=None)
    ap.add_argument("--peak-gbs", type=float, default=None, help="HBM denominator; default: MEASURED_PEAKS.json, else 6650")
    args = ap.parse_args()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    peak = args.peak_gbs
    if peak is None:
        p = os.path.join(root, "MEASURED_PEAKS.json")
        peak = json.load(open(p))["hbm_gbs"] if os.path.exists(p) else 6650.0
    import lantern_b200
    lib = lantern_b200.load()
    lib.init(0, 6 << 30)
    relu, add_op = 0, 0                                  # LTB_RELU, LTB_ADD (include/lantern_b200.h)
    flush_n = 64 << 20
    flush = lib.malloc(flush_n * 4)
    flush_out = lib.malloc(256)
    buf = ctypes.create_string_buffer(1 << 16)
    N = args.batch
    rng = np.random.default_rng(0)
    rows, totals = [], {}

    def dev(n, zero=False):
        if zero:
            return lib.malloc(n * 4)
        a = rng.standard_normal(n).astype(np.float32)
        p = lib.malloc_uninit(a.nbytes); lib.h2d(p, a.ctypes.data, a.nbytes); return p

    def timed(name, shape, count, nbytes, fn):
        fn(); fn(); lib.sync()
        lib.profile(1)
        for _ in range(args.reps):
            if not args.no_flush:
                lib.sum(flush, flush_out, flush_n)
            fn()
        lib.profile(0)
        lib.profile_report(buf, 1 << 16)
        kern = {}
        for line in buf.value.decode().strip().split("\n"):
            nm, cnt, ms = line.split("\t")
            if not (nm == "sum_kernel" and not args.no_flush):
                kern[nm] = float(ms) / args.reps * 1e3
        us = sum(kern.values())
        gbs = nbytes / us / 1e3
        rows.append({"op": name, "shape": shape, "count": count, "us": us, "bytes": nbytes, "gbs": gbs, "frac": gbs / peak, "kernels_us": kern})
        t = totals.setdefault(name, [0.0, 0.0]); t[0] += us * count; t[1] += nbytes * count
        print("%-14s %-16s x%-2d %8.1f us %8.1f GB/s %5.1f%%  %s" % (name, shape, count, us, gbs, 100 * gbs / peak,
              " ".join("%s=%.1f" % (k[:24], v) for k, v in kern.items())), flush=True)

    bn_shapes, add_shapes = shapes(N)
    for (c, h), count in bn_shapes.items():
        mark = lib.mark()
        hw = h * h; n = N * c * hw
        x, y, dy, dx = dev(n), dev(n, True), dev(n), dev(n, True)
        gamma, beta, rm, rv, sm, si, dg, db = dev(c), dev(c), dev(c, True), dev(c), dev(c, True), dev(c, True), dev(c, True), dev(c, True)
        tag = "%dx%dx%dx%d" % (N, c, h, h)
        timed("bn_fwd", tag, count, 8 * n, lambda: lib.bn_train_fwd(x, y, gamma, beta, rm, rv, sm, si, N, c, hw, 1e-5, 0.1))
        timed("bn_bwd", tag, count, 16 * n, lambda: lib.bn_bwd(x, dx, dy, gamma, dg, db, sm, si, N, c, hw))
        timed("relu", tag, count, 8 * n, lambda: lib.unary(relu, y, y, n))
        timed("relu_grad", tag, count, 12 * n, lambda: lib.unary_grad(relu, y, dy, y, dy, n, 1))
        lib.reset(mark)
    for (c, h), count in add_shapes.items():
        mark = lib.mark()
        n = N * c * h * h
        a, b, o, da, dbb, do = dev(n), dev(n), dev(n, True), dev(n, True), dev(n, True), dev(n)
        shp = (ctypes.c_int * 4)(N, c, h, h)
        tag = "%dx%dx%dx%d" % (N, c, h, h)
        timed("add", tag, count, 12 * n, lambda: lib.ew_binary(add_op, a, shp, b, shp, o, 4))
        timed("add_grad", tag, count, 24 * n, lambda: lib.ew_binary_grad(add_op, a, da, shp, b, dbb, shp, do, 4))
        lib.reset(mark)
    # 2x2 max-pool after the stem, and the SGD step over the parameter slab
    mark = lib.mark()
    c, h = 64, 32
    n = N * c * h * h
    x, y, idx, dx, dy = dev(n), dev(n // 4, True), lib.malloc(n), dev(n, True), dev(n // 4)
    timed("maxpool", "%dx%dx%dx%d" % (N, c, h, h), 1, 6 * n, lambda: lib.maxpool_fwd(x, y, idx, N, c, h, h, 2, 2, 2, 2, 0))
    timed("maxpool_bwd", "%dx%dx%dx%d" % (N, c, h, h), 1, 10 * n, lambda: lib.maxpool_bwd(dx, dy, idx, n // 4))
    lib.reset(mark)
    mark = lib.mark()
    n = 23520842
    xs, ds = dev(n), dev(n)
    timed("sgd", "%d params" % n, 1, 16 * n, lambda: lib.sgd_step(xs, ds, 0.0, n))
    lib.reset(mark)
    print()
    all_us = all_b = 0.0
    for name, (us, nb) in totals.items():
        print("TOTAL %-12s %8.3f ms per step  %8.1f GB/s  %5.1f%% of %.0f GB/s" % (name, us / 1e3, nb / us / 1e3, 100 * nb / us / 1e3 / peak, peak))
        all_us += us; all_b += nb
    print("TOTAL %-12s %8.3f ms per step  %8.1f GB/s  %5.1f%% of %.0f GB/s" % ("all", all_us / 1e3, all_b / all_us / 1e3, 100 * all_b / all_us / 1e3 / peak, peak))
    if args.json:
        json.dump({"peak_gbs": peak, "flush": not args.no_flush, "rows": rows}, open(args.json, "w"))
    lib.shutdown()


if __name__ == "__main__":
    main()
