"""Per-layer timing of the ResNet-50 (CIFAR shape) convolutions through the C ABI.

    python layer_bench.py [--batch 128] [--reps 10] [--math tf32|fp32] [--table FILE.md]

For every distinct convolution shape of the network it times forward, data-grad and weight-grad separately with the
library's launch profiler (CUDA events around every kernel on the launching stream), flushing the L2 cache between calls,
and prints the time of every kernel the call launched and the achieved TFLOP/s of the call (2*N*Cout*Ho*Wo*Cin*k*k FLOP).
With --table it also writes the rows as a markdown table with, per row, the time no layer-by-layer implementation can go
below on this GPU: the larger of FLOP / (measured TF32 rate) and (both operands + the result, read or written once) /
(measured copy bandwidth), and which of the two it is.
"""
import argparse
import ctypes
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def distinct_convs():
    import bench as mod                  # the workload arithmetic lives beside this file
    counts = {}
    for c in mod.resnet50_convs():
        counts[c] = counts.get(c, 0) + 1
    return counts


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--math", default="tf32")
    ap.add_argument("--json", default=None)
    ap.add_argument("--only", default=None, help="cin,cout,k,stride,h of the one shape to run")
    ap.add_argument("--table", default=None, help="write the rows as a markdown table to this file")
    args = ap.parse_args()
    import lantern_b200
    lib = lantern_b200.load()
    lib.init(0, 8 << 30)
    lib.set_math(1 if args.math == "tf32" else 0)
    flush_n = 64 << 20                                   # 256 MB of floats: larger than the 126 MB L2
    flush = lib.malloc(flush_n * 4)
    flush_out = lib.malloc(256)
    buf = ctypes.create_string_buffer(1 << 16)
    rows, tot = [], {"fwd": [0.0, 0.0], "dgrad": [0.0, 0.0], "wgrad": [0.0, 0.0]}
    N = args.batch
    only = tuple(int(v) for v in args.only.split(",")) if args.only else None
    for (ci, co, k, s, p, h), count in distinct_convs().items():
        if only and only != (ci, co, k, s, h):
            continue
        ho = (h + 2 * p - k) // s + 1
        flops = 2.0 * N * co * ho * ho * ci * k * k
        mark = lib.mark()
        rng = np.random.default_rng(0)
        def dev(shape):
            a = rng.standard_normal(shape).astype(np.float32)
            ptr = lib.malloc_uninit(a.nbytes); lib.h2d(ptr, a.ctypes.data, a.nbytes); lib.sync(); return ptr
        x, w, dy = dev((N, ci, h, h)), dev((co, ci, k, k)), dev((N, co, ho, ho))
        y, dx, dw = lib.malloc(N * co * ho * ho * 4), lib.malloc(N * ci * h * h * 4), lib.malloc(co * ci * k * k * 4)
        calls = {"fwd": lambda: lib.conv2d_fwd(x, w, 0, y, N, ci, h, h, co, k, k, s, s, p, p),
                 "dgrad": lambda: lib.conv2d_bwd(x, dx, w, 0, 0, dy, N, ci, h, h, co, k, k, s, s, p, p),
                 "wgrad": lambda: lib.conv2d_bwd(x, 0, w, dw, 0, dy, N, ci, h, h, co, k, k, s, s, p, p)}
        for name, fn in calls.items():
            if name == "dgrad" and ci == 3:
                continue                                  # the stem's input is a leaf: no data-grad in the training step
            fn(); fn(); lib.sync()
            lib.profile(1)
            for _ in range(args.reps):
                lib.sum(flush, flush_out, flush_n)        # a READ of 256 MB: evicts the operands and leaves clean lines behind
                fn()
            lib.profile(0)
            lib.profile_report(buf, 1 << 16)
            kern = {}
            for line in buf.value.decode().strip().split("\n"):
                nm, cnt, ms = line.split("\t")
                if nm != "sum_kernel":
                    kern[nm] = float(ms) / args.reps * 1e3          # microseconds per call
            us = sum(kern.values())
            nx, nw, ny = N * ci * h * h, co * ci * k * k, N * co * ho * ho
            moved = 4.0 * (nx + nw + ny) + (4.0 * nw if name == "wgrad" else 0.0)      # the weight gradient accumulates: dW is read and written
            rows.append({"shape": [ci, co, k, s, h], "count": count, "pass": name, "us": us, "tflops": flops / us / 1e6, "kernels_us": kern,
                         "flops": flops, "bytes": moved})
            tot[name][0] += us * count; tot[name][1] += flops * count
            print("cin %4d cout %4d k%d s%d h%2d x%d %-5s %8.1f us %7.1f TFLOP/s  %s" % (
                ci, co, k, s, h, count, name, us, flops / us / 1e6, " ".join("%s=%.1f" % (n[:28], v) for n, v in kern.items())), flush=True)
        lib.reset(mark)
    for name, (us, fl) in tot.items():
        print("TOTAL %-5s %.3f ms per step, %.1f TFLOP/s" % (name, us / 1e3, fl / us / 1e6 if us else 0))
    allus = sum(v[0] for v in tot.values()); allfl = sum(v[1] for v in tot.values())
    print("TOTAL all   %.3f ms per step, %.1f TFLOP/s" % (allus / 1e3, allfl / allus / 1e6))
    if args.json:
        json.dump(rows, open(args.json, "w"))
    if args.table:
        import bench as mod
        peaks = mod.measured_peaks()
        tf32, hbm = peaks["bf16_tflops_sustained"] / 2.0, peaks["hbm_gbs"]
        with open(args.table, "w") as f:
            f.write("| Cin | Cout | k | stride | H | layers | pass | us | TFLOP/s | of TF32 rate | bound us | bound by | us / bound | kernels |\n")
            f.write("|---|---|---|---|---|---|---|---|---|---|---|---|---|---|\n")
            t_us = t_bound = 0.0
            for r in rows:
                t_flop, t_byte = r["flops"] / (tf32 * 1e6), r["bytes"] / (hbm * 1e3)
                bound = max(t_flop, t_byte)
                t_us += r["us"] * r["count"]; t_bound += bound * r["count"]
                f.write("| %d | %d | %d | %d | %d | %d | %s | %.1f | %.1f | %.3f | %.1f | %s | %.1f | %d |\n" % (
                    *r["shape"], r["count"], r["pass"], r["us"], r["tflops"], r["tflops"] / tf32, bound,
                    "FLOP" if t_flop >= t_byte else "bytes", r["us"] / bound, len(r["kernels_us"])))
            f.write("\nbatch %d, %s math; rates used for the bound: TF32 %.0f TFLOP/s (half the %s bf16 figure), HBM %.0f GB/s; "
                    "all layers of a step: %.3f ms measured, %.3f ms bound\n" % (N, args.math, tf32, peaks["source"], hbm, t_us / 1e3, t_bound / 1e3))
    lib.shutdown()


if __name__ == "__main__":
    main()
