#!/usr/bin/env python
"""Benchmark of the ResNet-50 (CIFAR shape) training step through the lantern_b200 C ABI.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...
    python bench.py --impl reference ...        # the CPU path (oracle port of the reference's CPU backend) on the host cores
    --blocks R                                  # the K-step block is timed R times and the median block reported (default: >= 20, ~2 s)

One step = upload of one synthetic batch (128 x 3 x 32 x 32 per GPU, N(0,1), labels uniform 0..9) -> forward ->
backward -> loss read-back -> SGD (lr 0.1) over every parameter tensor, issued by the host program in
lantern_b200/hosts/models.cpp the way Lantern's generated code issues it, replayed from a recorded CUDA graph.
Prints ONE JSON line (rank 0).
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH = 128
LR = 0.1
METRIC = "train samples/s (ResNet-50 CIFAR shape, batch 128 per GPU)"


# --------------------------------------------------------------------------------------------- workload arithmetic
def resnet50_convs():
    """(Cin, Cout, k, stride, pad, Hin) for the 53 convolutions, in forward order."""
    convs = [(3, 64, 3, 1, 1, 32)]
    inpl, h = 64, 16
    for s, (planes, nblk) in enumerate(((64, 3), (128, 4), (256, 6), (512, 3))):
        for i in range(nblk):
            stride = 2 if (i == 0 and s > 0) else 1
            convs.append((inpl, planes, 1, 1, 0, h))
            convs.append((planes, planes, 3, stride, 1, h))
            ho = h // stride
            convs.append((planes, planes * 4, 1, 1, 0, ho))
            if i == 0:
                convs.append((inpl, planes * 4, 1, stride, 0, h))
            inpl, h = planes * 4, ho
    return convs


def step_flops(batch):
    """Algorithmic FLOPs of one training step: 2*N*Cout*Ho*Wo*Cin*k*k per conv pass; forward + weight-grad for all,
    data-grad for all but the stem (its input is a leaf); FC 2048x10 three times."""
    fwd = 0.0
    total = 0.0
    for (ci, co, k, s, p, h) in resnet50_convs():
        ho = (h + 2 * p - k) // s + 1
        f = 2.0 * batch * co * ho * ho * ci * k * k
        fwd += f
        total += 3 * f if ci != 3 else 2 * f
    fc = 2.0 * batch * 2048 * 10
    return fwd + fc, total + 3 * fc


def hbm_bound_bytes(batch):
    """Compulsory bytes of one training step for each class of HBM-bound kernel, keyed by a substring of the kernel's name:
    every distinct input read once, every output written once, one more read of a destination that is accumulated into,
    4 B per element.  With the look-ahead fusion on, the classes are the fused kernels the step really launches:
      bn_fwd*        batch-norm forward (+ ReLU in the same pass)          x, y                          8 B / element
      bn_bwd*        batch-norm backward; where an in-place ReLU gradient joined it the kernel also reads the ReLU output
                     and writes the masked gradient back                  x, dy, dx r/w (+ y, dy w)     16 (24) B / element
      relu_add_grad  ReLU gradient + residual-add gradient                y, d r/w, da r/w, db r/w      28 B / element
                     Gradient buffers of 2^20 elements and more are not zero-filled but written by the first operator that
                     would add into them (ltb_grad_unset: the host program's default), so for those tensors dx, da and db
                     are written only: 12 (20) and 20 B / element.  At fusion level 2 (the host program's default) an absorbed
                     ReLU gradient is not written back: 4 B / element less for the batch norms that absorb one (except the
                     two-sweep kernel of the 33 MB maps) and for relu_add_grad; and in the blocks without a shortcut convolution the
                     batch-norm backward of the last layer absorbs the add gradient altogether, and (level 3) the batch-norm forward of
                     that layer the residual add + ReLU (it reads the shortcut, 4 B / element more, and writes the sum
                     instead of its own result).
      map_vec4       residual add + ReLU                                  a, b, out                     12 B / element
      maxpool_*      2x2 max pool forward (x, y, idx) and backward        6 and 10 B / input element
      sgd_*          x -= lr d; d = 0                                     16 B / parameter"""
    el = {"bn": [], "add": []}
    for (ci, co, k, s, p, h) in resnet50_convs():
        ho = (h + 2 * p - k) // s + 1
        el["bn"].append(batch * co * ho * ho)
    bn_all = float(sum(el["bn"]))
    big = lambda n: n >= (1 << 20)                  # the host program's threshold for a deferred zero fill
    bn_bwd_bytes = float(sum((12.0 if big(n) else 16.0) * n for n in el["bn"]))
    relu_bn = 0.0                                   # BN outputs followed by an in-place ReLU: the stem, and conv1/conv2 of every block
    convs = resnet50_convs()
    i = 1
    relu_bn += el["bn"][0]
    for s_, (planes, nblk) in enumerate(((64, 3), (128, 4), (256, 6), (512, 3))):
        for b_ in range(nblk):
            relu_bn += el["bn"][i] + el["bn"][i + 1]
            i += 4 if b_ == 0 else 3
    add_shapes = ((256, 16, 3), (512, 8, 4), (1024, 4, 6), (2048, 2, 3))
    adds = sum(batch * c * h * h * n for (c, h, n) in add_shapes)
    add_grad_bytes = float(sum((20.0 if big(batch * c * h * h) else 28.0) * batch * c * h * h * n for (c, h, n) in add_shapes))
    pool_in = batch * 64 * 32 * 32
    params = 23520842
    add_grad_bytes -= 4.0 * adds                    # level 2: d is not rewritten
    two_sweep = float(batch * 64 * 32 * 32)         # the stem's map: its masked gradient is still written back
    # level 2, identity blocks (all but the first of each stage): the add gradient is absorbed by the batch-norm backward of the
    # block's last layer, which then also reads the block's output (the mask) and writes the shortcut's gradient: 8 B / element more
    # there, and no relu_add_grad launch (16 B / element) for those blocks
    absorbed = float(sum(batch * c * h * h * (n - 1) for (c, h, n) in add_shapes))
    add_grad_bytes -= 16.0 * absorbed
    bn_bwd_bytes += 8.0 * absorbed
    return {"bn_fwd": 8.0 * bn_all + 4.0 * absorbed, "bn_bwd": bn_bwd_bytes + 4.0 * relu_bn + 4.0 * two_sweep, "relu_add_grad": add_grad_bytes,
            "map_vec4": 12.0 * (adds - absorbed),
            "maxpool_fwd": 6.0 * pool_in, "maxpool_bwd": 10.0 * pool_in, "sgd": 16.0 * params}


STAGING_KERNELS = ("to_rows", "unfold", "permute_taps", "fold_", "pad_rows", "filter_forms", "channels_last")


# --------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown," \
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            if not self.rows:
                time.sleep(0.3)            # a very short timed region: give the sampler time for one line
            self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------------------------- CPU legs
CPU_BLAS = "none: the port's own register-tiled AVX2/FMA loops (4 x 16 tile, sequential sum over k per element) under OpenMP"


def cpu_steps(batch, steps, warmup, threads):
    """Time the CPU port (oracle/) of the same host program: `steps` training steps of `batch` samples."""
    from lantern_b200._ffi import BoundLibrary
    from lantern_b200.hosts import HostPrograms
    ora = BoundLibrary(os.path.join(ROOT, "oracle", "liblantern_oracle.so"), "ora_")
    ora.init(0, 12 << 30)
    ora.cdll.ora_set_threads(threads)
    m = HostPrograms(ora, os.path.join(ROOT, "oracle", "liblantern_oracle_hosts.so"), "orah_").model("resnet50", batch, seed=42)
    rng = np.random.default_rng(1)
    x = rng.standard_normal(batch * 3072).astype(np.float32)
    y = rng.integers(0, 10, batch).astype(np.int32)
    for _ in range(warmup):
        m.step(x, y, LR)
    t0 = time.perf_counter()
    for _ in range(steps):
        m.step(x, y, LR)
    dt = time.perf_counter() - t0
    m.close(); ora.shutdown()
    return dt / max(1, steps)


def reference_arm(args, rank):
    """The reference's CPU path for this step on the host cores.  Its own CPU backend cannot train ResNet-50 (batchNorm_grad
    is unimplemented there) and its generator needs a JVM, so what is timed is the CPU port of that backend (oracle/)
    running the same host program on the FULL 128-sample batch with every host thread; the number of steps is cut so that
    the run ends within a few minutes."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    probe = cpu_steps(BATCH, 1, 1, threads)         # one warm-up + one step: also sizes the run
    steps = max(1, min(args.steps, int(200 / max(probe, 1e-3))))
    warm = 1 if probe * (steps + args.warmup) > 200 else args.warmup
    sec = cpu_steps(BATCH, steps, warm, threads)
    v = BATCH / sec
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "samples/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
            "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "resnet50_cifar_train_step_sgd_lr0.1", "batch_per_gpu": BATCH, "global_batch": BATCH, "sample_per_step": BATCH,
                       "note": "the reference's CPU backend cannot train ResNet-50 (batchNorm_grad is unimplemented) and its Scala generator "
                               "needs a JVM; this arm times the CPU port of that backend (oracle/) running the same host program"},
            "cpu_baseline": {"value": v, "unit": "samples/s", "cores": threads, "kind": "port", "blas": CPU_BLAS,
                             "sample": "%d steps of the full %d-sample batch after %d warm-up, all host threads" % (steps, BATCH, warm)},
            "e2e": {"value": v, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--math", default="tf32", choices=["tf32", "fp32"])
    ap.add_argument("--blocks", type=int, default=0, help="timed blocks of --steps steps each; the median block is reported (0: enough for about 2 s)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0")); local = int(os.environ.get("LOCAL_RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
    args.warmup = max(3, args.warmup)
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    if args.gpus != world:
        raise SystemExit("--gpus %d needs %d ranks (launch with torch.distributed.run --nproc-per-node %d)" % (args.gpus, args.gpus, args.gpus))

    import torch
    import torch.distributed as dist
    import lantern_b200
    from lantern_b200.hosts import HostPrograms

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = lantern_b200.load()
    lib.init(local, 14 << 30)
    lib.set_math(1 if args.math == "tf32" else 0)
    stream = torch.cuda.Stream(device=local)
    lib.set_stream(stream.cuda_stream)
    if world > 1:
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            buf = ctypes.create_string_buffer(128)
            lib.comm_unique_id(buf)
            idt.copy_(torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        raw = bytes(idt.cpu().numpy().tobytes())
        lib.comm_init(rank, world, ctypes.create_string_buffer(raw, 128))

    model = HostPrograms(lib).model("resnet50", BATCH, seed=42)      # identical replica on every rank
    model.use_graph(True)
    rng = np.random.default_rng(1000 + rank)                          # each rank its own shard of the global batch
    pool = [(rng.standard_normal(BATCH * 3072).astype(np.float32), rng.integers(0, 10, BATCH).astype(np.int32)) for _ in range(4)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """One block: exactly `steps` steps between barrier + synchronize, CUDA events on the launching stream, max over ranks."""
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            a.record(stream)
            for i in range(steps):
                fn(i)
            b.record(stream)
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        barrier()
        if world > 1:
            t = torch.tensor([ms], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms = float(t.item())
        return ms

    def timed_blocks(make_fn, steps, first_ms=None):
        """Repeats the K-step block (20 blocks or more, until about 2 s are covered) and returns (median, all blocks): one block
        of 20 steps lasts under 0.1 s, too short to compare two boxes."""
        first = timed(make_fn(), steps) if first_ms is None else first_ms
        n = args.blocks if args.blocks > 0 else int(min(200, max(20, 2000.0 / max(first, 1e-3))))
        if world > 1:                               # every rank must run the same number of blocks
            t = torch.tensor([n], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX); n = int(t.item())
        blocks = [first] + [timed(make_fn(), steps) for _ in range(n - 1)]
        return float(np.median(blocks)), blocks

    # ---- value: device-resident batch, the recorded step replayed back to back
    model.set_resident(*pool[0])
    sampler = ClockSampler(local); sampler.start()        # sampled from the warm-up on: all of it is under the same load
    for _ in range(args.warmup):
        model.step_async(pool[0][0], pool[0][1], LR)
    lib.sync()
    l0 = lib.kernel_launches()
    ms, blocks = timed_blocks(lambda: (lambda i: model.step_async(pool[0][0], pool[0][1], LR)), args.steps)
    launches = (lib.kernel_launches() - l0) // len(blocks)
    loss_resident = model.last_loss()
    value = BATCH * world * args.steps / (ms / 1e3)
    exposed = ctypes.c_float(0.0)
    if world > 1:
        lib.comm_exposed_ms(ctypes.addressof(exposed))

    # ---- e2e: host buffers in, loss out, every step (upload + read-back inside the timed region)
    model.set_resident(None)
    losses = []

    # Model.submit copies the batch into pinned staging, queues its upload, the step and the 4-byte loss copy; the loss of
    # the step before is read while this one runs (two steps in flight), the last one before the timed region ends.
    def e2e_loop(steps):
        state = {"prev": None}

        def fn(i):
            x, y = pool[i % len(pool)]
            k = model.submit(x, y, LR)
            if state["prev"] is not None:
                losses.append(model.collect(state["prev"]))
            state["prev"] = k
            if i == steps - 1:
                losses.append(model.collect(k))
        return fn
    for i in range(3):
        e2e_loop(1)(0)
    ms_e2e, blocks_e2e = timed_blocks(lambda: e2e_loop(args.steps), args.steps)
    clocks = sampler.stop()
    e2e = BATCH * world * args.steps / (ms_e2e / 1e3)

    # ---- replicas: after all those updates every rank must hold the same trained parameters, bit for bit (batch-norm running
    #      statistics are each replica's own: the reference has no cross-replica batch norm)
    replicas_identical = None
    if world > 1:
        lib.sync()
        p = model.trained_params()
        chk = torch.tensor([float(p.astype(np.float64).sum()), float(np.abs(p).astype(np.float64).sum())], dtype=torch.float64, device="cuda")
        lo, hi = chk.clone(), chk.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        replicas_identical = bool(torch.equal(lo, hi))

    # ---- per-kernel timing of one eagerly issued step (CUDA events on the launching stream around every launch)
    model.use_graph(False)
    model.step(pool[0][0], pool[0][1], LR)
    lib.profile(1)
    prof_steps = 2
    for i in range(prof_steps):
        model.step(pool[i][0], pool[i][1], LR)
    lib.profile(0)
    buf = ctypes.create_string_buffer(1 << 16)
    lib.profile_report(buf, 1 << 16)
    kern = {}
    for line in buf.value.decode().strip().split("\n"):
        if line:
            name, cnt, tms = line.split("\t")
            kern[name] = (int(cnt) / prof_steps, float(tms) / prof_steps)
    status = lib.device_status()

    if rank == 0:
        peaks = measured_peaks()
        fwd_flops, flops = step_flops(BATCH)
        total_ms = sum(t for _, t in kern.values())
        contraction = {k: v for k, v in kern.items() if "gemm" in k}
        c_ms = sum(t for _, t in contraction.values()); c_n = sum(c for c, _ in contraction.values())
        staging = {k: v for k, v in kern.items() if any(tag in k for tag in STAGING_KERNELS)}
        s_ms = sum(t for _, t in staging.values()); s_n = sum(c for c, _ in staging.values())
        top = max(kern.items(), key=lambda kv: kv[1][1]) if kern else ("none", (0, 0.0))
        tf32_peak = peaks["bf16_tflops_sustained"] / 2.0
        # The dominant kernel's DRAM traffic comes from its ncu capture (profiles/tc_gemm_taps_conv64x64_3x3_batch512.md: a
        # batch-512 layer, because a batch-128 layer sits inside the 126 MB L2; traffic grows in proportion to the batch):
        # 33.8 MB read + 33.6 MB written per launch at batch 512 for 33.55 + 0.15 MB of operands and 33.55 MB of output.
        traffic_b512, algo_b512 = 33.8e6 + 33.6e6, (512 * 64 * 256 + 9 * 64 * 64 + 512 * 64 * 256) * 4.0
        roofline = {"bound": "tensor", "kernel": "contraction engine (all conv fwd/dgrad/wgrad and gemm launches of one step)",
                    "achieved": flops / (c_ms / 1e3) / 1e12 if c_ms else None, "peak": tf32_peak, "unit": "TFLOP/s",
                    "frac": (flops / (c_ms / 1e3) / 1e12 / tf32_peak) if c_ms else None,
                    "traffic": traffic_b512 * BATCH / 512.0, "algorithmic_bytes": algo_b512 * BATCH / 512.0,
                    "traffic_note": "DRAM bytes per launch of the 3x3 64->64 16x16 forward convolution, ncu capture at batch 512 scaled to batch %d" % BATCH,
                    "peak_source": "%s bf16 sustained / 2 (TF32 rate is half the bf16 rate)" % peaks["source"],
                    "launches_per_step": c_n, "ms_per_step": c_ms, "share_of_step_kernel_time": c_ms / total_ms if total_ms else None,
                    "frac_with_staging": (flops / ((c_ms + s_ms) / 1e3) / 1e12 / tf32_peak) if c_ms else None,
                    "whole_step_frac": value / world * (flops / BATCH) / 1e12 / tf32_peak,
                    "top_kernel": top[0][:80], "top_kernel_ms": top[1][1]}
        # HBM side: the streaming kernels of the same eagerly issued step, compulsory bytes over event-timed duration
        want = hbm_bound_bytes(BATCH)
        h_bytes = h_ms = 0.0; per_class = {}
        for tag, nbytes in want.items():
            t = sum(v[1] for k, v in kern.items() if tag in k)
            if t > 0:
                h_bytes += nbytes; h_ms += t
                per_class[tag] = {"ms": round(t, 4), "GB/s": round(nbytes / (t / 1e3) / 1e9, 1), "frac": round(nbytes / (t / 1e3) / 1e9 / peaks["hbm_gbs"], 3)}
        roofline_hbm = {"bound": "hbm", "kernel": "streaming kernels of one step (batch norm, ReLU/add fusions, pooling, SGD)",
                        "achieved": h_bytes / (h_ms / 1e3) / 1e9 if h_ms else None, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": (h_bytes / (h_ms / 1e3) / 1e9 / peaks["hbm_gbs"]) if h_ms else None,
                        "frac_of_nominal_8TBs": (h_bytes / (h_ms / 1e3) / 1e9 / 8000.0) if h_ms else None,
                        "bytes_per_step": h_bytes, "ms_per_step": h_ms, "peak_source": peaks["source"] + " copy bandwidth", "classes": per_class}
        line = {"metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": args.math if args.math == "tf32" else "f32", "data": "synthetic",
                "config": {"workload": "resnet50_cifar_train_step_sgd_lr0.1", "batch_per_gpu": BATCH, "global_batch": BATCH * world,
                           "parallelism": "dp%d" % world, "replay": "cuda_graph",
                           "library_switches": "look-ahead fusion level 3, operand cache, deferred zero fill of gradient buffers >= 4 MB, branch regions, split-K by atomics",
                           "l2": "per-step working set (~3 GB of activations and gradients) exceeds the 126 MB L2",
                           "step_gflop": flops / 1e9},
                "timing": {"blocks": len(blocks), "steps_per_block": args.steps, "block_ms_median": ms, "block_ms_min": min(blocks), "block_ms_max": max(blocks),
                           "timed_region_s": sum(blocks) / 1e3, "note": "value and ms_per_step are the median block of exactly `steps` steps"},
                "e2e": {"value": e2e, "unit": "samples/s", "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": BATCH * 3072 * 4 + BATCH * 4, "d2h_bytes_per_step": 4,
                        "blocks": len(blocks_e2e),
                        "note": "timed from before the first host-to-device copy to after the last loss read-back; the host-fed loop replays its own "
                                "recording of the step (the batch moves from two alternating staging blocks to a fixed device address), and two "
                                "recordings of the same step differ by up to 3 % in speed, so this figure can land on either side of `value`"},
                "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "roofline_hbm": roofline_hbm,
                "staging_ms_per_step": s_ms, "staging_launches_per_step": s_n, "device_status": status,
                "loss": {"resident_last": loss_resident, "e2e_first": losses[3] if len(losses) > 3 else None, "e2e_last": losses[-1]},
                "kernels_ms_per_step": {k[:60]: round(v[1], 4) for k, v in sorted(kern.items(), key=lambda kv: -kv[1][1])[:12]}}
        if world > 1:
            line["exposed_comm_ms"] = float(exposed.value)
            line["replicas_identical"] = replicas_identical
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            sec = cpu_steps(BATCH, 2, 1, threads)
            line["cpu_baseline"] = {"value": BATCH / sec, "unit": "samples/s", "cores": threads, "kind": "port", "blas": CPU_BLAS, "same_config": True,
                                    "sample": "2 steps of the full %d-sample batch after 1 warm-up, all host threads" % BATCH}
        print(json.dumps(line), flush=True)
    model.close()
    lib.shutdown()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
