"""Data-parallel step, world_size 2, on CPU: two gloo ranks run the host program of the SqueezeNet training step on
their own shard of a global batch through the CPU build of the ABI, with torch.distributed's all_reduce installed as
the communicator's transport. What is checked is the host logic the GPU ranks share with this build: the branch the
host program takes when the communicator has more than one rank, the bucket spans of the gradient slab, the 1/world
scaling (each rank's loss is a mean over its shard) and that both ranks hold identical parameters afterwards which
equal, to rounding, those of one process that trained on the whole batch.
"""
import ctypes
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

SHARD, STEPS, LR = 4, 2, 0.005


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _data(world):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((STEPS, world * SHARD, 3 * 32 * 32)).astype(np.float32)
    y = rng.integers(0, 10, (STEPS, world * SHARD)).astype(np.int32)
    return x, y


def _open_oracle():
    from lantern_b200._ffi import BoundLibrary
    from lantern_b200.hosts import HostPrograms
    ora = BoundLibrary(os.path.join(ROOT, "oracle", "liblantern_oracle.so"), "ora_")
    ora.init(0, 2 << 30)
    ora.set_math(0)
    hp = HostPrograms(ora, os.path.join(ROOT, "oracle", "liblantern_oracle_hosts.so"), "orah_")
    return ora, hp


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ora, hp = _open_oracle()
    calls = []

    @ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(ctypes.c_float), ctypes.c_int64)
    def transport(buf, n):
        a = np.ctypeslib.as_array(buf, shape=(n,))
        dist.all_reduce(torch.from_numpy(a))             # in place, sum over ranks
        calls.append(int(n))
        return 0
    ora.cdll.ora_comm_set_transport(transport)
    ora.comm_init(rank, world, ctypes.create_string_buffer(128))
    assert ora.comm_world() == world
    m = hp.model("squeezenet", SHARD, seed=42)
    x, y = _data(world)
    losses = []
    for s in range(STEPS):
        losses.append(m.step(x[s, rank * SHARD:(rank + 1) * SHARD].ravel(), y[s, rank * SHARD:(rank + 1) * SHARD], LR))
    np.save(os.path.join(out_dir, "params_%d.npy" % rank), m.slab_params())
    np.save(os.path.join(out_dir, "grads_%d.npy" % rank), m.slab_grads())
    np.save(os.path.join(out_dir, "losses_%d.npy" % rank), np.array(losses, np.float64))
    np.save(os.path.join(out_dir, "calls_%d.npy" % rank), np.array(calls, np.int64))
    m.close(); ora.comm_destroy(); ora.shutdown()
    dist.destroy_process_group()


def _whole_batch_worker(_, world, out_dir):
    ora, hp = _open_oracle()
    m = hp.model("squeezenet", world * SHARD, seed=42)
    np.save(os.path.join(out_dir, "init_params.npy"), m.slab_params())
    x, y = _data(world)
    whole = [m.step(x[s].ravel(), y[s], LR) for s in range(STEPS)]
    np.save(os.path.join(out_dir, "ref_params.npy"), m.slab_params())
    np.save(os.path.join(out_dir, "ref_losses.npy"), np.array(whole, np.float64))
    m.close(); ora.shutdown()


@pytest.mark.timeout(600)
def test_two_ranks_match_one_process_on_the_whole_batch(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    p0, p1 = np.load(tmp_path / "params_0.npy"), np.load(tmp_path / "params_1.npy")
    assert np.array_equal(p0, p1), "ranks diverged"
    assert not np.load(tmp_path / "grads_0.npy").any(), "the update must leave the gradient slab cleared"
    calls = np.load(tmp_path / "calls_0.npy")
    n = p0.size
    per_step = len(calls) // STEPS
    assert per_step >= 1 and calls[:per_step].sum() == n, "the buckets of one step must cover the slab exactly once"
    # the first sum of a step is the range the host program hands over during backward (the parameters of the last fire
    # modules and the classifier); the rest of the slab follows at the update, in buckets of whole 4 KiB blocks
    assert per_step >= 2 and all(c % 1024 == 0 for c in calls[1:per_step - 1])

    # one process, the whole batch: mean loss over 2*SHARD samples == mean of the two shard means
    mp.spawn(_whole_batch_worker, args=(world, str(tmp_path)), nprocs=1, join=True)
    ref, init, whole = np.load(tmp_path / "ref_params.npy"), np.load(tmp_path / "init_params.npy"), np.load(tmp_path / "ref_losses.npy")
    l0, l1 = np.load(tmp_path / "losses_0.npy"), np.load(tmp_path / "losses_1.npy")
    assert np.allclose((l0 + l1) / 2, whole, rtol=1e-4), ((l0 + l1) / 2, whole)
    # Two shard sums added together round differently from one sum over the whole batch (1e-7), and after the first update
    # a pre-activation within that distance of zero may fall on the other side of its ReLU in the second step, which switches
    # one gradient element on or off and shows in one filter row: nearly every parameter agrees to 1e-5, all of them to 2e-4.
    err = np.abs(p0 - ref) / np.abs(ref).max()
    assert (err > 1e-5).mean() < 1e-3 and err.max() < 2e-4, (float(err.max()), int((err > 1e-5).sum()))
    # and the steps did move the parameters by far more than that bound
    assert np.abs(p0 - init).max() / np.abs(ref).max() > 1e-3


def test_bucket_spans_cover_ragged_sizes(oracle_lib):
    """ltb::bucket_spans (csrc/buckets.h), through the CPU communicator with world 2 emulated by a doubling transport."""
    ora = oracle_lib
    seen = []

    @ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(ctypes.c_float), ctypes.c_int64)
    def transport(buf, n):
        a = np.ctypeslib.as_array(buf, shape=(n,)); a *= 2.0; seen.append(int(n)); return 0
    ora.cdll.ora_comm_set_transport(transport)
    ora.comm_init(0, 2, ctypes.create_string_buffer(128))
    try:
        for n in (1, 3, 1023, 1024, 1025, 8191, 8192, 8193, 100003, 23520842 // 64):
            seen.clear()
            x = np.ones(n, np.float32); d = np.arange(n, dtype=np.float32) % 7
            want = x - 0.5 * d                            # lr 0.5: x -= lr/2 * (2 d)
            ora.allreduce_sgd_step(x.ctypes.data, d.ctypes.data, 0.5, n)
            assert sum(seen) == n and len(seen) <= 8
            assert np.array_equal(x, want) and not d.any()
    finally:
        ora.comm_destroy()
        ora.cdll.ora_comm_set_transport(None)
