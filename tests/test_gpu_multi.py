"""Data-parallel training step on 2 GPUs through the C ABI: NCCL all-reduce of the gradient slab fused with the SGD
update. Needs two devices (skipped on a one-GPU box); each rank is its own process, as in production.

Checked: both ranks end with bit-identical parameters; those parameters equal, within the FP32 tolerance, what the CPU
oracle computes in one process on the whole batch (the mean over the global batch is the mean of the shard means);
eager issue and CUDA-graph replay of the step agree.
"""
import ctypes
import os
import sys
import time

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

SHARD, STEPS, LR = 4, 3, 0.005


def _device_count():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _data(world):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((STEPS, world * SHARD, 3 * 32 * 32)).astype(np.float32)
    y = rng.integers(0, 10, (STEPS, world * SHARD)).astype(np.int32)
    return x, y


def _gpu_worker(rank, world, out_dir, graph, name="squeezenet", math=0):
    os.environ["NCCL_NVLS_ENABLE"] = "0"        # plain peer transport: nothing stays bound to a multicast object if a rank dies
    import lantern_b200
    from lantern_b200.hosts import HostPrograms
    lib = lantern_b200.load()
    lib.init(rank, 2 << 30)
    lib.set_math(math)
    id_path = os.path.join(out_dir, "nccl_id_%s_%d.bin" % (name, int(graph)))
    buf = ctypes.create_string_buffer(128)
    if rank == 0:
        lib.comm_unique_id(buf)
        with open(id_path + ".tmp", "wb") as f:
            f.write(buf.raw)
        os.rename(id_path + ".tmp", id_path)
    else:
        deadline = time.time() + 120
        while not os.path.exists(id_path):
            if time.time() > deadline:
                raise RuntimeError("rank 0 never published the communicator id")
            time.sleep(0.05)
        buf = ctypes.create_string_buffer(open(id_path, "rb").read(), 128)
    lib.comm_init(rank, world, buf)
    assert lib.comm_world() == world
    m = HostPrograms(lib).model(name, SHARD, seed=42)
    m.use_graph(bool(graph))
    x, y = _data(world)
    losses = [m.step(x[s, rank * SHARD:(rank + 1) * SHARD].ravel(), y[s, rank * SHARD:(rank + 1) * SHARD], LR) for s in range(STEPS)]
    lib.sync()
    assert lib.device_status() == 0
    tag = "g%d_r%d" % (int(graph), rank)
    np.save(os.path.join(out_dir, "params_%s.npy" % tag), m.slab_params())
    np.save(os.path.join(out_dir, "trained_%s.npy" % tag), m.trained_params())
    np.save(os.path.join(out_dir, "state_%s.npy" % tag), np.concatenate([m.param(i) for i in range(m.num_params) if m.param_is_state(i)] + [np.zeros(0, np.float32)]))
    np.save(os.path.join(out_dir, "grads_%s.npy" % tag), m.slab_grads())
    np.save(os.path.join(out_dir, "losses_%s.npy" % tag), np.array(losses, np.float64))
    m.close(); lib.comm_destroy(); lib.shutdown()


def _oracle_worker(_, world, out_dir):
    from lantern_b200._ffi import BoundLibrary
    from lantern_b200.hosts import HostPrograms
    ora = BoundLibrary(os.path.join(ROOT, "oracle", "liblantern_oracle.so"), "ora_")
    ora.init(0, 2 << 30); ora.set_math(0)
    m = HostPrograms(ora, os.path.join(ROOT, "oracle", "liblantern_oracle_hosts.so"), "orah_").model("squeezenet", world * SHARD, seed=42)
    x, y = _data(world)
    losses = [m.step(x[s].ravel(), y[s], LR) for s in range(STEPS)]
    np.save(os.path.join(out_dir, "ref_params.npy"), m.slab_params())
    np.save(os.path.join(out_dir, "ref_losses.npy"), np.array(losses, np.float64))
    m.close(); ora.shutdown()


@pytest.mark.gpu
@pytest.mark.timeout(900)
def test_two_gpus_match_the_oracle_on_the_whole_batch(tmp_path):
    if _device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_oracle_worker, args=(world, str(tmp_path)), nprocs=1, join=True)
    ref, ref_losses = np.load(tmp_path / "ref_params.npy"), np.load(tmp_path / "ref_losses.npy")
    for graph in (0, 1):
        mp.spawn(_gpu_worker, args=(world, str(tmp_path), graph), nprocs=world, join=True)
        p0, p1 = np.load(tmp_path / ("params_g%d_r0.npy" % graph)), np.load(tmp_path / ("params_g%d_r1.npy" % graph))
        assert np.array_equal(p0, p1), "ranks diverged (graph=%d)" % graph
        assert not np.load(tmp_path / ("grads_g%d_r0.npy" % graph)).any()
        l0, l1 = np.load(tmp_path / ("losses_g%d_r0.npy" % graph)), np.load(tmp_path / ("losses_g%d_r1.npy" % graph))
        assert np.allclose((l0 + l1) / 2, ref_losses, rtol=1e-4), ((l0 + l1) / 2, ref_losses)
        err = np.abs(p0 - ref).max() / np.abs(ref).max()
        assert err < 5e-4, (graph, err)        # three steps of FP32 rounding in different summation orders (measured 1.6e-4)


@pytest.mark.gpu
@pytest.mark.timeout(900)
def test_two_gpus_keep_trained_parameters_identical_with_batch_norm(tmp_path):
    """A program with batch norm (stem + first bottleneck block of ResNet-50) on the tensor-core path, three data-parallel
    steps, eager and replayed: the trained parameters of the two ranks stay bit-identical (local gradients are summed by
    atomics in any order, but both ranks apply the same all-reduced sum), while the running statistics are each replica's
    own (different shards: they differ), as in the reference, which has no cross-replica batch norm."""
    if _device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    for graph in (0, 1):
        mp.spawn(_gpu_worker, args=(2, str(tmp_path), graph, "resnet50_prefix", 1), nprocs=2, join=True)
        t0, t1 = np.load(tmp_path / ("trained_g%d_r0.npy" % graph)), np.load(tmp_path / ("trained_g%d_r1.npy" % graph))
        assert t0.size > 70000 and np.array_equal(t0, t1), "trained parameters diverged (graph=%d)" % graph
        s0, s1 = np.load(tmp_path / ("state_g%d_r0.npy" % graph)), np.load(tmp_path / ("state_g%d_r1.npy" % graph))
        assert s0.size == 2 * (64 + 64 + 64 + 256 + 256) and not np.array_equal(s0, s1)
        assert not np.load(tmp_path / ("grads_g%d_r0.npy" % graph)).any()
