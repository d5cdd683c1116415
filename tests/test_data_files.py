"""Readers of the reference's data and parameter file formats, and training with two steps in flight.

Formats (synthetic files of the same layout stand in for the data sets, which are not redistributed here):
  * float data set: raw float32 samples + raw int32 targets, used as (x - mean) / std  (TensorDataLoader.scala:64-108)
  * CIFAR binary: 1 label byte + 3072 pixel bytes per record, x = byte / 255            (TensorDataLoader.scala:110-139)
  * parameter file: every float tensor back to back in declaration order                (ONNXLib.scala:157-185)
The CPU tests run the host programs on the oracle; the GPU tests run the same programs on the CUDA library.
"""
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORA_HOSTS = os.path.join(ROOT, "oracle", "liblantern_oracle_hosts.so")


def _cifar_file(path, n, rng, trailing=0):
    rec = rng.integers(0, 256, (n, 3073), dtype=np.uint8)
    rec[:, 0] = rng.integers(0, 10, n)
    with open(path, "wb") as f:
        f.write(rec.tobytes())
        f.write(b"\x07" * trailing)            # a partial record at the end of the file is ignored
    return rec


def _mnist_files(tmp, n, rng):
    x = rng.random((n, 784), dtype=np.float32)
    y = rng.integers(0, 10, n).astype(np.int32)
    xp, yp = os.path.join(tmp, "mnist_train.bin"), os.path.join(tmp, "mnist_train_target.bin")
    x.tofile(xp); y.tofile(yp)
    return xp, yp, x, y


def _programs(lib, oracle):
    from lantern_b200.hosts import HostPrograms
    return HostPrograms(lib, ORA_HOSTS, "orah_") if oracle else HostPrograms(lib)


def test_cifar_records_decode(oracle_lib, tmp_path):
    hp = _programs(oracle_lib, True)
    rng = np.random.default_rng(0)
    rec = _cifar_file(tmp_path / "data_batch_1.bin", 37, rng, trailing=100)
    ld = hp.cifar_loader(tmp_path / "data_batch_1.bin")
    assert ld.length == 37
    x, y = ld.batch(2, 8)                       # samples 16..23
    assert np.array_equal(y, rec[16:24, 0].astype(np.int32))
    assert np.array_equal(x.reshape(8, 3072), rec[16:24, 1:].astype(np.float32) / np.float32(255.0))
    with pytest.raises(IndexError):
        ld.batch(4, 8)                          # 37 samples hold four whole batches of 8: index 4 is the dropped remainder
    ld.close()
    with pytest.raises(OSError):
        hp.cifar_loader(tmp_path / "missing.bin")


def test_float_dataset_decode_and_length_check(oracle_lib, tmp_path):
    hp = _programs(oracle_lib, True)
    xp, yp, x, y = _mnist_files(str(tmp_path), 25, np.random.default_rng(1))
    ld = hp.float_loader(xp, yp, 784, mean=0.1307, std=0.3081)
    assert ld.length == 25
    bx, by = ld.batch(1, 10)
    assert np.array_equal(by, y[10:20])
    assert np.array_equal(bx.reshape(10, 784), (x[10:20] - np.float32(0.1307)) / np.float32(0.3081))
    ld.close()
    with open(xp, "ab") as f:
        f.write(b"\0\0\0\0")                   # one float too many: "Data length doesn't match"
    with pytest.raises(OSError):
        hp.float_loader(xp, yp, 784)


def _param_file_roundtrip(lib, oracle, tmp_path):
    hp = _programs(lib, oracle)
    mark = lib.mark()
    m = hp.model("mnist", 4, seed=42)
    path = tmp_path / "mnist.onnx.bin"
    m.save_params(path)
    counts = [m.hp.fn["model_param_count"](m.h, i) for i in range(m.num_params)]
    flat = np.fromfile(path, dtype=np.float32)
    assert flat.size == sum(counts) == 21840            # unpadded: conv 250+10, conv 5000+20, fc 16000+50, fc 500+10
    off = 0
    for i, c in enumerate(counts):                       # tensor i sits at the float offset of the tensors before it
        assert np.array_equal(flat[off:off + c], m.param(i)); off += c
    m.close(); lib.reset(mark)
    m2 = hp.model("mnist", 4, seed=7)                    # other weights, then the file
    assert not np.array_equal(m2.param(0), flat[:250])
    m2.load_params(path)
    off = 0
    for i, c in enumerate(counts):
        assert np.array_equal(flat[off:off + c], m2.param(i)); off += c
    with open(path, "ab") as f:
        f.write(b"\0\0\0\0")
    with pytest.raises(ValueError):
        m2.load_params(path)                             # a file of another size is not this model's
    m2.close(); lib.reset(mark)


def test_param_file_roundtrip_cpu(oracle_lib, tmp_path):
    oracle_lib.set_math(0)
    _param_file_roundtrip(oracle_lib, True, tmp_path)


def _two_in_flight_equals_blocking(lib, oracle, tmp_path, name, batch, steps, exact):
    hp = _programs(lib, oracle)
    rng = np.random.default_rng(2)
    mark = lib.mark()
    if name == "mnist":
        xp, yp, _, _ = _mnist_files(str(tmp_path), batch * steps + 3, rng)
        ld = hp.float_loader(xp, yp, 784, mean=0.1307, std=0.3081)
        lr = 5e-4
    else:
        _cifar_file(tmp_path / "cifar.bin", batch * steps + 3, rng)
        ld = hp.cifar_loader(tmp_path / "cifar.bin")
        lr = 0.005
    a = hp.model(name, batch, seed=42)
    if not oracle:
        a.use_graph(True)
    blocking = [a.step(*ld.batch(i, batch), lr) for i in range(steps)]
    pa = a.slab_params()
    a.close(); lib.reset(mark)
    b = hp.model(name, batch, seed=42)
    if not oracle:
        b.use_graph(True)
    fed = b.train_epoch(ld, lr)
    assert len(fed) == steps
    pb = b.slab_params()
    # submit / collect by hand, continuing from the epoch: collecting a step twice or too late is refused
    k0 = b.submit(*ld.batch(0, batch), lr)
    k1 = b.submit(*ld.batch(1, batch), lr)
    k2 = b.submit(*ld.batch(2, batch), lr)
    assert (k1, k2) == (k0 + 1, k0 + 2)
    with pytest.raises(RuntimeError):
        b.collect(k0)                                    # only the last two steps keep their loss
    l1, l2 = b.collect(k1), b.collect(k2)
    assert np.isfinite(l1) and np.isfinite(l2)
    again = b.step(*ld.batch(3, batch), lr)              # the blocking call still works afterwards
    assert np.isfinite(again)
    b.close(); ld.close(); lib.reset(mark)
    if exact:
        assert list(fed) == [np.float32(v) for v in blocking]
        assert np.array_equal(pa, pb)
    else:
        assert np.allclose(fed, blocking, rtol=2e-3, atol=0)
        # Two runs of the SAME blocking program already differ like this on the GPU: split-K partial sums are added atomically
        # in any order (1e-7 per operator), a max-pool or ReLU decision flips here and there, and five updates carry the flip
        # into a handful of the 806,144 parameters (measured, same process, blocking against blocking: largest difference
        # 3e-6 to 1.4e-3, up to 7 parameters beyond 1e-3).  So the bound is on all but one parameter in ten thousand, with
        # a gross-error guard on the rest.
        d, tol = np.abs(pa - pb), 2e-3 * np.abs(pa).max()
        assert (d > tol).mean() < 1e-4 and d.max() < 10 * tol, ((d > tol).sum(), d.max(), tol)


def test_two_steps_in_flight_equals_blocking_cpu(oracle_lib, tmp_path):
    oracle_lib.set_math(0)
    _two_in_flight_equals_blocking(oracle_lib, True, tmp_path, "mnist", 5, 6, exact=True)


@pytest.mark.gpu
def test_param_file_roundtrip_gpu(cuda_lib, tmp_path):
    _param_file_roundtrip(cuda_lib, False, tmp_path)


@pytest.mark.gpu
@pytest.mark.parametrize("name,batch,steps", [("mnist", 100, 6), ("squeezenet", 16, 5)])
def test_two_steps_in_flight_equals_blocking_gpu(cuda_lib, tmp_path, name, batch, steps):
    cuda_lib.set_math(0)                                 # FP32: the two runs differ by split-K summation order only
    try:
        _two_in_flight_equals_blocking(cuda_lib, False, tmp_path, name, batch, steps, exact=False)
        assert cuda_lib.device_status() == 0
    finally:
        cuda_lib.set_math(1)


@pytest.mark.gpu
def test_epoch_from_cifar_file_matches_oracle(cuda_lib, oracle_lib, tmp_path):
    """SqueezeNet trained from a CIFAR-format file with two steps in flight against the oracle's blocking steps."""
    rng = np.random.default_rng(3)
    batch, steps = 8, 4
    _cifar_file(tmp_path / "cifar.bin", batch * steps, rng)
    gpu = cuda_lib
    gpu.set_math(0); oracle_lib.set_math(0)
    mark_g, mark_o = gpu.mark(), oracle_lib.mark()
    try:
        hg, ho = _programs(gpu, False), _programs(oracle_lib, True)
        mg, mo = hg.model("squeezenet", batch, seed=42), ho.model("squeezenet", batch, seed=42)
        lg, lo = hg.cifar_loader(tmp_path / "cifar.bin"), ho.cifar_loader(tmp_path / "cifar.bin")
        got = mg.train_epoch(lg, 0.005)
        want = [mo.step(*lo.batch(i, batch), 0.005) for i in range(steps)]
        assert np.allclose(got, want, rtol=1e-3, atol=0), (got, want)
        mg.close(); mo.close(); lg.close(); lo.close()
        assert gpu.device_status() == 0
    finally:
        gpu.set_math(1); gpu.reset(mark_g); oracle_lib.reset(mark_o)


def test_empty_and_short_files(oracle_lib, tmp_path):
    """An empty data file has no samples and an epoch over it runs no step; a file shorter than one batch likewise."""
    hp = _programs(oracle_lib, True)
    oracle_lib.set_math(0)
    (tmp_path / "empty.bin").write_bytes(b"")
    ld = hp.cifar_loader(tmp_path / "empty.bin")
    assert ld.length == 0
    with pytest.raises(IndexError):
        ld.batch(0, 1)
    mark = oracle_lib.mark()
    m = hp.model("squeezenet", 4, seed=42)
    assert len(m.train_epoch(ld, 0.005)) == 0
    ld.close()
    _cifar_file(tmp_path / "three.bin", 3, np.random.default_rng(9))
    ld = hp.cifar_loader(tmp_path / "three.bin")
    assert ld.length == 3 and len(m.train_epoch(ld, 0.005)) == 0          # three samples do not fill a batch of four
    ld.close(); m.close(); oracle_lib.reset(mark)
