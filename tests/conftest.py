import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
ORACLE_SO = os.path.join(ROOT, "oracle", "liblantern_oracle.so")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _build_oracle():
    if not os.path.exists(ORACLE_SO):
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle")])


@pytest.fixture(scope="session")
def oracle_lib():
    """The CPU oracle (test infrastructure), bound through the same header as the product."""
    from lantern_b200._ffi import BoundLibrary
    _build_oracle()
    lib = BoundLibrary(ORACLE_SO, "ora_")
    lib.init(0, 10 << 30)            # untouched pages cost nothing; a ResNet-50 step at batch 128 needs about 4 GiB
    yield lib
    lib.shutdown()


@pytest.fixture()
def ora(oracle_lib):
    from lantern_b200.backend import Backend
    mark = oracle_lib.mark()
    oracle_lib.set_math(0)           # plain FP32: the reference's CPU backend; TF32 tests switch the emulation on themselves
    yield Backend(oracle_lib)
    oracle_lib.reset(mark)


@pytest.fixture(scope="session")
def cuda_lib():
    """The CUDA product library on device 0; absent library or device is an error, never a skip."""
    import lantern_b200
    lib = lantern_b200.load()
    lib.init(0, 16 << 30)            # of the 180 GB: the batch-128 steps with their staging blocks need about 6 GiB
    yield lib
    lib.shutdown()


@pytest.fixture()
def gpu(cuda_lib):
    from lantern_b200.backend import Backend
    mark = cuda_lib.mark()
    cuda_lib.set_math(1)
    yield Backend(cuda_lib)
    cuda_lib.sync()
    assert cuda_lib.device_status() == 0
    cuda_lib.reset(mark)
