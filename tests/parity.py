"""Helpers shared by the GPU parity tests: run the same calls on the CPU oracle and on the CUDA library."""
import numpy as np

FP32_RTOL = 1e-4      # FP32 CUDA-core paths: 1e-4 relative (north star)
TF32_RTOL = 2e-3      # TF32 tensor-core paths: 2e-3 relative


def rel_err(ref, got):
    """Max |got-ref| relative to the largest magnitude of the reference tensor (per-tensor relative error)."""
    ref = np.asarray(ref, dtype=np.float64); got = np.asarray(got, dtype=np.float64)
    assert ref.shape == got.shape, (ref.shape, got.shape)
    if ref.size == 0:
        return 0.0
    scale = max(np.abs(ref).max(), 1e-30)
    return float(np.abs(got - ref).max() / scale)


def assert_close(ref, got, rtol, what=""):
    assert np.all(np.isfinite(got)), what + ": non-finite values"
    e = rel_err(ref, got)
    assert e <= rtol, "%s: relative error %.3e > %.1e" % (what, e, rtol)


def both(fn, ora, gpu):
    """fn(backend) -> dict of numpy arrays; returns (oracle result, gpu result)."""
    return fn(ora), fn(gpu)


def check(fn, ora, gpu, rtol=FP32_RTOL, exact=()):
    a, b = both(fn, ora, gpu)
    assert a.keys() == b.keys()
    for k in a:
        if k in exact:
            assert np.array_equal(a[k], b[k]), "%s differs (bit-exact required)" % k
        else:
            assert_close(a[k], b[k], rtol, k)
