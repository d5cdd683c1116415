"""The allocation-free sum (ltb_sum_static_scratch) against ltb_sum. This file sorts last on purpose: the entry point
must work on a context that every other test has already used, and on a fresh one when the file runs alone."""
import numpy as np
import pytest


def _upload(lib, a):
    p = lib.malloc_uninit(a.nbytes)
    lib.h2d(p, a.ctypes.data, a.nbytes)
    return p


def _read1(lib, p):
    out = np.zeros(1, np.float32)
    lib.d2h(out.ctypes.data, p, 4)
    return out[0]


@pytest.mark.gpu
def test_static_scratch_sum_equals_sum_twice_in_a_row(cuda_lib):
    lib = cuda_lib
    mark = lib.mark()
    try:
        import torch
        rng = np.random.default_rng(5)
        torch.cuda.mem_get_info(0)                                  # the first query may itself set something up: not counted
        for n in (1, 1000, 65536, 65537, 1 << 20, (1 << 24) + 13):
            a = rng.standard_normal(n).astype(np.float32)
            x = _upload(lib, a)
            want, got = lib.malloc(256), lib.malloc(256)
            lib.sum(x, want, n)
            used = lib.arena_used()
            lib.sync()
            free_before = torch.cuda.mem_get_info(0)[0]             # cudaMemGetInfo: what the driver still has to give on this device
            for call in range(2):                                   # two calls in a row: the second reuses the scratch as the first left it
                lib.fill(got, -7.0, 1)
                lib.sum_static_scratch(x, got, n)
                lib.sync()
                assert _read1(lib, got) == _read1(lib, want), (n, call)
                assert abs(float(_read1(lib, got)) - float(a.astype(np.float64).sum())) <= 1e-4 * max(1.0, np.abs(a).sum())
            assert lib.arena_used() == used                         # no arena block taken either
            assert torch.cuda.mem_get_info(0)[0] == free_before     # and nothing obtained from the driver: the device's free memory is unchanged
        assert lib.device_status() == 0
    finally:
        lib.reset(mark)


@pytest.mark.gpu
def test_static_scratch_sum_rejects_sizes_beyond_its_limit(cuda_lib):
    from lantern_b200._ffi import LanternError
    lib = cuda_lib
    mark = lib.mark()
    try:
        x, out = lib.malloc(256), lib.malloc(256)
        lib.set_fatal(0)
        with pytest.raises(LanternError) as e:
            lib.sum_static_scratch(x, out, (1 << 30) + 1)           # refused before any launch: x is never read
        assert "limit" in str(e.value)
        lib.sync()
        assert lib.device_status() == 0
    finally:
        lib.reset(mark)
