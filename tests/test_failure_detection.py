"""Failure detection between ranks, on CPU (no GPU is faulted, trapped or hung anywhere).

The CUDA library bounds every host-side wait on a stream that carries collectives: it polls the stream, NCCL's
asynchronous error state and a deadline (lantern_b200/csrc/comm_wait.h, comm.cu), aborts the communicator when the
deadline passes or an error shows, returns LTB_E_COMM and refuses later collectives.  The CPU build of the same ABI
(oracle/) runs its transport behind the same `bounded_wait` with the same broken-communicator rule, so the policy is
exercised here with failures made on the host: a transport that never answers, one that reports an error, and a gloo
rank that leaves between two training steps."""
import ctypes
import os
import socket
import subprocess
import sys
import threading
import time

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
LTB_E_COMM = -5


def test_bounded_wait_policy(tmp_path):
    exe = str(tmp_path / "comm_wait_test")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-pthread", "-o", exe, os.path.join(ROOT, "tests", "comm_wait_test.cpp")])
    p = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    lines = p.stdout.strip().split("\n")
    assert p.returncode == 0 and len(lines) == 6 and all(l.startswith("ok ") for l in lines), p.stdout


def test_a_silent_or_failing_transport_gives_comm_error_and_breaks_the_communicator(oracle_lib):
    from lantern_b200 import LanternError
    ora = oracle_lib
    release = threading.Event()
    mode = {"kind": "hang"}

    @ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(ctypes.c_float), ctypes.c_int64)
    def transport(buf, n):
        if mode["kind"] == "hang":
            release.wait(30)                      # a peer that never joins the collective
            return 0
        if mode["kind"] == "error":
            return 1                              # a peer whose connection broke
        a = np.ctypeslib.as_array(buf, shape=(n,)); a *= 2.0
        return 0
    ora.cdll.ora_comm_set_transport(transport)
    x, d = np.ones(5000, np.float32), np.ones(5000, np.float32)
    try:
        for kind in ("hang", "error"):
            mode["kind"] = kind
            ora.comm_init(0, 2, ctypes.create_string_buffer(128))
            ora.comm_set_timeout_ms(300)
            t0 = time.perf_counter()
            with pytest.raises(LanternError) as e:
                ora.allreduce_sgd_step(x.ctypes.data, d.ctypes.data, 0.5, x.size)
            assert e.value.code == LTB_E_COMM and time.perf_counter() - t0 < 5.0
            assert ("timeout" in str(e.value)) == (kind == "hang")
            mode["kind"] = "ok"
            with pytest.raises(LanternError) as e:                 # broken: refused without touching the transport
                ora.allreduce_sum(d.ctypes.data, d.size)
            assert e.value.code == LTB_E_COMM and "aborted" in str(e.value)
            release.set(); time.sleep(0.05); release.clear()
            ora.comm_destroy()
        # a fresh communicator works again
        ora.comm_init(0, 2, ctypes.create_string_buffer(128))
        ora.comm_set_timeout_ms(60000)
        x[:] = 1; d[:] = 1
        ora.allreduce_sgd_step(x.ctypes.data, d.ctypes.data, 0.5, x.size)
        assert np.array_equal(x, np.full(5000, 0.5, np.float32)) and not d.any()
    finally:
        release.set()
        ora.comm_destroy()
        ora.cdll.ora_comm_set_transport(None)
        ora.comm_set_timeout_ms(60000)


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _rank(rank, world, port, out_dir):
    import datetime
    import torch
    import torch.distributed as dist
    from lantern_b200 import LanternError
    from lantern_b200._ffi import BoundLibrary
    from lantern_b200.hosts import HostPrograms
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    ora = BoundLibrary(os.path.join(ROOT, "oracle", "liblantern_oracle.so"), "ora_")
    ora.init(0, 1 << 30); ora.set_math(0)

    @ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(ctypes.c_float), ctypes.c_int64)
    def transport(buf, n):
        try:
            dist.all_reduce(torch.from_numpy(np.ctypeslib.as_array(buf, shape=(n,))))
            return 0
        except Exception:                          # the peer is gone: gloo raises (connection closed, or its own timeout)
            return 1
    ora.cdll.ora_comm_set_transport(transport)
    ora.comm_init(rank, world, ctypes.create_string_buffer(128))
    ora.comm_set_timeout_ms(20000)
    m = HostPrograms(ora, os.path.join(ROOT, "oracle", "liblantern_oracle_hosts.so"), "orah_").model("mnist", 4, seed=42)
    rng = np.random.default_rng(rank)
    x, y = rng.random(4 * 784, dtype=np.float32), rng.integers(0, 10, 4).astype(np.int32)
    m.step(x, y, 0.001)                            # step 1: both ranks present
    if rank == 1:                                  # leaves BETWEEN steps: nothing of its own is in flight
        dist.destroy_process_group()
        os._exit(0)
    t0 = time.perf_counter()
    status = "no error"
    ora.set_fatal(0)
    rc = ora.raw("allreduce_sum")(m.hp.fn["model_slab_grads"](m.h), 1024)      # the next collective of the rank that stayed
    waited = time.perf_counter() - t0
    rc2 = ora.raw("allreduce_sum")(m.hp.fn["model_slab_grads"](m.h), 1024)     # and the one after it: refused at once
    with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
        f.write("%d %d %.3f %s\n" % (rc, rc2, waited, ora.error_message()))
    os._exit(0)                                    # the process group cannot be torn down cleanly without its peer


@pytest.mark.timeout(300)
def test_a_rank_that_leaves_between_steps_surfaces_as_comm_error_on_the_other(tmp_path):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0, p.exitcode
    rc, rc2, waited, msg = open(tmp_path / "rank0.txt").read().split(" ", 3)
    assert int(rc) == LTB_E_COMM, msg
    assert float(waited) < 25.0                     # within the communicator's timeout (20 s), not for ever
    assert int(rc2) == LTB_E_COMM and "aborted" in msg
