"""Pins the oracle end to end against the reference's own implementation: the shipped generated MNIST CNN
program (compiled from its source into oracle/_ref/ by oracle/Makefile) and the hand-mirrored host program
running on the oracle must produce the same per-epoch loss on the same synthetic files, because both draw
weights and dropout masks from glibc rand() after srand(42) in the same order."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_BIN = os.path.join(ROOT, "oracle", "_ref", "mnist_cnn_cpu")
ORA_HOSTS = os.path.join(ROOT, "oracle", "liblantern_oracle_hosts.so")


@pytest.mark.skipif(not os.path.exists(REF_BIN), reason="oracle/_ref not built (reference checkout absent at build time)")
def test_mnist_loss_trajectory_matches_generated_program(oracle_lib, tmp_path):
    from lantern_b200.hosts import HostPrograms
    n = 600
    rng = np.random.default_rng(42)
    raw = rng.random((n, 784), dtype=np.float32)               # MNIST-shaped pixels in [0,1)
    tgt = rng.integers(0, 10, size=n).astype(np.int32)
    (tmp_path / "data" / "bin").mkdir(parents=True)
    (tmp_path / "run").mkdir()
    raw.tofile(tmp_path / "data" / "bin" / "mnist_train.bin")
    tgt.tofile(tmp_path / "data" / "bin" / "mnist_train_target.bin")
    subprocess.run([REF_BIN, "result.txt"], cwd=tmp_path / "run", check=True, stdout=subprocess.DEVNULL, timeout=600)
    lines = (tmp_path / "run" / "result.txt").read_text().split("\n")
    ref_losses = [float(v) for v in lines[1:5]]

    mark = oracle_lib.mark()
    hp = HostPrograms(oracle_lib, ORA_HOSTS, "orah_")
    model = hp.model("mnist", 100, seed=42)
    data = (raw - np.float32(0.1307)) / np.float32(0.3081)      # DataLoader.normalize, TensorDataLoader.scala:84-96
    ours = []
    for _ in range(4):
        tot = np.float32(0)
        for b in range(n // 100):
            tot += np.float32(model.step(data[b * 100:(b + 1) * 100], tgt[b * 100:(b + 1) * 100], 0.0005))
        ours.append(float(tot / np.float32(n)))
    model.close()
    oracle_lib.reset(mark)
    assert np.allclose(ours, ref_losses, rtol=2e-5, atol=1e-6), (ours, ref_losses)
    assert ours[-1] < ours[0]
