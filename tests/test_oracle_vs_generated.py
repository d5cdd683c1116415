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


REF_RNN_BIN = os.path.join(ROOT, "oracle", "_ref", "rnn_cpu")


@pytest.mark.skipif(not os.path.exists(REF_RNN_BIN), reason="oracle/_ref not built (reference checkout absent at build time)")
def test_rnn_loss_trajectory_matches_generated_program(oracle_lib, tmp_path):
    """The reference's shipped generated min-char-rnn (vocabulary 26, hidden 50, batch 20, 20 unrolled steps, Adagrad
    lr 0.1 clip 5; src/out/NIPS18evaluation/evaluationRNN/Lantern.cpp) against the hand-mirrored host program on the
    oracle at the same sizes, on the same text, from the same rand() stream (the program never calls srand: seed 1).
    Pins dot, broadcasting add, tanh, logSoftmax/NLL/sum and adagrad_update of the oracle end to end.
    The program opens `graham.txt` in its working directory and maps a byte c to the token c - 96 without any range
    check (its own text file contains spaces and newlines, i.e. negative tokens that index outside the one-hot row), so
    it is run here on a seeded synthetic text whose bytes 96..121 give exactly the tokens 0..25."""
    from lantern_b200.hosts import HostPrograms
    T, B, V = 20, 20, 26
    # A periodic text: with Adagrad at lr 0.1 the first steps on a text with real entropy send the loss UP for a dozen
    # iterations and the trajectory becomes chaotic (two builds of the same arithmetic drift apart by percents within ten
    # steps); on a learnable pattern the descent is monotone and rounding differences stay rounding differences.
    text = np.tile(np.array([3, 7, 1, 12, 20], np.int32), 700)        # 3500 tokens
    (tmp_path / "graham.txt").write_bytes(bytes((text + 96).astype(np.uint8)))
    out = subprocess.run([REF_RNN_BIN, "result.txt"], cwd=tmp_path, check=True, capture_output=True, text=True, timeout=600).stdout
    ref = {}
    for line in out.split("\n"):
        if line.startswith("iter "):
            it, loss = line[5:].split(", loss ")
            ref[int(it)] = float(loss)
    assert len(ref) == 51 and 0 in ref and 5000 in ref

    mark = oracle_lib.mark()
    oracle_lib.set_math(0)
    model = HostPrograms(oracle_lib, ORA_HOSTS, "orah_").model("rnn_26_50", B, seed=1)
    pos = -400
    steps = 2001                                                   # 21 comparison points
    ours = {}
    rows = np.arange(T)[:, None], np.arange(B)[None, :]
    for it in range(steps):
        pos += 400                                                 # Lantern.cpp:576-594
        if pos + 400 + 1 >= text.size:
            pos = 0
        ids = text[pos:pos + 400].reshape(B, T)                    # x71[b*20 + t]
        nxt = text[pos + 1:pos + 401].reshape(B, T)                # x72[b*20 + t]
        x = np.zeros((T, B, V), np.float32)
        x[rows[0], rows[1], ids.T] = 1.0                           # one-hot [t][b][id], Lantern.cpp:599-612
        loss = model.step(x.ravel(), np.ascontiguousarray(nxt.T).ravel(), 0.1)
        if it % 100 == 0:
            ours[it] = loss
    model.close()
    oracle_lib.reset(mark)
    got = [ours[k] for k in sorted(ours)]
    want = [ref[k] for k in sorted(ours)]
    assert abs(got[0] - 400 * np.log(26.0)) < 10.0                 # untrained: about ln 26 per prediction
    assert np.allclose(got[:2], want[:2], rtol=2e-5), list(zip(got[:2], want[:2]))
    assert np.allclose(got, want, rtol=5e-3, atol=1e-4), list(zip(got, want))
    assert got[-1] < 1e-3 * got[0]


REF_TREE_BIN = os.path.join(ROOT, "oracle", "_ref", "treelstm_cpu")


@pytest.mark.skipif(not os.path.exists(REF_TREE_BIN), reason="oracle/_ref not built (reference checkout absent at build time)")
def test_treelstm_loss_trajectory_matches_generated_program(oracle_lib, tmp_path):
    """The reference's shipped generated TreeLSTM sentiment program (src/out/NIPS18evaluation/evaluationTreeLSTM/Lantern/
    Lantern.cpp: embedding 300, hidden 150, 5 classes, one tree per step, hand-written Adagrad lr 0.05 without clipping,
    6 epochs) against the `treelstm_nips18` host program on the oracle, on synthetic files in the program's own formats
    (`small_glove.txt`: row count, then 300 floats per row; `array_tree.txt`: tree count, then per tree the node count
    and four rows scores / words / left child / right child). Same rand() stream (seed 1: the program never calls
    srand). Pins matrix-vector dot, sigmoid, tanh, elementwise product, the recursion and Adagrad of the oracle."""
    from lantern_b200.hosts import HostPrograms
    from tests.test_gpu_models import _random_tree
    rng = np.random.default_rng(77)
    vocab, n_trees = 60, 24
    emb = np.float32(rng.normal(0.0, 0.1, (vocab, 300)))
    with open(tmp_path / "small_glove.txt", "w") as f:
        f.write("%d\n" % vocab)
        for row in emb:
            f.write(" ".join("%.9g" % v for v in row) + "\n")
    trees = [_random_tree(rng, int(rng.integers(2, 9)), vocab=vocab) for _ in range(n_trees)]
    with open(tmp_path / "array_tree.txt", "w") as f:
        f.write("%d\n" % n_trees)
        for y in trees:
            n = int(y[0])
            f.write("%d\n" % n)
            for j in range(4):
                f.write(" ".join(str(int(v)) for v in y[1 + j * 99: 1 + j * 99 + n]) + "\n")
    out = subprocess.run([REF_TREE_BIN, "result.txt"], cwd=tmp_path, check=True, capture_output=True, text=True, timeout=900).stdout
    ref = [float(line.split("average_loss ")[1].split(",")[0]) for line in out.split("\n") if line.startswith("epoc ")]
    assert len(ref) == 6

    mark = oracle_lib.mark()
    oracle_lib.set_math(0)
    model = HostPrograms(oracle_lib, ORA_HOSTS, "orah_").model("treelstm_nips18", 1, seed=1)
    model.set_table(emb)
    x = np.zeros(1, np.float32)
    ours = []
    for epoch in range(6):
        avg = np.float32(0)
        for n, y in enumerate(trees):                              # average_loss = average_loss * n / (n + 1) + loss / (n + 1)
            loss = np.float32(model.step(x, y, 0.05))
            avg = np.float32(avg * np.float32(n) / np.float32(n + 1) + loss / np.float32(n + 1))
        ours.append(float(avg))
    model.close()
    oracle_lib.reset(mark)
    assert np.allclose(ours, ref, rtol=2e-4), list(zip(ours, ref))
    assert ours[-1] < ours[0]
